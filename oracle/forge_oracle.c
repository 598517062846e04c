/* CPU oracle for the forge_b200 parity tests - TEST INFRASTRUCTURE, never a product path.
 *
 * A plain-C restatement of the algorithms on Forge's quantized-inference path, each function
 * following the reference's own host test loop or kernel source (cited per function, paths
 * inside the Forge tree). Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg
 * may call into this file.
 *
 * Parity status:
 *   - integer functions (s32 GEMM, 2:4 prune/compress, metadata pack, pruned-dense GEMM) are
 *     exact and are pinned against the reference's own CPU test loops
 *     (tests/test_prune_compress.cu:11-47, tests/test_pack_metadata.cu:21-31) and, on a GPU,
 *     against the reference kernels compiled from their sources (oracle/_ref).
 *   - dequant is IEEE fp32 with the reference kernels' operation order and flush-to-zero,
 *     exact against the reference GPU kernels.
 *   - quantize uses IEEE divide where the reference's fast-math build uses
 *     div.approx / rcp.approx, so int8 values can differ by one step (the reference's own
 *     test allows +-1, tests/test_quantize.cu:80). Bit-exact pinning of the quantizer is done
 *     against the reference GPU kernel (oracle/_ref), not against this function.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- fp16 <-> fp32 (IEEE binary16, round-to-nearest-even), no compiler extensions ---- */

static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) return (uint16_t)(sign | (absx > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* rounds to inf */
    if (absx < 0x33000001u) return sign;                                   /* rounds to zero */
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_man;
    if (exp < -14) {                       /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        half_man = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    shift = 13;
    half_man = man >> shift;
    {
        const uint32_t rem = man & 0x1FFFu;
        if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1u))) half_man++;
    }
    /* half_man includes the implicit bit (0x400); a carry out of the mantissa bumps the exponent */
    return (uint16_t)(sign | (uint16_t)((((uint32_t)(exp + 15)) << 10) + (half_man - 0x400u)));
}

/* Flush-to-zero of subnormal fp32 values, as the .ftz PTX operations do on inputs and outputs. */
static float ftz(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7F800000u) == 0) x &= 0x80000000u;
    memcpy(&f, &x, 4);
    return f;
}
static float mul_ftz(float a, float b) { return ftz(ftz(a) * ftz(b)); }
static float fma_ftz(float a, float b, float c) { return ftz(fmaf(ftz(a), ftz(b), ftz(c))); }

uint16_t oracle_float_to_half(float f) { return float_to_half(f); }
float oracle_half_to_float(uint16_t h) { return half_to_float(h); }

/* ---- s32 GEMM: C[m,n] = sum_k A[m,k] * B[n,k]; tests/test_int8_dense_gemm.cu:35-39 ---- */
void oracle_int8_gemm_s32(const int8_t* A, const int8_t* B, int32_t* C, int M, int K, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        const int8_t* a = A + (size_t)m * K;
        for (int n = 0; n < N; n++) {
            const int8_t* b = B + (size_t)n * K;
            int32_t acc = 0;
            for (int k = 0; k < K; k++) acc += (int32_t)a[k] * (int32_t)b[k];
            C[(size_t)m * N + n] = acc;
        }
    }
}

/* ---- per-token quantize; tests/test_quantize.cu:28-42 with round-half-even
 * (tests/test_int8_sparse_gemm.cu:247-249), the rounding cvt.rni performs ---- */
void oracle_quantize(const uint16_t* x, int8_t* q, float* scales, int M, int K) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        const uint16_t* row = x + (size_t)m * K;
        float amax = 0.0f;
        for (int k = 0; k < K; k++) {
            const float v = fabsf(half_to_float(row[k]));
            if (v > amax) amax = v;
        }
        const float scale = (amax > 1e-8f ? amax : 1e-8f) / 127.0f;
        const float inv = 1.0f / scale;
        scales[m] = scale;
        for (int k = 0; k < K; k++) {
            int v = (int)nearbyintf(half_to_float(row[k]) * inv);
            if (v > 127) v = 127;
            if (v < -128) v = -128;
            q[(size_t)m * K + k] = (int8_t)v;
        }
    }
}

/* ---- standalone dequant + bias; src/quant/dequantize.cu:22-26 as compiled with fast-math:
 * fp16(fma.rn.ftz(mul.ftz(f32(acc), act_scale), f32(w_scale), f32(bias))) ---- */
void oracle_dequantize_bias(const int32_t* acc, const float* act_scale, const uint16_t* w_scale,
                            const uint16_t* bias, uint16_t* out, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            const float t = mul_ftz((float)acc[(size_t)m * N + n], act_scale[m]);
            const float w = half_to_float(w_scale[n]);
            const float o = bias ? fma_ftz(t, w, half_to_float(bias[n])) : mul_ftz(t, w);
            out[(size_t)m * N + n] = float_to_half(o);
        }
    }
}

/* ---- GEMM-epilogue dequant; src/gemm/int8_dense.cu:171-174, src/gemm/int8_sparse.cu:659-661:
 * fp16(fma.rn.ftz(f32(acc), mul.ftz(act_scale, f32(w_scale)), f32(bias))) ---- */
void oracle_dequantize_gemm_epilogue(const int32_t* acc, const float* act_scale, const uint16_t* w_scale,
                                     const uint16_t* bias, uint16_t* out, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            const float s = mul_ftz(act_scale[m], half_to_float(w_scale[n]));
            const float a = (float)acc[(size_t)m * N + n];
            const float o = bias ? fma_ftz(a, s, half_to_float(bias[n])) : mul_ftz(a, s);
            out[(size_t)m * N + n] = float_to_half(o);
        }
    }
}

/* ---- gated epilogue (no reference counterpart; the composition this library defines):
 * g = fma.rn.ftz(f32(acc_g), mul.ftz(act_scale, wg_scale), bg) and u likewise, both fp32 and
 * bit-reproducible here; h = SiLU(g) * u with SiLU(x) = x / (1 + exp(-x))
 * (include/forge/primitives/activation.cuh:66-69) evaluated in double; one rounding to fp16.
 * The GPU evaluates SiLU in fp32 with approximate exp/divide, so it is compared to this within
 * 1 fp16 ulp, not bit-exactly. ---- */
void oracle_gated_epilogue(const int32_t* acc_g, const int32_t* acc_u, const float* act_scale,
                           const uint16_t* wg_scale, const uint16_t* wu_scale, const uint16_t* bg, const uint16_t* bu,
                           uint16_t* out, int M, int N) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            const float sg = mul_ftz(act_scale[m], half_to_float(wg_scale[n]));
            const float su = mul_ftz(act_scale[m], half_to_float(wu_scale[n]));
            const float ag = (float)acc_g[(size_t)m * N + n], au = (float)acc_u[(size_t)m * N + n];
            const float g = bg ? fma_ftz(ag, sg, half_to_float(bg[n])) : mul_ftz(ag, sg);
            const float u = bu ? fma_ftz(au, su, half_to_float(bu[n])) : mul_ftz(au, su);
            const double h = ((double)g / (1.0 + exp(-(double)g))) * (double)u;
            out[(size_t)m * N + n] = float_to_half((float)h);
        }
    }
}

/* ---- 2:4 prune decision for one group; src/sparsity/prune_compress.cu:33-59 ---- */
static void prune_group(const int8_t* v, int* keep0, int* keep1) {
    int a[4];
    for (int i = 0; i < 4; i++) a[i] = abs((int)v[i]);
    int min1 = 0, min2 = 1;
    if (a[min1] > a[min2]) { int t = min1; min1 = min2; min2 = t; }
    for (int i = 2; i < 4; i++) {
        if (a[i] < a[min1]) { min2 = min1; min1 = i; }
        else if (a[i] < a[min2]) { min2 = i; }
    }
    int k[2], ki = 0;
    for (int i = 0; i < 4; i++) if (i != min1 && i != min2) k[ki++] = i;
    *keep0 = k[0];
    *keep1 = k[1];
}

/* ---- prune + compress; tests/test_prune_compress.cu:11-47 ---- */
void oracle_prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K) {
    const int gpr = K / 4;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < N; row++) {
        for (int g = 0; g < gpr; g++) {
            const int8_t* v = weight + (size_t)row * K + g * 4;
            int k0, k1;
            prune_group(v, &k0, &k1);
            compressed[(size_t)row * (K / 2) + g * 2] = v[k0];
            compressed[(size_t)row * (K / 2) + g * 2 + 1] = v[k1];
            metadata_raw[(size_t)row * gpr + g] = (uint8_t)(k0 | (k1 << 2));
        }
    }
}

/* ---- dense weight with the pruned positions zeroed; tests/test_int8_sparse_gemm.cu:26-44 ---- */
void oracle_prune_24_dense(const int8_t* weight, int8_t* pruned, int N, int K) {
    memset(pruned, 0, (size_t)N * K);
#pragma omp parallel for schedule(static)
    for (int row = 0; row < N; row++) {
        for (int g = 0; g < K / 4; g++) {
            const int8_t* v = weight + (size_t)row * K + g * 4;
            int k0, k1;
            prune_group(v, &k0, &k1);
            pruned[(size_t)row * K + g * 4 + k0] = v[k0];
            pruned[(size_t)row * K + g * 4 + k1] = v[k1];
        }
    }
}

/* ---- metadata pack; tests/test_pack_metadata.cu:21-31 ---- */
void oracle_pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K) {
    const int gpr = K / 4, cpr = K / 32;
    for (int row = 0; row < N; row++) {
        for (int c = 0; c < cpr; c++) {
            uint32_t p = 0;
            for (int g = 0; g < 8; g++) p |= ((uint32_t)(meta_raw[(size_t)row * gpr + c * 8 + g] & 0xF)) << (g * 4);
            meta_packed[(size_t)row * cpr + c] = p;
        }
    }
}

/* ---- 2:4-sparse s32 GEMM from the compressed form: out[m,n] = sum over groups of the two
 * kept weights times the activations their nibble selects (the contraction the reference's
 * mma.sp performs, src/gemm/int8_sparse.cu:549-569, restated on the public data layout) ---- */
void oracle_sparse_gemm_s32(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, int32_t* out, int M,
                            int K, int N_out) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++) {
        const int8_t* xr = x + (size_t)m * K;
        for (int n = 0; n < N_out; n++) {
            const int8_t* wc = W_comp + (size_t)n * (K / 2);
            const uint32_t* me = w_meta + (size_t)n * (K / 32);
            int32_t acc = 0;
            for (int g = 0; g < K / 4; g++) {
                const uint32_t nib = (me[g >> 3] >> (4 * (g & 7))) & 0xF;
                acc += (int32_t)wc[2 * g] * xr[4 * g + (nib & 3)] + (int32_t)wc[2 * g + 1] * xr[4 * g + (nib >> 2)];
            }
            out[(size_t)m * N_out + n] = acc;
        }
    }
}

/* ---- INT8 convolution callers of the GEMM ------------------------------------------------
 * src/nn/int8_conv2d.cu:41-80 (im2col with the row = one output position's patch, taps in
 * (c, kh, kw) order, zero outside the image) and :165-221 (per sample: im2col -> per-row
 * quantize -> GEMM + dequant + bias -> transpose to NCHW). The column matrix here holds all
 * samples one after the other: row = n * H_out * W_out + position. ---- */
static int conv_out_size(int in, int pad, int dil, int k, int stride) {
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
}

void oracle_im2col(const uint16_t* input, uint16_t* col, int N, int C_in, int H, int W, int kH, int kW, int padH,
                   int padW, int strideH, int strideW, int dilH, int dilW) {
    const int H_out = conv_out_size(H, padH, dilH, kH, strideH);
    const int W_out = conv_out_size(W, padW, dilW, kW, strideW);
    const int K = C_in * kH * kW;
    const long long rows = (long long)N * H_out * W_out;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < rows; r++) {
        const int n = (int)(r / ((long long)H_out * W_out));
        const int sp = (int)(r % ((long long)H_out * W_out));
        const int ho = sp / W_out, wo = sp % W_out;
        const uint16_t* in_n = input + (size_t)n * C_in * H * W;
        uint16_t* dst = col + (size_t)r * K;
        int k = 0;
        for (int c = 0; c < C_in; c++)
            for (int kh = 0; kh < kH; kh++)
                for (int kw = 0; kw < kW; kw++, k++) {
                    const int h = ho * strideH + kh * dilH - padH;
                    const int w = wo * strideW + kw * dilW - padW;
                    dst[k] = (h >= 0 && h < H && w >= 0 && w < W) ? in_n[((size_t)c * H + h) * W + w] : 0;
                }
    }
}

/* GEMM output (N*HW, C_out) fp16 -> NCHW; src/nn/int8_conv2d.cu:107-119 per sample. */
void oracle_rows_to_nchw(const uint16_t* gemm_out, uint16_t* output, int N, int HW, int C_out) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
        for (int s = 0; s < HW; s++)
            for (int c = 0; c < C_out; c++)
                output[((size_t)n * C_out + c) * HW + s] = gemm_out[((size_t)n * HW + s) * C_out + c];
}

/* Whole conv on the CPU with this file's quantizer (so +-1 int8 step from the GPU quantizer). */
void oracle_int8_conv2d(const uint16_t* input, const int8_t* weight, const uint16_t* w_scale, const uint16_t* bias,
                        uint16_t* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW,
                        int strideH, int strideW, int dilH, int dilW) {
    const int H_out = conv_out_size(H, padH, dilH, kH, strideH);
    const int W_out = conv_out_size(W, padW, dilW, kW, strideW);
    const int K = C_in * kH * kW;
    const long long rows = (long long)N * H_out * W_out;
    uint16_t* col = (uint16_t*)malloc((size_t)rows * K * 2);
    int8_t* q = (int8_t*)malloc((size_t)rows * K);
    float* as = (float*)malloc((size_t)rows * 4);
    int32_t* acc = (int32_t*)malloc((size_t)rows * C_out * 4);
    uint16_t* g = (uint16_t*)malloc((size_t)rows * C_out * 2);
    oracle_im2col(input, col, N, C_in, H, W, kH, kW, padH, padW, strideH, strideW, dilH, dilW);
    oracle_quantize(col, q, as, (int)rows, K);
    oracle_int8_gemm_s32(q, weight, acc, (int)rows, K, C_out);
    oracle_dequantize_gemm_epilogue(acc, as, w_scale, bias, g, (int)rows, C_out);
    oracle_rows_to_nchw(g, output, N, H_out * W_out, C_out);
    free(col); free(q); free(as); free(acc); free(g);
}

/* 2x2 stride-2 transposed conv, scatter step; src/nn/int8_conv_transpose2d.cu:70-101: GEMM output
 * (N*H*W, 4*C_out) fp16 computed with the channel scale replicated 4x and NO bias; column
 * n = co*4 + kh*2 + kw goes to output pixel (2h+kh, 2w+kw) of channel co; the bias is added in fp32
 * to the already rounded fp16 value and the sum is rounded to fp16 again. */
void oracle_conv_transpose_k2s2_scatter(const uint16_t* gemm_out, const uint16_t* bias, uint16_t* output, int N,
                                        int H, int W, int C_out) {
    const int Ng = 4 * C_out;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
        for (int h = 0; h < H; h++)
            for (int w = 0; w < W; w++)
                for (int j = 0; j < Ng; j++) {
                    const int co = j / 4, kh = (j % 4) / 2, kw = j % 2;
                    float v = half_to_float(gemm_out[(((size_t)n * H + h) * W + w) * Ng + j]);
                    if (bias) v = v + half_to_float(bias[co]);
                    output[(((size_t)n * C_out + co) * 2 * H + 2 * h + kh) * 2 * W + 2 * w + kw] = float_to_half(v);
                }
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1 for every rank; a baseline that is meant to use
 * the host's cores sets the count explicitly. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
