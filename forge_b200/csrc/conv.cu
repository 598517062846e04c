// INT8 convolution callers of the GEMM for sm_100a, as one fused implicit-GEMM kernel.
//
// Replaces forge::nn::int8_conv2d_forward (src/nn/int8_conv2d.cu:151-223: per sample im2col ->
// per-patch quantize -> INT8 GEMM + dequant + bias -> transpose to NCHW, four kernels and three
// workspace round trips) and forge::nn::int8_conv_transpose2d_k2s2_forward
// (src/nn/int8_conv_transpose2d.cu:140-191: NCHW->NHWC, quantize, GEMM against the repacked
// (4*C_out, C_in) weight, scatter + bias). Results are bit-identical to those pipelines: a GEMM row
// is one output position's patch, quantized per row with the quantizer's arithmetic, accumulated
// exactly in s32 and dequantised with the GEMM epilogue's association.
//
// One CTA = 128 output positions (over all samples: no per-sample loop) x up to 256 GEMM columns.
//   warps 0-3  thread t owns position t: pass 1 walks the patch for its absmax, pass 2 walks it
//              again (L1 hits; neighbouring threads read neighbouring pixels) and writes the int8
//              patch 16 taps at a time straight into the K-major 128-byte-swizzled operand layout
//              of a ring of 128-tap stages; afterwards the same thread reads its accumulator row
//              from TMEM (lane t) and stores NCHW (or the 2x2 scatter) directly - a warp store
//              covers 32 consecutive pixels of one channel plane.
//   warp 4     weight tiles into the ring: TMA when the (C_out, K) matrix allows it (K % 16 == 0,
//              aligned), plain loads into the same swizzled layout otherwise.
//   warp 5     TMEM allocation and tcgen05.mma kind::i8 (M = 128, N = columns, K = 32) issue.
// Nothing goes through global scratch: the workspace argument of the reference signatures is
// accepted and unused. Several CTAs are resident per SM, so one CTA's gather overlaps another's
// MMA and stores.
#include <algorithm>

#include "common.cuh"
#include "conv.cuh"
#include "gemm_dense.cuh"
#include "ptx.cuh"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int kRows = 128;                    // output positions per CTA (UMMA M)
constexpr int kStages = 3;
constexpr int kABytes = kRows * 128;          // one 128-tap slab of int8 patches
constexpr int kThreads = 192;

struct ConvShape {
    int N, C_in, H, W;
    int cols;                 // GEMM columns: C_out, or 4 * C_out for the 2x2 transposed conv
    int kH, kW, padH, padW, strideH, strideW, dilH, dilW;
    int H_out, W_out;         // of the GEMM rows (the input grid for the transposed conv)
    int K;                    // taps per patch: C_in * kH * kW
    long long rows;           // N * H_out * W_out
    int ct;                   // columns per CTA (multiple of 16, <= 256)
    int tmem_cols;            // power of two >= max(32, ct)
    int b_by_tma;
    int stages;               // ring depth: min(kStages, 128-tap slabs per patch)
    // input-tile variant: the CTA's positions form a TH x TW block of one sample's output grid and the
    // input window they read (all channels) is brought into shared memory by one TMA load
    int TW, tw_log2, TH, tiles_w, tiles_h;
    int IH, IWp;              // window rows; row pitch in elements (multiple of 8)
    int xoff;                 // window column of the first tap of position (.,0): the load starts 16-byte aligned
    int in_off, in_bytes;     // window's place in shared memory
};

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ uint32_t pack4(int q0, int q1, int q2, int q3) {
    return (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
           ((uint32_t)(q3 & 0xFF) << 24);
}

// The quantizer's value step; the byte in the low 8 bits.
__device__ __forceinline__ uint32_t quant_byte(float x, float inv_scale) {
    return static_cast<uint32_t>(quant_value(x, inv_scale)) & 0xFFu;
}

// Walks the taps of one patch in (c, kh, kw) order.
struct TapWalker {
    int c, kh, kw;
    __device__ __forceinline__ void reset() { c = 0; kh = 0; kw = 0; }
    __device__ __forceinline__ void next(const ConvShape& s) {
        if (++kw == s.kW) {
            kw = 0;
            if (++kh == s.kH) {
                kh = 0;
                ++c;
            }
        }
    }
};

__device__ __forceinline__ float load_tap(const __half* __restrict__ in_n, const ConvShape& s, const TapWalker& t,
                                          int h0, int w0) {
    const int h = h0 + t.kh * s.dilH;
    const int w = w0 + t.kw * s.dilW;
    if ((unsigned)h < (unsigned)s.H && (unsigned)w < (unsigned)s.W)
        return __half2float(__ldg(in_n + ((size_t)t.c * s.H + h) * s.W + w));
    return 0.f;
}

// MODE 0: conv2d, NCHW output. MODE 1: 2x2 stride-2 transposed conv, GEMM column n = co*4 + kh*2 + kw
// scattered to output pixel (2h+kh, 2w+kw), bias added after the fp16 rounding of the GEMM result
// as the reference's scatter kernel does.
// T: taps per channel (kH * kW) known at compile time - 1, 4 or 9 - or 0 for any other kernel size.
// HALO: input-tile variant (needs T > 0); otherwise taps are read from global memory.
template <int MODE, int T, bool HALO>
__global__ void __launch_bounds__(kThreads, HALO ? 4 : 3)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_in,
                  const ConvShape s, const __half* __restrict__ input,
                  const int8_t* __restrict__ weight, const __half* __restrict__ w_scale,
                  const __half* __restrict__ bias, __half* __restrict__ output, int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int stage_bytes = kABytes + s.ct * 128;
    float* s_ws = reinterpret_cast<float*>(smem + s.stages * stage_bytes);   // [ct] weight scales
    float* s_bias = s_ws + 256;                                             // [ct]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_bias + 256);
    uint64_t* full_bar = bars;                 // [kStages]: 4 gather warps + the weight loader
    uint64_t* empty_bar = bars + kStages;      // [kStages]: the MMA commit
    uint64_t* tmem_full = bars + 2 * kStages;  // [1]
    uint64_t* in_full = tmem_full + 1;         // [1]: the input window has landed
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(in_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
    const __half* in_tile = reinterpret_cast<const __half*>(smem + s.in_off);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 600);
        return;
    }
    // position block of this CTA (HALO): sample, block row, block column
    int t_smp = 0, t_bh = 0, t_bw = 0;
    if (HALO) {
        t_bw = blockIdx.x % s.tiles_w;
        const int rest = blockIdx.x / s.tiles_w;
        t_bh = rest % s.tiles_h;
        t_smp = rest / s.tiles_h;
    }
    const int n0 = blockIdx.y * s.ct;            // first GEMM column of this CTA
    const int num_kb = (s.K + 127) / 128;
    const bool has_bias = (bias != nullptr);

    // The loader thread sets up the barriers and starts the window and the first weight tiles at once,
    // so their latency overlaps the TMEM allocation and the rest of the prologue.
    const int b_prefetched = s.b_by_tma ? min(s.stages, num_kb) : 0;
    if (warp_id == 4 && lane == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(&full_bar[i], 5);
            mbar_init(&empty_bar[i], 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(in_full, 1);
        *abort_flag = 0;
        fence_mbar_init();
        if (HALO) {
            mbar_expect_tx(in_full, s.in_bytes);
            tma_load_4d(smem + s.in_off, &tm_in, in_full, t_bw * s.TW * s.strideW - s.padW - s.xoff,
                        t_bh * s.TH * s.strideH - s.padH, 0, t_smp);
        }
        for (int kb = 0; kb < b_prefetched; kb++) {
            mbar_expect_tx(&full_bar[kb], s.ct * 128);
            tma_load_2d(smem + kb * stage_bytes + kABytes, &tm_b, &full_bar[kb], kb * 128, n0);
        }
    }
    if (warp_id == 5) {
        tmem_alloc(tmem_base_slot, s.tmem_cols);
        tmem_relinquish();
    }
    // weight scales and bias of this CTA's columns: loaded now, parked in shared memory before the epilogue
    float r_ws[2] = {0.f, 0.f}, r_bias[2] = {0.f, 0.f};
    if (warp_id < 4) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = threadIdx.x + u * kRows;
            const int n = n0 + i;
            if (i < s.ct && n < s.cols) {
                const int co = (MODE == 1) ? (n >> 2) : n;
                r_ws[u] = __half2float(__ldg(w_scale + co));
                if (has_bias) r_bias[u] = __half2float(__ldg(bias + co));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp_id < 4) {
        // ------------------------------------------------------------ gather + quantize, then epilogue
        bool valid;
        int smp, sp, ho, wo;
        const int hw_out = s.H_out * s.W_out;
        if (HALO) {
            ho = t_bh * s.TH + (threadIdx.x >> s.tw_log2);
            wo = t_bw * s.TW + (threadIdx.x & (s.TW - 1));
            valid = ho < s.H_out && wo < s.W_out;
            smp = t_smp;
            sp = ho * s.W_out + wo;
        } else {
            const long long m = (long long)blockIdx.x * kRows + threadIdx.x;
            valid = m < s.rows;
            smp = valid ? (int)(m / hw_out) : 0;
            sp = valid ? (int)(m - (long long)smp * hw_out) : 0;
            ho = sp / s.W_out;
            wo = sp - ho * s.W_out;
        }
        const int h0 = ho * s.strideH - s.padH, w0 = wo * s.strideW - s.padW;
        const __half* in_n = input + (size_t)smp * s.C_in * s.H * s.W;

        const int r = threadIdx.x;
        bool ok = true;
        float scale, inv;
        if (T > 0) {
            // ---- fast path: the T tap offsets and their in-image flags are per-thread constants
            constexpr int G = (T == 1) ? 16 : (T == 4) ? 8 : 4;   // channels per group: ~32 loads in flight
            int off[T > 0 ? T : 1];
            uint32_t inside = 0;
            size_t plane;
            const __half* pc0;
            if (HALO) {
                // window-relative offsets; the TMA load zero-filled everything outside the image
                const int base = (threadIdx.x >> s.tw_log2) * s.strideH * s.IWp + (threadIdx.x & (s.TW - 1)) * s.strideW +
                                 s.xoff;
#pragma unroll
                for (int j = 0; j < T; j++) {
                    const int kh = j / s.kW, kw = j - kh * s.kW;
                    off[j] = base + kh * s.dilH * s.IWp + kw * s.dilW;
                }
                inside = 0xFFFFFFFFu;
                plane = (size_t)s.IH * s.IWp;
                pc0 = in_tile;
                if (!__all_sync(0xffffffffu, mbar_wait(in_full, 0, abort_flag))) {
                    atomicExch(status, 605);
                    ok = false;
                }
            } else {
#pragma unroll
                for (int j = 0; j < T; j++) {
                    const int kh = j / s.kW, kw = j - kh * s.kW;
                    const int h = h0 + kh * s.dilH, w = w0 + kw * s.dilW;
                    const bool in = valid && (unsigned)h < (unsigned)s.H && (unsigned)w < (unsigned)s.W;
                    off[j] = in ? h * s.W + w : 0;
                    inside |= in ? (1u << j) : 0u;
                }
                plane = (size_t)s.H * s.W;
                pc0 = in_n;
            }
            auto tap = [&](const __half* p, int j) -> float {
                if (HALO) return __half2float(p[off[j]]);
                return ((inside >> j) & 1u) ? __half2float(__ldg(p + off[j])) : 0.f;
            };
            float amax = 0.f;
            if (HALO) {
                // |x| maximum over the channels of every window pixel, two pixels per thread and step,
                // then the maximum over this position's T pixels. (Runs even after a failed wait so
                // that all four warps meet at the barrier; the result is then unused.)
                __half2* pmap = reinterpret_cast<__half2*>(smem + s.in_off + s.in_bytes);
                const __half2* win2 = reinterpret_cast<const __half2*>(in_tile);
                const int pairs = (s.IH * s.IWp) >> 1;
                for (int idx = threadIdx.x; idx < pairs; idx += kRows) {
                    __half2 mx = __float2half2_rn(0.f);
                    const __half2* pw = win2 + idx;
#pragma unroll 8
                    for (int c = 0; c < s.C_in; c++, pw += pairs) mx = __hmax2(mx, __habs2(*pw));
                    pmap[idx] = mx;
                }
                named_barrier_sync(1, kRows);
                const __half* pm = reinterpret_cast<const __half*>(pmap);
#pragma unroll
                for (int j = 0; j < T; j++) amax = max_ftz(amax, __half2float(pm[off[j]]));
            } else if (ok) {
                const __half* pc = pc0;
#pragma unroll G
                for (int c = 0; c < s.C_in; c++, pc += plane) {
#pragma unroll
                    for (int j = 0; j < T; j++) amax = max_ftz(amax, abs_ftz(tap(pc, j)));
                }
            }
            quant_scale(amax, scale, inv);

            // pass 2: G channels = G*T taps = G*T/4 whole 32-bit words of the patch row at a time
            int wi = 0;                 // word index within the patch row; 32 words = one 128-tap stage
            uint8_t* rowp = nullptr;
            auto emit = [&](uint32_t word) {
                if (!ok) return;
                if ((wi & 31) == 0) {
                    const int kb = wi >> 5;
                    const int stage = kb % s.stages;
                    if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], ((kb / s.stages) & 1) ^ 1, abort_flag))) {
                        atomicExch(status, 601);
                        ok = false;
                        return;
                    }
                    rowp = smem + stage * stage_bytes + r * 128;
                }
                *reinterpret_cast<uint32_t*>(rowp + ((((wi >> 2) & 7) ^ (r & 7)) << 4) + ((wi & 3) << 2)) = word;
                if ((wi & 31) == 31) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_bar[(wi >> 5) % s.stages]);
                }
                wi++;
            };
            const __half* pc = pc0;
            int c = 0;
            if (HALO) {
                // GC channels = GC*T taps = whole 16-byte chunks of the patch row
                constexpr int GC = (T == 4) ? 4 : 16;
                constexpr int TT = (T > 0) ? T : 1;
                const int plane_i = s.IH * s.IWp;
                for (; c + GC <= s.C_in; c += GC, pc += GC * plane) {
#pragma unroll
                    for (int ch = 0; ch < GC * T / 16; ch++) {
                        int q[16];
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const int tp = ch * 16 + i;     // tap within the group: channel tp / T, pixel tp % T
                            q[i] = cvt_rni_ftz(mul_ftz(__half2float(pc[(tp / TT) * plane_i + off[tp % TT]]), inv));
                        }
                        if (ok) {
                            if ((wi & 31) == 0) {
                                const int kb = wi >> 5;
                                const int stage = kb % s.stages;
                                if (!__all_sync(0xffffffffu,
                                                mbar_wait(&empty_bar[stage], ((kb / s.stages) & 1) ^ 1, abort_flag))) {
                                    atomicExch(status, 601);
                                    ok = false;
                                }
                                rowp = smem + stage * stage_bytes + r * 128;
                            }
                        }
                        if (ok) {
                            *reinterpret_cast<uint4*>(rowp + ((((wi >> 2) & 7) ^ (r & 7)) << 4)) =
                                make_uint4(pack4_sat(q[0], q[1], q[2], q[3]), pack4_sat(q[4], q[5], q[6], q[7]),
                                           pack4_sat(q[8], q[9], q[10], q[11]), pack4_sat(q[12], q[13], q[14], q[15]));
                            if ((wi & 31) == 28) {
                                fence_proxy_async_smem();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&full_bar[(wi >> 5) % s.stages]);
                            }
                            wi += 4;
                        }
                    }
                }
            }
            for (; c + G <= s.C_in; c += G, pc += G * plane) {
                uint32_t q[G * (T > 0 ? T : 1)];
#pragma unroll
                for (int cc = 0; cc < G; cc++) {
#pragma unroll
                    for (int j = 0; j < T; j++) {
                        q[cc * T + j] = quant_byte(tap(pc + cc * plane, j), inv);
                    }
                }
#pragma unroll
                for (int i = 0; i < G * T / 4; i++)
                    emit(q[4 * i] | (q[4 * i + 1] << 8) | (q[4 * i + 2] << 16) | (q[4 * i + 3] << 24));
            }
            {   // leftover channels (fewer than G): bytes collected with a running shift
                uint32_t word = 0;
                int nb = 0;
                for (; c < s.C_in; c++, pc += plane) {
#pragma unroll
                    for (int j = 0; j < T; j++) {
                        word |= quant_byte(tap(pc, j), inv) << (8 * nb);
                        if (++nb == 4) {
                            emit(word);
                            word = 0;
                            nb = 0;
                        }
                    }
                }
                if (nb != 0) emit(word);
            }
            // a last stage that is not full: taps past K meet zero weights, whatever is in them
            if (ok && (wi & 31) != 0) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_bar[(wi >> 5) % s.stages]);
            }
        } else {
            float amax = 0.f;
            TapWalker tw;
            if (valid) {
                tw.reset();
                for (int k = 0; k < s.K; k++, tw.next(s)) amax = max_ftz(amax, abs_ftz(load_tap(in_n, s, tw, h0, w0)));
            }
            quant_scale(amax, scale, inv);

            tw.reset();
            for (int kb = 0; kb < num_kb; kb++) {
                const int stage = kb % s.stages;
                const uint32_t phase = (kb / s.stages) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) {
                    atomicExch(status, 601);
                    ok = false;
                    break;
                }
                uint8_t* sa = smem + stage * stage_bytes + r * 128;
                int k = kb * 128;
#pragma unroll 1
                for (int ch = 0; ch < 8; ch++) {
                    uint32_t p[4] = {0u, 0u, 0u, 0u};
                    if (valid && k < s.K) {
                        int q[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            q[j] = 0;
                            if (k + j < s.K) {
                                q[j] = quant_value(load_tap(in_n, s, tw, h0, w0), inv);
                                tw.next(s);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++) p[j] = pack4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
                    }
                    k += 16;
                    *reinterpret_cast<uint4*>(sa + ((ch ^ (r & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
                }
                fence_proxy_async_smem();     // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_bar[stage]);
            }
        }

#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int i = threadIdx.x + u * kRows;
            if (i < s.ct) {
                s_ws[i] = r_ws[u];
                s_bias[i] = r_bias[u];
            }
        }
        named_barrier_sync(1, kRows);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(tmem_full, 0, abort_flag));
        if (!ok) {
            atomicExch(status, 602);
        } else {
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp_id * 32) << 16);
            for (int c0 = 0; c0 < s.ct; c0 += 32) {
                if (n0 + c0 >= s.cols) break;
                uint32_t v[32];
                tmem_ld_32x32b_x32(taddr + c0, v);
                tmem_ld_wait();
                if (!valid) continue;
                if (MODE == 0) {
                    __half* dst = output + ((size_t)smp * s.cols + n0 + c0) * hw_out + sp;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (n0 + c0 + j < s.cols) {
                            const float o = dequant_gemm(static_cast<int>(v[j]), mul_ftz(scale, s_ws[c0 + j]),
                                                         s_bias[c0 + j], has_bias);
                            dst[(size_t)j * hw_out] = __float2half_rn(o);
                        }
                    }
                } else {
                    const int c_out = s.cols >> 2;
                    const int W2 = 2 * s.W_out;
#pragma unroll
                    for (int g = 0; g < 8; g++) {          // 4 GEMM columns = one output channel's 2x2 block
                        const int co = ((n0 + c0) >> 2) + g;
                        if (co < c_out) {
                            const float sw = mul_ftz(scale, s_ws[c0 + 4 * g]);
                            float o[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                o[j] = __half2float(__float2half_rn(mul_ftz(static_cast<float>(static_cast<int>(v[4 * g + j])), sw)));
                                if (has_bias) o[j] = __fadd_rn(o[j], s_bias[c0 + 4 * g]);
                            }
                            __half* plane = output + ((size_t)smp * c_out + co) * (size_t)(4 * hw_out);
                            uint32_t* row0 = reinterpret_cast<uint32_t*>(plane + (size_t)(2 * ho) * W2 + 2 * wo);
                            uint32_t* row1 = reinterpret_cast<uint32_t*>(plane + (size_t)(2 * ho + 1) * W2 + 2 * wo);
                            *row0 = pack_half2(o[0], o[1]);
                            *row1 = pack_half2(o[2], o[3]);
                        }
                    }
                }
            }
            tc_fence_before();
        }
    } else if (warp_id == 4) {
        // ------------------------------------------------------------ input window, weight tiles
        bool ok = true;
        for (int kb = b_prefetched; kb < num_kb && ok; kb++) {
            const int stage = kb % s.stages;
            const uint32_t phase = (kb / s.stages) & 1;
            uint8_t* sb = smem + stage * stage_bytes + kABytes;
            if (s.b_by_tma) {
                if (lane == 0) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
                        atomicExch(status, 603);
                        ok = false;
                    } else {
                        mbar_expect_tx(&full_bar[stage], s.ct * 128);
                        tma_load_2d(sb, &tm_b, &full_bar[stage], kb * 128, n0);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
            } else {
                if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag))) {
                    atomicExch(status, 603);
                    ok = false;
                    break;
                }
                // only the 16-byte chunks the MMA steps of this slab read: 2 per 32-tap step
                const int taps = min(128, s.K - kb * 128);
                const int chunks = 2 * ((taps + 31) / 32);
                const bool vec = (s.K % 16 == 0) && aligned16_dev(weight);
                for (int idx = lane; idx < s.ct * chunks; idx += 32) {
                    const int row = idx / chunks, ch = idx - row * chunks;
                    const int n = n0 + row;
                    const int k0 = kb * 128 + ch * 16;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (n < s.cols && k0 < s.K) {
                        const int8_t* src = weight + (size_t)n * s.K + k0;
                        if (vec) {
                            v = __ldg(reinterpret_cast<const uint4*>(src));
                        } else {
                            uint32_t p[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (k0 + j < s.K) p[j >> 2] |= (uint32_t)(uint8_t)__ldg(src + j) << (8 * (j & 3));
                            v = make_uint4(p[0], p[1], p[2], p[3]);
                        }
                    }
                    *reinterpret_cast<uint4*>(sb + row * 128 + ((ch ^ (row & 7)) << 4)) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_bar[stage]);
            }
        }
    } else {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8(kRows, s.ct, false);
            bool ok = true;
            for (int kb = 0; kb < num_kb; kb++) {
                const int stage = kb % s.stages;
                const uint32_t phase = (kb / s.stages) & 1;
                if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                    atomicExch(status, 604);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + stage * stage_bytes);
                const uint64_t desc_a = make_desc_sw128(sa);
                const uint64_t desc_b = make_desc_sw128(sa + kABytes);
                const int steps = min(4, (s.K - kb * 128 + 31) / 32);   // taps past K are zero on both sides
                for (int k = 0; k < steps; k++)
                    umma_i8(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                tc_commit(&empty_bar[stage]);
            }
            if (ok) tc_commit(tmem_full);
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp_id == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, s.tmem_cols);
    }
}

}  // namespace

namespace {

inline int conv_out_size(int in, int pad, int dil, int k, int stride) {
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
}

constexpr int kMiscBytes = 2 * 256 * (int)sizeof(float) + 128;   // scales, bias, barriers
constexpr int kMaxSmem = 227 * 1024;

template <int MODE, int T, bool HALO>
int launch_kernel(const ConvShape& s, const CUtensorMap& tm_b, const CUtensorMap& tm_in, int smem, dim3 grid,
                  const __half* input, const int8_t* weight, const __half* w_scale, const __half* bias,
                  __half* output, cudaStream_t stream) {
    static int attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = conv_igemm_kernel<MODE, T, HALO>;
    if (!attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem) != cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = 1;
    }
    int* status = status_word();
    if (status == nullptr) return kLaunchFailed;
    // Never let more CTAs become resident on an SM than its 512 TMEM columns serve: a CTA that has to
    // wait inside tcgen05.alloc for another one's columns was measured to cost far more than the lost
    // occupancy. Shared memory is the lever: ask for enough that one CTA more would not fit.
    const int by_tmem = 512 / s.tmem_cols;
    const int floor_smem = (228 * 1024) / (by_tmem + 1) - 1024 + 16;
    smem = std::min(std::max(smem, floor_smem), kMaxSmem);
    kern<<<grid, kThreads, smem, stream>>>(tm_b, tm_in, s, input, weight, w_scale, bias, output, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

template <int MODE, int T>
int launch_conv(ConvShape s, const __half* input, const int8_t* weight, const __half* w_scale, const __half* bias,
                __half* output, cudaStream_t stream) {
    if (!device_is_sm100()) return kUnsupportedArch;
    if (input == nullptr || weight == nullptr || w_scale == nullptr || output == nullptr) return kBadPointer;
    if (s.H_out <= 0 || s.W_out <= 0 || s.K <= 0) return kOk;
    // 32-bit index arithmetic inside one sample and one weight row block
    if ((long long)s.C_in * s.H * s.W >= (1ll << 31) || (long long)s.cols * s.K >= (1ll << 31) ||
        (long long)s.H_out * s.W_out >= (1ll << 29))
        return kTooLarge;
    s.rows = (long long)s.N * s.H_out * s.W_out;
    const int n_blocks = (s.cols + 255) / 256;
    s.ct = (((s.cols + n_blocks - 1) / n_blocks) + 15) / 16 * 16;
    s.tmem_cols = 32;
    while (s.tmem_cols < s.ct) s.tmem_cols *= 2;
    // TMA for the weight tiles only when every row starts on a 32-byte sector: with 16- or 48-byte rows
    // the per-row requests of a 128-row box were measured to take microseconds per tile
    s.b_by_tma = (s.K % 32 == 0 && aligned16(weight)) ? 1 : 0;
    s.stages = std::min(kStages, (s.K + 127) / 128);
    const int ring_bytes = s.stages * (kABytes + s.ct * 128);

    CUtensorMap tm_b, tm_in;
    memset(&tm_b, 0, sizeof(tm_b));
    memset(&tm_in, 0, sizeof(tm_in));
    if (s.b_by_tma) {
        const uint64_t dims[2] = {(uint64_t)s.K, (uint64_t)s.cols};
        const uint64_t str[1] = {(uint64_t)s.K};
        const uint32_t box[2] = {128, (uint32_t)s.ct};
        if (!make_tmap(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weight, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }

    // Input-tile variant: TH x TW position blocks whose input window (all channels) is one TMA box.
    bool halo = false;
    if (T > 0 && s.W % 8 == 0 && aligned16(input) && s.C_in <= 256) {
        s.TW = (s.W_out >= 24) ? 32 : (s.W_out >= 12) ? 16 : 8;
        s.tw_log2 = (s.TW == 32) ? 5 : (s.TW == 16) ? 4 : 3;
        s.TH = kRows / s.TW;
        s.tiles_w = (s.W_out + s.TW - 1) / s.TW;
        s.tiles_h = (s.H_out + s.TH - 1) / s.TH;
        s.IH = (s.TH - 1) * s.strideH + (s.kH - 1) * s.dilH + 1;
        const int IW = (s.TW - 1) * s.strideW + (s.kW - 1) * s.dilW + 1;
        // the window starts at column bw*TW*strideW - padW; TW*strideW is a multiple of 8, so rounding
        // the start down to a multiple of 8 elements (16 bytes) shifts every tile by the same xoff
        s.xoff = ((-s.padW % 8) + 8) % 8;
        s.IWp = (IW + s.xoff + 7) / 8 * 8;
        s.in_off = ring_bytes + kMiscBytes;
        const long long in_bytes = (long long)s.C_in * s.IH * s.IWp * 2;
        const long long tiles = (long long)s.N * s.tiles_h * s.tiles_w;
        const long long pmap_bytes = (long long)s.IH * s.IWp * 2;   // per-pixel channel absmax of the window
        if (s.IH <= 256 && s.IWp <= 256 && s.in_off + in_bytes + pmap_bytes <= kMaxSmem && in_bytes <= 112 * 1024 &&
            tiles < (1ll << 31)) {
            s.in_bytes = (int)in_bytes;
            const uint64_t dims[4] = {(uint64_t)s.W, (uint64_t)s.H, (uint64_t)s.C_in, (uint64_t)s.N};
            const uint64_t str[3] = {(uint64_t)s.W * 2, (uint64_t)s.H * s.W * 2, (uint64_t)s.C_in * s.H * s.W * 2};
            const uint32_t box[4] = {(uint32_t)s.IWp, (uint32_t)s.IH, (uint32_t)s.C_in, 1};
            halo = make_tmap(&tm_in, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, input, dims, str, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
        }
    }
    if (halo) {
        dim3 grid((unsigned)(s.N * s.tiles_h * s.tiles_w), (unsigned)n_blocks);
        return launch_kernel<MODE, T, (T > 0)>(s, tm_b, tm_in, s.in_off + s.in_bytes + s.IH * s.IWp * 2, grid, input,
                                               weight, w_scale, bias, output, stream);
    }
    s.in_off = 0;
    s.in_bytes = 0;
    const long long tiles = (s.rows + kRows - 1) / kRows;
    if (tiles >= (1ll << 31)) return kTooLarge;
    dim3 grid((unsigned)tiles, (unsigned)n_blocks);
    return launch_kernel<MODE, T, false>(s, tm_b, tm_in, ring_bytes + kMiscBytes, grid, input, weight, w_scale, bias,
                                         output, stream);
}

}  // namespace

size_t int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW, int strideH,
                                  int strideW, int dilH, int dilW) {
    // the reference's figure (src/nn/int8_conv2d.cu:126-145), so callers that size their buffer
    // with it keep working; this implementation does not touch the buffer
    const long long M = (long long)conv_out_size(H, padH, dilH, kH, strideH) * conv_out_size(W, padW, dilW, kW, strideW);
    const long long K = (long long)C_in * kH * kW;
    return (size_t)(M * K * 2 + M * K + M * 4 + M * C_out * 2);
}

size_t int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out) {
    // src/nn/int8_conv_transpose2d.cu:103-117
    const long long M = (long long)H * W, Ng = 4ll * C_out;
    return (size_t)(M * C_in * 2 + M * C_in + M * 4 + Ng * 2 + M * Ng * 2);
}

int int8_conv2d_forward(const __half* input, const int8_t* weight, const __half* w_scale, const __half* bias,
                        __half* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW,
                        int strideH, int strideW, int dilH, int dilW, cudaStream_t stream) {
    if (N <= 0 || C_in <= 0 || C_out <= 0) return kOk;   // reference: silent no-op (int8_conv2d.cu:165)
    if (kH <= 0 || kW <= 0 || strideH <= 0 || strideW <= 0 || dilH <= 0 || dilW <= 0 || H <= 0 || W <= 0)
        return kBadShape;
    ConvShape s{};
    s.N = N; s.C_in = C_in; s.H = H; s.W = W; s.cols = C_out;
    s.kH = kH; s.kW = kW; s.padH = padH; s.padW = padW; s.strideH = strideH; s.strideW = strideW;
    s.dilH = dilH; s.dilW = dilW;
    s.H_out = conv_out_size(H, padH, dilH, kH, strideH);
    s.W_out = conv_out_size(W, padW, dilW, kW, strideW);
    s.K = C_in * kH * kW;
    switch (kH * kW) {
    case 1: return launch_conv<0, 1>(s, input, weight, w_scale, bias, output, stream);
    case 4: return launch_conv<0, 4>(s, input, weight, w_scale, bias, output, stream);
    case 9: return launch_conv<0, 9>(s, input, weight, w_scale, bias, output, stream);
    default: return launch_conv<0, 0>(s, input, weight, w_scale, bias, output, stream);
    }
}

int int8_conv_transpose2d_k2s2_forward(const __half* input, const int8_t* weight, const __half* w_scale,
                                       const __half* bias, __half* output, int N, int C_in, int H, int W, int C_out,
                                       cudaStream_t stream) {
    if (N <= 0 || C_in <= 0 || C_out <= 0) return kOk;   // int8_conv_transpose2d.cu:135
    if (H <= 0 || W <= 0) return kBadShape;
    if (C_out >= (1 << 28)) return kTooLarge;
    ConvShape s{};
    s.N = N; s.C_in = C_in; s.H = H; s.W = W; s.cols = 4 * C_out;
    s.kH = 1; s.kW = 1; s.padH = 0; s.padW = 0; s.strideH = 1; s.strideW = 1; s.dilH = 1; s.dilW = 1;
    s.H_out = H; s.W_out = W;
    s.K = C_in;
    return launch_conv<1, 1>(s, input, weight, w_scale, bias, output, stream);
}

}  // namespace fb200
