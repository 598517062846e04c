// 2:4-sparse INT8 GEMM for very few tokens (one or two by default, template instances up to four):
// a weight-streaming kernel on the CUDA cores.
//
// With so few tokens the call is a pass over the compressed weight (N_out x K/2 bytes) and its
// metadata (N_out x K/8 bytes) and nothing else: 0.625 bytes per weight element against a handful
// of integer operations. The tcgen05 kernel's fixed costs (tensor-map fetch, TMEM allocation,
// 128-row tiles that leave SMs idle when N_out / 128 < SM count, commit -> TMEM read -> store at
// the end) are then most of its time. Here every SM streams rows with plain 16-byte loads, many in
// flight per thread, and the 2:4 selection is a byte permute:
//
//   lane l of a warp owns the 32-deep K chunks l, l + 32, ... of the warp's current weight row:
//   16 compressed bytes (4 words of 4 weights = 2 groups each) + one metadata word (8 nibbles).
//   The 2-bit position fields of the metadata word are spread to nibbles, which makes them the
//   selector operands of four PRMT instructions that pick, from the 8 activation bytes of two
//   groups, the 4 bytes the 4 kept weights multiply; DP4A accumulates in int32. A lane needs the
//   same slice of the token rows for every weight row: for K <= 4096 it keeps that slice in
//   registers (re-reading it from shared memory per weight row costs more shared-memory bandwidth
//   than the weights cost HBM bandwidth), for larger K the token rows sit in shared memory.
//
// Exact int32 accumulation, the same fp32 epilogue as the tensor-core kernels: results are
// bit-identical to them. Replaces, for M <= 2, the reference's split-K small-M configurations
// (src/gemm/int8_sparse.cu:610-632, 885-920).
#include "common.cuh"
#include "gemv_common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"
#include "gemm_sparse.cuh"

namespace fb200 {

using namespace gemv;

namespace {

// 16 bits holding eight 2-bit fields -> 32 bits with each field in the low half of its own nibble.
__device__ __forceinline__ uint32_t spread_fields(uint32_t x) {
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    return x;
}

// acc += sum over the 4 weights of `w` (two groups: positions sel[0..1] of a_lo, sel[2..3] of a_hi)
__device__ __forceinline__ int dot_selected(uint32_t w, uint32_t a_lo, uint32_t a_hi, uint32_t sel, int acc) {
    return __dp4a(static_cast<int>(w), static_cast<int>(__byte_perm(a_lo, a_hi, sel)), acc);
}

// One weight row against the lane's activation chunks: 4 chunks of 32 K per lane and pass.
template <int MT>
__device__ __forceinline__ void gemv_chunk(const uint4& w, uint32_t meta, const uint4 (&a)[MT], const uint4 (&b)[MT],
                                           int (&acc)[MT]) {
    const uint32_t s_lo = spread_fields(meta & 0xFFFFu) | 0x44004400u;
    const uint32_t s_hi = spread_fields(meta >> 16) | 0x44004400u;
#pragma unroll
    for (int m = 0; m < MT; m++) {
        int s = acc[m];
        s = dot_selected(w.x, a[m].x, a[m].y, s_lo, s);
        s = dot_selected(w.y, a[m].z, a[m].w, s_lo >> 16, s);
        s = dot_selected(w.z, b[m].x, b[m].y, s_hi, s);
        s = dot_selected(w.w, b[m].z, b[m].w, s_hi >> 16, s);
        acc[m] = s;
    }
}

// K <= 4096: a lane's slice of every token row (at most 4 chunks of 32 bytes per token) is the same for
// every weight row, so it lives in registers for the whole kernel - no shared memory, no barrier.
// The next row's weights are requested before the current row is reduced.
// EPI 0: out is int32 (M, N_out); EPI 1: fp16 dequant (+ bias).
// FQ: `x` holds the FP16 activations instead (M rows of K halves) and `act_scale` is unused: every
// warp quantizes the token rows itself - it holds a whole row across its lanes, so the row maximum
// is a warp reduction - with the quantizer's exact arithmetic (quantize_rows_kernel), which makes
// the call bit-identical to quantize + GEMM without the second launch and the int8 round trip.
template <int MT, int EPI, bool FQ = false>
__global__ void __launch_bounds__(kGemvThreads)
sparse_gemv_reg_kernel(const int8_t* __restrict__ W_comp, const void* __restrict__ x_any,
                       const uint32_t* __restrict__ w_meta, const float* __restrict__ act_scale,
                       const __half* __restrict__ w_scale, const __half* __restrict__ bias, void* __restrict__ out,
                       int M, int K, int N_out) {
    const int chunks = K >> 5;   // <= 128
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kGemvWarps + warp;
    const int row_step = gridDim.x * kGemvWarps;
    if (!FQ && row0 >= N_out) return;   // FQ: every warp takes part in the block-wide quantization first

    uint4 wv[4], wn[4];
    uint32_t mv[4], mn[4];
    auto load_row = [&](int row, uint4 (&w)[4], uint32_t (&m)[4]) {
        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(W_comp) + (size_t)row * (K >> 1);
        const uint32_t* mrow = w_meta + (size_t)row * chunks;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = i * 32 + lane;
            if (c < chunks) {
                w[i] = ldg_stream16(wrow + (size_t)c * 16);
                m[i] = ldg_stream4(mrow + c);
            }
        }
    };
    RowScale rs = {0.f, 0.f}, rs_next = rs;
    if (row0 < N_out) {
        load_row(row0, wv, mv);   // in flight while the activations are fetched
        rs = load_row_scale<EPI>(w_scale, bias, row0);
        rs_next = rs;
    }
    const bool has_bias = bias != nullptr;
    // launched behind the quantizer of the same linear call: the first weight row is already in
    // flight; the activations and their scales are that kernel's output
    ptx::griddep_wait();
    float as[MT];
    uint4 xa[4][MT], xb[4][MT];
    if constexpr (!FQ) {
        const int8_t* x = static_cast<const int8_t*>(x_any);
#pragma unroll
        for (int m = 0; m < MT; m++) as[m] = (EPI == 1 && m < M) ? act_scale[m] : 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = i * 32 + lane;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                xa[i][m] = make_uint4(0, 0, 0, 0);
                xb[i][m] = make_uint4(0, 0, 0, 0);
                if (c < chunks && m < M) {
                    const uint4* p = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)c * 32);
                    xa[i][m] = p[0];
                    xb[i][m] = p[1];
                }
            }
        }
    } else {
        // The block quantizes each token row once into shared memory: thread t holds 16-byte pieces t and
        // t + 256 of the row (K <= 4096: at most 512 pieces), the row maximum is a warp reduction plus one
        // exchange through shared memory, and every lane then picks up its chunks as int8.
        const __half* xh = static_cast<const __half*>(x_any);
        __shared__ __align__(16) uint8_t xq_s[MT][4096];
        __shared__ float part[MT][kGemvWarps];
        const int nvec = K >> 3;
        uint4 hv[MT][2];
        float scale_m[MT], inv_m[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) {
            __half2 hmax = __float2half2_rn(0.f);
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int idx = threadIdx.x + u * kGemvThreads;
                hv[m][u] = make_uint4(0u, 0u, 0u, 0u);
                if (m < M && idx < nvec) hv[m][u] = __ldg(reinterpret_cast<const uint4*>(xh + (size_t)m * K) + idx);
                const __half2* h = reinterpret_cast<const __half2*>(&hv[m][u]);
#pragma unroll
                for (int e = 0; e < 4; e++) hmax = __hmax2(hmax, __habs2(h[e]));
            }
            float tmax = max_ftz(__low2float(hmax), __high2float(hmax));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tmax = max_ftz(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            if (lane == 0) part[m][warp] = tmax;
        }
        __syncthreads();
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float r = part[m][0];
#pragma unroll
            for (int w = 1; w < kGemvWarps; w++) r = max_ftz(r, part[m][w]);
            quant_scale(r, scale_m[m], inv_m[m]);
            as[m] = (m < M) ? scale_m[m] : 0.f;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int idx = threadIdx.x + u * kGemvThreads;
                if (idx < nvec) {
                    const __half2* h = reinterpret_cast<const __half2*>(&hv[m][u]);
                    int q[8];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(h[e]);
                        q[2 * e] = cvt_rni_ftz(mul_ftz(f.x, inv_m[m]));
                        q[2 * e + 1] = cvt_rni_ftz(mul_ftz(f.y, inv_m[m]));
                    }
                    *reinterpret_cast<uint2*>(&xq_s[m][idx * 8]) =
                        make_uint2(pack4_sat(q[0], q[1], q[2], q[3]), pack4_sat(q[4], q[5], q[6], q[7]));
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = i * 32 + lane;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                xa[i][m] = make_uint4(0, 0, 0, 0);
                xb[i][m] = make_uint4(0, 0, 0, 0);
                if (c < chunks && m < M) {
                    xa[i][m] = *reinterpret_cast<const uint4*>(&xq_s[m][c * 32]);
                    xb[i][m] = *reinterpret_cast<const uint4*>(&xq_s[m][c * 32 + 16]);
                }
            }
        }
    }

    for (int row = row0; row < N_out; row += row_step) {
        const int next = row + row_step;
        if (next < N_out) {
            load_row(next, wn, mn);
            rs_next = load_row_scale<EPI>(w_scale, bias, next);
        }
        int acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (i * 32 + lane < chunks) gemv_chunk<MT>(wv[i], mv[i], xa[i], xb[i], acc);
        }
        gemv_store<MT, EPI>(acc, lane, row, out, as, rs, has_bias, M, N_out);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wv[i] = wn[i];
            mv[i] = mn[i];
        }
        rs = rs_next;
    }
}

// Any K (token rows up to 96 KB): the token rows sit in shared memory, for each token two arrays of
// K/32 uint4 - bytes [0,16) and [16,32) of every 32-byte chunk - so that a warp's reads are conflict-free.
template <int MT, int EPI>
__global__ void __launch_bounds__(kGemvThreads)
sparse_gemv_smem_kernel(const int8_t* __restrict__ W_comp, const int8_t* __restrict__ x,
                        const uint32_t* __restrict__ w_meta, const float* __restrict__ act_scale,
                        const __half* __restrict__ w_scale, const __half* __restrict__ bias, void* __restrict__ out,
                        int M, int K, int N_out) {
    extern __shared__ uint4 xs[];   // [MT][2][K / 32]
    const int chunks = K >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kGemvWarps + warp;
    const int row_step = gridDim.x * kGemvWarps;
    const bool has_bias = bias != nullptr;

    // the first 128 chunks of a row are requested one row ahead (for K <= 4096 that is the whole row)
    uint4 wv[4], wn[4];
    uint32_t mv[4], mn[4];
    auto load_head = [&](int row, uint4 (&w)[4], uint32_t (&m)[4]) {
        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(W_comp) + (size_t)row * (K >> 1);
        const uint32_t* mrow = w_meta + (size_t)row * chunks;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = i * 32 + lane;
            if (c < chunks) {
                w[i] = ldg_stream16(wrow + (size_t)c * 16);
                m[i] = ldg_stream4(mrow + c);
            }
        }
    };
    RowScale rs = {0.f, 0.f}, rs_next = rs;
    if (row0 < N_out) {
        load_head(row0, wv, mv);   // in flight while the activations are staged
        rs = load_row_scale<EPI>(w_scale, bias, row0);
    }
    ptx::griddep_wait();   // see sparse_gemv_reg_kernel
    for (int i = threadIdx.x; i < MT * chunks * 2; i += kGemvThreads) {
        const int m = i / (chunks * 2);
        const int r = i - m * chunks * 2;
        const int c = r >> 1, half = r & 1;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)c * 32 + half * 16);
        xs[(m * 2 + half) * chunks + c] = v;
    }
    float as[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) as[m] = (EPI == 1 && m < M) ? act_scale[m] : 0.f;
    __syncthreads();

    for (int row = row0; row < N_out; row += row_step) {
        const int next = row + row_step;
        if (next < N_out) {
            load_head(next, wn, mn);
            rs_next = load_row_scale<EPI>(w_scale, bias, next);
        }
        int acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0;
        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(W_comp) + (size_t)row * (K >> 1);
        const uint32_t* mrow = w_meta + (size_t)row * chunks;
        for (int c0 = 0; c0 < chunks; c0 += 128) {
            if (c0 > 0) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int c = c0 + i * 32 + lane;
                    if (c < chunks) {
                        wv[i] = ldg_stream16(wrow + (size_t)c * 16);
                        mv[i] = ldg_stream4(mrow + c);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = c0 + i * 32 + lane;
                if (c < chunks) {
                    uint4 a[MT], b[MT];
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        a[m] = xs[(m * 2 + 0) * chunks + c];
                        b[m] = xs[(m * 2 + 1) * chunks + c];
                    }
                    gemv_chunk<MT>(wv[i], mv[i], a, b, acc);
                }
            }
        }
        gemv_store<MT, EPI>(acc, lane, row, out, as, rs, has_bias, M, N_out);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            wv[i] = wn[i];
            mv[i] = mn[i];
        }
        rs = rs_next;
    }
}

template <int MT, int EPI>
int launch_gemv(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out, cudaStream_t stream) {
    const long long blocks_for_rows = ((long long)N_out + kGemvWarps - 1) / kGemvWarps;
    // K <= 4096: token slices in registers (measured faster with the FP16 epilogue for one and two tokens);
    // larger K: token rows in shared memory. Knob 5 pins a variant (1 registers, 2 shared memory).
    const int pin = tuning_knob(kKnobGemvVariant);
    const bool in_regs = K <= 4096 && pin != 2;
    if (in_regs) {
        // resident CTAs per SM by register use; every warp has two rows of weights in flight
        const int per_sm = MT <= 2 ? 2 : 1;
        const int grid = (int)std::min<long long>(blocks_for_rows, (long long)sm_count() * per_sm);
        return launch_gemm(sparse_gemv_reg_kernel<MT, EPI>, dim3(grid), dim3(kGemvThreads), 0, stream, W_comp,
                           static_cast<const void*>(x), w_meta, act_scale, w_scale, bias, out, M, K, N_out) == cudaSuccess
                   ? kOk
                   : kLaunchFailed;
    }
    const size_t smem = (size_t)MT * K;   // MT token rows of K bytes
    auto kern = sparse_gemv_smem_kernel<MT, EPI>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && !attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = true;
    }
    const int per_sm = smem <= 16 * 1024 ? (MT == 1 ? 4 : 3) : (smem <= 48 * 1024 ? 2 : 1);
    const int grid = (int)std::min<long long>(blocks_for_rows, (long long)sm_count() * per_sm);
    return launch_gemm(kern, dim3(grid), dim3(kGemvThreads), smem, stream, W_comp, x, w_meta, act_scale, w_scale, bias, out,
                       M, K, N_out) == cudaSuccess
               ? kOk
               : kLaunchFailed;
}

}  // namespace

bool sparse_gemv_fits(int M, int K) {
    // beyond two tokens the tensor-core kernel wins (measured at N_out = 11008, K = 4096); knob 6 moves the limit
    const int max_tokens = tuning_knob(kKnobGemvMaxTokens) > 0 ? std::min(4, tuning_knob(kKnobGemvMaxTokens)) : 2;
    if (M < 1 || M > max_tokens || K % 32 != 0) return false;
    if (K <= 4096) return true;
    return M <= 2 && (size_t)M * K <= 96 * 1024;      // shared-memory kernel only
}

int sparse_gemv(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out, cudaStream_t stream,
                int epi) {
    const int mt = M <= 1 ? 1 : (M <= 2 ? 2 : 4);
#define FB200_GEMV(MT)                                                                                              \
    return epi == 0 ? launch_gemv<MT, 0>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream)     \
                    : launch_gemv<MT, 1>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream)
    if (mt == 1) { FB200_GEMV(1); }
    if (mt == 2) { FB200_GEMV(2); }
    FB200_GEMV(4);
#undef FB200_GEMV
}

// FP16 activations in, FP16 result out: the per-token quantization happens inside the streaming kernel
// (one or two tokens, K <= 4096, K % 32 == 0, x 16-byte aligned). Same bits as quantize + sparse GEMM.
bool sparse_gemv_fq_fits(int M, int K, const void* x) {
    return M >= 1 && M <= 2 && K % 32 == 0 && K <= 4096 && aligned16(x) && tuning_knob(kKnobGemvVariant) != 2 &&
           tuning_knob(kKnobSparseTile) == 0;
}

int sparse_gemv_fq(const int8_t* W_comp, const __half* x, const uint32_t* w_meta, const __half* w_scale,
                   const __half* bias, __half* out, int M, int K, int N_out, cudaStream_t stream) {
    if (W_comp == nullptr || x == nullptr || w_meta == nullptr || w_scale == nullptr || out == nullptr)
        return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    const long long blocks_for_rows = ((long long)N_out + kGemvWarps - 1) / kGemvWarps;
    const int grid = (int)std::min<long long>(blocks_for_rows, (long long)sm_count() * 2);
    cudaError_t e;
    if (M == 1)
        e = launch_gemm(sparse_gemv_reg_kernel<1, 1, true>, dim3(grid), dim3(kGemvThreads), 0, stream, W_comp,
                        static_cast<const void*>(x), w_meta, static_cast<const float*>(nullptr), w_scale, bias,
                        static_cast<void*>(out), M, K, N_out);
    else
        e = launch_gemm(sparse_gemv_reg_kernel<2, 1, true>, dim3(grid), dim3(kGemvThreads), 0, stream, W_comp,
                        static_cast<const void*>(x), w_meta, static_cast<const float*>(nullptr), w_scale, bias,
                        static_cast<void*>(out), M, K, N_out);
    return e == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace fb200
