// Dense INT8 GEMM for very few tokens (one or two by default): a weight-streaming kernel on the CUDA cores.
//
// With so few tokens int8_gemm_dequant / int8_linear is one pass over the weight (N x K bytes): the
// tcgen05 kernel has fixed costs (tensor-map fetch, TMEM allocation, a 128-row token tile that is almost
// empty) on top of the 7 us of HBM time of an 11008 x 4096 weight. Here every SM streams
// weight rows with 16-byte loads, one row ahead; the token rows (M x K bytes) sit in shared memory,
// where every warp reads them once per weight row (with dense weights that is one shared-memory byte
// per HBM byte and token, far from the shared-memory limit), and DP4A accumulates in int32.
//
// FQ: the activations arrive as FP16 and the block quantizes each token row into shared memory itself
// (the quantizer's exact arithmetic, quantize_rows_kernel), so int8_linear is one launch without the
// int8 round trip. Exact int32 accumulation and the tensor-core kernels' epilogue: bit-identical to
// them. The reference has no small-M dense path (src/gemm/int8_dense.cu:26-211 runs its 128 x 128
// tiles for every M).
#include "common.cuh"
#include "gemv_common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"

namespace fb200 {

using namespace gemv;

namespace {

constexpr int kHead = 8;   // 16-byte pieces per lane requested one row ahead: 8 x 32 lanes x 16 B = 4096 bytes of a row

template <int MT>
__device__ __forceinline__ void dot_piece(const uint4& w, const uint4* __restrict__ xs4, int pieces, int p, int M,
                                          int (&acc)[MT]) {
#pragma unroll
    for (int m = 0; m < MT; m++) {
        if (m < M) {
            const uint4 a = xs4[m * pieces + p];
            int s = acc[m];
            s = __dp4a(static_cast<int>(w.x), static_cast<int>(a.x), s);
            s = __dp4a(static_cast<int>(w.y), static_cast<int>(a.y), s);
            s = __dp4a(static_cast<int>(w.z), static_cast<int>(a.z), s);
            s = __dp4a(static_cast<int>(w.w), static_cast<int>(a.w), s);
            acc[m] = s;
        }
    }
}

// EPI 0: out is int32 (M, N); EPI 1: fp16 dequant (+ bias). FQ: x_any is FP16 (M, K), act_scale unused.
template <int MT, int EPI, bool FQ>
__global__ void __launch_bounds__(kGemvThreads, 2)
dense_gemv_kernel(const int8_t* __restrict__ W, const void* __restrict__ x_any, const float* __restrict__ act_scale,
                  const __half* __restrict__ w_scale, const __half* __restrict__ bias, void* __restrict__ out, int M,
                  int K, int N) {
    extern __shared__ __align__(16) uint8_t xs[];   // [M][K] int8
    __shared__ float as_s[MT];
    __shared__ float part[MT][kGemvWarps];
    uint4* xs4 = reinterpret_cast<uint4*>(xs);
    const int pieces = K >> 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kGemvWarps + warp;
    const int row_step = gridDim.x * kGemvWarps;
    const bool has_bias = bias != nullptr;

    uint4 wv[kHead], wn[kHead];
    auto load_head = [&](int row, uint4 (&w)[kHead]) {
        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(W) + (size_t)row * K;
#pragma unroll
        for (int j = 0; j < kHead; j++) {
            const int p = lane + 32 * j;
            if (p < pieces) w[j] = ldg_stream16(wrow + (size_t)p * 16);
        }
    };
    RowScale rs = {0.f, 0.f}, rs_next = rs;
    if (row0 < N) {
        load_head(row0, wv);   // in flight while the activations are staged
        rs = load_row_scale<EPI>(w_scale, bias, row0);
        rs_next = rs;
    }
    // launched behind a quantizer (launch_behind_quantizer): the weights above do not depend on it
    ptx::griddep_wait();

    if constexpr (!FQ) {
        const uint4* x4 = static_cast<const uint4*>(x_any);
        for (int i = threadIdx.x; i < M * pieces; i += kGemvThreads) xs4[i] = x4[i];
        if (threadIdx.x < MT) as_s[threadIdx.x] = (EPI == 1 && (int)threadIdx.x < M) ? act_scale[threadIdx.x] : 0.f;
    } else {
        // per token row: block-wide |x| maximum (packed-half, exact), then quantize into shared memory
        const __half* xh = static_cast<const __half*>(x_any);
        const int nvec = K >> 3;   // 16-byte pieces of 8 halves
        for (int m = 0; m < M; m++) {
            const uint4* row = reinterpret_cast<const uint4*>(xh + (size_t)m * K);
            __half2 hmax = __float2half2_rn(0.f);
            for (int i = threadIdx.x; i < nvec; i += kGemvThreads) {
                const uint4 v = __ldg(row + i);
                const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int e = 0; e < 4; e++) hmax = __hmax2(hmax, __habs2(h[e]));
            }
            float tmax = max_ftz(__low2float(hmax), __high2float(hmax));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tmax = max_ftz(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
            if (lane == 0) part[m][warp] = tmax;
        }
        __syncthreads();
        for (int m = 0; m < M; m++) {
            float r = part[m][0];
#pragma unroll
            for (int w = 1; w < kGemvWarps; w++) r = max_ftz(r, part[m][w]);
            float scale, inv;
            quant_scale(r, scale, inv);
            if (threadIdx.x == 0) as_s[m] = scale;
            const uint4* row = reinterpret_cast<const uint4*>(xh + (size_t)m * K);
            uint2* dst = reinterpret_cast<uint2*>(xs + (size_t)m * K);
            for (int i = threadIdx.x; i < nvec; i += kGemvThreads) {
                const uint4 v = __ldg(row + i);   // second read: L1 / L2
                const __half2* h = reinterpret_cast<const __half2*>(&v);
                int q[8];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(h[e]);
                    q[2 * e] = cvt_rni_ftz(mul_ftz(f.x, inv));
                    q[2 * e + 1] = cvt_rni_ftz(mul_ftz(f.y, inv));
                }
                dst[i] = make_uint2(pack4_sat(q[0], q[1], q[2], q[3]), pack4_sat(q[4], q[5], q[6], q[7]));
            }
        }
    }
    __syncthreads();
    float as[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) as[m] = (m < M) ? as_s[m] : 0.f;

    for (int row = row0; row < N; row += row_step) {
        const int next = row + row_step;
        if (next < N) {
            load_head(next, wn);
            rs_next = load_row_scale<EPI>(w_scale, bias, next);
        }
        int acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0;
#pragma unroll
        for (int j = 0; j < kHead; j++) {
            const int p = lane + 32 * j;
            if (p < pieces) dot_piece<MT>(wv[j], xs4, pieces, p, M, acc);
        }
        // K > 4096: the rest of the row, four pieces in flight per lane
        const uint8_t* wrow = reinterpret_cast<const uint8_t*>(W) + (size_t)row * K;
        for (int p0 = lane + 32 * kHead; p0 < pieces; p0 += 128) {
            uint4 t[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (p0 + 32 * u < pieces) t[u] = ldg_stream16(wrow + (size_t)(p0 + 32 * u) * 16);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (p0 + 32 * u < pieces) dot_piece<MT>(t[u], xs4, pieces, p0 + 32 * u, M, acc);
        }
        gemv_store<MT, EPI>(acc, lane, row, out, as, rs, has_bias, M, N);
#pragma unroll
        for (int j = 0; j < kHead; j++) wv[j] = wn[j];
        rs = rs_next;
    }
}

template <int MT, int EPI, bool FQ>
int launch_dense_gemv(const int8_t* W, const void* x, const float* act_scale, const __half* w_scale, const __half* bias,
                      void* out, int M, int K, int N, cudaStream_t stream) {
    auto kern = dense_gemv_kernel<MT, EPI, FQ>;
    const size_t smem = (size_t)M * K;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && !attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = true;
    }
    const long long blocks_for_rows = ((long long)N + kGemvWarps - 1) / kGemvWarps;
    const int per_sm = smem <= 96 * 1024 ? 2 : 1;
    const int grid = (int)std::min<long long>(blocks_for_rows, (long long)sm_count() * per_sm);
    return launch_gemm(kern, dim3(grid), dim3(kGemvThreads), smem, stream, W, x, act_scale, w_scale, bias, out, M, K,
                       N) == cudaSuccess
               ? kOk
               : kLaunchFailed;
}

template <int EPI, bool FQ>
int dispatch_dense_gemv(const int8_t* W, const void* x, const float* act_scale, const __half* w_scale,
                        const __half* bias, void* out, int M, int K, int N, cudaStream_t stream) {
    if (M <= 1) return launch_dense_gemv<1, EPI, FQ>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
    if (M <= 2) return launch_dense_gemv<2, EPI, FQ>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
    if (M <= 4) return launch_dense_gemv<4, EPI, FQ>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
    if (M <= 8) return launch_dense_gemv<8, EPI, FQ>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
    return launch_dense_gemv<16, EPI, FQ>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
}

}  // namespace

// Shapes the streaming kernel takes: one or two tokens (every warp re-reads the token rows from shared memory
// per weight row, so its time grows with M: 11008 x 4096, cold weights, 11.4 / 12.0 / 15.3 / 16.2 / 24.4 us at
// 1 / 2 / 3 / 4 / 8 tokens against 13.5 us for the tcgen05 kernel with 80-column tiles. Knob 9 moves the limit
// up to 16 or, negative, switches the kernel off), K a multiple of 16, the token rows within 200 KB of shared
// memory, 16-byte aligned operands; a pinned dense tile switches it off too.
bool dense_gemv_fits(int M, int K, const void* W, const void* x) {
    const int knob = tuning_knob(kKnobGemvDenseMaxTokens);
    const int max_tokens = knob > 0 ? std::min(16, knob) : (knob < 0 ? 0 : 2);
    return M >= 1 && M <= max_tokens && K % 16 == 0 && (size_t)M * K <= 200 * 1024 && aligned16(W) && aligned16(x) &&
           tuning_knob(kKnobDenseTile) == 0;
}

int dense_gemv(const int8_t* W, const int8_t* x, const float* act_scale, const __half* w_scale, const __half* bias,
               void* out, int M, int K, int N, cudaStream_t stream, int epi) {
    return epi == 0 ? dispatch_dense_gemv<0, false>(W, x, act_scale, w_scale, bias, out, M, K, N, stream)
                    : dispatch_dense_gemv<1, false>(W, x, act_scale, w_scale, bias, out, M, K, N, stream);
}

int dense_gemv_fq(const int8_t* W, const __half* x, const __half* w_scale, const __half* bias, __half* out, int M, int K,
                  int N, cudaStream_t stream) {
    return dispatch_dense_gemv<1, true>(W, x, nullptr, w_scale, bias, out, M, K, N, stream);
}

}  // namespace fb200
