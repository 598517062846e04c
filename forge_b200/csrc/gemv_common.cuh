// Pieces shared by the weight-streaming (CUDA-core) kernels for very few tokens: sparse_gemv.cu and
// dense_gemv.cu. A warp owns one weight row at a time; after the lanes' partial sums are reduced, lane 0
// applies the GEMM epilogue of the tensor-core kernels (same arithmetic, same bits).
#pragma once

#include "common.cuh"

namespace fb200 {
namespace gemv {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Per-row epilogue operands, requested together with the row's weights so that their latency is not
// paid after the reduction.
struct RowScale {
    float ws, bs;
};
template <int EPI>
__device__ __forceinline__ RowScale load_row_scale(const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                                                   int row) {
    RowScale r = {0.f, 0.f};
    if (EPI == 1) {
        r.ws = __half2float(w_scale[row]);
        if (bias != nullptr) r.bs = __half2float(bias[row]);
    }
    return r;
}

template <int MT, int EPI>
__device__ __forceinline__ void gemv_store(int (&acc)[MT], int lane, int row, void* __restrict__ out,
                                           const float (&as)[MT], const RowScale& rs, bool has_bias, int M, int N_out) {
#pragma unroll
    for (int m = 0; m < MT; m++) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
    }
    if (lane != 0) return;
    if (EPI == 0) {
#pragma unroll
        for (int m = 0; m < MT; m++)
            if (m < M) static_cast<int32_t*>(out)[(size_t)m * N_out + row] = acc[m];
    } else {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m < M) {
                const float o = dequant_gemm(acc[m], mul_ftz(as[m], rs.ws), rs.bs, has_bias);
                static_cast<__half*>(out)[(size_t)m * N_out + row] = __float2half_rn(o);
            }
        }
    }
}

}  // namespace gemv
}  // namespace fb200
