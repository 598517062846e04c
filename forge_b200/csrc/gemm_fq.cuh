// Internal declarations of the fused quantize + 2:4-sparse GEMM launcher (gemm_fq.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

// True when the fused kernel can take this problem: K a multiple of 128, K <= 1280 (the 128-token
// int8 block stays resident in shared memory) and a 16-byte aligned activation pointer.
bool sparse_fq_fits(int K, const void* x);

// out (M,N_out) fp16 = dequant(W24 x quantize(x)^T) in one kernel; bit-identical to quantize +
// sparse GEMM. No scratch buffers are touched.
int sparse_fq_linear(const __half* x, const int8_t* W_comp, const uint32_t* w_meta, const __half* w_scale,
                     const __half* bias, __half* out, int M, int K, int N_out, cudaStream_t stream);

}  // namespace fb200
