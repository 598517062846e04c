// Internal declarations of the dense INT8 GEMM launchers (gemm_dense.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

// out (M,N) s32 = A (M,K) s8 x B (N,K)^T s8. force_bn: 64/128/256 to pin the tile width, else auto.
int dense_gemm_s32(const int8_t* A, const int8_t* B, int32_t* out, int M, int K, int N, cudaStream_t stream,
                   int force_bn);

// out (M,N) fp16 = fp16((act_scale[m] * w_scale[n]) * acc + bias[n]).
int dense_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                       const __half* bias, __half* out, int M, int K, int N, cudaStream_t stream, int force_bn);

// Address of this device's status word (a file-scope __device__ int); nullptr on failure.
int* status_word();
// Reads the status word back (synchronising copy); clears it when reset != 0. -1 on failure.
int read_device_status(int reset);

}  // namespace fb200
