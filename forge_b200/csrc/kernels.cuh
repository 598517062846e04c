// Internal declarations of the non-GEMM launchers (quantize.cu, sparsity.cu). Each returns a
// fb200::Status code; argument meaning follows the reference function it replaces.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

int quantize_activation(const __half* input, int8_t* output, float* scales, int M, int K, cudaStream_t stream);
int dequantize_bias(const int32_t* input, const float* act_scale, const __half* w_scale, const __half* bias,
                    __half* output, int M, int N, cudaStream_t stream);
int prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K,
                      cudaStream_t stream);
int pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K, cudaStream_t stream);
// fp32 / fp16 weight (N,K) -> per-channel int8 (optional), 2:4 compressed values + packed metadata
// (optional) and fp16 scales, in one pass. Needs K % 32 == 0.
int prepare_weight(const void* w, int w_is_half, int8_t* w_int8, int8_t* W_comp, uint32_t* w_meta, __half* w_scale,
                   int N, int K, cudaStream_t stream);

}  // namespace fb200

// Kernels the reference declares publicly; same names, namespaces and parameter lists.
namespace forge { namespace quant {
__global__ void fused_quantize_activation_kernel(const __half* __restrict__ input, int8_t* __restrict__ output,
                                                 float* __restrict__ scales, int K);
__global__ void fused_dequantize_bias_kernel(const int32_t* __restrict__ input, const float* __restrict__ act_scale,
                                             const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                                             __half* __restrict__ output, int N);
}}
namespace forge { namespace sparsity {
__global__ void prune_compress_kernel(const int8_t* __restrict__ weight, int8_t* __restrict__ compressed,
                                      uint8_t* __restrict__ metadata_raw, int N, int K);
__global__ void pack_metadata_kernel(const uint8_t* __restrict__ meta_raw, uint32_t* __restrict__ meta_packed, int N,
                                     int K);
}}
