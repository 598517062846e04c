// Launchers of the fused INT8 convolution kernels (conv.cu). Return a fb200::Status code.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

namespace fb200 {

size_t int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW, int strideH,
                                  int strideW, int dilH, int dilW);
size_t int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out);

// input (N,C_in,H,W) fp16, weight (C_out, C_in*kH*kW) int8, w_scale / bias (C_out) fp16,
// output (N,C_out,H_out,W_out) fp16.
int int8_conv2d_forward(const __half* input, const int8_t* weight, const __half* w_scale, const __half* bias,
                        __half* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW,
                        int strideH, int strideW, int dilH, int dilW, cudaStream_t stream);

// 2x2 stride-2 transposed conv: weight (4*C_out, C_in) int8 with row co*4 + kh*2 + kw,
// output (N,C_out,2H,2W) fp16.
int int8_conv_transpose2d_k2s2_forward(const __half* input, const int8_t* weight, const __half* w_scale,
                                       const __half* bias, __half* output, int N, int C_in, int H, int W, int C_out,
                                       cudaStream_t stream);

}  // namespace fb200
