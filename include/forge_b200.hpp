// C++17 face of libforge_b200: the forge::gemm / forge::quant / forge::sparsity free functions
// of Forge's quantized-inference path and the two forge::nn INT8 convolutions that call it, with the reference's names, parameter order, defaults and
// void returns, implemented as inline forwards to the C ABI in forge_b200.h. Code written
// against the reference headers (include/forge/{gemm,quant,sparsity}/*.cuh in the Forge tree)
// compiles against this file unchanged and links with -lforge_b200.
//
// Differences a caller can observe:
//  - a non-zero status of the C call is remembered per thread (forge::b200::last_status()),
//    because the reference signatures return void;
//  - sparse_int8_gemm_plan never reports split_k > 1 (K is not split: the s32 accumulator in
//    tensor memory covers the whole reduction, so results are bit-identical for any request);
//  - additive functions int8_gemm_s32 / sparse_int8_gemm_s32 return the raw INT32 product.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

#include "forge_b200.h"

#define FORGE_SPARSE_GEMM_API_VERSION 3

namespace forge {

namespace b200 {
inline int& last_status_ref() {
    thread_local int status = 0;
    return status;
}
inline int last_status() { return last_status_ref(); }
inline void note(int status) {
    if (status != 0) last_status_ref() = status;
}
inline forge_stream_t st(cudaStream_t s) { return reinterpret_cast<forge_stream_t>(s); }
}  // namespace b200

namespace quant {

#ifdef __CUDACC__
// Kernels that are public in the reference; defined in libforge_b200 with the same launch
// contract (one block per row).
__global__ void fused_quantize_activation_kernel(const __half* __restrict__ input, int8_t* __restrict__ output,
                                                 float* __restrict__ scales, int K);
__global__ void fused_dequantize_bias_kernel(const int32_t* __restrict__ input, const float* __restrict__ act_scale,
                                             const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                                             __half* __restrict__ output, int N);
#endif

inline void fused_quantize_activation(const __half* input, int8_t* output, float* scales, int M, int K,
                                      cudaStream_t stream = nullptr) {
    b200::note(forge_fused_quantize_activation(input, output, scales, M, K, b200::st(stream)));
}

inline void fused_dequantize_bias(const int32_t* input, const float* act_scale, const __half* w_scale,
                                  const __half* bias, __half* output, int M, int N, cudaStream_t stream = nullptr) {
    b200::note(forge_fused_dequantize_bias(input, act_scale, w_scale, bias, output, M, N, b200::st(stream)));
}

}  // namespace quant

namespace sparsity {

#ifdef __CUDACC__
__global__ void prune_compress_kernel(const int8_t* __restrict__ weight, int8_t* __restrict__ compressed,
                                      uint8_t* __restrict__ metadata_raw, int N, int K);
__global__ void pack_metadata_kernel(const uint8_t* __restrict__ meta_raw, uint32_t* __restrict__ meta_packed, int N,
                                     int K);
#endif

inline void prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K,
                              cudaStream_t stream = nullptr) {
    b200::note(forge_prune_compress_24(weight, compressed, metadata_raw, N, K, b200::st(stream)));
}

inline void pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K,
                          cudaStream_t stream = nullptr) {
    b200::note(forge_pack_metadata(meta_raw, meta_packed, N, K, b200::st(stream)));
}

}  // namespace sparsity

namespace gemm {

// ---- dense
inline void int8_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                              const __half* bias, __half* output, int M, int K, int N,
                              cudaStream_t stream = nullptr) {
    b200::note(forge_int8_gemm_dequant(A, B, act_scale, w_scale, bias, output, M, K, N, b200::st(stream)));
}

inline void int8_linear(const __half* x, const int8_t* w_int8, const __half* w_scale, const __half* bias,
                        __half* output, int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale,
                        cudaStream_t stream = nullptr) {
    b200::note(forge_int8_linear(x, w_int8, w_scale, bias, output, M, K, N, scratch_a_int8, scratch_a_scale,
                                 b200::st(stream)));
}

inline void int8_dp4a_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                                   const __half* bias, __half* output, int M, int K, int N,
                                   cudaStream_t stream = nullptr) {
    b200::note(forge_int8_dp4a_gemm_dequant(A, B, act_scale, w_scale, bias, output, M, K, N, b200::st(stream)));
}

inline void int8_dp4a_linear(const __half* x, const int8_t* w_int8, const __half* w_scale, const __half* bias,
                             __half* output, int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale,
                             cudaStream_t stream = nullptr) {
    b200::note(forge_int8_dp4a_linear(x, w_int8, w_scale, bias, output, M, K, N, scratch_a_int8, scratch_a_scale,
                                      b200::st(stream)));
}

inline int get_compute_capability(int device = 0) { return forge_get_compute_capability(device); }
inline bool has_wmma_int8(int device = 0) { return forge_has_wmma_int8(device) != 0; }

inline void int8_gemm(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                      const __half* bias, __half* output, int M, int K, int N, cudaStream_t stream = nullptr) {
    b200::note(forge_int8_gemm(A, B, act_scale, w_scale, bias, output, M, K, N, b200::st(stream)));
}

inline void int8_gemm_s32(const int8_t* A, const int8_t* B, int32_t* output, int M, int K, int N,
                          cudaStream_t stream = nullptr) {
    b200::note(forge_int8_gemm_s32(A, B, output, M, K, N, b200::st(stream)));
}

// ---- 2:4 sparse
constexpr int kSparseTileAuto = FORGE_SPARSE_TILE_AUTO;
constexpr int kSparseTile256x128 = FORGE_SPARSE_TILE_256x128;
constexpr int kSparseTile128x128 = FORGE_SPARSE_TILE_128x128;
constexpr int kSparseTile128x64 = FORGE_SPARSE_TILE_128x64;
constexpr int kSparseNumTiles = FORGE_SPARSE_NUM_TILES;
constexpr int kSparseLinearAuto = FORGE_SPARSE_LINEAR_AUTO;
constexpr int kSparseLinearTwoPass = FORGE_SPARSE_LINEAR_TWO_PASS;
constexpr int kSparseLinearFused = FORGE_SPARSE_LINEAR_FUSED;

struct SparseGemmPlan {
    int tile;
    int split_k;
};

inline SparseGemmPlan sparse_int8_gemm_plan(int M, int K, int N_out, int split_k = 0, bool have_workspace = true,
                                            int tile = kSparseTileAuto) {
    SparseGemmPlan p{kSparseTile128x128, 1};
    b200::note(forge_sparse_int8_gemm_plan(M, K, N_out, split_k, have_workspace ? 1 : 0, tile, &p.tile, &p.split_k));
    return p;
}

inline void sparse_int8_gemm(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta,
                             const float* act_scale, const __half* w_scale, const __half* bias, __half* output, int M,
                             int K, int N_out, float* splitk_workspace = nullptr, int split_k = 1,
                             cudaStream_t stream = nullptr, int tile = kSparseTileAuto) {
    b200::note(forge_sparse_int8_gemm(W_comp, x_int8, w_meta, act_scale, w_scale, bias, output, M, K, N_out,
                                      splitk_workspace, split_k, b200::st(stream), tile));
}

inline bool sparse_int8_linear_fused(int M, int K, int N_out) {
    return forge_sparse_int8_linear_fused(M, K, N_out) != 0;
}

inline void sparse_int8_linear(const __half* x, const int8_t* W_comp, const uint32_t* w_meta, const __half* w_scale,
                               const __half* bias, __half* output, int M, int K, int N_out, int8_t* scratch_x_int8,
                               float* scratch_x_scale, float* splitk_workspace = nullptr, int split_k = 1,
                               cudaStream_t stream = nullptr, int path = kSparseLinearAuto) {
    b200::note(forge_sparse_int8_linear(x, W_comp, w_meta, w_scale, bias, output, M, K, N_out, scratch_x_int8,
                                        scratch_x_scale, splitk_workspace, split_k, b200::st(stream), path));
}

inline void splitk_reduce(const float* workspace, const __half* bias, __half* output, int M, int N_out,
                          cudaStream_t stream = nullptr) {
    b200::note(forge_splitk_reduce(workspace, bias, output, M, N_out, b200::st(stream)));
}

inline void sparse_int8_gemm_s32(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta, int32_t* output,
                                 int M, int K, int N_out, cudaStream_t stream = nullptr) {
    b200::note(forge_sparse_int8_gemm_s32(W_comp, x_int8, w_meta, output, M, K, N_out, b200::st(stream)));
}

}  // namespace gemm

namespace nn {

// include/forge/nn/int8_conv2d.cuh:24-30
inline size_t int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW,
                                         int strideH, int strideW, int dilH = 1, int dilW = 1) {
    return static_cast<size_t>(
        forge_int8_conv2d_workspace_size(C_in, H, W, C_out, kH, kW, padH, padW, strideH, strideW, dilH, dilW));
}

// include/forge/nn/int8_conv2d.cuh:42-54
inline void int8_conv2d_forward(const __half* input, const int8_t* weight, const __half* w_scale, const __half* bias,
                                __half* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                                int padW, int strideH, int strideW, int dilH, int dilW, void* workspace,
                                cudaStream_t stream = nullptr) {
    b200::note(forge_int8_conv2d_forward(input, weight, w_scale, bias, output, N, C_in, H, W, C_out, kH, kW, padH, padW,
                                         strideH, strideW, dilH, dilW, workspace, b200::st(stream)));
}

// include/forge/nn/int8_conv_transpose2d.cuh:25-26
inline size_t int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out) {
    return static_cast<size_t>(forge_int8_conv_transpose2d_k2s2_workspace_size(C_in, H, W, C_out));
}

// include/forge/nn/int8_conv_transpose2d.cuh:40-49
inline void int8_conv_transpose2d_k2s2_forward(const __half* input, const int8_t* weight, const __half* w_scale,
                                               const __half* bias, __half* output, int N, int C_in, int H, int W,
                                               int C_out, void* workspace, cudaStream_t stream = nullptr) {
    b200::note(forge_int8_conv_transpose2d_k2s2_forward(input, weight, w_scale, bias, output, N, C_in, H, W, C_out,
                                                        workspace, b200::st(stream)));
}

}  // namespace nn
}  // namespace forge
