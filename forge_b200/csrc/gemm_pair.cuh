// Internal declarations of the CTA-pair (cta_group::2) GEMM launchers (gemm_pair.cu).
// Preconditions are the TMA path's (checked by the callers in gemm_dense.cu / gemm_sparse.cu).
// Return a fb200::Status, or -1 when the device cannot co-schedule a pair of these CTAs.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

int dense_pair_s32(const int8_t* A, const int8_t* B, int32_t* out, int M, int K, int N, cudaStream_t stream);
int dense_pair_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                       const __half* bias, __half* out, int M, int K, int N, cudaStream_t stream);

// out[m][n] = SiLU(gate) * up of the two dequantised products, N output columns (256 x 128 per pair tile).
int dense_pair_gated(const int8_t* A, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                     const __half* wg_scale, const __half* wu_scale, const __half* bg, const __half* bu, __half* out,
                     int M, int K, int N, cudaStream_t stream);

// bt: tokens per pair tile, one of 128, 192, 224, 256.
int sparse_pair_s32(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, int32_t* out, int M, int K,
                    int N_out, cudaStream_t stream, int bt);
int sparse_pair_dequant(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                        const __half* w_scale, const __half* bias, __half* out, int M, int K, int N_out,
                        cudaStream_t stream, int bt);

// Copies the sparse pair kernel's probe counters (pair-kernel flag 4) to `out`.
int read_pair_probe(unsigned long long* out, int n);

struct OutDst;
// FP16 result written to every destination in `multi` (see sparse_epilogue.cuh).
int sparse_pair_dequant_multi(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                              const __half* w_scale, const __half* bias, const OutDst* multi, int M, int K, int N_out,
                              cudaStream_t stream);

// Gated (SiLU(gate) * up) sparse GEMM on CTA pairs; arguments as sparse_gemm_gated.
int sparse_pair_gated(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp, const uint32_t* wu_meta,
                      const int8_t* x, const float* act_scale, const __half* wg_scale, const __half* wu_scale,
                      const __half* bg, const __half* bu, __half* out, int M, int K, int N_out, cudaStream_t stream,
                      int bt);

}  // namespace fb200
