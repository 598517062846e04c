// Internal declarations of the 2:4-sparse INT8 GEMM launchers (gemm_sparse.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

// Which kernel a 2:4-sparse GEMM call runs: decided in one place for the GEMM's own dispatch and
// for the public plan query (forge_sparse_int8_gemm_plan).
struct SparseChoice {
    int kind;   // 0 = plain-CUDA kernel (shapes TMA cannot describe), 1 = one CTA per tile, 2 = CTA pair,
                // 3 = weight-streaming CUDA-core kernel for 1-2 tokens (sparse_gemv.cu)
    int bt;     // tokens per tile (kind 1: 32 / 64 / 128; kind 2: 128 / 192 / 224 / 256)
};
// tma_ok: K % 128 == 0 and 16-byte aligned operands; stream_ok: K % 32 == 0 and 16-byte aligned
// operands. force_bt: 0 = automatic (cost model), 32/64/128 pins the single-CTA tile, 1 = single CTA
// with 32 or 64 tokens, 1000 + BT pins the CTA-pair tile, 1000 = CTA pair with the model's width.
// allow_pair = false when the device cannot co-schedule the pair kernel.
SparseChoice sparse_choose(int M, int K, int N_out, bool tma_ok, bool stream_ok, int force_bt, bool allow_pair);

// The 1-4 token kernel: true when it can take the shape (K % 32 == 0, token rows fit shared memory).
bool sparse_gemv_fits(int M, int K);
// epi 0: out int32 (M,N_out); epi 1: fp16 dequant (+ bias). Needs 16-byte aligned W_comp / x, 4-byte w_meta.
int sparse_gemv(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out, cudaStream_t stream,
                int epi);

// One or two tokens of FP16 activations: per-token quantization inside the streaming kernel (same bits as
// quantize + sparse GEMM, no scratch). fits: M <= 2, K <= 4096, K % 32 == 0, x 16-byte aligned, no pinned tile.
bool sparse_gemv_fq_fits(int M, int K, const void* x);
int sparse_gemv_fq(const int8_t* W_comp, const __half* x, const uint32_t* w_meta, const __half* w_scale,
                   const __half* bias, __half* out, int M, int K, int N_out, cudaStream_t stream);

// out (M,N_out) s32 = x (M,K) s8 x W24 (N_out,K)^T, W24 given as W_comp (N_out,K/2) + w_meta (N_out,K/32).
// force_bt: 32/64/128 pins the token-tile width, anything else selects it automatically.
int sparse_gemm_s32(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, int32_t* out, int M, int K,
                    int N_out, cudaStream_t stream, int force_bt);

// out (M,N_out) fp16 = fp16((act_scale[m] * w_scale[n]) * acc + bias[n]).
int sparse_gemm_dequant(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                        const __half* w_scale, const __half* bias, __half* out, int M, int K, int N_out,
                        cudaStream_t stream, int force_bt);

// FP16 result (M,N_out) written into each of `n_outs` (<= 8) buffers with row pitch `ld_out`
// elements. The buffers may be peer-mapped memory of other GPUs: a column-sharded layer passes
// every rank's copy of the full output, offset to its own first column, and the epilogue's
// stores perform the all-gather. Needs K % 128 == 0 and 16-byte aligned operands.
int sparse_gemm_dequant_multi(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                              const __half* w_scale, const __half* bias, void* const* outs, int n_outs,
                              long long ld_out, int M, int K, int N_out, cudaStream_t stream);

// out (M,N_out) fp16 = fp16(SiLU(g) * u): gate and up projections (both 2:4 sparse, N_out rows
// each) of a gated MLP in one pass. Needs K % 128 == 0 and 16-byte aligned operands (kBadShape).
int sparse_gemm_gated(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp, const uint32_t* wu_meta,
                      const int8_t* x, const float* act_scale, const __half* wg_scale, const __half* wu_scale,
                      const __half* bg, const __half* bu, __half* out, int M, int K, int N_out, cudaStream_t stream,
                      int force_bt);

}  // namespace fb200
