/* forge_b200 - C ABI of the B200 (sm_100a) implementation of Forge's quantized-inference path.
 *
 * Every entry point takes plain device pointers, int shapes and a CUDA stream, enqueues its
 * work on that stream and returns without synchronising. Buffers are caller-owned; nothing
 * is allocated. Return value: 0 on success, otherwise a FORGE_B200_* status code. Sizes
 * <= 0 are a silent no-op that returns 0, as in the reference launchers.
 *
 * FP16 buffers are passed as `const void*` / `void*` (IEEE binary16, the layout of CUDA's
 * __half) so that this header stays plain C. `forge_stream_t` is a cudaStream_t.
 *
 * Each declaration names the reference interface it stands in for (path:line inside the
 * Forge source tree).
 */
#ifndef FORGE_B200_H
#define FORGE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* forge_stream_t;

enum {
    FORGE_B200_OK = 0,
    FORGE_B200_BAD_SHAPE = 1,
    FORGE_B200_BAD_POINTER = 2,
    FORGE_B200_UNSUPPORTED_ARCH = 3, /* the current device is not compute capability 10.x */
    FORGE_B200_LAUNCH_FAILED = 4,
    FORGE_B200_DEVICE_TIMEOUT = 5,   /* a bounded device-side wait ran out */
    FORGE_B200_TOO_LARGE = 6
};

/* ---------------------------------------------------------------- forge::quant */

/* forge::quant::fused_quantize_activation - include/forge/quant/quantize.cuh:23-29,
 * src/quant/quantize.cu:162-191. input (M,K) fp16 -> output (M,K) int8 + scales (M) fp32. */
int forge_fused_quantize_activation(const void* input, int8_t* output, float* scales, int M, int K,
                                    forge_stream_t stream);

/* forge::quant::fused_dequantize_bias - include/forge/quant/dequantize.cuh:22-30,
 * src/quant/dequantize.cu:30-45. input (M,N) int32, act_scale (M) fp32, w_scale/bias (N) fp16
 * (bias may be NULL) -> output (M,N) fp16. */
int forge_fused_dequantize_bias(const int32_t* input, const float* act_scale, const void* w_scale, const void* bias,
                                void* output, int M, int N, forge_stream_t stream);

/* ---------------------------------------------------------------- forge::gemm, dense */

/* forge::gemm::int8_gemm_dequant - include/forge/gemm/int8_dense.cuh:24-34,
 * src/gemm/int8_dense.cu:183-211. A (M,K) int8, B (N,K) int8 -> output (M,N) fp16 =
 * fp16((act_scale[m]*w_scale[n]) * sum_k A[m,k]B[n,k] + bias[n]). */
int forge_int8_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale,
                            const void* bias, void* output, int M, int K, int N, forge_stream_t stream);

/* forge::gemm::int8_gemm - include/forge/gemm/int8_gemm.cuh:25-35, src/gemm/int8_gemm.cu:27-46
 * (the reference dispatches on compute capability; here there is one backend). */
int forge_int8_gemm(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale, const void* bias,
                    void* output, int M, int K, int N, forge_stream_t stream);

/* forge::gemm::int8_dp4a_gemm_dequant - include/forge/gemm/int8_dp4a.cuh:25-35. Kept so callers
 * link; runs the same tensor-core kernel as forge_int8_gemm_dequant. */
int forge_int8_dp4a_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale,
                                 const void* bias, void* output, int M, int K, int N, forge_stream_t stream);

/* forge::gemm::int8_linear - include/forge/gemm/int8_dense.cuh:37-48, src/gemm/int8_dense.cu:213-232.
 * x (M,K) fp16 -> quantize into scratch_a_int8 (M,K) / scratch_a_scale (M) -> GEMM + dequant. */
int forge_int8_linear(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias, void* output,
                      int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale, forge_stream_t stream);

/* forge::gemm::int8_dp4a_linear - include/forge/gemm/int8_dp4a.cuh:38-50. Same as forge_int8_linear. */
int forge_int8_dp4a_linear(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias, void* output,
                           int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale,
                           forge_stream_t stream);

/* forge::gemm::get_compute_capability / has_wmma_int8 - include/forge/gemm/int8_gemm.cuh:18-21.
 * Unlike the reference (one cached value for all devices) the answer is per device. */
int forge_get_compute_capability(int device);
int forge_has_wmma_int8(int device);

/* Additive: raw INT32 GEMM output (M,N). The reference computes this only in its host test
 * loop, tests/test_int8_dense_gemm.cu:35-39. */
int forge_int8_gemm_s32(const int8_t* A, const int8_t* B, int32_t* output, int M, int K, int N,
                        forge_stream_t stream);

/* No counterpart in the reference. forge_int8_linear for callers that cannot provide the two
 * scratch buffers: code that runs where device allocation is off-limits (a plug-in under a host
 * framework whose allocator owns the GPU's memory, a serving loop that must not hit cudaMalloc's
 * device-wide synchronisation). The scratch lives in a fixed 16 MiB + 64 KiB array inside the
 * library image (resident in every context that loads the library until exit); the call
 * allocates nothing. Limits: M*K <= 16777216 and M <= 16384, otherwise FORGE_B200_TOO_LARGE.
 * All calls on a device share the array, so calls that may overlap on the GPU race - order
 * them. The first call on a device resolves the array's address; make it at start-up, before
 * any stream capture. Output is bit-identical to forge_int8_linear. */
int forge_int8_linear_static(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias,
                             void* output, int M, int K, int N, forge_stream_t stream);

/* ---------------------------------------------------------------- forge::gemm, 2:4 sparse */

/* Tile / path ids of include/forge/gemm/int8_sparse.cuh:26-31,74-76. */
enum {
    FORGE_SPARSE_TILE_AUTO = -1,
    FORGE_SPARSE_TILE_256x128 = 0,
    FORGE_SPARSE_TILE_128x128 = 1,
    FORGE_SPARSE_TILE_128x64 = 2,
    FORGE_SPARSE_NUM_TILES = 3,
    FORGE_SPARSE_LINEAR_AUTO = -1,
    FORGE_SPARSE_LINEAR_TWO_PASS = 0,
    FORGE_SPARSE_LINEAR_FUSED = 1
};

/* forge::gemm::sparse_int8_gemm_plan - include/forge/gemm/int8_sparse.cuh:33-50,
 * src/gemm/int8_sparse.cu:875-920. Writes the (tile, split_k) forge_sparse_int8_gemm will run,
 * chosen by the same routine the GEMM's own dispatch calls: a wave-aware cost model like the
 * reference's, with per-tile constants fitted on a B200. split_k is always 1: the s32 accumulator in
 * tensor memory covers the whole K range. The tcgen05 tile set is reported through the reference's
 * three ids: FORGE_SPARSE_TILE_256x128 = the CTA-pair kernel (256 weight rows x 192 or 224 tokens
 * per pair of SMs), 128x128 = one CTA with 128 tokens, 128x64 = one CTA with 64 or 32 tokens, and
 * also the answer for the weight-streaming kernel that takes 1-2 tokens and for shapes only the
 * plain-CUDA kernel takes (K % 128 != 0; the plan sees no pointers and assumes 16-byte aligned
 * operands). Passing the planned tile back to forge_sparse_int8_gemm runs exactly the kernel the
 * automatic path runs. */
int forge_sparse_int8_gemm_plan(int M, int K, int N_out, int split_k, int have_workspace, int tile, int* out_tile,
                                int* out_split_k);

/* forge::gemm::sparse_int8_gemm - include/forge/gemm/int8_sparse.cuh:57-71,
 * src/gemm/int8_sparse.cu:960-1003. W_comp (N_out,K/2) int8, x_int8 (M,K) int8,
 * w_meta (N_out,K/32) uint32 -> output (M,N_out) fp16. splitk_workspace: optional (M,N_out)
 * 4-byte-element buffer, overwritten by the call. */
int forge_sparse_int8_gemm(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta,
                           const float* act_scale, const void* w_scale, const void* bias, void* output, int M, int K,
                           int N_out, float* splitk_workspace, int split_k, forge_stream_t stream, int tile);

/* forge::gemm::sparse_int8_linear_fused - include/forge/gemm/int8_sparse.cuh:78-83. 1 or 0: whether the
 * automatic path of forge_sparse_int8_linear quantizes inside the GEMM kernel - the tcgen05 kernel for
 * narrow layers with K <= 1280 whose activation does not fit L2, the weight-streaming kernel for one and
 * two tokens with K <= 4096. Neither touches the scratch buffers. */
int forge_sparse_int8_linear_fused(int M, int K, int N_out);

/* forge::gemm::sparse_int8_linear - include/forge/gemm/int8_sparse.cuh:90-105,
 * src/gemm/int8_sparse.cu:1005-1043. */
int forge_sparse_int8_linear(const void* x, const int8_t* W_comp, const uint32_t* w_meta, const void* w_scale,
                             const void* bias, void* output, int M, int K, int N_out, int8_t* scratch_x_int8,
                             float* scratch_x_scale, float* splitk_workspace, int split_k, forge_stream_t stream,
                             int path);

/* forge::gemm::splitk_reduce - include/forge/gemm/int8_sparse.cuh:108-114,
 * src/gemm/int8_sparse.cu:945-958. output = fp16(workspace + bias[n]). */
int forge_splitk_reduce(const float* workspace, const void* bias, void* output, int M, int N_out,
                        forge_stream_t stream);

/* Additive: raw INT32 output (M,N_out) of the 2:4-sparse GEMM (the reference checks it only
 * through an FP64 host loop, tests/test_int8_sparse_gemm.cu:69-80). */
int forge_sparse_int8_gemm_s32(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta, int32_t* output,
                               int M, int K, int N_out, forge_stream_t stream);

/* Additive, no counterpart in the reference (which is single-GPU): forge_sparse_int8_gemm whose
 * FP16 result (M,N_out) is written into each of n_outs (1..8) buffers with row pitch ld_out
 * (elements, >= N_out). The buffers may be other GPUs' memory mapped into this process (CUDA
 * IPC / peer access): a layer sharded by output channels passes every rank's copy of the full
 * output, offset to its own first column, and the GEMM epilogue's stores carry out the
 * all-gather over NVLink while later tiles are still being computed. The caller orders the
 * ranks (nobody may read an output before every rank's kernel has finished). Needs K % 128 == 0
 * and 16-byte aligned operands (FORGE_B200_BAD_SHAPE otherwise). */
int forge_sparse_int8_gemm_multi(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta,
                                 const float* act_scale, const void* w_scale, const void* bias, void* const* outputs,
                                 int n_outs, long long ld_out, int M, int K, int N_out, forge_stream_t stream);

/* ---------------------------------------------------------------- gated MLP (additive) */

/* No counterpart in the reference (its only "gating" is an FP32 training op, src/nn/gating.cu).
 * Gate and up projections of a Llama-style MLP in one GEMM pass with the activation fused in
 * the epilogue: h[m,n] = fp16(SiLU(g) * u), g = (act_scale[m]*wg_scale[n]) * sum_k x[m,k]Wg[n,k] + bg[n],
 * u likewise from Wu; g, u and SiLU(g) = g / (1 + exp(-g)) are evaluated in fp32 and h is rounded
 * once. x_int8 (M,K), Wg / Wu (N,K) int8; bg / bu may be NULL. Needs K % 16 == 0, N % 8 == 0 and
 * 16-byte aligned operands (FORGE_B200_BAD_SHAPE otherwise). */
int forge_int8_gated_gemm(const int8_t* x_int8, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                          const void* wg_scale, const void* wu_scale, const void* bg, const void* bu, void* h_out,
                          int M, int K, int N, forge_stream_t stream);

/* The same with 2:4-sparse gate and up weights (compressed values + packed metadata as produced
 * by forge_prune_compress_24 / forge_pack_metadata). Needs K % 128 == 0. */
int forge_sparse_int8_gated_gemm(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp,
                                 const uint32_t* wu_meta, const int8_t* x_int8, const float* act_scale,
                                 const void* wg_scale, const void* wu_scale, const void* bg, const void* bu,
                                 void* h_out, int M, int K, int N_out, forge_stream_t stream);

/* Whole W8A8 gated MLP block: per-token quantize(x) -> gated GEMM -> per-token quantize(h) ->
 * down GEMM + dequant (+ bd). x (M,d_model) fp16 -> out (M,d_model) fp16. Wg / Wu (d_ffn,d_model),
 * Wd (d_model,d_ffn) int8 with fp16 per-channel scales. `workspace` is caller-owned device memory of
 * forge_w8a8_gated_mlp_workspace_bytes(M, d_model, d_ffn) bytes, 256-byte aligned; on return it
 * holds, in this order (each block padded to 256 bytes): int8 x (M*d_model), fp32 x scales (M),
 * fp16 h (M*d_ffn), int8 h (M*d_ffn), fp32 h scales (M). */
unsigned long long forge_w8a8_gated_mlp_workspace_bytes(int M, int d_model, int d_ffn);
int forge_w8a8_gated_mlp(const void* x, const int8_t* Wg, const int8_t* Wu, const int8_t* Wd, const void* wg_scale,
                         const void* wu_scale, const void* wd_scale, const void* bg, const void* bu, const void* bd,
                         void* out, int M, int d_model, int d_ffn, void* workspace, forge_stream_t stream);
int forge_sparse_w8a8_gated_mlp(const void* x, const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp,
                                const uint32_t* wu_meta, const int8_t* Wd_comp, const uint32_t* wd_meta,
                                const void* wg_scale, const void* wu_scale, const void* wd_scale, const void* bg,
                                const void* bu, const void* bd, void* out, int M, int d_model, int d_ffn,
                                void* workspace, forge_stream_t stream);

/* ---------------------------------------------------------------- forge::sparsity */

/* forge::sparsity::prune_compress_24 - include/forge/sparsity/prune_compress.cuh:23-30,
 * src/sparsity/prune_compress.cu:71-85. weight (N,K) int8 -> compressed (N,K/2) int8 +
 * metadata_raw (N*K/4) one nibble per byte. */
int forge_prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K,
                            forge_stream_t stream);

/* forge::sparsity::pack_metadata - include/forge/sparsity/pack_metadata.cuh:21-26,
 * src/sparsity/pack_metadata.cu:32-44. meta_raw (N*K/4) -> meta_packed (N,K/32) uint32. */
int forge_pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K, forge_stream_t stream);

/* Additive: weight preparation in one kernel. The reference does it with PyTorch ops followed by
 * prune_compress_24 + pack_metadata and a synchronize (python/forge/nn/linear.py:167-173,234-249).
 * weight (N,K) fp32 (weight_is_half = 0) or fp16 (1) -> per output channel scale = absmax/127
 * (floored at 1e-8), q = clamp(round_half_even(w / scale), +-127): w_int8 (N,K) (may be NULL),
 * w_scale (N) fp16, and - when W_comp is not NULL - the 2:4 pruned + compressed weight (N,K/2)
 * with its packed metadata (N,K/32). Needs K % 32 == 0 and 16-byte aligned outputs. */
int forge_prepare_weight(const void* weight, int weight_is_half, int8_t* w_int8, int8_t* W_comp, uint32_t* w_meta,
                         void* w_scale, int N, int K, forge_stream_t stream);

/* ---------------------------------------------------------------- convolution callers of the GEMM */

/* forge::nn::int8_conv2d_workspace_size - include/forge/nn/int8_conv2d.cuh:24-30,
 * src/nn/int8_conv2d.cu:126-145. Returns the reference's figure so existing callers keep sizing
 * their buffer the same way; forge_int8_conv2d_forward itself needs no scratch. */
unsigned long long forge_int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                                                   int padW, int strideH, int strideW, int dilH, int dilW);

/* forge::nn::int8_conv2d_forward - include/forge/nn/int8_conv2d.cuh:42-54, src/nn/int8_conv2d.cu:151-223.
 * input (N,C_in,H,W) fp16 NCHW, weight (C_out, C_in*kH*kW) int8, w_scale (C_out) fp16, bias (C_out)
 * fp16 or NULL, output (N,C_out,H_out,W_out) fp16. Each output position's patch is quantized per
 * row exactly as the reference quantizes its im2col rows; one fused kernel over all samples.
 * workspace is accepted for signature compatibility and may be NULL. */
int forge_int8_conv2d_forward(const void* input, const int8_t* weight, const void* w_scale, const void* bias,
                              void* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                              int padW, int strideH, int strideW, int dilH, int dilW, void* workspace,
                              forge_stream_t stream);

/* forge::nn::int8_conv_transpose2d_k2s2_workspace_size - include/forge/nn/int8_conv_transpose2d.cuh:25-26,
 * src/nn/int8_conv_transpose2d.cu:103-117 (the reference's figure; no scratch is needed here). */
unsigned long long forge_int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out);

/* forge::nn::int8_conv_transpose2d_k2s2_forward - include/forge/nn/int8_conv_transpose2d.cuh:40-49,
 * src/nn/int8_conv_transpose2d.cu:123-191. 2x2 kernel, stride 2: input (N,C_in,H,W) fp16, weight
 * (4*C_out, C_in) int8 with row co*4 + kh*2 + kw, w_scale / bias (C_out) fp16, output
 * (N,C_out,2H,2W) fp16; the bias is added after the fp16 rounding of the scaled product, as the
 * reference's scatter step does. workspace may be NULL. */
int forge_int8_conv_transpose2d_k2s2_forward(const void* input, const int8_t* weight, const void* w_scale,
                                             const void* bias, void* output, int N, int C_in, int H, int W, int C_out,
                                             void* workspace, forge_stream_t stream);

/* ---------------------------------------------------------------- diagnostics (additive) */

/* Every wait inside the tcgen05 kernels (on a TMA load, a tensor-core commit, a free pipeline
 * stage) is bounded at two seconds. A wait that runs out makes the kernel record a code in a
 * per-device status word and leave through its normal teardown, so the context stays usable; the
 * output of that launch is then incomplete.
 *
 * forge_b200_device_status: FORGE_B200_OK when no kernel on the current device has given up since
 * the last reset, FORGE_B200_DEVICE_TIMEOUT when one has (FORGE_B200_LAUNCH_FAILED when the word
 * cannot be read). forge_b200_device_status_raw returns the recorded code itself:
 *   100-104 dense GEMM, 200-204 2:4-sparse GEMM, 300-304 / 400-404 their CTA-pair forms,
 *   500-506 fused quantize + sparse GEMM, 600-605 convolution; within a range x00 = misaligned
 *   shared memory, x01 = producer waiting for a free stage, x02 = MMA issuer waiting for a drained
 *   accumulator, x03 = MMA issuer waiting for operands, x04 and up = epilogue / gather waits.
 * Both synchronise the device; reset != 0 clears the word after reading it. */
int forge_b200_device_status(int reset);
int forge_b200_device_status_raw(int reset);

const char* forge_b200_status_string(int status);

#ifdef __cplusplus
}
#endif

#endif /* FORGE_B200_H */
