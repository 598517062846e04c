// extern "C" boundary of libforge_b200.so: one symbol per reference entry point
// (declared and cited in include/forge_b200.h). Thin argument adaptation only.
#include "../../include/forge_b200.h"
#include "common.cuh"
#include "conv.cuh"
#include "gemm_dense.cuh"
#include "gemm_pair.cuh"
#include "gemm_sparse.cuh"
#include "gemm_fq.cuh"
#include "kernels.cuh"

using namespace fb200;

namespace {

inline int force_dense_bn() { return tuning_knob(kKnobDenseTile); }
inline int force_sparse_bt() { return tuning_knob(kKnobSparseTile); }

inline cudaStream_t S(forge_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
inline const __half* H(const void* p) { return static_cast<const __half*>(p); }
inline __half* H(void* p) { return static_cast<__half*>(p); }

// Tile id of the reference API -> tile knob of the tcgen05 kernels: the reference's 256-row weight
// tile is the CTA-pair kernel (256 weight rows per pair of SMs, 192 or 224 tokens by the cost model,
// knob 1000); its 128x128 tile is the single-CTA kernel with 128 tokens; its 128x64 tile the single-CTA
// kernel with 64 or 32 tokens by the cost model (knob 1) - and, for 1-2 tokens, the weight-streaming
// kernel (knob 0: the automatic choice).
inline int tile_to_bt(int tile, int M) {
    switch (tile) {
    case FORGE_SPARSE_TILE_256x128: return 1000;
    case FORGE_SPARSE_TILE_128x128: return 128;
    case FORGE_SPARSE_TILE_128x64: return M <= 2 ? 0 : 1;
    default: return 0;
    }
}

inline int choice_to_tile(const SparseChoice& c) {
    if (c.kind == 2) return FORGE_SPARSE_TILE_256x128;
    if (c.kind == 1 && c.bt == 128) return FORGE_SPARSE_TILE_128x128;
    return FORGE_SPARSE_TILE_128x64;
}

// fp32 workspace + bias -> fp16, the contract of the reference's splitk_reduce_kernel
// (src/gemm/int8_sparse.cu:99-111).
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, const __half* __restrict__ bias,
                                     __half* __restrict__ out, int N_out, long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = ws[i];
    if (bias != nullptr) v += __half2float(bias[i % N_out]);
    out[i] = __float2half_rn(v);
}

}  // namespace

extern "C" {

int forge_fused_quantize_activation(const void* input, int8_t* output, float* scales, int M, int K,
                                    forge_stream_t stream) {
    return quantize_activation(H(input), output, scales, M, K, S(stream));
}

int forge_fused_dequantize_bias(const int32_t* input, const float* act_scale, const void* w_scale, const void* bias,
                                void* output, int M, int N, forge_stream_t stream) {
    return dequantize_bias(input, act_scale, H(w_scale), H(bias), H(output), M, N, S(stream));
}

int forge_int8_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale,
                            const void* bias, void* output, int M, int K, int N, forge_stream_t stream) {
    return dense_gemm_dequant(A, B, act_scale, H(w_scale), H(bias), H(output), M, K, N, S(stream), force_dense_bn());
}

int forge_int8_gemm(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale, const void* bias,
                    void* output, int M, int K, int N, forge_stream_t stream) {
    return forge_int8_gemm_dequant(A, B, act_scale, w_scale, bias, output, M, K, N, stream);
}

int forge_int8_dp4a_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const void* w_scale,
                                 const void* bias, void* output, int M, int K, int N, forge_stream_t stream) {
    return forge_int8_gemm_dequant(A, B, act_scale, w_scale, bias, output, M, K, N, stream);
}

int forge_int8_linear(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias, void* output,
                      int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale, forge_stream_t stream) {
    if (M <= 0 || K <= 0 || N <= 0) return kOk;
    // very few tokens: the weight-streaming kernel quantizes the token rows itself (no scratch traffic)
    if (x != nullptr && w_int8 != nullptr && w_scale != nullptr && output != nullptr && dense_gemv_fits(M, K, w_int8, x) &&
        device_is_sm100())
        return dense_gemv_fq(w_int8, H(x), H(w_scale), H(bias), H(output), M, K, N, S(stream));
    const int r = quantize_activation(H(x), scratch_a_int8, scratch_a_scale, M, K, S(stream));
    if (r != kOk) return r;
    const BehindQuantizer dependent;
    return dense_gemm_dequant(scratch_a_int8, w_int8, scratch_a_scale, H(w_scale), H(bias), H(output), M, K, N,
                              S(stream), force_dense_bn());
}

int forge_int8_dp4a_linear(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias, void* output,
                           int M, int K, int N, int8_t* scratch_a_int8, float* scratch_a_scale,
                           forge_stream_t stream) {
    return forge_int8_linear(x, w_int8, w_scale, bias, output, M, K, N, scratch_a_int8, scratch_a_scale, stream);
}

int forge_get_compute_capability(int device) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) return 0;
    return major * 10 + minor;
}

int forge_has_wmma_int8(int device) { return forge_get_compute_capability(device) >= 80 ? 1 : 0; }

int forge_int8_gemm_s32(const int8_t* A, const int8_t* B, int32_t* output, int M, int K, int N,
                        forge_stream_t stream) {
    return dense_gemm_s32(A, B, output, M, K, N, S(stream), force_dense_bn());
}

int forge_sparse_int8_gemm_plan(int M, int K, int N_out, int split_k, int have_workspace, int tile, int* out_tile,
                                int* out_split_k) {
    // The K loop is never split: the exact s32 accumulation in TMEM covers the whole K range.
    (void)split_k;
    (void)have_workspace;
    if (tile >= FORGE_SPARSE_NUM_TILES) tile = FORGE_SPARSE_TILE_AUTO;   // reference: int8_sparse.cu:895
    int bt = force_sparse_bt();
    if (bt == 0 && tile >= 0) bt = tile_to_bt(tile, M);
    const SparseChoice c = sparse_choose(M, K, N_out, K % 128 == 0, K % 32 == 0, bt, true);
    if (out_tile) *out_tile = choice_to_tile(c);
    if (out_split_k) *out_split_k = 1;
    return kOk;
}

int forge_sparse_int8_gemm(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta,
                           const float* act_scale, const void* w_scale, const void* bias, void* output, int M, int K,
                           int N_out, float* splitk_workspace, int split_k, forge_stream_t stream, int tile) {
    (void)splitk_workspace;
    (void)split_k;
    int bt = force_sparse_bt();
    if (bt == 0 && tile >= 0 && tile < FORGE_SPARSE_NUM_TILES) bt = tile_to_bt(tile, M);
    return sparse_gemm_dequant(W_comp, x_int8, w_meta, act_scale, H(w_scale), H(bias), H(output), M, K, N_out,
                               S(stream), bt);
}

// Policy of the automatic path (the reference's is sp_use_fused, src/gemm/int8_sparse.cu:930-938: it fuses
// narrow layers whose activation does not fit L2 on an RTX 4090). Measured on B200 at M = 147456 the
// fused kernel beats quantize + pair GEMM for every K <= 1280 when N_out <= 640 (7-26 %: K = 1280,
// N_out = 320, the reference's showcase shape, 0.162 against 0.175 ms) and for K <= 1024 up to N_out = 1280
// (6-9 %); it loses at K = 1280, N_out = 1280 (its 64-token blocks re-stream the weights twice as often as
// the pair kernel's tiles and its N = 64 instructions run at a third of the tensor rate) and is on par or
// slower while the FP16 activation still fits L2 (M = 32768, K = 1280: 53 against 52 us; M = 2048: 22
// against 17 us). Hence: fuse when the kernel can take K, the activation does not fit L2, and the
// layer is narrow.
int forge_sparse_int8_linear_fused(int M, int K, int N_out) {
    // one and two tokens: the weight-streaming kernel quantizes the token rows itself (sparse_gemv_fq)
    if (M >= 1 && M <= 2 && N_out > 0 && K > 0 && K % 32 == 0 && K <= 4096) return 1;
    if (M <= 0 || N_out <= 0 || K <= 0 || K % 128 != 0 || K > 1280) return 0;
    if ((size_t)M * K * 2 <= l2_bytes()) return 0;
    return (N_out <= 640 || (N_out <= 1280 && K <= 1024)) ? 1 : 0;
}

int forge_sparse_int8_linear(const void* x, const int8_t* W_comp, const uint32_t* w_meta, const void* w_scale,
                             const void* bias, void* output, int M, int K, int N_out, int8_t* scratch_x_int8,
                             float* scratch_x_scale, float* splitk_workspace, int split_k, forge_stream_t stream,
                             int path) {
    if (M <= 0 || K <= 0 || N_out <= 0) return kOk;
    // Fused quantize + GEMM: forced, or chosen when the caller did not ask for a specific split-K
    // (same rule as the reference, int8_sparse.cu:1026-1034). It does not touch the scratch buffers.
    if (path != FORGE_SPARSE_LINEAR_TWO_PASS && split_k <= 1 && sparse_gemv_fq_fits(M, K, x) && aligned16(W_comp) &&
        (reinterpret_cast<uintptr_t>(w_meta) & 3) == 0)
        return sparse_gemv_fq(W_comp, H(x), w_meta, H(w_scale), H(bias), H(output), M, K, N_out, S(stream));
    const bool can_fuse = sparse_fq_fits(K, x) && aligned16(W_comp) && aligned16(w_meta);
    if (can_fuse && (path == FORGE_SPARSE_LINEAR_FUSED ||
                     (path == FORGE_SPARSE_LINEAR_AUTO && split_k <= 1 &&
                      forge_sparse_int8_linear_fused(M, K, N_out) != 0)))
        return sparse_fq_linear(H(x), W_comp, w_meta, H(w_scale), H(bias), H(output), M, K, N_out, S(stream));
    if (scratch_x_int8 == nullptr || scratch_x_scale == nullptr) return kBadPointer;
    const int r = quantize_activation(H(x), scratch_x_int8, scratch_x_scale, M, K, S(stream));
    if (r != kOk) return r;
    const BehindQuantizer dependent;
    return forge_sparse_int8_gemm(W_comp, scratch_x_int8, w_meta, scratch_x_scale, w_scale, bias, output, M, K, N_out,
                                  splitk_workspace, split_k, stream, FORGE_SPARSE_TILE_AUTO);
}

int forge_splitk_reduce(const float* workspace, const void* bias, void* output, int M, int N_out,
                        forge_stream_t stream) {
    if (M <= 0 || N_out <= 0) return kOk;
    if (workspace == nullptr || output == nullptr) return kBadPointer;
    const long long total = (long long)M * N_out;
    splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, S(stream)>>>(workspace, H(bias), H(output), N_out,
                                                                               total);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int forge_sparse_int8_gemm_s32(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta, int32_t* output,
                               int M, int K, int N_out, forge_stream_t stream) {
    return sparse_gemm_s32(W_comp, x_int8, w_meta, output, M, K, N_out, S(stream), force_sparse_bt());
}

int forge_sparse_int8_gemm_multi(const int8_t* W_comp, const int8_t* x_int8, const uint32_t* w_meta,
                                 const float* act_scale, const void* w_scale, const void* bias, void* const* outputs,
                                 int n_outs, long long ld_out, int M, int K, int N_out, forge_stream_t stream) {
    return sparse_gemm_dequant_multi(W_comp, x_int8, w_meta, act_scale, H(w_scale), H(bias), outputs, n_outs, ld_out,
                                     M, K, N_out, S(stream));
}

int forge_int8_gated_gemm(const int8_t* x_int8, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                          const void* wg_scale, const void* wu_scale, const void* bg, const void* bu, void* h_out,
                          int M, int K, int N, forge_stream_t stream) {
    return dense_gemm_gated(x_int8, Wg, Wu, act_scale, H(wg_scale), H(wu_scale), H(bg), H(bu), H(h_out), M, K, N,
                            S(stream));
}

int forge_sparse_int8_gated_gemm(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp,
                                 const uint32_t* wu_meta, const int8_t* x_int8, const float* act_scale,
                                 const void* wg_scale, const void* wu_scale, const void* bg, const void* bu,
                                 void* h_out, int M, int K, int N_out, forge_stream_t stream) {
    return sparse_gemm_gated(Wg_comp, wg_meta, Wu_comp, wu_meta, x_int8, act_scale, H(wg_scale), H(wu_scale), H(bg),
                             H(bu), H(h_out), M, K, N_out, S(stream), force_sparse_bt());
}

namespace {

inline size_t pad256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

struct MlpWorkspace {
    int8_t* xq;
    float* xs;
    __half* h;
    int8_t* hq;
    float* hs;
    size_t bytes;
};

inline MlpWorkspace carve_mlp_workspace(void* base, int M, int d_model, int d_ffn) {
    MlpWorkspace w;
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    w.xq = reinterpret_cast<int8_t*>(p + off);
    off += pad256((size_t)M * d_model);
    w.xs = reinterpret_cast<float*>(p + off);
    off += pad256((size_t)M * sizeof(float));
    w.h = reinterpret_cast<__half*>(p + off);
    off += pad256((size_t)M * d_ffn * sizeof(__half));
    w.hq = reinterpret_cast<int8_t*>(p + off);
    off += pad256((size_t)M * d_ffn);
    w.hs = reinterpret_cast<float*>(p + off);
    off += pad256((size_t)M * sizeof(float));
    w.bytes = off;
    return w;
}

}  // namespace

unsigned long long forge_w8a8_gated_mlp_workspace_bytes(int M, int d_model, int d_ffn) {
    if (M <= 0 || d_model <= 0 || d_ffn <= 0) return 0;
    return carve_mlp_workspace(nullptr, M, d_model, d_ffn).bytes;
}

int forge_w8a8_gated_mlp(const void* x, const int8_t* Wg, const int8_t* Wu, const int8_t* Wd, const void* wg_scale,
                         const void* wu_scale, const void* wd_scale, const void* bg, const void* bu, const void* bd,
                         void* out, int M, int d_model, int d_ffn, void* workspace, forge_stream_t stream) {
    if (M <= 0 || d_model <= 0 || d_ffn <= 0) return kOk;
    if (x == nullptr || workspace == nullptr || out == nullptr) return kBadPointer;
    const MlpWorkspace w = carve_mlp_workspace(workspace, M, d_model, d_ffn);
    int r = quantize_activation(H(x), w.xq, w.xs, M, d_model, S(stream));
    if (r != kOk) return r;
    launch_behind_quantizer(true);
    r = dense_gemm_gated(w.xq, Wg, Wu, w.xs, H(wg_scale), H(wu_scale), H(bg), H(bu), w.h, M, d_model, d_ffn,
                         S(stream));
    launch_behind_quantizer(false);
    if (r != kOk) return r;
    r = quantize_activation(w.h, w.hq, w.hs, M, d_ffn, S(stream));
    if (r != kOk) return r;
    const BehindQuantizer dependent;
    return dense_gemm_dequant(w.hq, Wd, w.hs, H(wd_scale), H(bd), H(out), M, d_ffn, d_model, S(stream),
                              force_dense_bn());
}

int forge_sparse_w8a8_gated_mlp(const void* x, const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp,
                                const uint32_t* wu_meta, const int8_t* Wd_comp, const uint32_t* wd_meta,
                                const void* wg_scale, const void* wu_scale, const void* wd_scale, const void* bg,
                                const void* bu, const void* bd, void* out, int M, int d_model, int d_ffn,
                                void* workspace, forge_stream_t stream) {
    if (M <= 0 || d_model <= 0 || d_ffn <= 0) return kOk;
    if (x == nullptr || workspace == nullptr || out == nullptr) return kBadPointer;
    const MlpWorkspace w = carve_mlp_workspace(workspace, M, d_model, d_ffn);
    int r = quantize_activation(H(x), w.xq, w.xs, M, d_model, S(stream));
    if (r != kOk) return r;
    launch_behind_quantizer(true);
    r = sparse_gemm_gated(Wg_comp, wg_meta, Wu_comp, wu_meta, w.xq, w.xs, H(wg_scale), H(wu_scale), H(bg), H(bu), w.h,
                          M, d_model, d_ffn, S(stream), force_sparse_bt());
    launch_behind_quantizer(false);
    if (r != kOk) return r;
    r = quantize_activation(w.h, w.hq, w.hs, M, d_ffn, S(stream));
    if (r != kOk) return r;
    const BehindQuantizer dependent;
    return sparse_gemm_dequant(Wd_comp, w.hq, wd_meta, w.hs, H(wd_scale), H(bd), H(out), M, d_ffn, d_model, S(stream),
                               force_sparse_bt());
}

int forge_prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K,
                            forge_stream_t stream) {
    return prune_compress_24(weight, compressed, metadata_raw, N, K, S(stream));
}

int forge_pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K, forge_stream_t stream) {
    return pack_metadata(meta_raw, meta_packed, N, K, S(stream));
}

int forge_prepare_weight(const void* weight, int weight_is_half, int8_t* w_int8, int8_t* W_comp, uint32_t* w_meta,
                         void* w_scale, int N, int K, forge_stream_t stream) {
    return prepare_weight(weight, weight_is_half, w_int8, W_comp, w_meta, H(w_scale), N, K, S(stream));
}

unsigned long long forge_int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                                                   int padW, int strideH, int strideW, int dilH, int dilW) {
    return int8_conv2d_workspace_size(C_in, H, W, C_out, kH, kW, padH, padW, strideH, strideW, dilH, dilW);
}

int forge_int8_conv2d_forward(const void* input, const int8_t* weight, const void* w_scale, const void* bias,
                              void* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                              int padW, int strideH, int strideW, int dilH, int dilW, void* workspace,
                              forge_stream_t stream) {
    (void)workspace;
    return int8_conv2d_forward(static_cast<const __half*>(input), weight, static_cast<const __half*>(w_scale),
                               static_cast<const __half*>(bias), static_cast<__half*>(output), N, C_in, H, W, C_out, kH, kW, padH,
                               padW, strideH, strideW, dilH, dilW, S(stream));
}

unsigned long long forge_int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out) {
    return int8_conv_transpose2d_k2s2_workspace_size(C_in, H, W, C_out);
}

int forge_int8_conv_transpose2d_k2s2_forward(const void* input, const int8_t* weight, const void* w_scale,
                                             const void* bias, void* output, int N, int C_in, int H, int W, int C_out,
                                             void* workspace, forge_stream_t stream) {
    (void)workspace;
    return int8_conv_transpose2d_k2s2_forward(static_cast<const __half*>(input), weight,
                                              static_cast<const __half*>(w_scale), static_cast<const __half*>(bias),
                                              static_cast<__half*>(output), N, C_in, H, W, C_out,
                                              S(stream));
}

const char* forge_b200_status_string(int status) {
    switch (status) {
    case kOk: return "ok";
    case kBadShape: return "bad shape";
    case kBadPointer: return "required pointer is null";
    case kUnsupportedArch: return "device is not sm_100";
    case kLaunchFailed: return "kernel launch or driver call failed";
    case kDeviceTimeout: return "a device-side wait ran out";
    case kTooLarge: return "exceeds a fixed capacity";
    default: return "unknown status";
    }
}

}  // extern "C"
