// extern "C" shim around the reference's own GPU launchers, so the parity tests can call the
// reference kernels (compiled for sm_100a from their sources, unmodified) through ctypes.
// TEST INFRASTRUCTURE: built by oracle/build.py into oracle/_ref/libforge_ref.so, only when
// the reference source tree is present; loaded only by tests/ and bench.py's comparison legs.
#include <forge/gemm/int8_dense.cuh>
#include <forge/gemm/int8_dp4a.cuh>
#include <forge/gemm/int8_gemm.cuh>
#include <forge/gemm/int8_sparse.cuh>
#include <forge/nn/int8_conv2d.cuh>
#include <forge/nn/int8_conv_transpose2d.cuh>
#include <forge/quant/dequantize.cuh>
#include <forge/quant/quantize.cuh>
#include <forge/sparsity/pack_metadata.cuh>
#include <forge/sparsity/prune_compress.cuh>

extern "C" {

void ref_fused_quantize_activation(const void* in, int8_t* out, float* scales, int M, int K, void* stream) {
    forge::quant::fused_quantize_activation((const __half*)in, out, scales, M, K, (cudaStream_t)stream);
}
// the two-pass kernel launched directly, as tests/test_quantize.cu:54-55 does
void ref_quantize_two_pass(const void* in, int8_t* out, float* scales, int M, int K, void* stream) {
    int threads = ((K + 31) / 32) * 32;
    if (threads > 256) threads = 256;
    forge::quant::fused_quantize_activation_kernel<<<M, threads, 0, (cudaStream_t)stream>>>((const __half*)in, out,
                                                                                            scales, K);
}
void ref_fused_dequantize_bias(const int32_t* in, const float* as, const void* ws, const void* bias, void* out, int M,
                               int N, void* stream) {
    forge::quant::fused_dequantize_bias(in, as, (const __half*)ws, (const __half*)bias, (__half*)out, M, N,
                                        (cudaStream_t)stream);
}
void ref_int8_gemm_dequant(const int8_t* A, const int8_t* B, const float* as, const void* ws, const void* bias,
                           void* out, int M, int K, int N, void* stream) {
    forge::gemm::int8_gemm_dequant(A, B, as, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N,
                                   (cudaStream_t)stream);
}
void ref_int8_linear(const void* x, const int8_t* w, const void* ws, const void* bias, void* out, int M, int K, int N,
                     int8_t* sa, float* ss, void* stream) {
    forge::gemm::int8_linear((const __half*)x, w, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N, sa,
                             ss, (cudaStream_t)stream);
}
void ref_sparse_int8_gemm(const int8_t* Wc, const int8_t* x, const uint32_t* meta, const float* as, const void* ws,
                          const void* bias, void* out, int M, int K, int N, float* wksp, int split_k, void* stream,
                          int tile) {
    forge::gemm::sparse_int8_gemm(Wc, x, meta, as, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N,
                                  wksp, split_k, (cudaStream_t)stream, tile);
}
void ref_sparse_int8_linear(const void* x, const int8_t* Wc, const uint32_t* meta, const void* ws, const void* bias,
                            void* out, int M, int K, int N, int8_t* sx, float* ss, float* wksp, int split_k,
                            void* stream, int path) {
    forge::gemm::sparse_int8_linear((const __half*)x, Wc, meta, (const __half*)ws, (const __half*)bias, (__half*)out,
                                    M, K, N, sx, ss, wksp, split_k, (cudaStream_t)stream, path);
}
void ref_splitk_reduce(const float* wksp, const void* bias, void* out, int M, int N, void* stream) {
    forge::gemm::splitk_reduce(wksp, (const __half*)bias, (__half*)out, M, N, (cudaStream_t)stream);
}
// the dispatch front end and the legacy dp4a backend (src/gemm/int8_gemm.cu, src/gemm/int8_dp4a.cu)
void ref_int8_gemm(const int8_t* A, const int8_t* B, const float* as, const void* ws, const void* bias, void* out,
                   int M, int K, int N, void* stream) {
    forge::gemm::int8_gemm(A, B, as, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N,
                           (cudaStream_t)stream);
}
void ref_int8_dp4a_gemm_dequant(const int8_t* A, const int8_t* B, const float* as, const void* ws, const void* bias,
                                void* out, int M, int K, int N, void* stream) {
    forge::gemm::int8_dp4a_gemm_dequant(A, B, as, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N,
                                        (cudaStream_t)stream);
}
void ref_int8_dp4a_linear(const void* x, const int8_t* w, const void* ws, const void* bias, void* out, int M, int K,
                          int N, int8_t* sa, float* ss, void* stream) {
    forge::gemm::int8_dp4a_linear((const __half*)x, w, (const __half*)ws, (const __half*)bias, (__half*)out, M, K, N,
                                  sa, ss, (cudaStream_t)stream);
}
int ref_get_compute_capability(int device) { return forge::gemm::get_compute_capability(device); }
int ref_has_wmma_int8(int device) { return forge::gemm::has_wmma_int8(device) ? 1 : 0; }
void ref_prune_compress_24(const int8_t* w, int8_t* c, uint8_t* m, int N, int K, void* stream) {
    forge::sparsity::prune_compress_24(w, c, m, N, K, (cudaStream_t)stream);
}
void ref_pack_metadata(const uint8_t* raw, uint32_t* packed, int N, int K, void* stream) {
    forge::sparsity::pack_metadata(raw, packed, N, K, (cudaStream_t)stream);
}

// The two in-library callers of the INT8 GEMM (src/nn/int8_conv2d.cu, src/nn/int8_conv_transpose2d.cu).
unsigned long long ref_int8_conv2d_workspace_size(int C_in, int H, int W, int C_out, int kH, int kW, int padH, int padW,
                                                  int strideH, int strideW, int dilH, int dilW) {
    return forge::nn::int8_conv2d_workspace_size(C_in, H, W, C_out, kH, kW, padH, padW, strideH, strideW, dilH, dilW);
}
void ref_int8_conv2d_forward(const void* input, const int8_t* weight, const void* w_scale, const void* bias,
                             void* output, int N, int C_in, int H, int W, int C_out, int kH, int kW, int padH,
                             int padW, int strideH, int strideW, int dilH, int dilW, void* workspace, void* stream) {
    forge::nn::int8_conv2d_forward((const __half*)input, weight, (const __half*)w_scale, (const __half*)bias,
                                   (__half*)output, N, C_in, H, W, C_out, kH, kW, padH, padW, strideH, strideW, dilH,
                                   dilW, workspace, (cudaStream_t)stream);
}
unsigned long long ref_int8_conv_transpose2d_k2s2_workspace_size(int C_in, int H, int W, int C_out) {
    return forge::nn::int8_conv_transpose2d_k2s2_workspace_size(C_in, H, W, C_out);
}
void ref_int8_conv_transpose2d_k2s2_forward(const void* input, const int8_t* weight, const void* w_scale,
                                            const void* bias, void* output, int N, int C_in, int H, int W, int C_out,
                                            void* workspace, void* stream) {
    forge::nn::int8_conv_transpose2d_k2s2_forward((const __half*)input, weight, (const __half*)w_scale,
                                                  (const __half*)bias, (__half*)output, N, C_in, H, W, C_out,
                                                  workspace, (cudaStream_t)stream);
}

}  // extern "C"
