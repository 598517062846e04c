// Compile-and-link check of the C++ face: code written against the reference's headers and
// call style (tests/test_int8_sparse_gemm.cu, tests/test_quantize.cu, tests/test_int8_conv2d.cu in the Forge tree) must
// build against include/forge/... and link with libforge_b200.so. Not executed on CPU boxes.
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

using namespace forge;

int main(int argc, char**) {
    if (argc < 100) return 0;   // link check only
    __half* h = nullptr;
    int8_t* i8 = nullptr;
    int32_t* i32 = nullptr;
    float* f = nullptr;
    uint8_t* u8 = nullptr;
    uint32_t* u32 = nullptr;
    quant::fused_quantize_activation(h, i8, f, 1, 8);
    quant::fused_quantize_activation_kernel<<<1, 32>>>(h, i8, f, 8);
    quant::fused_dequantize_bias(i32, f, h, nullptr, h, 1, 8);
    quant::fused_dequantize_bias_kernel<<<1, 32>>>(i32, f, h, h, h, 8);
    sparsity::prune_compress_24(i8, i8, u8, 1, 64);
    sparsity::prune_compress_kernel<<<1, 32>>>(i8, i8, u8, 1, 64);
    sparsity::pack_metadata(u8, u32, 1, 64);
    sparsity::pack_metadata_kernel<<<1, 32>>>(u8, u32, 1, 64);
    gemm::int8_gemm_dequant(i8, i8, f, h, nullptr, h, 1, 64, 16);
    gemm::int8_linear(h, i8, h, h, h, 1, 64, 16, i8, f);
    gemm::int8_dp4a_gemm_dequant(i8, i8, f, h, h, h, 1, 64, 16);
    gemm::int8_dp4a_linear(h, i8, h, h, h, 1, 64, 16, i8, f);
    gemm::int8_gemm(i8, i8, f, h, h, h, 1, 64, 16);
    const gemm::SparseGemmPlan plan = gemm::sparse_int8_gemm_plan(1, 64, 16, 0, true, gemm::kSparseTile128x64);
    gemm::sparse_int8_gemm(i8, i8, u32, f, h, h, h, 1, 64, 16, f, plan.split_k, nullptr, plan.tile);
    gemm::sparse_int8_linear(h, i8, u32, h, h, h, 1, 64, 16, i8, f, nullptr, 0, nullptr, gemm::kSparseLinearTwoPass);
    gemm::splitk_reduce(f, h, h, 1, 16);
    // tests/test_int8_conv2d.cu:142-150, tests/test_int8_special_conv.cu (call style of the conv callers)
    void* ws = nullptr;
    const size_t conv_ws = nn::int8_conv2d_workspace_size(8, 16, 16, 16, 3, 3, 1, 1, 1, 1);
    nn::int8_conv2d_forward(h, i8, h, h, h, 1, 8, 16, 16, 16, 3, 3, 1, 1, 1, 1, 1, 1, ws);
    const size_t convt_ws = nn::int8_conv_transpose2d_k2s2_workspace_size(32, 16, 16, 64);
    nn::int8_conv_transpose2d_k2s2_forward(h, i8, h, nullptr, h, 1, 32, 16, 16, 64, ws);
    if (conv_ws + convt_ws == 0) return 1;
    return gemm::has_wmma_int8() && gemm::sparse_int8_linear_fused(1, 64, 16) && FORGE_SPARSE_GEMM_API_VERSION == 3;
}
