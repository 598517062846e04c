// forge_int8_linear_static: the W8A8 linear layer for callers that cannot supply scratch memory.
//
// forge_int8_linear needs two caller-owned scratch buffers (the int8 copy of the activations
// and the per-token scales). Some callers have nowhere to get them from: a plug-in running
// under a host framework whose allocator already owns the GPU's memory and lends none to
// third-party code, or a latency-critical serving loop in which cudaMalloc is off-limits
// because it synchronises the whole device. This variant keeps that scratch in a fixed array
// inside the library image instead. It allocates nothing - no cudaMalloc / cudaFree, no
// allocating library call - and the caller still passes every input and the output.
//
// Cost and limits: the array (16 MiB + 64 KiB) is part of every CUDA context that loads
// libforge_b200 and stays resident until the process exits. Requests with M*K > 16 Mi
// elements or M > 16384 tokens are rejected with FORGE_B200_TOO_LARGE. All calls on a device
// share the one array: two calls whose kernels can overlap on the GPU (different streams, no
// ordering between them) race on it - order them yourself. Nothing in the array has to start at
// zero: the quantizer overwrites all M*K bytes and M scales before the GEMM reads them, so
// whatever an earlier call left behind is never observed.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress,
// with that device current). Make that first call on a device during start-up, outside any
// stream capture.
#include "../../include/forge_b200.h"
#include "common.cuh"
#include "gemm_dense.cuh"
#include "gemm_pair.cuh"
#include "kernels.cuh"

namespace {

constexpr size_t kMaxActBytes = 16u << 20;   // int8 activations: M*K <= 16 Mi
constexpr int kMaxTokens = 16384;            // per-token fp32 scales
constexpr size_t kScratchBytes = kMaxActBytes + sizeof(float) * kMaxTokens;

// In host code this name is only a handle for the symbol API, never a device address.
static __device__ __align__(256) unsigned char g_linear_scratch[kScratchBytes];

// Device address of g_linear_scratch on the current device, looked up once per device.
unsigned char* scratch_base() {
    static unsigned char* base[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (base[dev] == nullptr) {
        unsigned char* p = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_linear_scratch) != cudaSuccess) return nullptr;
        base[dev] = p;
    }
    return base[dev];
}

}  // namespace

extern "C" int forge_int8_linear_static(const void* x, const int8_t* w_int8, const void* w_scale, const void* bias,
                                        void* output, int M, int K, int N, forge_stream_t stream) {
    using namespace fb200;
    if (M <= 0 || K <= 0 || N <= 0) return kOk;
    if (x == nullptr || w_int8 == nullptr || w_scale == nullptr || output == nullptr) return kBadPointer;
    if (static_cast<size_t>(M) * static_cast<size_t>(K) > kMaxActBytes || M > kMaxTokens) return kTooLarge;
    unsigned char* base = scratch_base();
    if (base == nullptr) return kLaunchFailed;
    int8_t* act_int8 = reinterpret_cast<int8_t*>(base);
    float* act_scale = reinterpret_cast<float*>(base + kMaxActBytes);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int r = quantize_activation(static_cast<const __half*>(x), act_int8, act_scale, M, K, s);
    if (r != kOk) return r;
    const BehindQuantizer dependent;
    return dense_gemm_dequant(act_int8, w_int8, act_scale, static_cast<const __half*>(w_scale),
                              static_cast<const __half*>(bias), static_cast<__half*>(output), M, K, N, s,
                              tuning_knob(kKnobDenseTile));
}
