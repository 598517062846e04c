// Internal declarations of the dense INT8 GEMM launchers (gemm_dense.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fb200 {

// out (M,N) s32 = A (M,K) s8 x B (N,K)^T s8. force_bn: 64/128/256 to pin the tile width, else auto.
int dense_gemm_s32(const int8_t* A, const int8_t* B, int32_t* out, int M, int K, int N, cudaStream_t stream,
                   int force_bn);

// out (M,N) fp16 = fp16((act_scale[m] * w_scale[n]) * acc + bias[n]).
int dense_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                       const __half* bias, __half* out, int M, int K, int N, cudaStream_t stream, int force_bn);

// out (M,N) fp16 = fp16(SiLU(g) * u), g = (act_scale*wg_scale)*acc_g + bg, u likewise from Wu: the
// gate and up projections of a gated MLP in one GEMM pass. Wg, Wu (N,K) s8; bg / bu may be null.
// Needs K % 16 == 0, N % 8 == 0 and 16-byte aligned A, Wg, Wu, out (else kBadShape).
// Weight-streaming CUDA-core kernel for very few tokens (dense_gemv.cu). epi 0: out int32 (M,N); 1: fp16 dequant
// (+ bias). dense_gemv_fq: FP16 activations, quantized inside the kernel (the bits of quantize + GEMM).
bool dense_gemv_fits(int M, int K, const void* W, const void* x);
int dense_gemv(const int8_t* W, const int8_t* x, const float* act_scale, const __half* w_scale, const __half* bias,
               void* out, int M, int K, int N, cudaStream_t stream, int epi);
int dense_gemv_fq(const int8_t* W, const __half* x, const __half* w_scale, const __half* bias, __half* out, int M, int K,
                  int N, cudaStream_t stream);

int dense_gemm_gated(const int8_t* A, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                     const __half* wg_scale, const __half* wu_scale, const __half* bg, const __half* bu, __half* out,
                     int M, int K, int N, cudaStream_t stream);

// Address of this device's status word (a file-scope __device__ int); nullptr on failure.
int* status_word();
// Reads the status word back (synchronising copy); clears it when reset != 0. -1 on failure.
int read_device_status(int reset);

// Process-wide integer knobs (tuning.h); 0 = default behaviour.
enum TuningKnob : int {
    kKnobDenseTile = 0,        // pinned dense tile width
    kKnobSparseTile = 1,       // pinned sparse token-tile width
    kKnobMaxPairs = 2,         // CTA-pair kernels: launch at most this many pairs
    kKnobPairFlags = 3,        // CTA-pair kernels, measurement only: selects one of the instantiated variants
                               // (flag values kFlag... in gemm_pair.cu; e.g. 1 = operands stay resident after
                               // the first ring fill - wrong results, tensor-core side alone - 4 = the sparse
                               // MMA thread records its wait clocks, 128 = stores issued by the epilogue warps)
    kKnobLastPairs = 4,        // written by the launcher: CTA pairs of the last pair-kernel launch
    kKnobGemvVariant = 5,      // 1-4 token sparse kernel: 1 = token slices in registers, 2 = in shared memory
    kKnobGemvMaxTokens = 6,    // 1-4 token sparse kernel: largest M it takes (default 2)
    kKnobDenseBand = 7,        // dense CTA-pair kernel: 256-row blocks per raster band
    kKnobGemvDenseMaxTokens = 9,  // dense streaming kernel: largest M it takes (default 2, at most 16; negative: never)
    kKnobDenseOneAtom = 10,    // dense single-CTA kernel: 1 = one K atom per stage also for M <= 128 (measurement)
    kKnobDependentLaunch = 8,  // CTA-pair kernels as programmatic dependents: 0 = where requested, 1 = always, 2 = never
};
int tuning_knob(int key);
void set_tuning_knob(int key, int value);

// Quantize -> GEMM chains. launch_behind_quantizer(true): the calling thread's next GEMM launch directly
// follows, on the same stream, the per-token quantizer whose output it reads, and may be launched as
// that kernel's programmatic dependent: it starts while the quantizer drains, streams its weights at
// once and executes griddepcontrol.wait before its first access to the activations and their scales.
// The request is consumed by the launch (take_behind_quantizer); false withdraws it. Knob 8 overrides.
void launch_behind_quantizer(bool on);
bool take_behind_quantizer();
struct BehindQuantizer {
    BehindQuantizer() { launch_behind_quantizer(true); }
    ~BehindQuantizer() { launch_behind_quantizer(false); }
};

// kern<<<grid, block, smem, stream>>>(args...), with the programmatic-serialization attribute when the
// calling thread asked for it.
template <typename Kern, typename... Args>
inline cudaError_t launch_gemm(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = take_behind_quantizer() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace fb200
