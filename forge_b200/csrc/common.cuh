// Shared host/device helpers for the forge_b200 kernels: status codes, exact-arithmetic
// helpers that pin the rounding/flush behaviour of the reference's fast-math build, and
// the host side of TMA (tensor-map encoding through the driver entry point).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

namespace fb200 {

// Status codes returned by every extern "C" entry point (0 = ok).
enum Status : int {
    kOk = 0,
    kBadShape = 1,         // negative size, or a size the entry point documents as unsupported
    kBadPointer = 2,       // required pointer is null
    kUnsupportedArch = 3,  // current device is not sm_100
    kLaunchFailed = 4,     // cudaGetLastError() after the launch, or a driver call, failed
    kDeviceTimeout = 5,    // a bounded device-side wait ran out (read back from the status word)
    kTooLarge = 6,         // exceeds a documented fixed capacity
};

constexpr int kNumSMsB200 = 148;

inline int sm_count() {
    static int cache[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int& n = cache[dev & 63];
    if (n == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = kNumSMsB200;
    }
    return n;
}

inline size_t l2_bytes() {
    static int cache[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    int& n = cache[dev & 63];
    if (n == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrL2CacheSize, dev);
        if (n <= 0) n = 1;
    }
    return (size_t)n;
}

// True when the current device can run the tcgen05 kernels (compute capability 10.x).
inline bool device_is_sm100() {
    static int cache[64] = {};   // 0 unknown, 1 yes, 2 no
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    int& c = cache[dev & 63];
    if (c == 0) {
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        c = (major == 10) ? 1 : 2;
    }
    return c == 1;
}

// ---------------------------------------------------------------------------------------
// Arithmetic with the exact PTX operations the reference build (-use_fast_math) emits.
// Written as inline PTX so the result does not depend on this library's compile flags.

__device__ __forceinline__ float mul_ftz(float a, float b) {
    float r;
    asm("mul.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float fma_ftz(float a, float b, float c) {
    float r;
    asm("fma.rn.ftz.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float max_ftz(float a, float b) {
    float r;
    asm("max.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float abs_ftz(float a) {
    float r;
    asm("abs.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}
__device__ __forceinline__ float div_approx_ftz(float a, float b) {
    float r;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float rcp_approx_ftz(float a) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    return r;
}
__device__ __forceinline__ int cvt_rni_ftz(float a) {
    int r;
    asm("cvt.rni.ftz.s32.f32 %0, %1;" : "=r"(r) : "f"(a));
    return r;
}

// Per-token scale and its reciprocal from the row's absolute maximum.
__device__ __forceinline__ void quant_scale(float amax, float& scale, float& inv_scale) {
    scale = div_approx_ftz(max_ftz(amax, 1e-8f), 127.0f);
    inv_scale = rcp_approx_ftz(scale);
}
__device__ __forceinline__ int quant_value(float x, float inv_scale) {
    int q = cvt_rni_ftz(mul_ftz(x, inv_scale));
    return max(-128, min(127, q));
}

// Four s32 values -> four saturated s8 bytes (first value in the low byte): the quantizer's clamp
// to [-128, 127] and the byte packing in two instructions.
__device__ __forceinline__ uint32_t pack4_sat(int q0, int q1, int q2, int q3) {
    uint32_t hi, d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(q3), "r"(q2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(q1), "r"(q0), "r"(hi));
    return d;
}

// GEMM-epilogue dequantisation: (act_scale * w_scale) * acc (+ bias), one fp16 rounding.
__device__ __forceinline__ float dequant_gemm(int acc, float as_ws, float bias, bool has_bias) {
    const float a = static_cast<float>(acc);
    return has_bias ? fma_ftz(a, as_ws, bias) : mul_ftz(a, as_ws);
}

// SiLU(g) * u in fp32: g / (1 + exp(-g)) * u, with the fast exponential and division (the
// composition is this library's own; the reference has no gated epilogue). One fp16 rounding
// happens at the caller.
__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
    return *reinterpret_cast<const uint32_t*>(&h);
}

// ---------------------------------------------------------------------------------------
// TMA tensor maps (host).

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
    static PFN_encodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
    return fn;
}

// Encodes a tiled tensor map of up to 3 dimensions. dims/box are in elements (innermost
// first), strides_bytes[i] is the byte stride of dimension i+1. Returns false on failure.
// Encoding costs about a microsecond of host time per map and a launch needs three to five of
// them, which matters for microsecond-sized problems, so each host thread keeps the last maps it
// built (keyed by every encode argument; a map depends on nothing else).
inline bool make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    struct Key {
        const void* base;
        uint64_t dims[4];
        uint64_t strides[3];
        uint32_t box[4];
        int dtype, rank, swizzle;
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        bool valid;
    };
    constexpr int kSlots = 64;
    thread_local Entry cache[kSlots] = {};
    Key k = {};
    k.base = base;
    k.dtype = (int)dtype;
    k.rank = rank;
    k.swizzle = (int)swizzle;
    for (int i = 0; i < rank; i++) {
        k.dims[i] = dims[i];
        k.box[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; i++) k.strides[i] = strides_bytes[i];
    uint64_t h = reinterpret_cast<uintptr_t>(base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.dims[0] * 31 + k.dims[1]) * 0xC2B2AE3D27D4EB4Full + k.box[0] * 131 + k.box[1] * 17 + k.box[2] +
         (uint64_t)k.swizzle * 7 + (uint64_t)k.dtype * 3 + k.dims[2] * 1315423911ull + k.dims[3] * 2654435761ull +
         k.box[3] * 977;
    Entry& e = cache[(h >> 32) % kSlots];
    if (e.valid && memcmp(&e.key, &k, sizeof(Key)) == 0) {
        *out = e.map;
        return true;
    }
    PFN_encodeTiled fn = get_encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdim[4];
    cuuint64_t gstr[3];
    cuuint32_t bx[4];
    cuuint32_t es[4] = {1, 1, 1, 1};
    for (int i = 0; i < rank; i++) {
        gdim[i] = dims[i];
        bx[i] = box[i];
    }
    for (int i = 0; i + 1 < rank; i++) gstr[i] = strides_bytes[i];
    const CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    e.key = k;
    e.map = *out;
    e.valid = true;
    return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace fb200
