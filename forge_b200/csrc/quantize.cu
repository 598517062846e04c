// Per-token FP16 -> INT8 quantizer and INT32 -> FP16 dequant + bias for sm_100a.
//
// Replaces forge::quant::fused_quantize_activation (reference src/quant/quantize.cu:8-191) and
// forge::quant::fused_dequantize_bias (reference src/quant/dequantize.cu:8-45).
//
// Arithmetic is the reference's, operation for operation (its build uses -use_fast_math):
//   amax  = max_k |f32(x_k)|
//   scale = div.approx.ftz(max.ftz(amax, 1e-8), 127)      inv = rcp.approx.ftz(scale)
//   q     = clamp(cvt.rni.ftz.s32(mul.ftz(f32(x_k), inv)), -128, 127)
//   deq   = fp16_rn(fma.rn.ftz(mul.ftz(act_scale, f32(acc)), f32(w_scale), f32(bias)))
//
// Both kernels are HBM-bound. The quantizer keeps a whole row in registers (one read of the
// input) with up to eight 16-byte loads in flight per thread; rows are spread over 1..32 warps
// so that K up to 65536 takes the single-read path.
#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

// --------------------------------------------------------------------------------------------
// Kernels that are public declarations in the reference headers keep their name, namespace,
// parameter list and launch contract (reference include/forge/quant/quantize.cuh:17-21,
// include/forge/quant/dequantize.cuh:17-23): one block per row, any block size that is a
// multiple of 32.
namespace forge { namespace quant {

__global__ void fused_quantize_activation_kernel(const __half* __restrict__ input, int8_t* __restrict__ output,
                                                 float* __restrict__ scales, int K) {
    using namespace fb200;
    const int row = blockIdx.x;
    const __half* in_row = input + (size_t)row * K;
    int8_t* out_row = output + (size_t)row * K;

    float tmax = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) tmax = max_ftz(tmax, abs_ftz(__half2float(in_row[k])));
    for (int off = 16; off > 0; off >>= 1) tmax = max_ftz(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));

    __shared__ float warp_max[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_max[warp] = tmax;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float v = (lane < nwarps) ? warp_max[lane] : 0.0f;
    for (int off = 16; off > 0; off >>= 1) v = max_ftz(v, __shfl_xor_sync(0xffffffffu, v, off));

    float scale, inv;
    quant_scale(v, scale, inv);
    if (threadIdx.x == 0) scales[row] = scale;
    for (int k = threadIdx.x; k < K; k += blockDim.x)
        out_row[k] = static_cast<int8_t>(quant_value(__half2float(in_row[k]), inv));
}

__global__ void fused_dequantize_bias_kernel(const int32_t* __restrict__ input, const float* __restrict__ act_scale,
                                             const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                                             __half* __restrict__ output, int N) {
    using namespace fb200;
    const int row = blockIdx.x;
    const int32_t* in_row = input + (size_t)row * N;
    __half* out_row = output + (size_t)row * N;
    const float a = act_scale[row];
    for (int col = threadIdx.x; col < N; col += blockDim.x) {
        const float t = mul_ftz(static_cast<float>(in_row[col]), a);
        const float w = __half2float(w_scale[col]);
        const float o = (bias != nullptr) ? fma_ftz(t, w, __half2float(bias[col])) : mul_ftz(t, w);
        out_row[col] = __float2half_rn(o);
    }
}

}}  // namespace forge::quant

namespace fb200 {

namespace {

// One row per TPR threads, the row in registers as VPT 16-byte vectors per thread.
// BLOCK threads per block, BLOCK / TPR rows per block.
template <int VPT, int TPR, int BLOCK, bool STREAM>
__global__ void __launch_bounds__(BLOCK)
quantize_rows_kernel(const __half* __restrict__ input, int8_t* __restrict__ output, float* __restrict__ scales,
                     int M, int K) {
    constexpr int ROWS = BLOCK / TPR;
    constexpr int WPR = TPR / 32;   // warps per row
    // a GEMM launched behind this kernel as a programmatic dependent may start its set-up now
    ptx::griddep_launch_dependents();
    const int sub = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const long long row = (long long)blockIdx.x * ROWS + sub;
    const bool live = row < M;
    const int nvec = K >> 3;
    const uint4* in_row = reinterpret_cast<const uint4*>(input + (size_t)(live ? row : 0) * K);
    uint2* out_row = reinterpret_cast<uint2*>(output + (size_t)(live ? row : 0) * K);

    uint4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int idx = t + i * TPR;
        if (live && idx < nvec) v[i] = STREAM ? __ldcs(in_row + idx) : __ldg(in_row + idx);
        else v[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    // |x| maximum in packed half precision: exact (no rounding in abs / max, NaNs are skipped like
    // max.ftz.f32 skips them, fp16 subnormals are normal fp32 numbers so nothing is flushed)
    __half2 hmax = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const __half2* h = reinterpret_cast<const __half2*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; j++) hmax = __hmax2(hmax, __habs2(h[j]));
    }
    float tmax = max_ftz(__low2float(hmax), __high2float(hmax));
    for (int off = 16; off > 0; off >>= 1) tmax = max_ftz(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
    if (WPR > 1) {
        __shared__ float part[BLOCK / 32];
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) part[warp] = tmax;
        __syncthreads();
        const int first = sub * WPR;
        float r = part[first];
#pragma unroll
        for (int w = 1; w < WPR; w++) r = max_ftz(r, part[first + w]);
        tmax = r;
    }
    float scale, inv;
    quant_scale(tmax, scale, inv);
    if (live && t == 0) scales[row] = scale;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int idx = t + i * TPR;
        if (live && idx < nvec) {
            const __half2* h = reinterpret_cast<const __half2*>(&v[i]);
            int q[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                q[2 * j] = cvt_rni_ftz(mul_ftz(f.x, inv));          // the clamp to [-128, 127] is the pack's
                q[2 * j + 1] = cvt_rni_ftz(mul_ftz(f.y, inv));
            }
            out_row[idx] = make_uint2(pack4_sat(q[0], q[1], q[2], q[3]), pack4_sat(q[4], q[5], q[6], q[7]));
        }
    }
}

template <int VPT, int TPR, int BLOCK>
void launch_rows(const __half* in, int8_t* out, float* scales, int M, int K, bool stream_loads, cudaStream_t s) {
    constexpr int ROWS = BLOCK / TPR;
    const unsigned grid = (unsigned)(((long long)M + ROWS - 1) / ROWS);
    if (stream_loads) quantize_rows_kernel<VPT, TPR, BLOCK, true><<<grid, BLOCK, 0, s>>>(in, out, scales, M, K);
    else quantize_rows_kernel<VPT, TPR, BLOCK, false><<<grid, BLOCK, 0, s>>>(in, out, scales, M, K);
}

template <int TPR, int BLOCK>
void launch_rows_vpt(int vpt, const __half* in, int8_t* out, float* scales, int M, int K, bool st, cudaStream_t s) {
    if (vpt <= 1) launch_rows<1, TPR, BLOCK>(in, out, scales, M, K, st, s);
    else if (vpt <= 2) launch_rows<2, TPR, BLOCK>(in, out, scales, M, K, st, s);
    else if (vpt <= 4) launch_rows<4, TPR, BLOCK>(in, out, scales, M, K, st, s);
    else if (vpt <= 6) launch_rows<6, TPR, BLOCK>(in, out, scales, M, K, st, s);
    else launch_rows<8, TPR, BLOCK>(in, out, scales, M, K, st, s);
}

// 8 outputs per thread: 32 bytes of s32 in, 16 bytes of fp16 out.
template <bool HAS_BIAS>
__global__ void __launch_bounds__(256)
dequant_vec_kernel(const int32_t* __restrict__ input, const float* __restrict__ act_scale,
                   const __half* __restrict__ w_scale, const __half* __restrict__ bias, __half* __restrict__ output,
                   long long total_vec, int nvec_row) {
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= total_vec) return;
    const long long row = id / nvec_row;
    const int cv = (int)(id - row * nvec_row);
    const int4* in = reinterpret_cast<const int4*>(input) + id * 2;
    const int4 a0 = __ldcs(in), a1 = __ldcs(in + 1);
    const float as = act_scale[row];
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w_scale) + cv);
    uint4 bv = make_uint4(0u, 0u, 0u, 0u);
    if (HAS_BIAS) bv = __ldg(reinterpret_cast<const uint4*>(bias) + cv);
    const int acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
    const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 w = __half22float2(w2[j]);
        const float2 b = __half22float2(b2[j]);
        const float t0 = mul_ftz(static_cast<float>(acc[2 * j]), as);
        const float t1 = mul_ftz(static_cast<float>(acc[2 * j + 1]), as);
        const float r0 = HAS_BIAS ? fma_ftz(t0, w.x, b.x) : mul_ftz(t0, w.x);
        const float r1 = HAS_BIAS ? fma_ftz(t1, w.y, b.y) : mul_ftz(t1, w.y);
        o[j] = pack_half2(r0, r1);
    }
    reinterpret_cast<uint4*>(output)[id] = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace

int quantize_activation(const __half* input, int8_t* output, float* scales, int M, int K, cudaStream_t stream) {
    if (M <= 0 || K <= 0) return kOk;   // reference: silent no-op (quantize.cu:170)
    if (input == nullptr || output == nullptr || scales == nullptr) return kBadPointer;
    const bool vec_ok = (K % 8 == 0) && (K <= 65536) && aligned16(input) &&
                        (reinterpret_cast<uintptr_t>(output) % 8 == 0);
    if (!vec_ok) {
        int threads = std::min(256, ((K + 31) / 32) * 32);
        if (threads < 32) threads = 32;
        forge::quant::fused_quantize_activation_kernel<<<M, threads, 0, stream>>>(input, output, scales, K);
        return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
    }
    const int nvec = K / 8;
    // evict-first loads once the input cannot stay in L2 anyway
    const bool st = (size_t)M * K * sizeof(__half) > l2_bytes();
    // threads per row: the fewest (a power of two >= 32) that hold the row in <= 8 vectors each
    int tpr = 32;
    while (tpr < 1024 && nvec > tpr * 8) tpr <<= 1;
    const int vpt = (nvec + tpr - 1) / tpr;
    switch (tpr) {
    case 32:   launch_rows_vpt<32, 256>(vpt, input, output, scales, M, K, st, stream); break;
    case 64:   launch_rows_vpt<64, 256>(vpt, input, output, scales, M, K, st, stream); break;
    case 128:  launch_rows_vpt<128, 256>(vpt, input, output, scales, M, K, st, stream); break;
    case 256:  launch_rows_vpt<256, 256>(vpt, input, output, scales, M, K, st, stream); break;
    case 512:  launch_rows_vpt<512, 512>(vpt, input, output, scales, M, K, st, stream); break;
    default:   launch_rows_vpt<1024, 1024>(vpt, input, output, scales, M, K, st, stream); break;
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int dequantize_bias(const int32_t* input, const float* act_scale, const __half* w_scale, const __half* bias,
                    __half* output, int M, int N, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return kOk;   // reference: silent no-op (dequantize.cu:40)
    if (input == nullptr || act_scale == nullptr || w_scale == nullptr || output == nullptr) return kBadPointer;
    const bool vec_ok = (N % 8 == 0) && aligned16(input) && aligned16(output) && aligned16(w_scale) &&
                        (bias == nullptr || aligned16(bias));
    if (!vec_ok) {
        int threads = std::min(256, ((N + 31) / 32) * 32);
        if (threads < 32) threads = 32;
        forge::quant::fused_dequantize_bias_kernel<<<M, threads, 0, stream>>>(input, act_scale, w_scale, bias,
                                                                              output, N);
        return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
    }
    const int nvec_row = N / 8;
    const long long total = (long long)M * nvec_row;
    const unsigned grid = (unsigned)((total + 255) / 256);
    if (bias != nullptr)
        dequant_vec_kernel<true><<<grid, 256, 0, stream>>>(input, act_scale, w_scale, bias, output, total, nvec_row);
    else
        dequant_vec_kernel<false><<<grid, 256, 0, stream>>>(input, act_scale, w_scale, bias, output, total,
                                                            nvec_row);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace fb200
