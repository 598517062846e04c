// 2:4 magnitude prune + compress, and metadata packing, for sm_100a.
//
// Replaces forge::sparsity::prune_compress_24 (reference src/sparsity/prune_compress.cu:9-85)
// and forge::sparsity::pack_metadata (reference src/sparsity/pack_metadata.cu:8-44). Outputs are
// byte-identical to the reference: per group of 4 along K the two smallest magnitudes are
// dropped (scan order and strict '<' comparisons as in prune_compress.cu:39-50), the two kept
// values are stored in ascending position order, and the group's nibble is idx0 | idx1 << 2;
// pack_metadata puts nibble g of each run of 8 at bits [4g, 4g+4) of one uint32.
//
// Both are HBM-bound streaming kernels; the launchers use 16-byte accesses (8 groups, or 16
// nibbles, per thread) whenever the shape and pointers allow it.
#include "common.cuh"
#include "kernels.cuh"

namespace fb200 {

// Decides one group of four signed bytes packed in `w` (byte i = position i).
// Returns the nibble; `kept` receives the two surviving bytes (low byte = lower position).
//
// The reference scan (prune_compress.cu:39-50: start with positions 0/1 ordered by magnitude,
// then strict '<' replacements for positions 2 and 3) drops exactly the two smallest elements
// under the order (|value|, position) - checked exhaustively over all 129^4 magnitude tuples -
// so the two dropped positions are the two smallest of the keys (|value| << 2) | position, found
// with a five-comparator min/max network instead of a data-dependent scan.
__device__ __forceinline__ uint32_t prune_group(uint32_t w, uint32_t& kept) {
    const uint32_t a = __vabs4(w);   // per-byte |x|; |-128| = 128 (no saturation), as abs((int)x)
    const uint32_t k0 = (a & 0xFFu) << 2;
    const uint32_t k1 = ((a >> 6) & 0x3FCu) | 1u;
    const uint32_t k2 = ((a >> 14) & 0x3FCu) | 2u;
    const uint32_t k3 = ((a >> 22) & 0x3FCu) | 3u;
    const uint32_t lo01 = min(k0, k1), hi01 = max(k0, k1);
    const uint32_t lo23 = min(k2, k3), hi23 = max(k2, k3);
    const uint32_t d1 = min(lo01, lo23);                            // smallest key
    const uint32_t d2 = min(max(lo01, lo23), min(hi01, hi23));      // second smallest
    const uint32_t keep = ~((1u << (d1 & 3u)) | (1u << (d2 & 3u))) & 0xFu;   // exactly two bits set
    const int p0 = __ffs(keep) - 1;                // lower kept position
    const int p1 = 31 - __clz(keep);               // higher kept position
    kept = ((w >> (8 * p0)) & 0xFF) | (((w >> (8 * p1)) & 0xFF) << 8);
    return (uint32_t)(p0 | (p1 << 2));
}

// Two groups at once (wA, wB): the same decision with the keys of both groups in the two 16-bit
// lanes of a register, so that every min / max of the network serves two groups, and with the
// surviving bytes picked by one PRMT whose selector is computed (no variable shifts, no bit
// scans). The kernel is bound by the integer ALU pipe (92 % busy with prune_group), not by HBM.
// `comp` receives the compressed word of both groups (A in the low half), the return value holds
// the two nibbles in its 16-bit lanes.
__device__ __forceinline__ uint32_t prune_pair(uint32_t wA, uint32_t wB, uint32_t& comp) {
    const uint32_t aA = __vabs4(wA), aB = __vabs4(wB);
    // key_i = (|x_i| << 2) | i, lane 0: group A, lane 1: group B
    const uint32_t k0 = (__byte_perm(aA, aB, 0x4400) & 0x00FF00FFu) * 4u;
    const uint32_t k1 = (__byte_perm(aA, aB, 0x5511) & 0x00FF00FFu) * 4u + 0x00010001u;
    const uint32_t k2 = (__byte_perm(aA, aB, 0x6622) & 0x00FF00FFu) * 4u + 0x00020002u;
    const uint32_t k3 = (__byte_perm(aA, aB, 0x7733) & 0x00FF00FFu) * 4u + 0x00030003u;
    const uint32_t lo01 = __vminu2(k0, k1), hi01 = __vmaxu2(k0, k1);
    const uint32_t lo23 = __vminu2(k2, k3), hi23 = __vmaxu2(k2, k3);
    const uint32_t h1 = __vmaxu2(hi01, hi23);                                   // largest key
    const uint32_t h2 = __vimax3_u16x2(__vminu2(hi01, hi23), lo01, lo23);       // second largest
    const uint32_t pa = h1 & 0x00030003u, pb = h2 & 0x00030003u;                // the two kept positions
    const uint32_t p0 = __vminu2(pa, pb), p1 = __vmaxu2(pa, pb);
    // PRMT selector per lane: byte 0 <- position p0, byte 1 <- position p1, bytes 2, 3 <- zero
    const uint32_t sel = p1 * 16u + p0 + 0x44004400u;
    const uint32_t keptA = __byte_perm(wA, 0u, sel);
    const uint32_t keptB = __byte_perm(wB, 0u, sel >> 16);
    comp = __byte_perm(keptA, keptB, 0x5410);
    return p1 * 4u + p0;
}

}  // namespace fb200

// Public kernel declarations of the reference headers (include/forge/sparsity/prune_compress.cuh:16-21,
// include/forge/sparsity/pack_metadata.cuh:15-19): one thread per group / per output word.
namespace forge { namespace sparsity {

__global__ void prune_compress_kernel(const int8_t* __restrict__ weight, int8_t* __restrict__ compressed,
                                      uint8_t* __restrict__ metadata_raw, int N, int K) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int groups_per_row = K / 4;
    const long long total = (long long)N * groups_per_row;
    if (idx >= total) return;
    const long long row = idx / groups_per_row;
    const int group = (int)(idx - row * groups_per_row);
    const int8_t* p = weight + row * K + group * 4;
    const uint32_t w = (uint32_t)(uint8_t)p[0] | ((uint32_t)(uint8_t)p[1] << 8) | ((uint32_t)(uint8_t)p[2] << 16) |
                       ((uint32_t)(uint8_t)p[3] << 24);
    uint32_t kept;
    const uint32_t nib = fb200::prune_group(w, kept);
    int8_t* c = compressed + row * (K / 2) + group * 2;
    c[0] = (int8_t)(kept & 0xFF);
    c[1] = (int8_t)(kept >> 8);
    metadata_raw[idx] = (uint8_t)nib;
}

__global__ void pack_metadata_kernel(const uint8_t* __restrict__ meta_raw, uint32_t* __restrict__ meta_packed, int N,
                                     int K) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int groups_per_row = K / 4;
    const int chunks_per_row = K / 32;
    const long long total = (long long)N * chunks_per_row;
    if (idx >= total) return;
    const long long row = idx / chunks_per_row;
    const int chunk = (int)(idx - row * chunks_per_row);
    const uint8_t* p = meta_raw + row * groups_per_row + chunk * 8;
    uint32_t packed = 0;
#pragma unroll
    for (int g = 0; g < 8; g++) packed |= ((uint32_t)(p[g] & 0xF)) << (g * 4);
    meta_packed[idx] = packed;
}

}}  // namespace forge::sparsity

namespace fb200 {

namespace {

// 16 weight bytes (4 groups) per piece -> 8 compressed bytes + 4 nibble bytes; a thread takes four
// pieces 256 apart, so every load and store of a warp is one contiguous run (512 / 256 / 128 bytes)
// and four loads are in flight per thread. Valid when K % 4 == 0 (groups tile the flat array) and
// N*K % 16 == 0.
__global__ void __launch_bounds__(256)
prune_compress_vec_kernel(const uint4* __restrict__ weight, uint2* __restrict__ compressed,
                          uint32_t* __restrict__ metadata_raw, long long npieces) {
    const long long first = (long long)blockIdx.x * 1024 + threadIdx.x;
    uint4 w[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const long long p = first + u * 256;
        w[u] = (p < npieces) ? __ldcs(weight + p) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const long long p = first + u * 256;
        if (p >= npieces) break;
        uint32_t comp[2];
        const uint32_t nib01 = prune_pair(w[u].x, w[u].y, comp[0]);
        const uint32_t nib23 = prune_pair(w[u].z, w[u].w, comp[1]);
        __stcs(compressed + p, make_uint2(comp[0], comp[1]));
        __stcs(metadata_raw + p, __byte_perm(nib01, nib23, 0x6420));   // one nibble byte per group
    }
}

// 16 nibble bytes per piece -> two packed words; two pieces 256 apart per thread. Valid when
// K % 32 == 0 and N*K/4 % 16 == 0.
__global__ void __launch_bounds__(256)
pack_metadata_vec_kernel(const uint4* __restrict__ meta_raw, uint2* __restrict__ meta_packed, long long npieces) {
    const long long first = (long long)blockIdx.x * 512 + threadIdx.x;
    uint4 r[2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const long long p = first + u * 256;
        r[u] = (p < npieces) ? __ldcs(meta_raw + p) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
        const long long p = first + u * 256;
        if (p >= npieces) break;
        const uint32_t w[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
        uint32_t out[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            // four nibbles, one per byte -> neighbours merged into bytes 0 and 2 -> one PRMT gathers
            // those bytes of both words: eight nibbles in order
            const uint32_t xa = w[2 * h] & 0x0F0F0F0Fu, xb = w[2 * h + 1] & 0x0F0F0F0Fu;
            out[h] = __byte_perm(xa | (xa >> 4), xb | (xb >> 4), 0x6420);
        }
        __stcs(meta_packed + p, make_uint2(out[0], out[1]));
    }
}

// One pass from a floating-point weight to everything a W8A8 layer stores: per-output-channel
// symmetric quantisation (scale = absmax / 127 floored at 1e-8, round half to even, clamp +-127,
// scale kept as fp16 - the recipe of the reference's Python modules,
// python/forge/nn/linear.py:167-173,234-249, with IEEE divides so the values equal torch's), then
// 2:4 prune + compress + metadata pack of the int8 row. One block per weight row; a thread turns
// 32 consecutive weights (8 groups) into 16 compressed bytes and one packed metadata word.
__device__ __forceinline__ float load_w(const float* p) { return __ldg(p); }
__device__ __forceinline__ float load_w(const __half* p) { return __half2float(__ldg(p)); }

template <typename T>
__global__ void __launch_bounds__(256)
prepare_weight_kernel(const T* __restrict__ w, int8_t* __restrict__ w_int8, int8_t* __restrict__ W_comp,
                      uint32_t* __restrict__ w_meta, __half* __restrict__ w_scale, int K) {
    const int row = blockIdx.x;
    const T* wr = w + (size_t)row * K;
    float amax = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(load_w(wr + k)));
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = part[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, part[i]);
    const float scale = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
    if (threadIdx.x == 0) w_scale[row] = __float2half_rn(scale);
    for (int c = threadIdx.x; c < K / 32; c += blockDim.x) {     // c: run of 32 weights
        uint32_t q[8];
#pragma unroll
        for (int g = 0; g < 8; g++) {
            uint32_t word = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float v = rintf(__fdiv_rn(load_w(wr + c * 32 + g * 4 + i), scale));
                const int qi = (int)fminf(fmaxf(v, -127.f), 127.f);
                word |= ((uint32_t)qi & 0xFFu) << (8 * i);
            }
            q[g] = word;
        }
        if (w_int8 != nullptr) {
            uint4* d = reinterpret_cast<uint4*>(w_int8 + (size_t)row * K + c * 32);
            d[0] = make_uint4(q[0], q[1], q[2], q[3]);
            d[1] = make_uint4(q[4], q[5], q[6], q[7]);
        }
        if (W_comp != nullptr) {
            uint32_t comp[4];
            uint32_t meta = 0;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const uint32_t nib2 = prune_pair(q[2 * g], q[2 * g + 1], comp[g]);
                meta |= ((nib2 & 0xFu) | ((nib2 >> 12) & 0xF0u)) << (8 * g);   // nibbles 2g and 2g+1
            }
            *reinterpret_cast<uint4*>(W_comp + (size_t)row * (K / 2) + c * 16) =
                make_uint4(comp[0], comp[1], comp[2], comp[3]);
            w_meta[(size_t)row * (K / 32) + c] = meta;
        }
    }
}

}  // namespace

int prune_compress_24(const int8_t* weight, int8_t* compressed, uint8_t* metadata_raw, int N, int K,
                      cudaStream_t stream) {
    if (N <= 0 || K <= 0) return kOk;   // reference: silent no-op (prune_compress.cu:79)
    if (weight == nullptr || compressed == nullptr || metadata_raw == nullptr) return kBadPointer;
    const long long bytes = (long long)N * K;
    const bool vec_ok = (K % 4 == 0) && (bytes % 16 == 0) && aligned16(weight) &&
                        (reinterpret_cast<uintptr_t>(compressed) % 8 == 0) &&
                        (reinterpret_cast<uintptr_t>(metadata_raw) % 4 == 0);
    if (vec_ok) {
        const long long n = bytes / 16;
        prune_compress_vec_kernel<<<(unsigned)((n + 1023) / 1024), 256, 0, stream>>>(
            reinterpret_cast<const uint4*>(weight), reinterpret_cast<uint2*>(compressed),
            reinterpret_cast<uint32_t*>(metadata_raw), n);
    } else {
        const long long groups = (long long)N * (K / 4);
        if (groups == 0) return kOk;
        forge::sparsity::prune_compress_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, stream>>>(
            weight, compressed, metadata_raw, N, K);
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int pack_metadata(const uint8_t* meta_raw, uint32_t* meta_packed, int N, int K, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return kOk;   // reference: silent no-op (pack_metadata.cu:38)
    if (meta_raw == nullptr || meta_packed == nullptr) return kBadPointer;
    const long long nibbles = (long long)N * (K / 4);
    const bool vec_ok = (K % 32 == 0) && (nibbles % 16 == 0) && aligned16(meta_raw) &&
                        (reinterpret_cast<uintptr_t>(meta_packed) % 8 == 0);
    if (vec_ok) {
        const long long n = nibbles / 16;
        pack_metadata_vec_kernel<<<(unsigned)((n + 511) / 512), 256, 0, stream>>>(
            reinterpret_cast<const uint4*>(meta_raw), reinterpret_cast<uint2*>(meta_packed), n);
    } else {
        const long long words = (long long)N * (K / 32);
        if (words == 0) return kOk;
        forge::sparsity::pack_metadata_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>(meta_raw,
                                                                                                  meta_packed, N, K);
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int prepare_weight(const void* w, int w_is_half, int8_t* w_int8, int8_t* W_comp, uint32_t* w_meta, __half* w_scale,
                   int N, int K, cudaStream_t stream) {
    if (N <= 0 || K <= 0) return kOk;
    if (w == nullptr || w_scale == nullptr || (w_int8 == nullptr && W_comp == nullptr)) return kBadPointer;
    if (W_comp != nullptr && w_meta == nullptr) return kBadPointer;
    if (K % 32 != 0 || (w_int8 != nullptr && !aligned16(w_int8)) || (W_comp != nullptr && !aligned16(W_comp)))
        return kBadShape;
    if (w_is_half)
        prepare_weight_kernel<__half><<<N, 256, 0, stream>>>(static_cast<const __half*>(w), w_int8, W_comp, w_meta,
                                                            w_scale, K);
    else
        prepare_weight_kernel<float><<<N, 256, 0, stream>>>(static_cast<const float*>(w), w_int8, W_comp, w_meta,
                                                           w_scale, K);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace fb200
