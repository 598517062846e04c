// Epilogue of the 2:4-sparse GEMM kernels. The sparse operand is the MMA's A operand, so the
// accumulator is the transpose of the output: TMEM lane = weight row n (an output COLUMN),
// TMEM column = token m (an output ROW). After tcgen05.ld a thread holds 32 consecutive tokens
// of one output column, and the 32 lanes of a warp hold 32 consecutive columns - so a plain
// store per token writes 32 consecutive elements (64 or 128 contiguous bytes) per warp
// instruction: coalesced without any staging in shared memory.
#pragma once

#include "common.cuh"

namespace fb200 {

// v[j]: accumulator of token (m_first + j) for output column n. EPI 0: raw s32, 1: fp16 dequant.
// as_lane: act_scale[m_first + lane] (0 past the end), broadcast per token with a shuffle.
template <int EPI>
__device__ __forceinline__ void store_transposed_chunk(const uint32_t (&v)[32], void* __restrict__ out, int N_out,
                                                       int M, int n, int m_first, float as_lane, float ws, float bs,
                                                       bool has_bias) {
    const int valid = min(32, M - m_first);   // warp-uniform
    const bool col_ok = n < N_out;
    // interior chunks (the common case) take the unguarded path: no per-element branches
    const bool full = (valid == 32) && __all_sync(0xffffffffu, col_ok);
    if (EPI == 0) {
        int32_t* p = static_cast<int32_t*>(out) + (size_t)m_first * N_out + n;
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j++) __stcs(p + (size_t)j * N_out, static_cast<int32_t>(v[j]));
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                if (j < valid && col_ok) p[(size_t)j * N_out] = static_cast<int32_t>(v[j]);
            }
        }
    } else {
        __half* p = static_cast<__half*>(out) + (size_t)m_first * N_out + n;
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float as = __shfl_sync(0xffffffffu, as_lane, j);
                const float o = dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias);
                // streaming store: the output is not read again by this kernel and must not push
                // the activations out of L2
                __stcs(reinterpret_cast<unsigned short*>(p + (size_t)j * N_out),
                       __half_as_ushort(__float2half_rn(o)));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float as = __shfl_sync(0xffffffffu, as_lane, j);
                if (j < valid && col_ok) {
                    const float o = dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias);
                    p[(size_t)j * N_out] = __float2half_rn(o);
                }
            }
        }
    }
}


// Destinations of the FP16 result: up to 8 buffers with a common row pitch. With one entry
// this is the ordinary output; with several, entry d is typically GPU d's copy of the full
// (M, N) output, peer-mapped over NVLink, and `ptr[d]` already points at this rank's first
// column - the epilogue then performs the all-gather of a column-sharded layer as plain
// peer stores, tile by tile, while the tensor cores work on the next tile.
struct OutDst {
    void* ptr[8];
    long long ld;   // row pitch in elements
    int count;
    int vec;        // 1: every ptr is 16-byte aligned and ld % 8 == 0 -> 16-byte row-segment stores
};

// As store_transposed_chunk<1>, to every destination.
__device__ __forceinline__ void store_transposed_chunk_multi(const uint32_t (&v)[32], const OutDst& dst, int N_out,
                                                             int M, int n, int m_first, float as_lane, float ws,
                                                             float bs, bool has_bias) {
    const int valid = min(32, M - m_first);
    const bool col_ok = n < N_out;
    __half h[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
        const float as = __shfl_sync(0xffffffffu, as_lane, j);
        h[j] = __float2half_rn(dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias));
    }
    if (!col_ok) return;
    for (int d = 0; d < dst.count; d++) {
        __half* p = static_cast<__half*>(dst.ptr[d]) + (size_t)m_first * dst.ld + n;
#pragma unroll
        for (int j = 0; j < 32; j++) {
            if (j < valid) p[(size_t)j * dst.ld] = h[j];
        }
    }
}

// Multi-destination store with wide segments, for the four warps that together hold one
// 32-token x 128-column chunk (one warp per TMEM lane quarter). The chunk is transposed through
// `stage` (32 rows x 256 bytes) so that a half-warp then owns one whole 256-byte output row
// segment and writes it to every destination with 16-byte stores: peer writes over NVLink travel
// as 256-byte contiguous runs instead of 64-byte ones. Two 128-thread named barriers bracket
// the transpose; all four warps always reach them (ok = false: synchronise only).
__device__ __forceinline__ void store_chunk_multi_vec(bool ok, const uint32_t (&v)[32], const OutDst& dst,
                                                      uint8_t* stage, int bar_id, int q, int N_out, int M,
                                                      int n_base, int m_first, float as_lane, float ws, float bs,
                                                      bool has_bias) {
    const int lane = threadIdx.x & 31;
    if (ok) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float as = __shfl_sync(0xffffffffu, as_lane, j);
            const float o = dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias);
            *reinterpret_cast<__half*>(stage + j * 256 + (q * 32 + lane) * 2) = __float2half_rn(o);
        }
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (ok) {
        const int valid = min(32, M - m_first);
        const int col = n_base + (lane & 15) * 8;          // first of this lane's 8 columns
        const bool col_ok = col + 8 <= N_out;              // N_out % 8 == 0 on this path
        uint4 seg[4];
        int rows[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            rows[i] = q * 8 + 2 * i + (lane >> 4);
            seg[i] = *reinterpret_cast<const uint4*>(stage + rows[i] * 256 + (lane & 15) * 16);
        }
        for (int d = 0; d < dst.count; d++) {
            __half* base = static_cast<__half*>(dst.ptr[d]) + (size_t)m_first * dst.ld + col;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (rows[i] < valid && col_ok) *reinterpret_cast<uint4*>(base + (size_t)rows[i] * dst.ld) = seg[i];
            }
        }
    }
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
}

// Gated (SiLU(gate) * up) epilogue of the sparse kernels. A 128-row weight tile holds 64 gate
// rows (TMEM lanes 0-63) followed by the 64 up rows of the same output columns (lanes 64-127), so
// gate and up of one output sit in two different warps. Both warps dequantise their 32 tokens in
// fp32, then swap halves through `xbuf` (2 x 16 tokens x 32 lanes fp32, 4 KB): the gate warp
// receives u of tokens 0-15 and finishes those, the up warp receives g of tokens 16-31 and
// finishes these - each combines, rounds once to fp16 and stores 16 tokens. Two 64-thread named
// barriers bracket the swap; both warps always reach them (a warp whose wait failed passes
// ok = false and only synchronises).
__device__ __forceinline__ void gated_chunk(bool is_gate, bool ok, const uint32_t (&v)[32], float* xbuf, int bar_id,
                                            __half* __restrict__ out, int N_out, int M, int n, int m_first,
                                            float as_lane, float ws, float bs, bool has_bias) {
    const int lane = threadIdx.x & 31;
    float d[32];
    float* give = xbuf + (is_gate ? 512 : 0);   // gate hands over g[16..31], up hands over u[0..15]
    float* take = xbuf + (is_gate ? 0 : 512);
    if (ok) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float as = __shfl_sync(0xffffffffu, as_lane, j);
            d[j] = dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias);
        }
#pragma unroll
        for (int j = 0; j < 16; j++) give[j * 32 + lane] = is_gate ? d[16 + j] : d[j];
    }
    asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
    if (ok) {
        const int first = is_gate ? 0 : 16;          // the 16 tokens this warp finishes
        const int valid = min(32, M - m_first);
        const bool col_ok = n < N_out;
        __half* p = out + (size_t)(m_first + first) * N_out + n;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const float other = take[j * 32 + lane];
            const float h = is_gate ? silu_mul(d[j], other) : silu_mul(other, d[16 + j]);
            if (first + j < valid && col_ok) p[(size_t)j * N_out] = __float2half_rn(h);
        }
    }
    asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");
}

}  // namespace fb200
