// 2:4 structured-sparse INT8 GEMM for sm_100a:
//   out[m, n] = sum_k W24[n, k] * x[m, k]      (W24 = the 2:4-pruned weight)
// from the compressed weight W_comp (N_out, K/2), the packed metadata w_meta (N_out, K/32)
// and int8 activations x (M, K).
//
// Replaces forge::gemm::sparse_int8_gemm (reference src/gemm/int8_sparse.cu:139-720, 960-1003,
// a warp-synchronous mma.sp kernel) and adds an INT32-output form.
//
// Design: persistent CTAs walking tiles of 128 weight rows x BT tokens. The sparse operand
// must be the A operand of tcgen05.mma.sp, so weight rows sit on the TMEM lanes and the
// accumulator is the transpose of the output tile.
//   warp 0   : TMA producer. Per 256-deep K slab: compressed weights (128 rows x 128 bytes,
//              128B swizzle), activations (two 128-byte-wide swizzled atoms of BT rows) and the
//              metadata slab (128 rows x 32 bytes, fetched as two 16-byte columns so that it
//              lands as unswizzled 8-row x 16-byte core matrices).
//   warp 1   : MMA issuer: four tcgen05.mma.sp kind::i8 (M=128, N=BT, K=64) per slab.
//   last warp: metadata copies. One tcgen05.cp per slab moves the metadata into TMEM as soon as it
//              has landed (its own barrier) - the public w_meta layout (row-major uint32, nibble g
//              at bits [4g,4g+4)) is already what the tensor core expects per lane: 2 columns per
//              64-deep step. Issued from the MMA thread the copies sit in the MMA stream and cost
//              about a fifth of a compute-bound kernel's time.
//   warps 2-9: epilogue. tcgen05.ld (lane = weight row, registers = tokens), dequantise, and
//              store straight to global memory: for one token the 32 lanes of a warp hold 32
//              consecutive output columns, so every warp store is one contiguous segment.
#include "common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"
#include "gemm_sparse.cuh"
#include "gemm_pair.cuh"
#include "sparse_epilogue.cuh"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int BW = 128;          // weight rows per tile (UMMA M)
constexpr int SLAB_K = 256;      // logical K per pipeline stage
constexpr int kEpiWarps = 8;             // two warps per TMEM lane quarter, alternating 32-token chunks
constexpr int kThreads = 96 + 32 * kEpiWarps;   // TMA, MMA, epilogue warps, metadata-copy warp
constexpr int kMetaBytes = BW * 32;        // 128 rows x 32 bytes per slab

constexpr int kXbufBytes = 4 * 32 * 32 * (int)sizeof(float);   // gated epilogue: 4 warp pairs x 4 KB

template <int BT, int EPI = 0>
struct SparseCfg {
    static constexpr int kABytes = BW * 128;
    static constexpr int kBAtomBytes = BT * 128;
    static constexpr int kStageBytes = kABytes + 2 * kBAtomBytes + kMetaBytes;
    static constexpr int kAccBufs = (2 * BT + 32 <= 512) ? 2 : 1;
    static constexpr int kBarBytes = 320;   // up to 8 stages x 4 barriers + 4 accumulator barriers + 2 words
    static constexpr int kFixed = kBarBytes + (EPI == 2 ? kXbufBytes : 0);
    static constexpr int kStagesMax = (232448 - kFixed) / kStageBytes;
    static constexpr int kStages = kStagesMax > 8 ? 8 : kStagesMax;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFixed;
    static constexpr int kMetaCols = 8 * kStages;             // 8 TMEM columns of metadata per stage
    static constexpr int kAccCols = kAccBufs * BT;
    static constexpr int kTmemNeed = kAccCols + kMetaCols;
    static constexpr int kTmemCols = kTmemNeed <= 64 ? 64 : kTmemNeed <= 128 ? 128 : kTmemNeed <= 256 ? 256 : 512;
    static_assert(kStages >= 2, "pipeline needs at least two stages");
    static_assert(kTmemNeed <= 512, "TMEM capacity");
    static_assert(kStageBytes % 1024 == 0, "stage buffers must keep 1024-byte alignment");
};

struct TileCoord {
    int w_blk, t_blk;
};

// Bands of 8 weight-row blocks, token-block major inside a band: concurrently running tiles
// share weight slabs and activation slabs in L2.
__device__ __forceinline__ TileCoord tile_coord(int t, int w_blocks, int t_blocks) {
    constexpr int kGroup = 8;
    const int band_tiles = kGroup * t_blocks;
    const int band = t / band_tiles;
    const int first_w = band * kGroup;
    const int rows = min(kGroup, w_blocks - first_w);
    const int r = t - band * band_tiles;
    TileCoord c;
    c.w_blk = first_w + r % rows;
    c.t_blk = r / rows;
    return c;
}

// EPI: 0 = raw s32 output, 1 = fp16 dequant (+ optional bias),
//      2 = gated: the 128-row weight tile is 64 rows of a gate weight (tm_w / tm_meta) followed by
//          the same 64 rows of an up weight (tm_w2 / tm_meta2); output = fp16(SiLU(g) * u), 64
//          output columns per tile.
template <int BT, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
sparse_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ CUtensorMap tm_meta, const __grid_constant__ CUtensorMap tm_w2,
                   const __grid_constant__ CUtensorMap tm_meta2, void* __restrict__ out, const OutDst multi,
                   const float* __restrict__ act_scale, const __half* __restrict__ w_scale,
                   const __half* __restrict__ bias, const __half* __restrict__ w_scale2,
                   const __half* __restrict__ bias2, int M, int N_out, int K, int* __restrict__ status) {
    using Cfg = SparseCfg<BT, EPI>;
    constexpr int TILE_W = (EPI == 2) ? BW / 2 : BW;   // output columns per tile
    extern __shared__ __align__(1024) uint8_t smem[];

    uint8_t* smem_stage = smem;
    float* smem_xbuf = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes +
                                                 (EPI == 2 ? kXbufBytes : 0));
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + Cfg::kStages;
    uint64_t* tmem_full = bars + 2 * Cfg::kStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint64_t* meta_full = tmem_empty + 2;                 // the stage's metadata slab has landed
    uint64_t* meta_ready = meta_full + Cfg::kStages;      // ... is in tensor memory and the operands have landed
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(meta_ready + Cfg::kStages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 200);
        return;
    }

    const int w_blocks = (N_out + TILE_W - 1) / TILE_W;
    const int t_blocks = (M + BT - 1) / BT;
    const int num_tiles = w_blocks * t_blocks;
    const int num_kb = (K + SLAB_K - 1) / SLAB_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&meta_full[s], 1);
            mbar_init(&meta_ready[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp_id == 0 && lane == 0) {
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_x);
        prefetch_tensormap(&tm_meta);
    }
    if (warp_id == 1) {
        tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_meta = tmem_base + Cfg::kAccCols;

    if (warp_id == 0) {
        // ------------------------------------------------------------------ TMA producer
        // Iterations are numbered over this CTA's (tile, K slab) sequence. A stage's loads come in two
        // parts - weights + metadata, then the two activation atoms - because the weights are static
        // while the activations may be the output of a quantizer this kernel was launched behind
        // (launch_behind_quantizer): the first ring fill requests all its weight slabs at once, then
        // waits for that kernel (griddepcontrol.wait; immediate in an ordinary launch), then requests
        // the activations. With few tokens the call is a pass over the weights, which so starts
        // under the quantizer's tail.
        if (lane == 0) {
            const int my_tiles = (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
            const int total = my_tiles * num_kb;
            auto issue = [&](int it, bool weights, bool acts) {
                const int stage = it % Cfg::kStages;
                const int t = blockIdx.x + (it / num_kb) * gridDim.x;
                const int kb = it % num_kb;
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks);
                uint8_t* sa = smem_stage + stage * Cfg::kStageBytes;
                uint8_t* sb = sa + Cfg::kABytes;
                uint8_t* sm = sb + 2 * Cfg::kBAtomBytes;
                if (weights) {
                    mbar_expect_tx(&meta_full[stage], kMetaBytes);
                    mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes - kMetaBytes);
                    if (EPI == 2) {
                        // 64 gate rows then 64 up rows; metadata per 16-byte column: [gate 64 rows][up 64 rows]
                        const int w_row = tc.w_blk * TILE_W;
#pragma unroll
                        for (int c = 0; c < 2; c++) {
                            tma_load_3d(sm + c * 2048, &tm_meta, &meta_full[stage], 0, w_row, kb * 2 + c);
                            tma_load_3d(sm + c * 2048 + 1024, &tm_meta2, &meta_full[stage], 0, w_row, kb * 2 + c);
                        }
                        tma_load_2d(sa, &tm_w, &full_bar[stage], kb * (SLAB_K / 2), w_row);
                        tma_load_2d(sa + Cfg::kABytes / 2, &tm_w2, &full_bar[stage], kb * (SLAB_K / 2), w_row);
                    } else {
                        tma_load_3d(sm, &tm_meta, &meta_full[stage], 0, tc.w_blk * BW, kb * 2);
                        tma_load_2d(sa, &tm_w, &full_bar[stage], kb * (SLAB_K / 2), tc.w_blk * BW);
                    }
                }
                if (acts) {
                    tma_load_2d(sb, &tm_x, &full_bar[stage], kb * SLAB_K, tc.t_blk * BT);
                    tma_load_2d(sb + Cfg::kBAtomBytes, &tm_x, &full_bar[stage], kb * SLAB_K + 128, tc.t_blk * BT);
                }
            };
            const int pre = min(Cfg::kStages, total);   // the ring starts empty: no wait for these stages
            for (int it = 0; it < pre; it++) issue(it, true, false);
            griddep_wait();
            for (int it = 0; it < pre; it++) issue(it, false, true);
            for (int it = pre; it < total; it++) {
                const int stage = it % Cfg::kStages;
                const uint32_t phase = (uint32_t)(it / Cfg::kStages) & 1u;
                if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
                    atomicExch(status, 201);
                    break;
                }
                issue(it, true, true);
            }
        }
    } else if (warp_id == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(BW, BT, true);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local++) {
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag)) {
                    atomicExch(status, 202);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * BT;
                for (int kb = 0; kb < num_kb; kb++) {
                    // meta_ready[s]: the slab's metadata is in tensor memory and its operands have landed
                    if (!mbar_wait(&meta_ready[stage], phase, abort_flag)) {
                        atomicExch(status, 203);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_stage + stage * Cfg::kStageBytes);
                    const uint32_t sb = sa + Cfg::kABytes;
                    const uint32_t te = tmem_meta + 8 * stage;
                    const uint64_t desc_a = make_desc_sw128(sa);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // step j: 32 compressed bytes of A, 64 bytes of B (atom j/2, half j%2), 2 metadata columns
                        const uint64_t desc_b = make_desc_sw128(sb + (j >> 1) * Cfg::kBAtomBytes) + 4 * (j & 1);
                        umma_i8_sp(tmem_acc, desc_a + 2 * j, desc_b, te + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[stage]);
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) tc_commit(&tmem_full[buf]);
            }
        }
    } else if (warp_id == kThreads / 32 - 1) {
        // ------------------------------------------------------------------ metadata copies
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&meta_full[stage], phase, abort_flag)) {
                        atomicExch(status, 205);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sm = smem_u32(smem_stage + stage * Cfg::kStageBytes) + Cfg::kABytes +
                                        2 * Cfg::kBAtomBytes;
                    // two 16-byte columns of 128 rows -> 8 TMEM columns
                    tmem_cp_128x256b(tmem_meta + 8 * stage, make_desc_noswizzle(sm, 2048, 128));
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        atomicExch(status, 206);
                        ok = false;
                        break;
                    }
                    tc_commit(&meta_ready[stage]);
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp_id & 3;                 // TMEM lane quarter this warp may read
        const int chunk0 = (warp_id - 2) >> 2;     // 0 or 1: which alternate chunks this warp takes
        const bool has_bias = (bias != nullptr);
        int local = 0;
        griddep_wait();   // the token scales may be the output of the quantizer this kernel was launched behind
        if (EPI == 2) {
            // lanes 0-63 hold gate rows, lanes 64-127 the up rows of the same output columns
            const bool is_gate = q < 2;
            const int pair = (q & 1) + 2 * chunk0;
            float* xbuf = smem_xbuf + pair * 1024;
            const __half* my_scale = is_gate ? w_scale : w_scale2;
            const __half* my_bias = is_gate ? bias : bias2;
            bool ok = true;   // after a failed wait: keep meeting the partner warp at the barriers
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n = tc.w_blk * TILE_W + (q & 1) * 32 + lane;
                const int m0 = tc.t_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (n < N_out) {
                    ws = __half2float(my_scale[n]);
                    if (my_bias != nullptr) bs = __half2float(my_bias[n]);
                }
                if (ok) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], acc_phase, abort_flag));
                    if (!ok) atomicExch(status, 204);
                }
                if (ok) tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kEpiWarps / 4) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M) break;
                    uint32_t v[32];
                    float as_lane = 0.f;
                    if (ok) {
                        tmem_ld_32x32b_x32(taddr + c * 32, v);
                        if (m_first + lane < M) as_lane = act_scale[m_first + lane];
                        tmem_ld_wait();
                    }
                    gated_chunk(is_gate, ok, v, xbuf, 4 + pair, static_cast<__half*>(out), N_out, M, n, m_first,
                                as_lane, ws, bs, my_bias != nullptr);
                }
                if (ok) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                }
            }
        } else {
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n = tc.w_blk * BW + q * 32 + lane;   // this thread's weight row = output column
                const int m0 = tc.t_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (EPI == 1 && n < N_out) {
                    ws = __half2float(w_scale[n]);
                    if (has_bias) bs = __half2float(bias[n]);
                }
                // warp-uniform outcome: the TMEM loads below are .sync.aligned
                if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], acc_phase, abort_flag))) {
                    atomicExch(status, 204);
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kEpiWarps / 4) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M) break;   // warp-uniform: the rest of the tile is past the last token
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    float as_lane = 0.f;
                    if (EPI == 1 && m_first + lane < M) as_lane = act_scale[m_first + lane];
                    tmem_ld_wait();
                    if (EPI == 1 && multi.count > 0)
                        store_transposed_chunk_multi(v, multi, N_out, M, n, m_first, as_lane, ws, bs, has_bias);
                    else
                        store_transposed_chunk<EPI>(v, out, N_out, M, n, m_first, as_lane, ws, bs, has_bias);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp_id == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// Plain-CUDA kernel for shapes the TMA path cannot describe (K % 128 != 0, misaligned
// pointers or row pitches). One thread per output element, decoding the nibbles directly.
template <int EPI>
__global__ void sparse_gemm_ragged_kernel(const int8_t* __restrict__ W_comp, const int8_t* __restrict__ x,
                                          const uint32_t* __restrict__ w_meta, const float* __restrict__ act_scale,
                                          const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                                          void* __restrict__ out, int M, int K, int N_out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N_out) return;
    const int m = (int)(idx / N_out), n = (int)(idx % N_out);
    const int8_t* wc = W_comp + (size_t)n * (K / 2);
    const uint32_t* me = w_meta + (size_t)n * (K / 32);
    const int8_t* xr = x + (size_t)m * K;
    int acc = 0;
    for (int g = 0; g < K / 4; g++) {
        const uint32_t nib = (me[g >> 3] >> (4 * (g & 7))) & 0xF;
        acc += (int)wc[2 * g] * (int)xr[4 * g + (nib & 3)] + (int)wc[2 * g + 1] * (int)xr[4 * g + (nib >> 2)];
    }
    if (EPI == 0) {
        reinterpret_cast<int32_t*>(out)[idx] = acc;
    } else {
        const float s = mul_ftz(act_scale[m], __half2float(w_scale[n]));
        const float o = dequant_gemm(acc, s, bias ? __half2float(bias[n]) : 0.f, bias != nullptr);
        reinterpret_cast<__half*>(out)[idx] = __float2half_rn(o);
    }
}

template <int BT, int EPI>
int launch_sparse(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                  const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out,
                  cudaStream_t stream, const int8_t* W_comp2 = nullptr, const uint32_t* w_meta2 = nullptr,
                  const __half* w_scale2 = nullptr, const __half* bias2 = nullptr, const OutDst* multi = nullptr) {
    using Cfg = SparseCfg<BT, EPI>;
    constexpr int TILE_W = (EPI == 2) ? BW / 2 : BW;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = sparse_gemm_kernel<BT, EPI>;
    if (!attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = true;
    }
    CUtensorMap tm_w, tm_x, tm_meta, tm_w2, tm_meta2;
    {
        const uint64_t dims[2] = {(uint64_t)K / 2, (uint64_t)N_out};
        const uint64_t str[1] = {(uint64_t)K / 2};
        const uint32_t box[2] = {128, TILE_W};
        if (!make_tmap(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, W_comp, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
        if (!make_tmap(&tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (EPI == 2) ? W_comp2 : W_comp, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {128, BT};
        if (!make_tmap(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        // (4 words, N_out rows, K/128 column groups). Plain: one box = 2 column groups of 128 rows x 16
        // bytes. Gated: one box = 1 column group of 64 rows (gate and up halves are placed separately).
        const uint64_t dims[3] = {4, (uint64_t)N_out, (uint64_t)K / 128};
        const uint64_t str[2] = {(uint64_t)K / 8, 16};
        const uint32_t box[3] = {4, (uint32_t)TILE_W, (uint32_t)((EPI == 2) ? 1 : 2)};
        if (!make_tmap(&tm_meta, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w_meta, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
        if (!make_tmap(&tm_meta2, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (EPI == 2) ? w_meta2 : w_meta, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
    }
    int* status = status_word();
    if (status == nullptr) return kLaunchFailed;
    const long long tiles = (long long)((N_out + TILE_W - 1) / TILE_W) * ((M + BT - 1) / BT);
    const int grid = (int)std::min<long long>(tiles, sm_count());
    OutDst md = {};
    if (multi != nullptr) md = *multi;
    return launch_gemm(kern, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, tm_w, tm_x, tm_meta, tm_w2, tm_meta2, out,
                       md, act_scale, w_scale, bias, w_scale2, bias2, M, N_out, K, status) == cudaSuccess
               ? kOk
               : kLaunchFailed;
}

template <int EPI>
int sparse_dispatch(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                    const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out,
                    cudaStream_t stream, int force_bt) {
    if (M <= 0 || K <= 0 || N_out <= 0) return kOk;   // reference: silent no-op (int8_sparse.cu:976)
    if (W_comp == nullptr || x == nullptr || w_meta == nullptr || out == nullptr) return kBadPointer;
    if (EPI == 1 && (act_scale == nullptr || w_scale == nullptr)) return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    const bool aligned = aligned16(W_comp) && aligned16(x) && aligned16(w_meta);
    const bool tma_ok = (K % 128 == 0) && aligned;
    SparseChoice c = sparse_choose(M, K, N_out, tma_ok, aligned, force_bt, true);
    if (c.kind == 3)
        return sparse_gemv(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream, EPI);
    if (c.kind == 0) {
        const long long total = (long long)M * N_out;
        sparse_gemm_ragged_kernel<EPI><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
            W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out);
        return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
    }
    if (c.kind == 2) {
        const int r = (EPI == 0) ? sparse_pair_s32(W_comp, x, w_meta, static_cast<int32_t*>(out), M, K, N_out,
                                                   stream, c.bt)
                                 : sparse_pair_dequant(W_comp, x, w_meta, act_scale, w_scale, bias,
                                                       static_cast<__half*>(out), M, K, N_out, stream, c.bt);
        if (r >= 0) return r;
        c = sparse_choose(M, K, N_out, true, aligned, force_bt, false);   // no pair of these CTAs fits on this device
    }
    const int bt = c.bt;
    switch (bt) {
    case 128: return launch_sparse<128, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    case 64:  return launch_sparse<64, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    default:  return launch_sparse<32, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    }
}

}  // namespace

// Cost model of the tile choice, the counterpart of the reference's wave-aware model
// (src/gemm/int8_sparse.cu:885-920, fitted there to an RTX 4090): a launch of variant v costs
//     c0_v + waves_v * (a_v * ksteps + b_v)   microseconds,
// waves_v = ceil(tiles_v / co-resident tiles), ksteps = ceil(K / 256). The constants are a
// non-negative least-squares fit (relative errors) to single launches with cold L2 on a B200 over the reference's
// benchmark grid ((K, N) in {(1536,6144), (6144,1536), (1280,5120), (5120,1280)} x M in {64, 1024, 4096,
// 8192}), the 11008 x 4096 weight at M = 8 ... 8192, the 4096 <-> 14336 and 8192 -> 28672 layers at
// M = 8192 and four square shapes; on those points the model's pick is the best measured variant or
// within 0.3 % of it (sum of times 2581 us, the same as the per-point best).
struct TileCost {
    int bt;
    bool pair;
    float c0, a, b;
};
constexpr TileCost kTileCosts[] = {
    {32, false, 9.82f, 0.271f, 0.349f},  {64, false, 10.60f, 0.281f, 0.421f}, {128, false, 10.50f, 0.410f, 0.800f},
    {192, true, 12.18f, 0.417f, 0.938f}, {224, true, 11.64f, 0.447f, 1.276f},
};

// force_bt: 0 = free choice; 1 = one CTA per tile, 32 or 64 tokens; 32 / 64 / 128 = that single-CTA tile;
// 1000 = CTA pair, width by the model; 1000 + BT = that pair tile.
SparseChoice sparse_choose(int M, int K, int N_out, bool tma_ok, bool stream_ok, int force_bt, bool allow_pair) {
    // One or two tokens: the call is a pass over the weights; the CUDA-core streaming kernel has less
    // fixed cost than the tensor-core kernel (sparse_gemv.cu).
    if (force_bt == 0 && stream_ok && sparse_gemv_fits(M, K)) return {3, 0};
    if (!tma_ok) return {0, 0};
    if (force_bt > 1000) {
        if (allow_pair) return {2, force_bt - 1000};
        force_bt = 0;
    }
    if (force_bt == 32 || force_bt == 64 || force_bt == 128) return {1, force_bt};
    const int sms = sm_count();
    const float ksteps = (float)((K + SLAB_K - 1) / SLAB_K);
    SparseChoice best = {1, 128};
    float best_cost = 3.0e38f;
    for (const TileCost& t : kTileCosts) {
        if (t.pair && (!allow_pair || force_bt == 1)) continue;
        if (!t.pair && force_bt == 1000 && allow_pair) continue;
        if (force_bt == 1 && t.bt > 64) continue;
        const long long tiles = t.pair ? (long long)((N_out + 2 * BW - 1) / (2 * BW)) * ((M + t.bt - 1) / t.bt)
                                       : (long long)((N_out + BW - 1) / BW) * ((M + t.bt - 1) / t.bt);
        const long long slots = t.pair ? sms / 2 : sms;
        const float waves = (float)((tiles + slots - 1) / slots);
        const float cost = t.c0 + waves * (t.a * ksteps + t.b);
        if (cost < best_cost) {
            best_cost = cost;
            best = {t.pair ? 2 : 1, t.bt};
        }
    }
    return best;
}

int sparse_gemm_s32(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, int32_t* out, int M, int K,
                    int N_out, cudaStream_t stream, int force_bt) {
    return sparse_dispatch<0>(W_comp, x, w_meta, nullptr, nullptr, nullptr, out, M, K, N_out, stream, force_bt);
}

int sparse_gemm_dequant(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                        const __half* w_scale, const __half* bias, __half* out, int M, int K, int N_out,
                        cudaStream_t stream, int force_bt) {
    return sparse_dispatch<1>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream, force_bt);
}

int sparse_gemm_dequant_multi(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                              const __half* w_scale, const __half* bias, void* const* outs, int n_outs,
                              long long ld_out, int M, int K, int N_out, cudaStream_t stream) {
    if (M <= 0 || K <= 0 || N_out <= 0 || n_outs <= 0) return kOk;
    if (W_comp == nullptr || x == nullptr || w_meta == nullptr || act_scale == nullptr || w_scale == nullptr ||
        outs == nullptr)
        return kBadPointer;
    if (n_outs > 8 || ld_out < N_out) return kBadShape;
    if (!device_is_sm100()) return kUnsupportedArch;
    if (K % 128 != 0 || !aligned16(W_comp) || !aligned16(x) || !aligned16(w_meta)) return kBadShape;
    OutDst md = {};
    md.count = n_outs;
    md.ld = ld_out;
    md.vec = (ld_out % 8 == 0 && N_out % 8 == 0) ? 1 : 0;
    for (int d = 0; d < n_outs; d++) {
        if (outs[d] == nullptr) return kBadPointer;
        md.ptr[d] = outs[d];
        if (!aligned16(outs[d])) md.vec = 0;
    }
    if (M >= 1024 && N_out >= 512) {
        const int r = sparse_pair_dequant_multi(W_comp, x, w_meta, act_scale, w_scale, bias, &md, M, K, N_out, stream);
        if (r >= 0) return r;
    }
    if (M > 64)
        return launch_sparse<128, 1>(W_comp, x, w_meta, act_scale, w_scale, bias, nullptr, M, K, N_out, stream, nullptr,
                                     nullptr, nullptr, nullptr, &md);
    return launch_sparse<32, 1>(W_comp, x, w_meta, act_scale, w_scale, bias, nullptr, M, K, N_out, stream, nullptr,
                                nullptr, nullptr, nullptr, &md);
}

int sparse_gemm_gated(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp, const uint32_t* wu_meta,
                      const int8_t* x, const float* act_scale, const __half* wg_scale, const __half* wu_scale,
                      const __half* bg, const __half* bu, __half* out, int M, int K, int N_out, cudaStream_t stream,
                      int force_bt) {
    if (M <= 0 || K <= 0 || N_out <= 0) return kOk;
    if (Wg_comp == nullptr || wg_meta == nullptr || Wu_comp == nullptr || wu_meta == nullptr || x == nullptr ||
        act_scale == nullptr || wg_scale == nullptr || wu_scale == nullptr || out == nullptr)
        return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    // TMA path only: K a multiple of 128, 16-byte aligned operands
    if (K % 128 != 0 || !aligned16(Wg_comp) || !aligned16(Wu_comp) || !aligned16(wg_meta) || !aligned16(wu_meta) ||
        !aligned16(x))
        return kBadShape;
    if (force_bt == 0 && M >= 1024 && N_out >= 256) {
        const int r = sparse_pair_gated(Wg_comp, wg_meta, Wu_comp, wu_meta, x, act_scale, wg_scale, wu_scale, bg, bu,
                                        out, M, K, N_out, stream, 224);
        if (r >= 0) return r;
    }
    if (force_bt > 1000) {
        const int r = sparse_pair_gated(Wg_comp, wg_meta, Wu_comp, wu_meta, x, act_scale, wg_scale, wu_scale, bg, bu,
                                        out, M, K, N_out, stream, force_bt - 1000);
        if (r >= 0) return r;
    }
    const int bt = (force_bt == 32 || force_bt == 64 || force_bt == 128) ? force_bt : (M > 64 ? 128 : (M > 32 ? 64 : 32));
    switch (bt) {
    case 128: return launch_sparse<128, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                           Wu_comp, wu_meta, wu_scale, bu);
    case 64:  return launch_sparse<64, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                          Wu_comp, wu_meta, wu_scale, bu);
    default:  return launch_sparse<32, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                          Wu_comp, wu_meta, wu_scale, bu);
    }
}

}  // namespace fb200
