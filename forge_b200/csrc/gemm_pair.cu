// CTA-pair (tcgen05 cta_group::2) variants of the dense and 2:4-sparse INT8 GEMMs.
//
// Two CTAs on neighbouring SMs form a cluster and share one UMMA tile: the dense kernel
// computes 256 x 256 outputs per pair, the sparse kernel 256 weight rows x BT tokens. Each CTA
// stages only its own half of BOTH operands (128 rows of the M-side operand, N/2 rows of the
// N-side operand) in its shared memory with ordinary TMA loads - no cluster multicast - and
// the leader CTA's single MMA thread issues tcgen05.mma.cta_group::2, which reads both CTAs'
// shared memory and writes both CTAs' tensor memory. Per output this halves the N-side operand
// bytes a CTA has to pull from L2, which is what limits the single-CTA kernels.
//
// Barrier protocol (per pipeline stage s; "leader" = cluster rank 0):
//   full[s]   lives in the leader. The leader's first producer arms it with the byte count of both
//             CTAs' operand loads; every operand TMA load of either CTA reports its bytes to it.
//   empty[s]  one per CTA. After the MMAs that read stage s the leader's MMA thread issues ONE
//             tcgen05.commit whose arrival is delivered to the barrier at the same shared-memory
//             offset in both CTAs; each CTA's producers wait on their own. (Two commits, one per
//             CTA, cost the sparse MMA stream about 70 clocks each - measured.)
//   tmem_full[b]  one per CTA, committed by the leader after a tile's last MMA.
//   tmem_empty[b] lives in the leader; the epilogue warps of both CTAs arrive on it.
//   sparse kernel only:
//   meta_full[s]  lives in the leader; armed with the bytes of both CTAs' metadata slabs, which
//                 report to it instead of full[s].
//   meta_ready[s] lives in the leader; committed by the metadata-copy thread (below) once the
//                 slab is in tensor memory AND full[s] has completed - the only barrier the MMA
//                 thread waits on per stage.
// Every wait is bounded; a wait that runs out sets the CTA's abort flag and the device status
// word, and all roles fall through to the common teardown (cluster barrier, TMEM free).
#include "common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"
#include "gemm_pair.cuh"
#include "sparse_epilogue.cuh"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int kThreads = 224;   // TMA warp, MMA warp, 4 epilogue warps, second TMA warp
constexpr int kEpiWarps = 4;
constexpr int kEpiThreads = 128;
// sparse kernel: epilogue warps per CTA - two per TMEM lane quarter, four for the gated epilogue
// (measured: the heavier SiLU epilogue gains from 16 warps, the plain one loses a little)
__host__ __device__ constexpr int sp_epi_warps(int epi) { return epi == 2 ? 16 : 8; }
// TMA warp, MMA warp, the epilogue warps, second TMA warp, metadata-copy warp
__host__ __device__ constexpr int sp_threads(int epi) { return 128 + 32 * sp_epi_warps(epi); }
constexpr int kSpEpiWarpsMax = 16;
// weight-row blocks per raster band of the sparse kernel: the activations are re-read from DRAM
// once per band, the band's weights stay in L2
constexpr int kSparseBand = 16;
// row blocks (of 256) per raster band of the dense pair kernel
constexpr int kDenseBand = 16;

// Shared bookkeeping at the tail of dynamic shared memory.
struct PairBars {
    uint64_t* full;        // [stages], used in the leader
    uint64_t* empty;       // [stages]
    uint64_t* tmem_full;   // [2]
    uint64_t* tmem_empty;  // [2], used in the leader
    uint64_t* meta_full;   // [stages], used in the leader (sparse kernel)
    uint64_t* meta_ready;  // [stages], used in the leader (sparse kernel)
    uint32_t* tmem_slot;
    volatile int* abort_flag;
};

__device__ __forceinline__ PairBars carve_bars(uint8_t* p, int stages) {
    PairBars b;
    uint64_t* q = reinterpret_cast<uint64_t*>(p);
    b.full = q;
    b.empty = q + stages;
    b.tmem_full = q + 2 * stages;
    b.tmem_empty = b.tmem_full + 2;
    b.meta_full = b.tmem_empty + 2;
    b.meta_ready = b.meta_full + stages;
    b.tmem_slot = reinterpret_cast<uint32_t*>(b.meta_ready + stages);
    b.abort_flag = reinterpret_cast<volatile int*>(b.tmem_slot + 1);
    return b;
}

__device__ __forceinline__ void init_bars(const PairBars& b, int stages, int epi_warps) {
    for (int s = 0; s < stages; s++) {
        mbar_init(&b.full[s], 1);
        mbar_init(&b.empty[s], 1);
        mbar_init(&b.meta_full[s], 1);
        mbar_init(&b.meta_ready[s], 1);
    }
    for (int i = 0; i < 2; i++) {
        mbar_init(&b.tmem_full[i], 1);
        mbar_init(&b.tmem_empty[i], 2 * epi_warps);
    }
    *b.abort_flag = 0;
    fence_mbar_init();
}

// Launch flags (measurement only; 0 in normal operation).
constexpr int kFlagResident = 1;    // stop loading after the first ring fill: the MMAs re-read resident stages
                                    // (wrong results; the time of the tensor-core side alone)
constexpr int kFlagTwoCommits = 2;  // free a stage with one tcgen05.commit per CTA instead of one commit
                                    // delivered to both CTAs' barriers
constexpr int kFlagProbe = 4;       // sparse: pair 0's MMA thread records where its clocks go (g_pair_probe)
constexpr int kFlagNoSplit = 8;     // dense: never cut the last wave's tiles in halves
constexpr int kFlagOneProducer = 16; // dense: warp 0 issues both TMA loads of a stage, the second producer idles
constexpr int kFlagNoEpilogue = 32;  // sparse: the epilogue warps free the accumulator without reading or storing it
constexpr int kFlagNoMetaCopy = 64;  // sparse: the copy thread signals meta_ready without issuing the tcgen05.cp
constexpr int kFlagEpiNoLoad = 256;   // sparse, with 128: the epilogue stores without reading tensor memory
constexpr int kFlagEpiNoStore = 512;  // sparse, with 128: the epilogue reads tensor memory and stores nothing
constexpr int kFlagEpiMathOnly = 2048; // sparse, with 128: the epilogue computes its results and stores none
constexpr int kFlagDirectStores = 128;   // sparse: the warps store the output themselves (the earlier epilogue)
constexpr int kFlagClusterRelease = 65536;  // sparse: free the accumulator with a cluster-scope release (the earlier form)

// kFlagProbe: [0] total clocks of the MMA thread's loop, [1] waiting for operands, [2] waiting for a
// drained accumulator, [3] stages, [4] tiles
__device__ unsigned long long g_pair_probe[8];

struct TileCoord {
    int a_blk, b_blk;   // block index along the M-side operand / the N-side operand
};

// Bands of `group` blocks of the M-side operand, N-side block major inside a band.
__device__ __forceinline__ TileCoord tile_coord(int t, int a_blocks, int b_blocks, int group) {
    const int band_tiles = group * b_blocks;
    const int band = t / band_tiles;
    const int first = band * group;
    const int rows = min(group, a_blocks - first);
    const int r = t - band * band_tiles;
    TileCoord c;
    c.a_blk = first + r % rows;
    c.b_blk = r / rows;
    return c;
}

// Work items of the dense pair kernel. The tiles are 256 x 256; when the last wave would leave more
// than half of the pairs idle (0 < tiles % pairs <= pairs / 2), the tiles of that wave are cut into
// two 256 x 128 halves so that the wave takes half as long (4096^3 on 74 pairs: 3.46 -> 3.5 waves
// instead of 4).
struct DenseWork {
    int full;     // items [0, full) are whole tiles
    int items;    // items [full, items) are halves of tiles full + (i - full) / 2
};
__host__ __device__ inline DenseWork dense_work(int tiles, int pairs, bool allow_split) {
    DenseWork w;
    const int rem = tiles % pairs;
    const bool split = allow_split && tiles > pairs && rem > 0 && 2 * rem <= pairs;
    w.full = split ? tiles - rem : tiles;
    w.items = split ? tiles + rem : tiles;
    return w;
}
struct DenseItem {
    int tile;
    int n_off;    // first column inside the tile (0 or 128)
    int n_cols;   // 256 or 128
};
__device__ __forceinline__ DenseItem dense_item(int i, const DenseWork& w) {
    DenseItem it;
    if (i < w.full) {
        it.tile = i;
        it.n_off = 0;
        it.n_cols = 256;
    } else {
        it.tile = w.full + ((i - w.full) >> 1);
        it.n_off = ((i - w.full) & 1) * 128;
        it.n_cols = 128;
    }
    return it;
}

// ============================================================================================
// Dense: 256 x 256 outputs per pair. CTA r holds A rows [128r, 128r+128) and B rows
// [128r, 128r+128) of the tile; its TMEM receives output rows [128r, 128r+128) x 256 columns.

struct DensePairCfg {
    static constexpr int kStages = 6;
    static constexpr int kABytes = 128 * 128;
    static constexpr int kBBytes = 128 * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kEpiBufs = 2;
    static constexpr int kEpiBufBytes = 32 * 128;
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiBufBytes;
    static constexpr int kScaleBytes = 2 * 256 * 2 * (int)sizeof(__half);
    static constexpr int kBarBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kScaleBytes + kBarBytes;
    static constexpr int kTmemCols = 512;
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory limit");
};

// FLAGS is a template parameter, 0 in production: the single-thread MMA issue loop must carry no run-time
// flag test (one around the commits cost 15 % of the kernel's time at 8192^3). The measurement variants
// are separate instantiations, selected by the launcher from the tuning knob.
template <int EPI, int FLAGS>
__global__ void __launch_bounds__(kThreads, 1)
dense_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_b_half, const __grid_constant__ CUtensorMap tm_c,
                  const float* __restrict__ act_scale,
                  const __half* __restrict__ w_scale, const __half* __restrict__ bias,
                  const __half* __restrict__ w_scale2, const __half* __restrict__ bias2, int M, int N, int K,
                  int band, int* __restrict__ status) {
    // EPI 2 (gated): the pair's B tile is 128 rows of the gate weight (staged by CTA 0, map tm_b)
    // followed by the same 128 rows of the up weight (staged by CTA 1, map tm_b_half), so every
    // accumulator row holds gate and up of 128 output columns and the epilogue writes
    // SiLU(gate) * up for a 256 x 128 output tile. N counts output columns.
    using Cfg = DensePairCfg;
    constexpr int flags = FLAGS | (EPI == 2 ? kFlagNoSplit : 0);
    constexpr int BN = 256;
    constexpr int TILE_N = (EPI == 2) ? BN / 2 : BN;   // output columns per tile
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* smem_ab = smem;
    uint8_t* smem_epi = smem + Cfg::kStages * Cfg::kStageBytes;
    __half* smem_scale = reinterpret_cast<__half*>(smem_epi + Cfg::kEpiBytes);
    const PairBars bars = carve_bars(smem_epi + Cfg::kEpiBytes + Cfg::kScaleBytes, Cfg::kStages);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = (rank == 0);
    const bool aligned = (smem_u32(smem) & 1023u) == 0;   // same in both CTAs of the pair
    if (!aligned) {
        if (threadIdx.x == 0) atomicExch(status, 300);
        return;
    }

    const int m_blocks = (M + 255) / 256;
    const int n_blocks = (N + TILE_N - 1) / TILE_N;
    const int num_kb = (K + 127) / 128;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const DenseWork work = dense_work(m_blocks * n_blocks, num_pairs, (flags & kFlagNoSplit) == 0);
    const int num_tiles = work.items;   // work items: whole tiles, then halves of the last wave's tiles

    if (threadIdx.x == 0) init_bars(bars, Cfg::kStages, kEpiWarps);
    if (warp_id == 0 && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_c);
    }
    if (warp_id == 1) {
        tmem_alloc_pair(bars.tmem_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *bars.tmem_slot;
    // When the launch is a programmatic dependent of the quantizer that produces this GEMM's
    // activations (launch_behind_quantizer), everything above ran under that kernel's tail. The
    // threads that read that kernel's output - the producer of the A slabs and the epilogue warps
    // (token scales) - execute griddepcontrol.wait first; the weight slabs stream at once. In an
    // ordinary launch the wait returns immediately.

    // Two TMA producers per CTA: warp 0 loads the A slab and arms the stage's barrier with the byte
    // count of the whole stage (both CTAs), the last warp loads the B slab.
    const bool second = (warp_id == kThreads / 32 - 1);
    const bool one_producer = (flags & kFlagOneProducer) != 0;
    if (warp_id == 0 || second) {
        // ------------------------------------------------------------------ TMA producers (both CTAs)
        if (lane == 0 && !(second && one_producer)) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            if (!second) griddep_wait();   // A is the preceding quantizer's output; B (weights) is not
            for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
                const DenseItem item = dense_item(t, work);
                const TileCoord tc = tile_coord(item.tile, m_blocks, n_blocks, band);
                const bool half = item.n_cols == 128;
                for (int kb = 0; kb < num_kb; kb++, it++) {
                    if (!mbar_wait(&bars.empty[stage], phase ^ 1, bars.abort_flag)) {
                        atomicExch(status, 301);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem_ab + stage * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    const uint32_t full_leader = mapa_shared(smem_u32(&bars.full[stage]), 0);
                    if ((flags & kFlagResident) != 0 && it >= Cfg::kStages) {
                        if (leader && !second) mbar_arrive(&bars.full[stage]);
                    } else if (!second) {
                        if (leader)
                            mbar_expect_tx(&bars.full[stage], 2 * (Cfg::kABytes + (half ? Cfg::kBBytes / 2 : Cfg::kBBytes)));
                        tma_load_2d_pair(sa, &tm_a, full_leader, kb * 128, tc.a_blk * 256 + (int)rank * 128);
                        if (one_producer && EPI != 2) {
                            if (half)
                                tma_load_2d_pair(sb, &tm_b_half, full_leader, kb * 128,
                                                 tc.b_blk * 256 + item.n_off + (int)rank * 64);
                            else
                                tma_load_2d_pair(sb, &tm_b, full_leader, kb * 128, tc.b_blk * 256 + (int)rank * 128);
                        }
                    } else if (EPI == 2) {
                        // CTA 0: 128 gate rows, CTA 1: the same rows of the up weight
                        tma_load_2d_pair(sb, leader ? &tm_b : &tm_b_half, full_leader, kb * 128, tc.b_blk * TILE_N);
                    } else if (half) {
                        // each CTA stages 64 of the 128 B rows of a half tile
                        tma_load_2d_pair(sb, &tm_b_half, full_leader, kb * 128,
                                         tc.b_blk * 256 + item.n_off + (int)rank * 64);
                    } else {
                        tma_load_2d_pair(sb, &tm_b, full_leader, kb * 128, tc.b_blk * 256 + (int)rank * 128);
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp_id == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            constexpr uint32_t idesc_full = make_idesc_i8(256, BN, false);
            constexpr uint32_t idesc_half = make_idesc_i8(256, BN / 2, false);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = pair_id; t < num_tiles && ok; t += num_pairs, local++) {
                const uint32_t idesc = dense_item(t, work).n_cols == 128 ? idesc_half : idesc_full;
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                if (!mbar_wait(&bars.tmem_empty[buf], acc_phase ^ 1, bars.abort_flag)) {
                    atomicExch(status, 302);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&bars.full[stage], phase, bars.abort_flag)) {
                        atomicExch(status, 303);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_ab + stage * Cfg::kStageBytes);
                    const uint64_t desc_a = make_desc_sw128(sa);
                    const uint64_t desc_b = make_desc_sw128(sa + Cfg::kABytes);
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_i8_pair(tmem_acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    const uint32_t e = smem_u32(&bars.empty[stage]);
                    if ((flags & kFlagTwoCommits) == 0) {
                        tc_commit_pair_mask(e, 3);
                    } else {
                        tc_commit_pair(mapa_shared(e, 0));
                        tc_commit_pair(mapa_shared(e, 1));
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) {
                    const uint32_t f = smem_u32(&bars.tmem_full[buf]);
                    tc_commit_pair(mapa_shared(f, 0));
                    tc_commit_pair(mapa_shared(f, 1));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp_id & 3;
        const int epi_tid = (warp_id - 2) * 32 + lane;
        uint8_t* my_stage = smem_epi + (warp_id - 2) * Cfg::kEpiBufs * Cfg::kEpiBufBytes;
        constexpr int CH = (EPI == 0) ? 32 : 64;
        const bool has_bias = (bias != nullptr);
        const uint64_t store_policy = l2_policy_evict_first();   // outputs must not push operands out of L2
        int local = 0;
        int sbuf = 0;
        bool ok = true;
        griddep_wait();   // the token scales are the preceding quantizer's output
        for (int t = pair_id; t < num_tiles; t += num_pairs, local++) {
            const DenseItem item = dense_item(t, work);
            const TileCoord tc = tile_coord(item.tile, m_blocks, n_blocks, band);
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int row0 = tc.a_blk * 256 + (int)rank * 128;
            const int row = row0 + q * 32 + lane;
            const int n0 = tc.b_blk * TILE_N + item.n_off;
            // EPI 1: [w_scale BN][bias BN]; EPI 2: [gate scale][gate bias][up scale][up bias], TILE_N each
            __half* s_ws = smem_scale + buf * 2 * BN;
            __half* s_bias = s_ws + TILE_N;
            __half* s_ws2 = s_bias + TILE_N;
            __half* s_bias2 = s_ws2 + TILE_N;
            float as = 0.f;
            if (EPI != 0) {
                if (ok) {
                    for (int i = epi_tid; i < TILE_N; i += kEpiThreads) {
                        const int n = n0 + i;
                        s_ws[i] = (n < N) ? w_scale[n] : __float2half(0.f);
                        s_bias[i] = (has_bias && n < N) ? bias[n] : __float2half(0.f);
                        if (EPI == 2) {
                            s_ws2[i] = (n < N) ? w_scale2[n] : __float2half(0.f);
                            s_bias2[i] = (bias2 != nullptr && n < N) ? bias2[n] : __float2half(0.f);
                        }
                    }
                    as = (row < M) ? act_scale[row] : 0.f;
                }
                named_barrier_sync(1, kEpiThreads);
            }
            if (ok) {
                ok = __all_sync(0xffffffffu, mbar_wait(&bars.tmem_full[buf], acc_phase, bars.abort_flag));
                if (!ok) atomicExch(status, 304);
            }
            if (!ok) continue;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < (EPI == 2 ? TILE_N : item.n_cols) / CH; c++) {
                uint32_t packed[32];
                if (EPI == 0) {
                    tmem_ld_32x32b_x32(taddr + c * CH, packed);
                    tmem_ld_wait();
                } else if (EPI == 2) {
                    const bool has_bias2 = (bias2 != nullptr);
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {   // two 32-column halves of the 64-column staged row
                        uint32_t vg[32], vu[32];
                        const int col = c * CH + hh * 32;
                        tmem_ld_32x32b_x32(taddr + col, vg);
                        tmem_ld_32x32b_x32(taddr + TILE_N + col, vu);
                        tmem_ld_wait();
                        const __half2* gs2 = reinterpret_cast<const __half2*>(s_ws + col);
                        const __half2* gb2 = reinterpret_cast<const __half2*>(s_bias + col);
                        const __half2* us2 = reinterpret_cast<const __half2*>(s_ws2 + col);
                        const __half2* ub2 = reinterpret_cast<const __half2*>(s_bias2 + col);
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const float2 gw = __half22float2(gs2[i]), gb = __half22float2(gb2[i]);
                            const float2 uw = __half22float2(us2[i]), ub = __half22float2(ub2[i]);
                            const float g0 = dequant_gemm(static_cast<int>(vg[2 * i]), mul_ftz(as, gw.x), gb.x, has_bias);
                            const float g1 =
                                dequant_gemm(static_cast<int>(vg[2 * i + 1]), mul_ftz(as, gw.y), gb.y, has_bias);
                            const float u0 = dequant_gemm(static_cast<int>(vu[2 * i]), mul_ftz(as, uw.x), ub.x, has_bias2);
                            const float u1 =
                                dequant_gemm(static_cast<int>(vu[2 * i + 1]), mul_ftz(as, uw.y), ub.y, has_bias2);
                            packed[hh * 16 + i] = pack_half2(silu_mul(g0, u0), silu_mul(g1, u1));
                        }
                    }
                } else {
                    uint32_t va[32], vb[32];
                    tmem_ld_32x32b_x32(taddr + c * CH, va);
                    tmem_ld_32x32b_x32(taddr + c * CH + 32, vb);
                    tmem_ld_wait();
                    const __half2* ws2 = reinterpret_cast<const __half2*>(s_ws + c * CH);
                    const __half2* bs2 = reinterpret_cast<const __half2*>(s_bias + c * CH);
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float2 w = __half22float2(ws2[i]);
                        const float2 b = __half22float2(bs2[i]);
                        packed[i] = pack_half2(
                            dequant_gemm(static_cast<int>(va[2 * i]), mul_ftz(as, w.x), b.x, has_bias),
                            dequant_gemm(static_cast<int>(va[2 * i + 1]), mul_ftz(as, w.y), b.y, has_bias));
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float2 w = __half22float2(ws2[16 + i]);
                        const float2 b = __half22float2(bs2[16 + i]);
                        packed[16 + i] = pack_half2(
                            dequant_gemm(static_cast<int>(vb[2 * i]), mul_ftz(as, w.x), b.x, has_bias),
                            dequant_gemm(static_cast<int>(vb[2 * i + 1]), mul_ftz(as, w.y), b.y, has_bias));
                    }
                }
                uint8_t* stg = my_stage + sbuf * Cfg::kEpiBufBytes;
                if (lane == 0) tma_store_wait_read<Cfg::kEpiBufs - 1>();
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int chunk = j ^ (lane & 7);
                    *reinterpret_cast<uint4*>(stg + lane * 128 + chunk * 16) =
                        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d_hint(&tm_c, stg, n0 + c * CH, row0 + q * 32, store_policy);
                    tma_store_commit();
                }
                sbuf = (sbuf + 1) % Cfg::kEpiBufs;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote_cta_scope(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
        }
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    if (*bars.abort_flag != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // neither CTA frees TMEM or exits while the peer can still touch it
    if (warp_id == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// ============================================================================================
// 2:4 sparse: 256 weight rows x BT tokens per pair. CTA r holds compressed weight rows
// [128r, 128r+128) with their metadata, and token rows [r*BT/2, (r+1)*BT/2) of the tile; its
// TMEM receives weight rows [128r, 128r+128) x BT token columns.

constexpr int kXbufBytes = (kSpEpiWarpsMax / 2) * 32 * 32 * (int)sizeof(float);   // gated epilogue: 4 KB per warp pair

template <int BT, int EPI = 0>
struct SparsePairCfg {
    static constexpr int HT = BT / 2;                       // tokens staged per CTA
    static constexpr int kABytes = 128 * 128;
    static constexpr int kBAtomBytes = HT * 128;
    static constexpr int kMetaBytes = 128 * 32;
    static constexpr int kStageBytes = kABytes + 2 * kBAtomBytes + kMetaBytes;
    static constexpr int kBarBytes = 256;
    // EPI 2: gate/up exchange buffers; EPI 1: two 8 KB transposition buffers of the multi-destination store
    static constexpr int kFixed = kBarBytes + (EPI == 2 ? kXbufBytes : (EPI == 1 ? 16384 : 0));
    static constexpr int kStagesMax = (232448 - kFixed) / kStageBytes;
    static constexpr int kStages = kStagesMax > 6 ? 6 : kStagesMax;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFixed;
    static constexpr int kMetaCols = 8 * kStages;
    static constexpr int kAccBufs = (2 * BT + kMetaCols <= 512) ? 2 : 1;
    static constexpr int kAccCols = kAccBufs * BT;
    static constexpr int kTmemCols = 512;
    static_assert(BT % 32 == 0 && BT <= 256, "pair MMA needs N % 32 == 0, N <= 256");
    static_assert(kBAtomBytes % 1024 == 0 && kStageBytes % 1024 == 0, "1024-byte aligned operand atoms");
    static_assert(kStages >= 3, "pipeline depth");
    static_assert(kAccCols + kMetaCols <= 512, "TMEM capacity");
};

template <int BT, int EPI, int FLAGS>
__global__ void __launch_bounds__(sp_threads(EPI), 1)
sparse_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ CUtensorMap tm_meta, const __grid_constant__ CUtensorMap tm_w2,
                   const __grid_constant__ CUtensorMap tm_meta2, const __grid_constant__ CUtensorMap tm_out,
                   int out_tma, void* __restrict__ out, const OutDst multi,
                   const float* __restrict__ act_scale, const __half* __restrict__ w_scale,
                   const __half* __restrict__ bias, const __half* __restrict__ w_scale2,
                   const __half* __restrict__ bias2, int M, int N_out, int K, int* __restrict__ status) {
    constexpr int flags = FLAGS;   // see dense_pair_kernel
    // EPI 2 (gated): each CTA's 128-row weight tile is 64 gate rows followed by the 64 up rows of the
    // same output columns, so a pair produces 128 output columns per tile.
    using Cfg = SparsePairCfg<BT, EPI>;
    constexpr int HT = Cfg::HT;
    constexpr int CTA_W = (EPI == 2) ? 64 : 128;   // output columns per CTA
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* smem_stage = smem;
    float* smem_xbuf = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes);
    uint8_t* smem_tr = smem + Cfg::kStages * Cfg::kStageBytes;   // EPI 1: transposition buffers
    const PairBars bars = carve_bars(smem + Cfg::kStages * Cfg::kStageBytes + (Cfg::kFixed - Cfg::kBarBytes),
                                     Cfg::kStages);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = (rank == 0);
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 400);
        return;
    }

    const int w_blocks = (N_out + 2 * CTA_W - 1) / (2 * CTA_W);
    const int t_blocks = (M + BT - 1) / BT;
    const int num_tiles = w_blocks * t_blocks;
    const int num_kb = (K + 255) / 256;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    constexpr int kSpEpiWarps = sp_epi_warps(EPI);
    if (threadIdx.x == 0) init_bars(bars, Cfg::kStages, kSpEpiWarps);
    if (warp_id == 0 && lane == 0) {
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_x);
        prefetch_tensormap(&tm_meta);
    }
    if (warp_id == 1) {
        tmem_alloc_pair(bars.tmem_slot, Cfg::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *bars.tmem_slot;
    const uint32_t tmem_meta = tmem_base + Cfg::kAccCols;

    // Two TMA producers per CTA. One iteration of a producer (wait for the free stage, arm, issue) costs
    // the issuing thread about 310 clocks plus 60-100 per additional load, whatever the box size
    // (measured), and the MMAs of a stage take 500: a single thread issuing a stage's four loads is
    // slower than the tensor cores. Warp 0 loads the weight slab and its metadata and arms both
    // barriers with the byte counts of both CTAs; the second-to-last warp loads the two activation
    // atoms. (A third producer warp was measured: no gain, and its registers cost the epilogue.)
    const int n_warps = sp_threads(EPI) / 32;
    const int producer = warp_id == 0 ? 0 : (warp_id == n_warps - 2 ? 1 : -1);
    const bool copy_warp = (warp_id == n_warps - 1);
    if (producer >= 0) {
        // ------------------------------------------------------------------ TMA producers (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            // as in dense_pair_kernel: only the activation producer waits for the preceding quantizer
            if (producer == 1) griddep_wait();
            for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks, kSparseBand);
                const int w_row = tc.a_blk * 2 * CTA_W + (int)rank * CTA_W;
                const int t_row = tc.b_blk * BT + (int)rank * HT;
                for (int kb = 0; kb < num_kb; kb++, it++) {
                    if (!mbar_wait(&bars.empty[stage], phase ^ 1, bars.abort_flag)) {
                        atomicExch(status, 401);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem_stage + stage * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    uint8_t* sm = sb + 2 * Cfg::kBAtomBytes;
                    const uint32_t full_leader = mapa_shared(smem_u32(&bars.full[stage]), 0);
                    const uint32_t meta_leader = mapa_shared(smem_u32(&bars.meta_full[stage]), 0);
                    if ((flags & kFlagResident) != 0 && it >= Cfg::kStages) {
                        if (leader && producer == 0) {
                            mbar_arrive(&bars.meta_full[stage]);
                            mbar_arrive(&bars.full[stage]);
                        }
                    } else if (producer == 0) {
                        if (leader) {
                            mbar_expect_tx(&bars.meta_full[stage], 2 * Cfg::kMetaBytes);
                            mbar_expect_tx(&bars.full[stage], 2 * (Cfg::kStageBytes - Cfg::kMetaBytes));
                        }
                        if (EPI == 2) {
#pragma unroll
                            for (int c = 0; c < 2; c++) {
                                tma_load_3d_pair(sm + c * 2048, &tm_meta, meta_leader, 0, w_row, kb * 2 + c);
                                tma_load_3d_pair(sm + c * 2048 + 1024, &tm_meta2, meta_leader, 0, w_row, kb * 2 + c);
                            }
                            tma_load_2d_pair(sa, &tm_w, full_leader, kb * 128, w_row);
                            tma_load_2d_pair(sa + Cfg::kABytes / 2, &tm_w2, full_leader, kb * 128, w_row);
                        } else {
                            tma_load_3d_pair(sm, &tm_meta, meta_leader, 0, w_row, kb * 2);
                            tma_load_2d_pair(sa, &tm_w, full_leader, kb * 128, w_row);
                        }
                    } else {
                        tma_load_2d_pair(sb, &tm_x, full_leader, kb * 256, t_row);
                        tma_load_2d_pair(sb + Cfg::kBAtomBytes, &tm_x, full_leader, kb * 256 + 128, t_row);
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp_id == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (leader && lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(256, BT, true);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            int it = 0;
            bool ok = true;
            const bool probe = (flags & kFlagProbe) != 0 && pair_id == 0;
            long long wait_ops = 0, wait_acc = 0;
            const long long t_begin = probe ? clock64() : 0;
            for (int t = pair_id; t < num_tiles && ok; t += num_pairs, local++) {
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                long long w0 = probe ? clock64() : 0;
                if (!mbar_wait(&bars.tmem_empty[buf], acc_phase ^ 1, bars.abort_flag)) {
                    atomicExch(status, 402);
                    ok = false;
                    break;
                }
                if (probe) wait_acc += clock64() - w0;
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * BT;
                for (int kb = 0; kb < num_kb; kb++, it++) {
                    w0 = probe ? clock64() : 0;
                    // meta_ready[s]: the stage's metadata is in tensor memory and its operand loads have landed
                    if (!mbar_wait(&bars.meta_ready[stage], phase, bars.abort_flag)) {
                        atomicExch(status, 403);
                        ok = false;
                        break;
                    }
                    if (probe) wait_ops += clock64() - w0;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_stage + stage * Cfg::kStageBytes);
                    const uint32_t sb = sa + Cfg::kABytes;
                    const uint32_t te = tmem_meta + 8 * stage;
                    const uint64_t desc_a = make_desc_sw128(sa);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint64_t desc_b = make_desc_sw128(sb + (j >> 1) * Cfg::kBAtomBytes) + 4 * (j & 1);
                        umma_i8_sp_pair(tmem_acc, desc_a + 2 * j, desc_b, te + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    const uint32_t e = smem_u32(&bars.empty[stage]);
                    if ((flags & kFlagTwoCommits) == 0) {
                        tc_commit_pair_mask(e, 3);
                    } else {
                        tc_commit_pair(mapa_shared(e, 0));
                        tc_commit_pair(mapa_shared(e, 1));
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) {
                    const uint32_t f = smem_u32(&bars.tmem_full[buf]);
                    tc_commit_pair(mapa_shared(f, 0));
                    tc_commit_pair(mapa_shared(f, 1));
                }
            }
            if (probe) {
                g_pair_probe[0] = (unsigned long long)(clock64() - t_begin);
                g_pair_probe[1] = (unsigned long long)wait_ops;
                g_pair_probe[2] = (unsigned long long)wait_acc;
                g_pair_probe[3] = (unsigned long long)it;
                g_pair_probe[4] = (unsigned long long)local;
            }
        }
    } else if (copy_warp) {
        // ------------------------------------------------------------------ metadata copies (leader only)
        // A thread of its own moves each stage's metadata slab (both CTAs' 128 rows x 32 bytes) into
        // tensor memory with one tcgen05.cp as soon as the slab has landed - while the stage's
        // operand loads are still in flight - and commits to meta_ready[s] after full[s]. Issued from
        // the MMA thread instead, the copies sit in the MMA stream and cost about a fifth of the
        // kernel's time (measured at 8192^3).
        if (leader && lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&bars.meta_full[stage], phase, bars.abort_flag)) {
                        atomicExch(status, 405);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sm = smem_u32(smem_stage + stage * Cfg::kStageBytes) + Cfg::kABytes +
                                        2 * Cfg::kBAtomBytes;
                    // two 16-byte columns of 128 rows -> 8 TMEM columns
                    if ((flags & kFlagNoMetaCopy) == 0 || kb + (t - pair_id) < Cfg::kStages)
                        tmem_cp_128x256b_pair(tmem_meta + 8 * stage, make_desc_noswizzle(sm, 2048, 128));
                    if (!mbar_wait(&bars.full[stage], phase, bars.abort_flag)) {
                        atomicExch(status, 406);
                        ok = false;
                        break;
                    }
                    tc_commit_pair(mapa_shared(smem_u32(&bars.meta_ready[stage]), 0));
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp_id & 3;
        const int chunk0 = (warp_id - 2) >> 2;
        const bool has_bias = (bias != nullptr);
        int local = 0;
        griddep_wait();   // the token scales are the preceding quantizer's output
        if (EPI == 2) {
            const bool is_gate = q < 2;
            const int pair = (q & 1) + 2 * chunk0;   // 0 .. kSpEpiWarps/2 - 1
            float* xbuf = smem_xbuf + pair * 1024;
            const __half* my_scale = is_gate ? w_scale : w_scale2;
            const __half* my_bias = is_gate ? bias : bias2;
            bool ok = true;   // after a failed wait: keep meeting the partner warp at the barriers
            for (int t = pair_id; t < num_tiles; t += num_pairs, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks, kSparseBand);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n = tc.a_blk * 2 * CTA_W + (int)rank * CTA_W + (q & 1) * 32 + lane;
                const int m0 = tc.b_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (n < N_out) {
                    ws = __half2float(my_scale[n]);
                    if (my_bias != nullptr) bs = __half2float(my_bias[n]);
                }
                if (ok) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars.tmem_full[buf], acc_phase, bars.abort_flag));
                    if (!ok) atomicExch(status, 404);
                }
                if (ok) tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kSpEpiWarps / 4) {
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
                    if (lane == 0) mbar_arrive_remote_cta_scope(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
                }
            }
        } else if (EPI == 1 && multi.count > 0 && multi.vec != 0) {
            // several destinations (peer GPUs): wide row-segment stores through a transposition buffer
            uint8_t* stage = smem_tr + chunk0 * 8192;
            bool ok = true;   // after a failed wait: keep meeting the group at the barriers
            for (int t = pair_id; t < num_tiles; t += num_pairs, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks, kSparseBand);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n_base = tc.a_blk * 256 + (int)rank * 128;
                const int n = n_base + q * 32 + lane;
                const int m0 = tc.b_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (n < N_out) {
                    ws = __half2float(w_scale[n]);
                    if (has_bias) bs = __half2float(bias[n]);
                }
                if (ok) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars.tmem_full[buf], acc_phase, bars.abort_flag));
                    if (!ok) atomicExch(status, 404);
                }
                if (ok) tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kSpEpiWarps / 4) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M) break;
                    uint32_t v[32];
                    float as_lane = 0.f;
                    if (ok) {
                        tmem_ld_32x32b_x32(taddr + c * 32, v);
                        if (m_first + lane < M) as_lane = act_scale[m_first + lane];
                        tmem_ld_wait();
                    }
                    store_chunk_multi_vec(ok, v, multi, stage, 8 + chunk0, q, N_out, M, n_base, m_first, as_lane, ws,
                                          bs, has_bias);
                }
                if (ok) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote_cta_scope(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
                }
            }
        } else if (EPI == 1 && out_tma != 0 && (flags & kFlagDirectStores) == 0) {
            // FP16 output through shared memory and TMA stores: each warp transposes its 32 tokens x 32
            // columns into a 2 KB buffer (one 64-byte row per token) and one thread hands the box to the
            // copy engine, which also clips it at the edges of the output. Stores issued by the warps
            // themselves cost the tensor pipe 11 % of the kernel's time at 8192^3 (measured, whatever
            // their width or cache policy).
            uint8_t* stg = smem_tr + (warp_id - 2) * 2048;
            const uint64_t store_policy = l2_policy_evict_first();
            for (int t = pair_id; t < num_tiles; t += num_pairs, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks, kSparseBand);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n_warp = tc.a_blk * 256 + (int)rank * 128 + q * 32;
                const int n = n_warp + lane;
                const int m0 = tc.b_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (n < N_out) {
                    ws = __half2float(w_scale[n]);
                    if (has_bias) bs = __half2float(bias[n]);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(&bars.tmem_full[buf], acc_phase, bars.abort_flag))) {
                    atomicExch(status, 404);
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kSpEpiWarps / 4) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M || n_warp >= N_out || (flags & kFlagNoEpilogue) != 0) break;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    const float as_lane = (m_first + lane < M) ? act_scale[m_first + lane] : 0.f;
                    if (lane == 0) tma_store_wait_read<0>();   // the previous box has left the buffer
                    tmem_ld_wait();
                    __syncwarp();
                    // (16-byte staging stores after an 8 x 8 lane transpose were measured: slower, the
                    // shuffles put the epilogue on the critical path of short-K shapes)
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float as = __shfl_sync(0xffffffffu, as_lane, j);
                        const float o = dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias);
                        *reinterpret_cast<__half*>(stg + j * 64 + lane * 2) = __float2half_rn(o);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d_hint(&tm_out, stg, n_warp, m_first, store_policy);
                        tma_store_commit();
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote_cta_scope(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
            }
            if (lane == 0) tma_store_wait_all<0>();
        } else {
            for (int t = pair_id; t < num_tiles; t += num_pairs, local++) {
                const TileCoord tc = tile_coord(t, w_blocks, t_blocks, kSparseBand);
                const int buf = (Cfg::kAccBufs == 2) ? (local & 1) : 0;
                const uint32_t acc_phase = (Cfg::kAccBufs == 2) ? ((local >> 1) & 1) : (local & 1);
                const int n = tc.a_blk * 256 + (int)rank * 128 + q * 32 + lane;
                const int m0 = tc.b_blk * BT;
                float ws = 0.f, bs = 0.f;
                if (EPI == 1 && n < N_out) {
                    ws = __half2float(w_scale[n]);
                    if (has_bias) bs = __half2float(bias[n]);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(&bars.tmem_full[buf], acc_phase, bars.abort_flag))) {
                    atomicExch(status, 404);
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = chunk0; c < BT / 32; c += kSpEpiWarps / 4) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M || (flags & kFlagNoEpilogue) != 0) break;
                    uint32_t v[32];
                    if ((flags & kFlagEpiNoLoad) == 0) {
                        tmem_ld_32x32b_x32(taddr + c * 32, v);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = (uint32_t)(j ^ lane);
                    }
                    float as_lane = 0.f;
                    if (EPI == 1 && m_first + lane < M) as_lane = act_scale[m_first + lane];
                    if ((flags & kFlagEpiNoLoad) == 0) tmem_ld_wait();
                    if ((flags & kFlagEpiNoStore) != 0) continue;
                    if ((flags & kFlagEpiMathOnly) != 0) {
                        // the epilogue's arithmetic without its stores (one store that never happens)
                        unsigned sum = 0;
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float as = __shfl_sync(0xffffffffu, as_lane, j);
                            sum += __half_as_ushort(__float2half_rn(
                                dequant_gemm(static_cast<int>(v[j]), mul_ftz(as, ws), bs, has_bias)));
                        }
                        if (sum == 0xfedcba98u) static_cast<unsigned*>(out)[n] = sum;
                        continue;
                    }
                    if (EPI == 1 && multi.count > 0)
                        store_transposed_chunk_multi(v, multi, N_out, M, n, m_first, as_lane, ws, bs, has_bias);
                    else
                        store_transposed_chunk<EPI>(v, out, N_out, M, n, m_first, as_lane, ws, bs, has_bias);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    // CTA scope: the MMA thread consumes tensor memory (ordered by the tcgen05 fences),
                    // not this warp's global stores - a cluster-scope release would first wait for
                    // those to be acknowledged (measured 2 % of the kernel at 8192^3)
                    if ((flags & kFlagClusterRelease) != 0) mbar_arrive_cluster(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
                    else mbar_arrive_remote_cta_scope(mapa_shared(smem_u32(&bars.tmem_empty[buf]), 0));
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (*bars.abort_flag != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp_id == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    }
}

// ============================================================================================
// Host side.

// Launches `kern` as clusters of two CTAs; grid = 2 x min(tiles, co-resident clusters).
// Returns kOk, kLaunchFailed, or -1 when no cluster of this kernel fits (caller falls back to the
// single-CTA kernel).
template <typename Kern, typename... Args>
int launch_pairs(Kern kern, int threads, int smem_bytes, long long tiles, cudaStream_t stream,
                 int* max_pairs_cache, Args... args) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = take_behind_quantizer() ? 2 : 1;
    int& max_pairs = max_pairs_cache[dev & 63];
    if (max_pairs == 0) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess)
            return kLaunchFailed;
        cfg.gridDim = dim3(2 * sm_count(), 1, 1);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            max_pairs = -1;
        } else {
            max_pairs = n;
        }
    }
    if (max_pairs < 0) return -1;
    int pairs = (int)std::min<long long>(tiles, max_pairs);
    const int cap = tuning_knob(kKnobMaxPairs);
    if (cap > 0 && cap < pairs) pairs = cap;
    set_tuning_knob(kKnobLastPairs, pairs);
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
    return e == cudaSuccess ? kOk : kLaunchFailed;
}

template <int EPI>
int launch_dense_pair(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                      const __half* bias, void* out, int M, int K, int N, cudaStream_t stream,
                      const int8_t* B2 = nullptr, const __half* w_scale2 = nullptr, const __half* bias2 = nullptr) {
    static int max_pairs[64] = {};
    CUtensorMap tm_a, tm_b, tm_b_half, tm_c;
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {128, 128};
        if (!make_tmap(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {128, 128};
        if (!make_tmap(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, B, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
        const uint64_t str[1] = {(uint64_t)K};
        // EPI 0/1: 64-row boxes for the halves of a split tile; EPI 2: the up weight, whole 128-row slabs
        const uint32_t box[2] = {128, (uint32_t)((EPI == 2) ? 128 : 64)};
        if (!make_tmap(&tm_b_half, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (EPI == 2) ? B2 : B, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t esz = (EPI == 0) ? 4 : 2;
        const uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)N * esz};
        const uint32_t box[2] = {(uint32_t)(128 / esz), 32};
        const CUtensorMapDataType dt = (EPI == 0) ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        if (!make_tmap(&tm_c, dt, 2, out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B)) return kLaunchFailed;
    }
    int* status = status_word();
    if (status == nullptr) return kLaunchFailed;
    constexpr int TILE_N = (EPI == 2) ? 128 : 256;
    // a band's rows of A are re-read from L2 by every wave and should stay there: 16 blocks up to
    // K = 8192, 8 beyond (K = 14336: 584 -> less DRAM read per launch, 1 % faster; 8 at K = 8192: 1 % slower)
    const int band = tuning_knob(kKnobDenseBand) > 0 ? tuning_knob(kKnobDenseBand)
                                                     : ((long long)kDenseBand * 256 * K > (40ll << 20) ? kDenseBand / 2 : kDenseBand);
    const long long tiles = (long long)((M + 255) / 256) * ((N + TILE_N - 1) / TILE_N);
    const int flags = (EPI == 2) ? 0 : tuning_knob(kKnobPairFlags);
#define FB200_DENSE_VARIANT(F)                                                                                        \
    if (flags == F) {                                                                                                 \
        static int mp[64] = {};                                                                                       \
        return launch_pairs(dense_pair_kernel<EPI, F>, kThreads, DensePairCfg::kSmemBytes, tiles, stream, mp, tm_a, tm_b, \
                            tm_b_half, tm_c, act_scale, w_scale, bias, w_scale2, bias2, M, N, K, band, status);       \
    }
    if constexpr (EPI != 2) {
        FB200_DENSE_VARIANT(1) FB200_DENSE_VARIANT(2) FB200_DENSE_VARIANT(3) FB200_DENSE_VARIANT(8)
        FB200_DENSE_VARIANT(16) FB200_DENSE_VARIANT(18)
    }
#undef FB200_DENSE_VARIANT
    if constexpr (EPI == 2)
        return launch_pairs(dense_pair_kernel<2, kFlagNoSplit>, kThreads, DensePairCfg::kSmemBytes, tiles, stream,
                            max_pairs, tm_a, tm_b, tm_b_half, tm_c, act_scale, w_scale, bias, w_scale2, bias2, M, N, K,
                            band, status);
    // The half-tile bookkeeping costs about 2 % where no tile is ever cut (8192^3): the instantiation
    // without it runs unless this launch's last wave will be split.
    {
        static int mp_probe[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        const int pairs_known = mp_probe[dev & 63] > 0 ? mp_probe[dev & 63] : max_pairs[dev & 63];
        const int cap = tuning_knob(kKnobMaxPairs);
        int pairs = pairs_known > 0 ? (int)std::min<long long>(tiles, pairs_known) : 0;
        if (cap > 0 && cap < pairs) pairs = cap;
        const bool will_split = pairs > 0 && dense_work((int)tiles, pairs, true).items != (int)tiles;
        if (!will_split && pairs > 0)
            return launch_pairs(dense_pair_kernel<EPI, kFlagNoSplit>, kThreads, DensePairCfg::kSmemBytes, tiles, stream,
                                mp_probe, tm_a, tm_b, tm_b_half, tm_c, act_scale, w_scale, bias, w_scale2, bias2, M, N, K,
                                band, status);
    }
    return launch_pairs(dense_pair_kernel<EPI, 0>, kThreads, DensePairCfg::kSmemBytes, tiles, stream, max_pairs, tm_a, tm_b,
                        tm_b_half, tm_c, act_scale, w_scale, bias, w_scale2, bias2, M, N, K, band, status);
}

template <int BT, int EPI>
int launch_sparse_pair(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                       const __half* w_scale, const __half* bias, void* out, int M, int K, int N_out,
                       cudaStream_t stream, const int8_t* W_comp2 = nullptr, const uint32_t* w_meta2 = nullptr,
                       const __half* w_scale2 = nullptr, const __half* bias2 = nullptr,
                       const OutDst* multi = nullptr) {
    using Cfg = SparsePairCfg<BT, EPI>;
    constexpr int CTA_W = (EPI == 2) ? 64 : 128;
    static int max_pairs[64] = {};
    CUtensorMap tm_w, tm_x, tm_meta, tm_w2, tm_meta2;
    {
        const uint64_t dims[2] = {(uint64_t)K / 2, (uint64_t)N_out};
        const uint64_t str[1] = {(uint64_t)K / 2};
        const uint32_t box[2] = {128, (uint32_t)CTA_W};
        if (!make_tmap(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, W_comp, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
        if (!make_tmap(&tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (EPI == 2) ? W_comp2 : W_comp, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {128, (uint32_t)Cfg::HT};
        if (!make_tmap(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[3] = {4, (uint64_t)N_out, (uint64_t)K / 128};
        const uint64_t str[2] = {(uint64_t)K / 8, 16};
        const uint32_t box[3] = {4, (uint32_t)CTA_W, (uint32_t)((EPI == 2) ? 1 : 2)};
        if (!make_tmap(&tm_meta, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w_meta, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
        if (!make_tmap(&tm_meta2, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (EPI == 2) ? w_meta2 : w_meta, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
    }
    int* status = status_word();
    if (status == nullptr) return kLaunchFailed;
    const long long tiles = (long long)((N_out + 2 * CTA_W - 1) / (2 * CTA_W)) * ((M + BT - 1) / BT);
    OutDst md = {};
    if (multi != nullptr) md = *multi;
    // FP16 output as 32-token x 32-column boxes for the TMA-store epilogue (single destination only)
    CUtensorMap tm_out = tm_x;
    int out_tma = 0;
    if (EPI == 1 && multi == nullptr && N_out % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const uint64_t dims[2] = {(uint64_t)N_out, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)N_out * 2};
        const uint32_t box[2] = {32, 32};
        if (!make_tmap(&tm_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, out, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
        out_tma = 1;
    }
    const int flags = tuning_knob(kKnobPairFlags);
#define FB200_SPARSE_VARIANT(F)                                                                                       \
    if (flags == F) {                                                                                                 \
        static int mp[64] = {};                                                                                       \
        return launch_pairs(sparse_pair_kernel<BT, EPI, F>, sp_threads(EPI), Cfg::kSmemBytes, tiles, stream, mp, tm_w, tm_x, \
                            tm_meta, tm_w2, tm_meta2, tm_out, out_tma, out, md, act_scale, w_scale, bias, w_scale2, bias2, M, N_out, K, \
                            status);                                                                                  \
    }
    if (BT == 224 && EPI == 1) {   // measurement variants exist for the default tile only
        FB200_SPARSE_VARIANT(1) FB200_SPARSE_VARIANT(2) FB200_SPARSE_VARIANT(3) FB200_SPARSE_VARIANT(4)
        FB200_SPARSE_VARIANT(5) FB200_SPARSE_VARIANT(32) FB200_SPARSE_VARIANT(33) FB200_SPARSE_VARIANT(37)
        FB200_SPARSE_VARIANT(65) FB200_SPARSE_VARIANT(65536) FB200_SPARSE_VARIANT(128)
        // the three splits of the direct-store epilogue (128 + 256 / 512 / 2048)
        FB200_SPARSE_VARIANT(384) FB200_SPARSE_VARIANT(640) FB200_SPARSE_VARIANT(2176)
    }
#undef FB200_SPARSE_VARIANT
    return launch_pairs(sparse_pair_kernel<BT, EPI, 0>, sp_threads(EPI), Cfg::kSmemBytes, tiles, stream, max_pairs, tm_w,
                        tm_x, tm_meta, tm_w2, tm_meta2, tm_out, out_tma, out, md, act_scale, w_scale, bias, w_scale2, bias2,
                        M, N_out, K, status);
}

template <int EPI>
int sparse_pair_dispatch(int bt, const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta,
                         const float* act_scale, const __half* w_scale, const __half* bias, void* out, int M, int K,
                         int N_out, cudaStream_t stream) {
    switch (bt) {
    case 128: return launch_sparse_pair<128, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    case 192: return launch_sparse_pair<192, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    case 256: return launch_sparse_pair<256, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    default:  return launch_sparse_pair<224, EPI>(W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
    }
}

}  // namespace

int read_pair_probe(unsigned long long* out, int n) {
    if (n > 8) n = 8;
    return cudaMemcpyFromSymbol(out, g_pair_probe, sizeof(unsigned long long) * n) == cudaSuccess ? kOk : kLaunchFailed;
}

int dense_pair_s32(const int8_t* A, const int8_t* B, int32_t* out, int M, int K, int N, cudaStream_t stream) {
    return launch_dense_pair<0>(A, B, nullptr, nullptr, nullptr, out, M, K, N, stream);
}

int dense_pair_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                       const __half* bias, __half* out, int M, int K, int N, cudaStream_t stream) {
    return launch_dense_pair<1>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
}

int dense_pair_gated(const int8_t* A, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                     const __half* wg_scale, const __half* wu_scale, const __half* bg, const __half* bu, __half* out,
                     int M, int K, int N, cudaStream_t stream) {
    return launch_dense_pair<2>(A, Wg, act_scale, wg_scale, bg, out, M, K, N, stream, Wu, wu_scale, bu);
}

int sparse_pair_s32(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, int32_t* out, int M, int K,
                    int N_out, cudaStream_t stream, int bt) {
    return sparse_pair_dispatch<0>(bt, W_comp, x, w_meta, nullptr, nullptr, nullptr, out, M, K, N_out, stream);
}

int sparse_pair_dequant(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                        const __half* w_scale, const __half* bias, __half* out, int M, int K, int N_out,
                        cudaStream_t stream, int bt) {
    return sparse_pair_dispatch<1>(bt, W_comp, x, w_meta, act_scale, w_scale, bias, out, M, K, N_out, stream);
}

int sparse_pair_dequant_multi(const int8_t* W_comp, const int8_t* x, const uint32_t* w_meta, const float* act_scale,
                              const __half* w_scale, const __half* bias, const OutDst* multi, int M, int K, int N_out,
                              cudaStream_t stream) {
    return launch_sparse_pair<224, 1>(W_comp, x, w_meta, act_scale, w_scale, bias, nullptr, M, K, N_out, stream,
                                      nullptr, nullptr, nullptr, nullptr, multi);
}

int sparse_pair_gated(const int8_t* Wg_comp, const uint32_t* wg_meta, const int8_t* Wu_comp, const uint32_t* wu_meta,
                      const int8_t* x, const float* act_scale, const __half* wg_scale, const __half* wu_scale,
                      const __half* bg, const __half* bu, __half* out, int M, int K, int N_out, cudaStream_t stream,
                      int bt) {
    switch (bt) {
    case 128: return launch_sparse_pair<128, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                                Wu_comp, wu_meta, wu_scale, bu);
    case 192: return launch_sparse_pair<192, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                                Wu_comp, wu_meta, wu_scale, bu);
    default:  return launch_sparse_pair<224, 2>(Wg_comp, x, wg_meta, act_scale, wg_scale, bg, out, M, K, N_out, stream,
                                                Wu_comp, wu_meta, wu_scale, bu);
    }
}

}  // namespace fb200
