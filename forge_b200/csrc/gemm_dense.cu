// Dense INT8 GEMM for sm_100a: out[m,n] = sum_k A[m,k] * B[n,k].
//
// Replaces forge::gemm::int8_gemm_dequant (reference src/gemm/int8_dense.cu:26-211, a wmma
// kernel) and adds an INT32-output form the reference only has as a host test loop
// (tests/test_int8_dense_gemm.cu:35-39).
//
// Design: persistent CTAs (one per SM), each walking 128 x BN output tiles.
//   warp 0   : TMA producer. Loads 128-byte-deep K slabs of A (128 rows) and B (BN rows)
//              into a 4-stage shared-memory ring, 128B-swizzled, K-major.
//   warp 1   : MMA issuer. One thread issues tcgen05.mma kind::i8 (M=128, N=BN, K=32), four per
//              stage, accumulating s32 in TMEM; tcgen05.commit releases the stage.
//   warps 2-5: epilogue. tcgen05.ld the accumulator (lane = output row), dequantise in
//              registers, stage 128-byte row pieces in swizzled shared memory and TMA-store.
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.
#include "common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"
#include "gemm_pair.cuh"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;   // bytes of K per stage = one 128B swizzle atom = 4 UMMAs of K=32
constexpr int UMMA_K = 32;
constexpr int kThreads = 192;
constexpr int kEpiWarps = 4;
constexpr int kEpiBufBytes = 32 * 128;   // one epilogue staging buffer: 32 rows x 128 bytes

// KA: 128-byte K atoms per pipeline stage. 1 for the general kernel; 2 for calls with one block of token rows,
// which are passes over the weights whose pace is set by the TMA-issuing threads (about 310 clocks per stage
// and thread plus 80 per further load, whatever the box size): stages twice as deep and a second producer
// thread for the weight slabs halve the issue cost per byte.
template <int BN, int KA = 1>
struct DenseCfg {
    static constexpr int kABytes = BLOCK_M * BLOCK_K * KA;
    static constexpr int kBBytes = BN * BLOCK_K * KA;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kEpiBufs = 2;
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiBufBytes;
    static constexpr int kScaleBytes = 2 * BN * 2 * (int)sizeof(__half);   // [2 tiles in flight][w_scale, bias][BN]
    static constexpr int kBarBytes = 256;
    static constexpr int kStagesFit = (232448 - kEpiBytes - kScaleBytes - kBarBytes) / kStageBytes;
    static constexpr int kStages = (KA == 1) ? ((BN == 256) ? 4 : 6) : (kStagesFit > 6 ? 6 : kStagesFit);
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kScaleBytes + kBarBytes;
    static constexpr int kTmemCols = (2 * BN <= 128) ? 128 : (2 * BN <= 256 ? 256 : 512);   // power of two >= 2 * BN
    static constexpr int kThreads = (KA == 1) ? 192 : 224;   // KA 2: a seventh warp issues the B loads
    static_assert(kStages >= 3, "pipeline depth");
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KB shared memory limit");
    static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns: power of two <= 512");
};

struct TileCoord {
    int m_blk, n_blk;
};

// Grouped raster: tiles are visited in bands of 16 row-blocks, column-block major inside a
// band, so the tiles running concurrently share A and B slabs in L2.
__device__ __forceinline__ TileCoord tile_coord(int t, int m_blocks, int n_blocks) {
    constexpr int kGroup = 16;
    const int band_tiles = kGroup * n_blocks;
    const int band = t / band_tiles;
    const int first_m = band * kGroup;
    const int rows = min(kGroup, m_blocks - first_m);
    const int r = t - band * band_tiles;
    TileCoord c;
    c.m_blk = first_m + r % rows;
    c.n_blk = r / rows;
    return c;
}

// EPI: 0 = raw s32 output, 1 = fp16 dequant (+ optional bias),
//      2 = gated: the B tile is 128 rows of a gate weight followed by the same 128 rows of an up
//          weight (tm_b / tm_b2), so accumulator columns c and 128 + c belong to output column c of
//          the same token; the epilogue writes fp16(SiLU(g) * u) with g, u dequantised in fp32.
template <int BN, int EPI, int KA>
__global__ void __launch_bounds__((DenseCfg<BN, KA>::kThreads), 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_c,
                  const float* __restrict__ act_scale, const __half* __restrict__ w_scale,
                  const __half* __restrict__ bias, const __half* __restrict__ w_scale2,
                  const __half* __restrict__ bias2, void* __restrict__ out, int M, int N, int K, int a_rows,
                  int* __restrict__ status) {
    // a_rows: rows of the A slab a TMA load fetches (128; 32 or 64 when M is that small: the other rows of
    // the 128-row MMA operand keep whatever the buffer holds - their accumulator lanes are never stored)
    using Cfg = DenseCfg<BN, KA>;
    extern __shared__ __align__(1024) uint8_t smem[];

    uint8_t* smem_ab = smem;
    uint8_t* smem_epi = smem + Cfg::kStages * Cfg::kStageBytes;
    __half* smem_scale = reinterpret_cast<__half*>(smem_epi + Cfg::kEpiBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_epi + Cfg::kEpiBytes + Cfg::kScaleBytes);
    uint64_t* full_bar = bars;                         // [kStages]
    uint64_t* empty_bar = bars + Cfg::kStages;         // [kStages]
    uint64_t* tmem_full = bars + 2 * Cfg::kStages;     // [2]
    uint64_t* tmem_empty = tmem_full + 2;              // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts need a 1024-byte aligned base
        if (threadIdx.x == 0) atomicExch(status, 100);
        return;
    }

    const int m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
    constexpr int TILE_N = (EPI == 2) ? BN / 2 : BN;   // output columns per tile
    const int n_blocks = (N + TILE_N - 1) / TILE_N;
    const int num_tiles = m_blocks * n_blocks;
    const int num_kb = (K + BLOCK_K * KA - 1) / (BLOCK_K * KA);

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp_id == 0 && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        if (EPI == 2) prefetch_tensormap(&tm_b2);
        prefetch_tensormap(&tm_c);
    }
    if (warp_id == 1) {
        tmem_alloc(tmem_base_slot, Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    constexpr int kBWarp = Cfg::kThreads / 32 - 1;   // KA 2: the warp that issues the B (weight) loads
    if (warp_id == 0 || (KA == 2 && warp_id == kBWarp)) {
        // ------------------------------------------------------------------ TMA producer(s)
        const bool loads_a = (warp_id == 0);
        const bool loads_b = (KA == 1) || (warp_id == kBWarp);
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // launched behind the quantizer of the same linear call (launch_behind_quantizer): the
            // set-up above ran under that kernel's tail; A is its output (the weights are not)
            if (loads_a) griddep_wait();
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const TileCoord tc = tile_coord(t, m_blocks, n_blocks);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
                        atomicExch(status, 101);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem_ab + stage * Cfg::kStageBytes;
                    uint8_t* sb = sa + Cfg::kABytes;
                    if (loads_a) {
                        // the arming thread: bytes of every load of the stage (A atoms of a_rows rows, B atoms)
                        mbar_expect_tx(&full_bar[stage], KA * (a_rows * BLOCK_K + BN * BLOCK_K));
#pragma unroll
                        for (int j = 0; j < KA; j++)
                            tma_load_2d(sa + j * (BLOCK_M * BLOCK_K), &tm_a, &full_bar[stage], (kb * KA + j) * BLOCK_K,
                                        tc.m_blk * BLOCK_M);
                    }
                    if (loads_b) {
                        if (EPI == 2) {
                            tma_load_2d(sb, &tm_b, &full_bar[stage], kb * BLOCK_K, tc.n_blk * TILE_N);
                            tma_load_2d(sb + Cfg::kBBytes / 2, &tm_b2, &full_bar[stage], kb * BLOCK_K, tc.n_blk * TILE_N);
                        } else {
#pragma unroll
                            for (int j = 0; j < KA; j++)
                                tma_load_2d(sb + j * (BN * BLOCK_K), &tm_b, &full_bar[stage], (kb * KA + j) * BLOCK_K,
                                            tc.n_blk * BN);
                        }
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp_id == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(BLOCK_M, BN, false);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, local++) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag)) {
                    atomicExch(status, 102);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + buf * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        atomicExch(status, 103);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_ab + stage * Cfg::kStageBytes);
#pragma unroll
                    for (int j = 0; j < KA; j++) {
                        const uint64_t desc_a = make_desc_sw128(sa + j * (BLOCK_M * BLOCK_K));
                        const uint64_t desc_b = make_desc_sw128(sa + Cfg::kABytes + j * (BN * BLOCK_K));
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; k++) {
                            // advancing the start address by 32 bytes (>>4 = 2) steps one UMMA_K inside the atom
                            umma_i8(tmem_acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | j | k) != 0 ? 1u : 0u);
                        }
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
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp_id & 3;               // TMEM lane quarter this warp may read
        const int epi_tid = (warp_id - 2) * 32 + lane;
        uint8_t* my_stage = smem_epi + (warp_id - 2) * Cfg::kEpiBufs * kEpiBufBytes;
        constexpr int CH = (EPI == 0) ? 32 : 64;   // output columns per 128-byte staged row
        const bool has_bias = (bias != nullptr);
        int local = 0;
        int sbuf = 0;
        griddep_wait();   // the token scales are that kernel's output too
        // After a failed wait this warp keeps walking its tiles without touching TMEM, so it
        // still meets the other epilogue warps at every named barrier.
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, local++) {
            const TileCoord tc = tile_coord(t, m_blocks, n_blocks);
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int row = tc.m_blk * BLOCK_M + q * 32 + lane;
            const int n0 = tc.n_blk * TILE_N;
            // EPI 1: [w_scale BN][bias BN]; EPI 2: [gate scale][gate bias][up scale][up bias], TILE_N each
            __half* s_ws = smem_scale + buf * 2 * BN;
            __half* s_bias = s_ws + TILE_N;
            __half* s_ws2 = s_bias + TILE_N;
            __half* s_bias2 = s_ws2 + TILE_N;
            float as = 0.f;
            if (EPI != 0) {
                if (ok) {
                    for (int i = epi_tid; i < TILE_N; i += kEpiWarps * 32) {
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
                named_barrier_sync(1, kEpiWarps * 32);
            }
            if (ok) {
                // warp-uniform outcome: the TMEM loads below are .sync.aligned
                ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], acc_phase, abort_flag));
                if (!ok) atomicExch(status, 104);
            }
            if (!ok) continue;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int c = 0; c < TILE_N / CH; c++) {
                uint32_t packed[32];
                if (EPI == 0) {
                    tmem_ld_32x32b_x32(taddr + c * CH, packed);
                    tmem_ld_wait();
                } else if (EPI == 1) {
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
                } else {
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
                }
                uint8_t* stg = my_stage + sbuf * kEpiBufBytes;
                // the TMA store that last read this buffer must be done with it
                if (lane == 0) tma_store_wait_read<Cfg::kEpiBufs - 1>();
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int chunk = j ^ (lane & 7);   // 128B swizzle: 16-byte chunk index XOR row%8
                    *reinterpret_cast<uint4*>(stg + lane * 128 + chunk * 16) =
                        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tm_c, stg, n0 + c * CH, tc.m_blk * BLOCK_M + q * 32);
                    tma_store_commit();
                }
                sbuf = (sbuf + 1) % Cfg::kEpiBufs;
            }
            // Tile widths that are not a multiple of the staged chunk (BN = 80, 96, 112: chosen so that a
            // few-token call's tiles fit one wave) end in 16-column pieces written with plain stores.
            if constexpr (EPI != 2 && TILE_N % CH != 0) {
#pragma unroll 1
                for (int col = (TILE_N / CH) * CH; col < TILE_N; col += 16) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(taddr + col, v);
                    tmem_ld_wait();
                    const int n = n0 + col;
                    if (row < M && n < N) {   // N % 16 == 0 on this path: a piece is inside or outside as a whole
                        if (EPI == 0) {
                            int4* dst = reinterpret_cast<int4*>(static_cast<int32_t*>(out) + (size_t)row * N + n);
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                dst[i] = make_int4((int)v[4 * i], (int)v[4 * i + 1], (int)v[4 * i + 2], (int)v[4 * i + 3]);
                        } else {
                            uint32_t h[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const float2 w = __half22float2(reinterpret_cast<const __half2*>(s_ws + col)[i]);
                                const float2 b = __half22float2(reinterpret_cast<const __half2*>(s_bias + col)[i]);
                                h[i] = pack_half2(
                                    dequant_gemm(static_cast<int>(v[2 * i]), mul_ftz(as, w.x), b.x, has_bias),
                                    dequant_gemm(static_cast<int>(v[2 * i + 1]), mul_ftz(as, w.y), b.y, has_bias));
                            }
                            uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(out) + (size_t)row * N + n);
                            dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
                            dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
                        }
                    }
                }
            }
            // accumulator fully read: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        if (lane == 0) tma_store_wait_all<0>();
    }

    // ---------------------------------------------------------------------- teardown
    if (*abort_flag != 0) {
        // give loads still in flight time to land before the CTA's shared memory is released
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

// Plain-CUDA kernel for shapes the TMA path cannot describe (K or N not a multiple of the
// 16-byte TMA stride granule, misaligned base pointers). One thread per output element.
template <int EPI>
__global__ void dense_gemm_ragged_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B,
                                         const float* __restrict__ act_scale, const __half* __restrict__ w_scale,
                                         const __half* __restrict__ bias, void* __restrict__ out, int M, int N,
                                         int K) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N) return;
    const int m = (int)(idx / N), n = (int)(idx % N);
    const int8_t* a = A + (size_t)m * K;
    const int8_t* b = B + (size_t)n * K;
    int acc = 0;
    for (int k = 0; k < K; k++) acc += (int)a[k] * (int)b[k];
    if (EPI == 0) {
        reinterpret_cast<int32_t*>(out)[idx] = acc;
    } else {
        const float s = mul_ftz(act_scale[m], __half2float(w_scale[n]));
        const float o = dequant_gemm(acc, s, bias ? __half2float(bias[n]) : 0.f, bias != nullptr);
        reinterpret_cast<__half*>(out)[idx] = __float2half_rn(o);
    }
}

template <int BN, int EPI, int KA = 1>
int launch_dense(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale, const __half* bias,
                 void* out, int M, int K, int N, cudaStream_t stream, const int8_t* B2 = nullptr,
                 const __half* w_scale2 = nullptr, const __half* bias2 = nullptr) {
    using Cfg = DenseCfg<BN, KA>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = dense_gemm_kernel<BN, EPI, KA>;
    if (!attr_set[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = true;
    }
    constexpr int TILE_N = (EPI == 2) ? BN / 2 : BN;
    const int a_rows = (EPI != 2 && M <= 32) ? 32 : ((EPI != 2 && M <= 64) ? 64 : BLOCK_M);
    CUtensorMap tm_a, tm_b, tm_b2, tm_c;
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {BLOCK_K, (uint32_t)a_rows};
        if (!make_tmap(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
        const uint64_t str[1] = {(uint64_t)K};
        const uint32_t box[2] = {BLOCK_K, TILE_N};
        if (!make_tmap(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, B, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
        if (!make_tmap(&tm_b2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (EPI == 2) ? B2 : B, dims, str, box,
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
    const int m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
    const int n_blocks = (N + TILE_N - 1) / TILE_N;
    const long long tiles = (long long)m_blocks * n_blocks;
    const int grid = (int)std::min<long long>(tiles, sm_count());
    return launch_gemm(kern, dim3(grid), dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tm_a, tm_b, tm_b2, tm_c, act_scale,
                       w_scale, bias, w_scale2, bias2, out, M, N, K, a_rows, status) == cudaSuccess
               ? kOk
               : kLaunchFailed;
}

template <int EPI>
int dense_dispatch(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                   const __half* bias, void* out, int M, int K, int N, cudaStream_t stream, int force_bn) {
    if (M <= 0 || K <= 0 || N <= 0) return kOk;   // reference: silent no-op (int8_dense.cu:195)
    if (A == nullptr || B == nullptr || out == nullptr) return kBadPointer;
    if (EPI == 1 && (act_scale == nullptr || w_scale == nullptr)) return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    // very few tokens: one pass over the weights on the CUDA cores (dense_gemv.cu)
    if (force_bn == 0 && dense_gemv_fits(M, K, B, A))
        return dense_gemv(B, A, act_scale, w_scale, bias, out, M, K, N, stream, EPI);
    const int out_esz = (EPI == 0) ? 4 : 2;
    const bool tma_ok = (K % 16 == 0) && ((long long)N * out_esz % 16 == 0) && aligned16(A) && aligned16(B) &&
                        aligned16(out);
    if (!tma_ok) {
        const long long total = (long long)M * N;
        const int block = 256;
        const long long grid = (total + block - 1) / block;
        dense_gemm_ragged_kernel<EPI><<<(unsigned)grid, block, 0, stream>>>(A, B, act_scale, w_scale, bias, out, M,
                                                                           N, K);
        return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
    }
    // The CTA-pair kernel (256 x 256 outputs per pair of SMs; knob 512) once there are enough such
    // tiles for every SM pair: measured 7 % faster than 128 x 256 tiles at 8192^3, burst and sustained.
    const long long pair_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    // (not for a single block of token rows: half of every 256-row pair tile would be empty - N = 28672, K = 8192,
    // 64 tokens: 66.6 us against 62.5 us with 128 x 128 tiles)
    if (force_bn == 512 || (force_bn == 0 && pair_tiles >= sm_count() / 2 && K >= 512 && M > BLOCK_M)) {
        const int r = (EPI == 0) ? dense_pair_s32(A, B, static_cast<int32_t*>(out), M, K, N, stream)
                                 : dense_pair_dequant(A, B, act_scale, w_scale, bias, static_cast<__half*>(out), M,
                                                      K, N, stream);
        if (r >= 0) return r;
    }
    // Tile width: the widest tile that still gives every SM work.
    int bn = force_bn;
    if ((bn == 80 || bn == 96 || bn == 112) && N % 16 != 0) bn = 64;   // the narrow widths end in 16-column pieces
    if (bn != 64 && bn != 80 && bn != 96 && bn != 112 && bn != 128 && bn != 256) {
        const long long m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
        const int sms = sm_count();
        if (m_blocks * ((N + 255) / 256) * 5 >= sms * 3) bn = 256;   // >= 60 % of the SMs busy: wide tiles still win
        else if (m_blocks * ((N + 127) / 128) >= sms) bn = 128;
        else bn = 64;
    }
    // One block of token rows (M <= 128): the call is a pass over the weights and its time is that of the SM with
    // the most weight columns - 11008 columns in 64-wide tiles are 172 tiles, two waves on 148 SMs. Tile widths in
    // steps of 16 columns: take the narrowest width whose tiles fit one wave, if that beats the default's waves x width
    // (N = 28672, K = 8192, 64 tokens: two waves of 128 measured 6 % faster than two of 112).
    if (force_bn == 0 && bn <= 128 && M <= BLOCK_M && N % 16 == 0) {
        const int sms = sm_count();
        int best = bn, best_cost = ((N + bn - 1) / bn + sms - 1) / sms * bn;
        for (int w = 64; w <= 128; w += 16) {
            if ((N + w - 1) / w > sms) continue;   // only widths that fit one wave (with more, the model is too coarse)
            if (w < best_cost) {
                best = w;
                best_cost = w;
            }
        }
        bn = best;
    }
    // One block of token rows in 64-column tiles: stages of two K atoms and a second producer thread (DenseCfg),
    // four stages deep. N = 4096, K = 14336, 16-128 tokens: 31.4 -> 24.0-24.9 us; N = K = 4096: 12.0 -> 10.2 us.
    // The wider tiles have room for three such stages only and gain nothing (80 columns, N = 11008, K = 4096:
    // 13.4 -> 13.4 us at 16 tokens, 13.8 -> 14.2 us at 128). Knob 10 = 1 keeps the one-atom form for comparison.
    if (M <= BLOCK_M && bn == 64 && tuning_knob(kKnobDenseOneAtom) == 0)
        return launch_dense<64, EPI, 2>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    switch (bn) {
    case 256: return launch_dense<256, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    case 128: return launch_dense<128, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    case 112: return launch_dense<112, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    case 96:  return launch_dense<96, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    case 80:  return launch_dense<80, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    default:  return launch_dense<64, EPI>(A, B, act_scale, w_scale, bias, out, M, K, N, stream);
    }
}

}  // namespace

int dense_gemm_s32(const int8_t* A, const int8_t* B, int32_t* out, int M, int K, int N, cudaStream_t stream,
                   int force_bn) {
    return dense_dispatch<0>(A, B, nullptr, nullptr, nullptr, out, M, K, N, stream, force_bn);
}

int dense_gemm_dequant(const int8_t* A, const int8_t* B, const float* act_scale, const __half* w_scale,
                       const __half* bias, __half* out, int M, int K, int N, cudaStream_t stream, int force_bn) {
    return dense_dispatch<1>(A, B, act_scale, w_scale, bias, out, M, K, N, stream, force_bn);
}

int dense_gemm_gated(const int8_t* A, const int8_t* Wg, const int8_t* Wu, const float* act_scale,
                     const __half* wg_scale, const __half* wu_scale, const __half* bg, const __half* bu, __half* out,
                     int M, int K, int N, cudaStream_t stream) {
    if (M <= 0 || K <= 0 || N <= 0) return kOk;
    if (A == nullptr || Wg == nullptr || Wu == nullptr || act_scale == nullptr || wg_scale == nullptr ||
        wu_scale == nullptr || out == nullptr)
        return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    // TMA path only: K a multiple of 16, N a multiple of 8, 16-byte aligned operands
    if (K % 16 != 0 || N % 8 != 0 || !aligned16(A) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(out))
        return kBadShape;
    // CTA-pair kernel (256 tokens x 128 output columns per pair of SMs; dense tile knob 512 forces it, any other
    // forced tile keeps the single-CTA kernel) once every pair has a tile
    const int force_bn = tuning_knob(kKnobDenseTile);
    const long long pair_tiles = (long long)((M + 255) / 256) * ((N + 127) / 128);
    if (force_bn == 512 || (force_bn == 0 && pair_tiles >= sm_count() / 2 && K >= 512)) {
        const int r = dense_pair_gated(A, Wg, Wu, act_scale, wg_scale, wu_scale, bg, bu, out, M, K, N, stream);
        if (r >= 0) return r;
    }
    return launch_dense<256, 2>(A, Wg, act_scale, wg_scale, bg, out, M, K, N, stream, Wu, wu_scale, bu);
}

}  // namespace fb200
