// Fused per-token quantize + 2:4-sparse INT8 GEMM + dequant for sm_100a: the FP16 activation is
// read once and its INT8 copy never goes to global memory.
//
// Replaces the reference's sparse_gemm_fq_kernel path of forge::gemm::sparse_int8_linear
// (src/gemm/int8_sparse.cu:258-333, 723-736, 833-850; K <= 1280). Output is bit-identical to the
// two-pass path: the quantizer arithmetic is the standalone kernel's, the GEMM and epilogue are
// the sparse kernel's.
//
// Each persistent CTA walks blocks of 64 tokens. Sixteen quantizer warps turn a block's FP16 rows
// (whole row in registers, 16-byte loads, warp-shuffle absmax) into INT8 written straight into
// shared memory in the layout the tensor core reads - K-major atoms of 64 rows x 128 bytes with
// the 128-byte swizzle - and leave the per-token scales in shared memory. There are two such block
// buffers: while the MMA thread runs every 128-row weight tile against one block (compressed
// weights and metadata stream through a 3-stage TMA ring), the quantizer warps are already
// fetching and converting the next one, so the kernel is paced by the one pass over the FP16
// activation. A thread of its own moves each stage's metadata into tensor memory; four epilogue
// warps drain the double-buffered accumulator with the transposed direct-store epilogue of the
// sparse kernel.
#include "common.cuh"
#include "ptx.cuh"
#include "gemm_dense.cuh"
#include "gemm_fq.cuh"
#include "sparse_epilogue.cuh"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int BT = 64;                  // tokens per block (UMMA N)
constexpr int BW = 128;                 // weight rows per tile (UMMA M)
constexpr int kMaxK = 1280;             // a block: up to 10 atoms of 8 KB, two blocks resident
constexpr int kEpiWarps = 4;
constexpr int kQuantWarps = 16;
constexpr int kRowsPerQuantWarp = BT / kQuantWarps;
// warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-21 quantizers, warp 22 metadata copies
constexpr int kFirstQuantWarp = 2 + kEpiWarps;
constexpr int kCopyWarp = kFirstQuantWarp + kQuantWarps;
constexpr int kThreads = 32 * (kCopyWarp + 1);
constexpr int kStages = 3;
constexpr int kABytes = BW * 128;
constexpr int kMetaBytes = BW * 32;
constexpr int kStageBytes = kABytes + kMetaBytes;    // 20 KB
constexpr int kAtomBytes = BT * 128;                 // 8 KB
constexpr int kScaleSlots = 2;                       // per-token scales, one set per block buffer
constexpr int kScaleBytes = kScaleSlots * BT * (int)sizeof(float);
constexpr int kBarBytes = 320;
constexpr int kAccCols = 2 * BT;
constexpr int kTmemCols = 256;                       // 128 accumulator + 24 metadata columns
constexpr int kChunksPerLane = 3;                    // 16-value chunks per lane per row: K <= 3*32*16

inline int fq_smem_bytes(int K) {
    return 2 * (K / 128) * kAtomBytes + kStages * kStageBytes + kScaleBytes + kBarBytes;
}
static_assert(2 * (kMaxK / 128) * kAtomBytes + kStages * kStageBytes + kScaleBytes + kBarBytes <= 232448,
              "exceeds the 227 KB shared memory limit");

__global__ void __launch_bounds__(kThreads, 1)
sparse_fq_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_meta,
                 const __half* __restrict__ x, __half* __restrict__ out, const __half* __restrict__ w_scale,
                 const __half* __restrict__ bias, int M, int N_out, int K, int stream_x, int* __restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int n_atoms = K / 128;
    const int block_bytes = n_atoms * kAtomBytes;
    uint8_t* smem_b = smem;                                   // two resident int8 token blocks
    uint8_t* smem_stage = smem + 2 * block_bytes;             // weight + metadata ring
    float* smem_as = reinterpret_cast<float*>(smem_stage + kStages * kStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(smem_as) + kScaleBytes);
    uint64_t* full_bar = bars;                  // [kStages] weights of the stage have landed
    uint64_t* empty_bar = full_bar + kStages;   // [kStages]
    uint64_t* meta_full = empty_bar + kStages;  // [kStages] metadata of the stage has landed
    uint64_t* meta_ready = meta_full + kStages; // [kStages] ... is in tensor memory and the weights have landed
    uint64_t* tmem_full = meta_ready + kStages; // [2]
    uint64_t* tmem_empty = tmem_full + 2;       // [2]
    uint64_t* b_full = tmem_empty + 2;          // [2] the token block is quantized and resident
    uint64_t* b_empty = b_full + 2;             // [2] every MMA that reads the block has completed and the
                                                //     epilogue warps have read its scales for the last time
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(b_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp_id = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if ((smem_u32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(status, 500);
        return;
    }

    const int w_blocks = (N_out + BW - 1) / BW;
    const int t_blocks = (M + BT - 1) / BT;
    const int num_kb = (K + 255) / 256;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
            mbar_init(&meta_full[s], 1);
            mbar_init(&meta_ready[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiWarps);
            mbar_init(&b_full[b], kQuantWarps);
            mbar_init(&b_empty[b], 1 + kEpiWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp_id == 0 && lane == 0) {
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_meta);
    }
    if (warp_id == 1) {
        tmem_alloc(tmem_base_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const uint32_t tmem_meta = tmem_base + kAccCols;

    if (warp_id == 0) {
        // ------------------------------------------------------------------ TMA producer: weights + metadata
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tb = blockIdx.x; tb < t_blocks && ok; tb += gridDim.x) {
                for (int wb = 0; wb < w_blocks && ok; wb++) {
                    for (int kb = 0; kb < num_kb; kb++) {
                        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) {
                            atomicExch(status, 501);
                            ok = false;
                            break;
                        }
                        uint8_t* sa = smem_stage + stage * kStageBytes;
                        mbar_expect_tx(&meta_full[stage], kMetaBytes);
                        mbar_expect_tx(&full_bar[stage], kABytes);
                        tma_load_3d(sa + kABytes, &tm_meta, &meta_full[stage], 0, wb * BW, kb * 2);
                        tma_load_2d(sa, &tm_w, &full_bar[stage], kb * 128, wb * BW);
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp_id == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(BW, BT, true);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;       // tiles issued by this CTA (accumulator buffer / phase)
            int blocks = 0;      // token blocks started (block buffer / phase)
            bool ok = true;
            for (int tb = blockIdx.x; tb < t_blocks && ok; tb += gridDim.x, blocks++) {
                const int bbuf = blocks & 1;
                if (!mbar_wait(&b_full[bbuf], (blocks >> 1) & 1, abort_flag)) {
                    atomicExch(status, 505);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sb0 = smem_u32(smem_b) + bbuf * block_bytes;
                for (int wb = 0; wb < w_blocks && ok; wb++, local++) {
                    const int buf = local & 1;
                    const uint32_t acc_phase = (local >> 1) & 1;
                    if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag)) {
                        atomicExch(status, 502);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tmem_acc = tmem_base + buf * BT;
                    for (int kb = 0; kb < num_kb; kb++) {
                        if (!mbar_wait(&meta_ready[stage], phase, abort_flag)) {
                            atomicExch(status, 503);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sa = smem_u32(smem_stage + stage * kStageBytes);
                        const uint32_t te = tmem_meta + 8 * stage;
                        const uint64_t desc_a = make_desc_sw128(sa);
                        const uint32_t sb = sb0 + (2 * kb) * kAtomBytes;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            // a K tail of 128 (odd atom count) reads one atom past the block for j >= 2 (the other
                            // block buffer or the weight ring: finite int8 bytes); the weights and metadata of that
                            // half are TMA zero fill, so it adds nothing
                            const uint64_t desc_b = make_desc_sw128(sb + (j >> 1) * kAtomBytes) + 4 * (j & 1);
                            umma_i8_sp(tmem_acc, desc_a + 2 * j, desc_b, te + 2 * j, idesc, (kb | j) != 0 ? 1u : 0u);
                        }
                        tc_commit(&empty_bar[stage]);
                        if (++stage == kStages) {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                    if (ok) tc_commit(&tmem_full[buf]);
                }
                if (ok) tc_commit(&b_empty[bbuf]);   // the block buffer may be overwritten
            }
        }
    } else if (warp_id == kCopyWarp) {
        // ------------------------------------------------------------------ metadata copies
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tb = blockIdx.x; tb < t_blocks && ok; tb += gridDim.x) {
                for (int i = 0; i < w_blocks * num_kb; i++) {
                    if (!mbar_wait(&meta_full[stage], phase, abort_flag)) {
                        atomicExch(status, 507);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sm = smem_u32(smem_stage + stage * kStageBytes) + kABytes;
                    tmem_cp_128x256b(tmem_meta + 8 * stage, make_desc_noswizzle(sm, 2048, 128));
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) {
                        atomicExch(status, 508);
                        ok = false;
                        break;
                    }
                    tc_commit(&meta_ready[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp_id >= kFirstQuantWarp) {
        // ------------------------------------------------------------------ quantizers
        const int qw = warp_id - kFirstQuantWarp;  // rows [4*qw, 4*qw+4) of every block
        const int n_chunks = K / 16;               // 16-value chunks per row
        int blocks = 0;
        for (int tb = blockIdx.x; tb < t_blocks; tb += gridDim.x, blocks++) {
            const int m0 = tb * BT;
            const int bbuf = blocks & 1;
            uint8_t* dst_block = smem_b + bbuf * block_bytes;
            float* s_as = smem_as + bbuf * BT;
            bool dead = false;
#pragma unroll 1
            for (int rr = 0; rr < kRowsPerQuantWarp; rr += 2) {
                uint4 v[2][kChunksPerLane][2];
                __half2 hmax[2];
                // every load of the two rows is issued before anything consumes one (a loop that mixed the
                // loads with the running maximum made each load wait for the previous one's use)
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int r = qw * kRowsPerQuantWarp + rr + u;
                    const int row = min(m0 + r, M - 1);
                    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * K);
#pragma unroll
                    for (int i = 0; i < kChunksPerLane; i++) {
                        const int c = lane + 32 * i;
                        const bool live = c < n_chunks;
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            v[u][i][hh] = make_uint4(0u, 0u, 0u, 0u);
                            if (live) v[u][i][hh] = stream_x ? __ldcs(src + 2 * c + hh) : __ldg(src + 2 * c + hh);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    hmax[u] = __float2half2_rn(0.f);
#pragma unroll
                    for (int i = 0; i < kChunksPerLane; i++) {
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            const __half2* h = reinterpret_cast<const __half2*>(&v[u][i][hh]);
#pragma unroll
                            for (int j = 0; j < 4; j++) hmax[u] = __hmax2(hmax[u], __habs2(h[j]));
                        }
                    }
                }
                // the loads above are in flight while this warp waits for the block buffer to be free
                if (rr == 0) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&b_empty[bbuf], ((blocks >> 1) & 1) ^ 1, abort_flag))) {
                        atomicExch(status, 506);
                        dead = true;
                        break;
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    float amax = max_ftz(__low2float(hmax[u]), __high2float(hmax[u]));
                    for (int o = 16; o > 0; o >>= 1) amax = max_ftz(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    float scale, inv;
                    quant_scale(amax, scale, inv);
                    const int r = qw * kRowsPerQuantWarp + rr + u;
                    if (lane == 0) s_as[r] = scale;
#pragma unroll
                    for (int i = 0; i < kChunksPerLane; i++) {
                        const int c = lane + 32 * i;
                        if (c < n_chunks) {
                            uint32_t p[4];
#pragma unroll
                            for (int hh = 0; hh < 2; hh++) {
                                const __half2* h = reinterpret_cast<const __half2*>(&v[u][i][hh]);
                                int q[8];
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    const float2 f = __half22float2(h[j]);
                                    q[2 * j] = cvt_rni_ftz(mul_ftz(f.x, inv));       // clamped by the saturating pack
                                    q[2 * j + 1] = cvt_rni_ftz(mul_ftz(f.y, inv));
                                }
                                p[hh * 2] = pack4_sat(q[0], q[1], q[2], q[3]);
                                p[hh * 2 + 1] = pack4_sat(q[4], q[5], q[6], q[7]);
                            }
                            // chunk c = 16 bytes at k = 16c: atom c/8, 16-byte slot (c%8) ^ (r%8) of row r
                            uint8_t* dst = dst_block + (c >> 3) * kAtomBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                            *reinterpret_cast<uint4*>(dst) = make_uint4(p[0], p[1], p[2], p[3]);
                        }
                    }
                }
            }
            if (dead) break;
            fence_proxy_async_smem();     // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[bbuf]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2-5)
        const int q = warp_id & 3;                 // TMEM lane quarter
        const bool has_bias = (bias != nullptr);
        int local = 0;
        int blocks = 0;
        bool ok = true;
        for (int tb = blockIdx.x; tb < t_blocks && ok; tb += gridDim.x, blocks++) {
            const int m0 = tb * BT;
            const float* s_as = smem_as + (blocks & 1) * BT;
            // the block's scales were written before the quantizers' arrivals on b_full (the quantizers
            // cannot start the block after next in this buffer before this warp's arrival on b_empty below,
            // so the phase waited for here is always the barrier's latest)
            if (!__all_sync(0xffffffffu, mbar_wait(&b_full[blocks & 1], (blocks >> 1) & 1, abort_flag))) {
                atomicExch(status, 509);
                break;
            }
            for (int wb = 0; wb < w_blocks; wb++, local++) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                const int n = wb * BW + q * 32 + lane;
                float ws = 0.f, bs = 0.f;
                if (n < N_out) {
                    ws = __half2float(w_scale[n]);
                    if (has_bias) bs = __half2float(bias[n]);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], acc_phase, abort_flag))) {
                    atomicExch(status, 504);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BT;
#pragma unroll 1
                for (int c = 0; c < BT / 32; c++) {
                    const int m_first = m0 + c * 32;
                    if (m_first >= M) break;
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    const float as_lane = s_as[c * 32 + lane];
                    tmem_ld_wait();
                    store_transposed_chunk<1>(v, out, N_out, M, n, m_first, as_lane, ws, bs, has_bias);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
            if (ok) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&b_empty[blocks & 1]);   // done with this block's scales
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
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

bool sparse_fq_fits(int K, const void* x) { return K > 0 && K % 128 == 0 && K <= kMaxK && aligned16(x); }

int sparse_fq_linear(const __half* x, const int8_t* W_comp, const uint32_t* w_meta, const __half* w_scale,
                     const __half* bias, __half* out, int M, int K, int N_out, cudaStream_t stream) {
    if (M <= 0 || K <= 0 || N_out <= 0) return kOk;
    if (x == nullptr || W_comp == nullptr || w_meta == nullptr || w_scale == nullptr || out == nullptr)
        return kBadPointer;
    if (!device_is_sm100()) return kUnsupportedArch;
    if (!sparse_fq_fits(K, x) || !aligned16(W_comp) || !aligned16(w_meta)) return kBadShape;
    static int attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int smem = fq_smem_bytes(K);
    if (attr_set[dev & 63] < smem) {
        if (cudaFuncSetAttribute(sparse_fq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fq_smem_bytes(kMaxK)) !=
            cudaSuccess)
            return kLaunchFailed;
        attr_set[dev & 63] = fq_smem_bytes(kMaxK);
    }
    CUtensorMap tm_w, tm_meta;
    {
        const uint64_t dims[2] = {(uint64_t)K / 2, (uint64_t)N_out};
        const uint64_t str[1] = {(uint64_t)K / 2};
        const uint32_t box[2] = {128, BW};
        if (!make_tmap(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, W_comp, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return kLaunchFailed;
    }
    {
        const uint64_t dims[3] = {4, (uint64_t)N_out, (uint64_t)K / 128};
        const uint64_t str[2] = {(uint64_t)K / 8, 16};
        const uint32_t box[3] = {4, BW, 2};
        if (!make_tmap(&tm_meta, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w_meta, dims, str, box,
                       CU_TENSOR_MAP_SWIZZLE_NONE))
            return kLaunchFailed;
    }
    int* status = status_word();
    if (status == nullptr) return kLaunchFailed;
    const int t_blocks = (M + BT - 1) / BT;
    const int grid = std::min(t_blocks, sm_count());
    const int stream_x = ((size_t)M * K * 2 > l2_bytes()) ? 1 : 0;
    sparse_fq_kernel<<<grid, kThreads, smem, stream>>>(tm_w, tm_meta, x, out, w_scale, bias, M, N_out, K, stream_x,
                                                       status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace fb200
