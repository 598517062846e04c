// Built-in ceiling probes (internal, see tuning.h): two small kernels that measure, on the device the
// library runs on, the two rates that bound the GEMM kernels - so that a benchmark can state its
// roofline denominators from this GPU instead of from a data sheet.
//
//   mma rate    one thread issues a long run of tcgen05.mma kind::i8 instructions (dense K=32 or
//               2:4-sparse K=64; one CTA with M=128 or a CTA pair with M=256) on operands that stay in
//               shared memory, optionally with the per-stage tcgen05.commit of the real kernels, and
//               reports clocks per instruction. Nothing is loaded or stored: this is the tensor pipe's
//               own rate, the upper bound of any kernel built from these instructions.
//   tma ingest  every CTA streams 128 x 128-byte tiles of one L2-resident matrix through a ring of
//               shared-memory stages with up to four TMA-issuing threads and reports bytes per clock:
//               what the L2 -> SM path delivers to one SM when `ctas` SMs pull at once.
//
// Every wait is bounded; the probes touch only their own buffers.
#include "../../include/forge_b200.h"
#include "common.cuh"
#include "gemm_dense.cuh"
#include "ptx.cuh"
#include "tuning.h"

namespace fb200 {

using namespace ptx;

namespace {

constexpr int kMmaStages = 2;
constexpr int kMmaStageBytes = 80 * 1024;   // A 16 KB | B: two 128-byte-wide atoms of up to 256 rows

// out[0] = clocks from the first issue to the completion of the last instruction.
// COMMITS is a compile-time parameter on purpose: a run-time branch around the commits changed the code of
// the issue loop enough to double the measured clocks per instruction.
template <int PAIR, int COMMITS>
__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int n, int sparse, int iters, unsigned long long* out, int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t done_bar;
    __shared__ uint64_t stage_bar[kMmaStages];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;
    for (int i = threadIdx.x; i < kMmaStages * kMmaStageBytes / 4; i += blockDim.x) {
        uint32_t v = 0x44444444u;   // as metadata: valid 2:4 nibbles (positions 0 and 1)
        if (i >= 1024) {            // operands: pseudo-random bytes (the first 4 KB stay valid metadata)
            v = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
            v ^= v >> 15; v *= 2246822519u; v ^= v >> 13; v *= 3266489917u; v ^= v >> 16;
        }
        reinterpret_cast<uint32_t*>(smem)[i] = v;
    }
    if (threadIdx.x == 0) {
        mbar_init(&done_bar, 1);
        for (int s = 0; s < kMmaStages; s++) mbar_init(&stage_bar[s], 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(&tmem_slot, 512); tmem_relinquish_pair(); }
        else { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0 && lane == 0 && rank == 0) {
        if (sparse) {   // metadata columns 480.. from the first 4 KB of shared memory
            for (int c = 0; c < kMmaStages; c++) {
                const uint64_t d = make_desc_noswizzle(smem_u32(smem), 2048, 128);
                if (PAIR) tmem_cp_128x256b_pair(tmem_base + 480 + 8 * c, d);
                else tmem_cp_128x256b(tmem_base + 480 + 8 * c, d);
            }
        }
        const uint32_t idesc = make_idesc_i8(PAIR ? 256 : 128, n, sparse != 0);
        const uint32_t b_atom = (PAIR ? n / 2 : n) * 128;
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            const int stage = (i >> 2) % kMmaStages;
            const int j = i & 3;
            const uint32_t sa = smem_u32(smem + stage * kMmaStageBytes);
            const uint32_t sb = sa + 16384;
            const uint32_t acc = tmem_base + ((i >> 7) & 1) * (n <= 224 ? n : 0);
            const uint64_t desc_a = make_desc_sw128(sa) + 2 * j;
            if (sparse) {
                const uint64_t desc_b = make_desc_sw128(sb + (j >> 1) * b_atom) + 4 * (j & 1);
                if (PAIR) umma_i8_sp_pair(acc, desc_a, desc_b, tmem_base + 480 + 8 * stage + 2 * j, idesc, 1u);
                else umma_i8_sp(acc, desc_a, desc_b, tmem_base + 480 + 8 * stage + 2 * j, idesc, 1u);
            } else {
                const uint64_t desc_b = make_desc_sw128(sb) + 2 * j;
                if (PAIR) umma_i8_pair(acc, desc_a, desc_b, idesc, 1u);
                else umma_i8(acc, desc_a, desc_b, idesc, 1u);
            }
            if (j == 3 && COMMITS > 0) {   // the per-stage commits of the GEMM kernels
                if (PAIR) {
                    if (COMMITS == 1) tc_commit_pair_mask(smem_u32(&stage_bar[stage]), 3);
                    else { tc_commit_pair(mapa_shared(smem_u32(&stage_bar[stage]), 0)); tc_commit_pair(mapa_shared(smem_u32(&stage_bar[stage]), 1)); }
                } else {
                    tc_commit(&stage_bar[stage]);
                }
            }
        }
        if (PAIR) tc_commit_pair(mapa_shared(smem_u32(&done_bar), 0)); else tc_commit(&done_bar);
        if (!mbar_wait(&done_bar, 0, &abort_flag)) atomicExch(status, 901);
        if (blockIdx.x == 0) out[0] = (unsigned long long)(clock64() - t0);
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
    }
}

constexpr int kRingBytes = 192 * 1024;
constexpr int kBox = 128 * 128;

// out[cta] = clocks the CTA needed for `iters` tiles per producer.
__global__ void __launch_bounds__(256, 1)
tma_ingest_kernel(const __grid_constant__ CUtensorMap tm, int rows, int kcols, int iters, int producers,
                  unsigned long long* out, int* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t full[64], empty[64];
    __shared__ int abort_flag;
    const int stages = (kRingBytes / producers) / kBox;   // per producer
    if (threadIdx.x == 0) {
        for (int s = 0; s < 64; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane != 0) return;
    if (warp < producers) {
        int stage = 0; uint32_t phase = 0;
        uint8_t* ring = smem + warp * (kRingBytes / producers);
        int cx = 0, cy = (int)(((blockIdx.x * producers + warp) * 37) % (rows / 128)) * 128;
        for (int i = 0; i < iters; i++) {
            if (!mbar_wait(&empty[warp * 16 + stage], phase ^ 1, &abort_flag)) { atomicExch(status, 902); break; }
            mbar_expect_tx(&full[warp * 16 + stage], kBox);
            tma_load_2d(ring + stage * kBox, &tm, &full[warp * 16 + stage], cx, cy);
            cx += 128;
            if (cx >= kcols) { cx = 0; cy += 128; if (cy >= rows) cy = 0; }
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
    } else if (warp >= 4 && warp < 4 + producers) {
        const int w = warp - 4;
        const long long t0 = clock64();
        int stage = 0; uint32_t phase = 0;
        for (int i = 0; i < iters; i++) {
            if (!mbar_wait(&full[w * 16 + stage], phase, &abort_flag)) { atomicExch(status, 903); break; }
            mbar_arrive(&empty[w * 16 + stage]);
            if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (w == 0) out[blockIdx.x] = (unsigned long long)(clock64() - t0);
    }
}

// Result buffer of the probes: a file-scope device array (nothing is allocated).
__device__ unsigned long long g_probe_out[256];

unsigned long long* probe_buffer() {
    static unsigned long long* buf[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (buf[dev & 63] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_probe_out) != cudaSuccess) return nullptr;
        buf[dev & 63] = static_cast<unsigned long long*>(p);
    }
    return buf[dev & 63];
}

}  // namespace

}  // namespace fb200

extern "C" {

// Clocks per instruction, or a negative status. Synchronises the device.
double forge_b200_probe_mma_rate(int pair, int n, int sparse, int commits, int ctas) {
    using namespace fb200;
    if (!device_is_sm100()) return -FORGE_B200_UNSUPPORTED_ARCH;
    if (n < 16 || n > 256 || n % 16 != 0 || ctas < 1 || commits < 0 || commits > 2) return -FORGE_B200_BAD_SHAPE;
    unsigned long long* out = probe_buffer();
    int* status = status_word();
    if (out == nullptr || status == nullptr) return -FORGE_B200_LAUNCH_FAILED;
    const int iters = 8192;
    const int smem = kMmaStages * kMmaStageBytes;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pair ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    if (pair) ctas = (ctas + 1) & ~1;
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaErrorInvalidValue;
#define FB200_RATE(P, C)                                                                                  \
    if ((pair != 0) == (P != 0) && commits == C) {                                                        \
        cudaFuncSetAttribute(mma_rate_kernel<P, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);   \
        e = cudaLaunchKernelEx(&cfg, mma_rate_kernel<P, C>, n, sparse, iters, out, status);               \
    }
    FB200_RATE(0, 0) FB200_RATE(0, 1) FB200_RATE(0, 2) FB200_RATE(1, 0) FB200_RATE(1, 1) FB200_RATE(1, 2)
#undef FB200_RATE
    if (e != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return -FORGE_B200_LAUNCH_FAILED;
    unsigned long long clocks = 0;
    if (cudaMemcpy(&clocks, out, sizeof(clocks), cudaMemcpyDeviceToHost) != cudaSuccess) return -FORGE_B200_LAUNCH_FAILED;
    return (double)clocks / iters;
}

// Mean bytes per clock and CTA over `ctas` CTAs streaming tiles of `matrix` (rows x kcols int8, 16-byte
// aligned, kcols % 128 == 0, rows % 128 == 0) with `producers` (1, 2 or 4) TMA-issuing threads each.
double forge_b200_probe_tma_ingest(const void* matrix, int rows, int kcols, int producers, int ctas) {
    using namespace fb200;
    if (!device_is_sm100()) return -FORGE_B200_UNSUPPORTED_ARCH;
    if (matrix == nullptr || rows < 128 || rows % 128 != 0 || kcols < 128 || kcols % 128 != 0 ||
        (producers != 1 && producers != 2 && producers != 4) || ctas < 1 || ctas > 256)
        return -FORGE_B200_BAD_SHAPE;
    unsigned long long* out = probe_buffer();
    int* status = status_word();
    if (out == nullptr || status == nullptr) return -FORGE_B200_LAUNCH_FAILED;
    CUtensorMap tm;
    const uint64_t dims[2] = {(uint64_t)kcols, (uint64_t)rows};
    const uint64_t str[1] = {(uint64_t)kcols};
    const uint32_t box[2] = {128, 128};
    if (!make_tmap(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, matrix, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return -FORGE_B200_LAUNCH_FAILED;
    cudaFuncSetAttribute(tma_ingest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    const int iters = (32 << 20) / kBox / producers;   // 32 MB per CTA
    tma_ingest_kernel<<<ctas, 256, kRingBytes>>>(tm, rows, kcols, iters, producers, out, status);
    if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return -FORGE_B200_LAUNCH_FAILED;
    unsigned long long clocks[256];
    if (cudaMemcpy(clocks, out, sizeof(unsigned long long) * ctas, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -FORGE_B200_LAUNCH_FAILED;
    double sum = 0;
    for (int i = 0; i < ctas; i++) sum += (double)clocks[i];
    return (double)iters * producers * kBox / (sum / ctas);
}

}  // extern "C"
