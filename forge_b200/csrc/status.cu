// Per-device status word the GEMM kernels write when a bounded wait runs out, the host-side
// getters, and the library's process-wide tuning knobs (internal, see tuning.h).
#include <atomic>

#include "../../include/forge_b200.h"
#include "common.cuh"
#include "gemm_dense.cuh"
#include "gemm_pair.cuh"
#include "ptx.cuh"
#include "tuning.h"

namespace fb200 {

__device__ int g_status_word = 0;

int* status_word() {
    static int* words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    int*& w = words[dev & 63];
    if (w == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        w = static_cast<int*>(p);
    }
    return w;
}

int read_device_status(int reset) {
    int* w = status_word();
    if (w == nullptr) return -1;
    int v = 0;
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (reset && v != 0) cudaMemset(w, 0, sizeof(int));
    return v;
}

namespace {

constexpr int kNumKnobs = 16;
std::atomic<int> g_knobs[kNumKnobs];

// One thread waits on a barrier that nothing signals; the wait gives up after `budget_ns`.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long budget_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !ptx::mbar_wait(&bar, 0, &abort_flag, budget_ns)) atomicExch(status, 900);
}

}  // namespace

void set_tuning_knob(int key, int value) {
    if (key >= 0 && key < kNumKnobs) g_knobs[key].store(value, std::memory_order_relaxed);
}

namespace {
thread_local bool g_behind_quantizer = false;
}
void launch_behind_quantizer(bool on) { g_behind_quantizer = on; }
bool take_behind_quantizer() {
    const int knob = tuning_knob(kKnobDependentLaunch);   // 0: as requested, 1: always, 2: never
    const bool take = knob == 1 || (knob == 0 && g_behind_quantizer);
    g_behind_quantizer = false;
    return take;
}

int tuning_knob(int key) { return (key >= 0 && key < kNumKnobs) ? g_knobs[key].load(std::memory_order_relaxed) : 0; }

}  // namespace fb200

extern "C" {

int forge_b200_device_status_raw(int reset) { return fb200::read_device_status(reset); }

int forge_b200_device_status(int reset) {
    const int v = fb200::read_device_status(reset);
    if (v == 0) return FORGE_B200_OK;
    return v < 0 ? FORGE_B200_LAUNCH_FAILED : FORGE_B200_DEVICE_TIMEOUT;
}

void forge_b200_set_tuning(int key, int value) {
    if (key >= 0 && key < fb200::kNumKnobs) fb200::g_knobs[key].store(value, std::memory_order_relaxed);
}
int forge_b200_get_tuning(int key) { return fb200::tuning_knob(key); }
void forge_b200_set_dense_tile(int bn) { forge_b200_set_tuning(fb200::kKnobDenseTile, bn); }
void forge_b200_set_sparse_tile(int bt) { forge_b200_set_tuning(fb200::kKnobSparseTile, bt); }

int forge_b200_read_probe(unsigned long long* out, int n) { return fb200::read_pair_probe(out, n); }

int forge_b200_selftest_wait_timeout(unsigned budget_us, void* stream) {
    int* status = fb200::status_word();
    if (status == nullptr) return FORGE_B200_LAUNCH_FAILED;
    if (budget_us > 10000u) budget_us = 10000u;
    fb200::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        status, static_cast<unsigned long long>(budget_us) * 1000ull);
    return cudaGetLastError() == cudaSuccess ? FORGE_B200_OK : FORGE_B200_LAUNCH_FAILED;
}

}  // extern "C"
