// Per-device status word the GEMM kernels write when a bounded wait runs out.
#include "common.cuh"
#include "gemm_dense.cuh"

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

}  // namespace fb200
