// Library-wide state: last-error text, launch counter, device properties.
#include <atomic>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace nb {
std::atomic<uint64_t> g_launch_count{0};
}

static thread_local char g_err[512] = "";

int nb_set_error(int code, const char* msg) {
    std::snprintf(g_err, sizeof(g_err), "%s", msg ? msg : "");
    return code;
}

int nb_set_cuda_error(cudaError_t e) {
    std::snprintf(g_err, sizeof(g_err), "CUDA error %d: %s", (int)e, cudaGetErrorString(e));
    return NB_ERR_CUDA;
}

int nb_num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

extern "C" const char* nb_last_error(void) { return g_err; }
extern "C" int nb_version(void) { return 1; }
extern "C" int nb_built_arch(void) { return 100; }
extern "C" uint64_t nb_launch_count(void) { return nb::g_launch_count.load(); }

// Asynchronous zero fill of a device range on the caller's stream (cudaMemsetAsync), so host code that
// drives the library needs no other runtime for it.
extern "C" int nb_zero_async(void* d_ptr, int64_t bytes, void* stream) {
    if (bytes < 0 || (bytes > 0 && !d_ptr)) return nb_set_error(NB_ERR_INVALID, "nb_zero_async: null pointer or negative size");
    if (bytes == 0) return NB_OK;
    cudaError_t e = cudaMemsetAsync(d_ptr, 0, (size_t)bytes, (cudaStream_t)stream);
    if (e != cudaSuccess) return nb_set_cuda_error(e);
    return NB_OK;
}
