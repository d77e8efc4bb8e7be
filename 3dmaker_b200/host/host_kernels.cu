#include "host_kernels.h"

#include <atomic>

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

template <class T>
__global__ void __launch_bounds__(256) repitch_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, int64_t rows, int src_dim,
                                                           int dst_dim) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * dst_dim) return;
    int64_t r = i / dst_dim;
    int c = (int)(i % dst_dim);
    dst[i] = c < src_dim ? src[r * src_dim + c] : T(0);
}

template <class T>
static void repitch(const T* src, T* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream) {
    if (rows <= 0) return;
    int64_t total = rows * dst_dim;
    repitch_rows_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(src, dst, rows, src_dim, dst_dim);
    g_launch_count++;
}

void pad_rows_half(const half* src, half* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream) {
    repitch<half>(src, dst, rows, src_dim, dst_dim, stream);
}
void pad_rows_float(const float* src, float* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream) {
    repitch<float>(src, dst, rows, src_dim, dst_dim, stream);
}
void unpad_rows_float(const float* src, float* dst, int64_t rows, int src_dim, int dst_dim, cudaStream_t stream) {
    repitch<float>(src, dst, rows, src_dim, dst_dim, stream);
}

}  // namespace nb
