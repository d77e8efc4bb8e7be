// Spatial ordering of a sample batch: a permutation that lists the samples brick by brick, the 16^3 bricks of the unit
// cube in Morton order.
//
// The field kernels gather (forward) and reduce (backward) 8 corners per level and sample.  In arrival order every one
// of those is a trip to L2; when the samples of a tile sit next to each other in space, the corners they need on the
// coarser levels form a small box that a CTA can keep in shared memory (field_fused.cu, field_backward_tc.cu).  This
// file only produces the order; the kernels work with any order and use what locality they find.
//
// The reference has the same idea in its legacy path - Morton keys from the sample position and a radix sort of the
// whole batch (modules/NeRF/processRays.cu:70-81, 412-448, nothing in its training or rendering loop calls it).  Here
// the key is 12 bits (4 per axis), so the sort is one counting pass: histogram, exclusive scan, placement.  Samples of
// one brick keep no particular order among themselves.
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

constexpr int BRICKS = 4096;          // 16 x 16 x 16
constexpr int ORDER_CHUNK = 2048;     // samples per CTA
constexpr int ORDER_THREADS = 256;

// bits of v (4 of them) spread to every third position
__device__ __forceinline__ uint32_t spread4(uint32_t v) { return (v & 1u) | ((v & 2u) << 2) | ((v & 4u) << 4) | ((v & 8u) << 6); }

__device__ __forceinline__ uint32_t brick_key(const float* __restrict__ pos4, int64_t i) {
    const float4 p = ld_nc_f4(pos4 + i * 4);
    const uint32_t x = (uint32_t)max(0, min(15, __float2int_rd(p.x * 16.0f)));
    const uint32_t y = (uint32_t)max(0, min(15, __float2int_rd(p.y * 16.0f)));
    const uint32_t z = (uint32_t)max(0, min(15, __float2int_rd(p.z * 16.0f)));
    return spread4(x) | (spread4(y) << 1) | (spread4(z) << 2);
}

__global__ void __launch_bounds__(ORDER_THREADS) brick_count_kernel(const float* __restrict__ pos4, int64_t n, uint32_t* __restrict__ hist) {
    __shared__ uint32_t s_cnt[BRICKS];
    for (int b = threadIdx.x; b < BRICKS; b += ORDER_THREADS) s_cnt[b] = 0u;
    __syncthreads();
    const int64_t first = (int64_t)blockIdx.x * ORDER_CHUNK;
#pragma unroll
    for (int j = 0; j < ORDER_CHUNK / ORDER_THREADS; j++) {
        const int64_t i = first + j * ORDER_THREADS + threadIdx.x;
        if (i < n) atomicAdd(&s_cnt[brick_key(pos4, i)], 1u);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < BRICKS; b += ORDER_THREADS) {
        const uint32_t c = s_cnt[b];
        if (c != 0u) atomicAdd(&hist[b], c);
    }
}

// cursor[b] = number of samples in bricks before b (one block of 1024 threads, 4 bricks each)
__global__ void __launch_bounds__(1024) brick_scan_kernel(const uint32_t* __restrict__ hist, uint32_t* __restrict__ cursor) {
    __shared__ uint32_t s_warp[32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint4 h = reinterpret_cast<const uint4*>(hist)[t];
    const uint32_t mine = h.x + h.y + h.z + h.w;
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        s_warp[lane] = w;
    }
    __syncthreads();
    const uint32_t before = (warp > 0 ? s_warp[warp - 1] : 0u) + incl - mine;
    reinterpret_cast<uint4*>(cursor)[t] = make_uint4(before, before + h.x, before + h.x + h.y, before + h.x + h.y + h.z);
}

// Every CTA ranks its samples inside their bricks in shared memory, takes one range per brick from the global cursor
// and writes the sample numbers there.
__global__ void __launch_bounds__(ORDER_THREADS) brick_place_kernel(const float* __restrict__ pos4, int64_t n, uint32_t* __restrict__ cursor,
                                                                    uint32_t* __restrict__ perm) {
    __shared__ uint32_t s_cnt[BRICKS];
    __shared__ uint32_t s_base[BRICKS];
    for (int b = threadIdx.x; b < BRICKS; b += ORDER_THREADS) s_cnt[b] = 0u;
    __syncthreads();
    const int64_t first = (int64_t)blockIdx.x * ORDER_CHUNK;
    uint32_t key[ORDER_CHUNK / ORDER_THREADS], rank[ORDER_CHUNK / ORDER_THREADS];
#pragma unroll
    for (int j = 0; j < ORDER_CHUNK / ORDER_THREADS; j++) {
        const int64_t i = first + j * ORDER_THREADS + threadIdx.x;
        key[j] = 0u; rank[j] = 0u;
        if (i < n) {
            key[j] = brick_key(pos4, i);
            rank[j] = atomicAdd(&s_cnt[key[j]], 1u);
        }
    }
    __syncthreads();
    for (int b = threadIdx.x; b < BRICKS; b += ORDER_THREADS) {
        const uint32_t c = s_cnt[b];
        if (c != 0u) s_base[b] = atomicAdd(&cursor[b], c);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < ORDER_CHUNK / ORDER_THREADS; j++) {
        const int64_t i = first + j * ORDER_THREADS + threadIdx.x;
        if (i < n) perm[s_base[key[j]] + rank[j]] = (uint32_t)i;
    }
}

}  // namespace nb

using namespace nb;

extern "C" int64_t nb_sample_order_scratch_bytes(void) { return (int64_t)2 * BRICKS * sizeof(uint32_t); }

extern "C" int nb_sample_order(const float* d_pos4, int64_t n, uint32_t* d_perm, void* d_scratch, void* stream) {
    if (!d_pos4 || !d_perm || !d_scratch || n < 0) return nb_set_error(NB_ERR_INVALID, "nb_sample_order: null pointer or negative count");
    if (n > 0xffffffffLL) return nb_set_error(NB_ERR_LIMIT, "nb_sample_order: more than 2^32 - 1 samples");
    if ((reinterpret_cast<uintptr_t>(d_pos4) & 15u) || (reinterpret_cast<uintptr_t>(d_scratch) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_sample_order: positions and scratch must be 16-byte aligned");
    if (n == 0) return NB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* hist = reinterpret_cast<uint32_t*>(d_scratch);
    uint32_t* cursor = hist + BRICKS;
    NB_CUDA(cudaMemsetAsync(hist, 0, BRICKS * sizeof(uint32_t), st));
    const unsigned grid = (unsigned)((n + ORDER_CHUNK - 1) / ORDER_CHUNK);
    brick_count_kernel<<<grid, ORDER_THREADS, 0, st>>>(d_pos4, n, hist);
    NB_CHECK_LAUNCH();
    brick_scan_kernel<<<1, 1024, 0, st>>>(hist, cursor);
    NB_CHECK_LAUNCH();
    brick_place_kernel<<<grid, ORDER_THREADS, 0, st>>>(d_pos4, n, cursor, d_perm);
    NB_CHECK_LAUNCH();
    g_launch_count += 3;
    return NB_OK;
}
