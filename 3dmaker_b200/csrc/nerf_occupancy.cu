// Occupancy grid maintenance: jittered cell samples, per-cell density maximum, decayed master grid, the
// thresholded level-0 bitfield of every cascade, its OR-pooled mip pyramid and the list of occupied cells.
//
// Replaces sampleAABB, sampleOccupiedAABB, updateTmpGrid, updateMasterGrid, updateOccupancyGrid,
// bitfield_max_pool, extractActiveCells (modules/NeRF/otherKernels.cu:591-888), the cub::DeviceReduce::Sum of
// the master grid (otherKernels.cu:696-698) and InstantNerf::buildMipmaps (InstantNerf.cu:1177-1204).
//
// Bit layout (what the marcher reads): bit = cascade * S + level_offset + z * res^2 + y * res + x, LSB first,
// S = cells of one cascade's whole pyramid.
//
// Differences from the reference, on purpose:
//  * the mean density comes from a deterministic two-stage tree sum kept in fp64 (the reference's CUB sum has
//    no fixed order); the mean only enters the threshold min(bar, mean);
//  * the occupied-cell list is appended with one atomic per warp (lanes in cell order) instead of one per cell;
//    as in the reference the order of the list is not fixed, only the set of cells is;
//  * all levels of the pyramid are pooled by one launch per level covering every cascade.
#include <atomic>

#include <curand_kernel.h>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__device__ __forceinline__ float3 occ_contract_pos(float3 pos, float3 aabb_min, float3 aabb_max) {
    float3 aabb_extent = make_float3(aabb_max.x - aabb_min.x, aabb_max.y - aabb_min.y, aabb_max.z - aabb_min.z);
    float3 rel_pos = make_float3((pos.x - aabb_min.x) / aabb_extent.x, (pos.y - aabb_min.y) / aabb_extent.y,
                                 (pos.z - aabb_min.z) / aabb_extent.z);
    float3 norm_pos = make_float3(rel_pos.x * 2.0f - 1.0f, rel_pos.y * 2.0f - 1.0f, rel_pos.z * 2.0f - 1.0f);
    float3 contracted;
    contracted.x = fabsf(norm_pos.x) <= 1.0f ? norm_pos.x : (2.0f - 1.0f / fabsf(norm_pos.x)) * copysignf(1.0f, norm_pos.x);
    contracted.y = fabsf(norm_pos.y) <= 1.0f ? norm_pos.y : (2.0f - 1.0f / fabsf(norm_pos.y)) * copysignf(1.0f, norm_pos.y);
    contracted.z = fabsf(norm_pos.z) <= 1.0f ? norm_pos.z : (2.0f - 1.0f / fabsf(norm_pos.z)) * copysignf(1.0f, norm_pos.z);
    return make_float3(fmaxf(0.0f, fminf((contracted.x + 2.0f) * 0.25f, 1.0f)), fmaxf(0.0f, fminf((contracted.y + 2.0f) * 0.25f, 1.0f)),
                       fmaxf(0.0f, fminf((contracted.z + 2.0f) * 0.25f, 1.0f)));
}

__device__ __forceinline__ void write_cell_sample(float4* __restrict__ samples_vec, int idx, int cell_idx, float4 rnd, float3 aabbMin,
                                                  float3 aabbMax, uint3 gridResolution) {
    int cells_per_level = gridResolution.x * gridResolution.y * gridResolution.z;
    int cascade = cell_idx / cells_per_level;
    int local_cell = cell_idx % cells_per_level;
    int gridX = local_cell % gridResolution.x;
    int gridY = (local_cell / gridResolution.x) % gridResolution.y;
    int gridZ = local_cell / (gridResolution.x * gridResolution.y);
    float cascade_scale = exp2f((float)cascade);
    float3 c_aabb_min = make_float3(aabbMin.x * cascade_scale, aabbMin.y * cascade_scale, aabbMin.z * cascade_scale);
    float3 c_aabb_max = make_float3(aabbMax.x * cascade_scale, aabbMax.y * cascade_scale, aabbMax.z * cascade_scale);
    float3 cellSize = make_float3((c_aabb_max.x - c_aabb_min.x) / gridResolution.x, (c_aabb_max.y - c_aabb_min.y) / gridResolution.y,
                                  (c_aabb_max.z - c_aabb_min.z) / gridResolution.z);
    float3 pos = make_float3(c_aabb_min.x + (gridX + rnd.x) * cellSize.x, c_aabb_min.y + (gridY + rnd.y) * cellSize.y,
                             c_aabb_min.z + (gridZ + rnd.z) * cellSize.z);
    pos = occ_contract_pos(pos, aabbMin, aabbMax);
    st_cs_v4(&samples_vec[idx], make_uint4(__float_as_uint(pos.x), __float_as_uint(pos.y), __float_as_uint(pos.z), (uint32_t)cell_idx));
}

__global__ void __launch_bounds__(256) sample_cells_kernel(float4* __restrict__ samples, float3 aabbMin, float3 aabbMax, uint3 gridResolution,
                                                           int N, int totalCells, int cellOffset, unsigned long long seed) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N) return;
    curandStatePhilox4_32_10_t state;
    curand_init(seed, idx, 0, &state);
    float4 rnd = curand_uniform4(&state);
    int cell_idx;
    if (N == totalCells) cell_idx = cellOffset + idx;
    else cell_idx = cellOffset + min((int)(rnd.w * totalCells), totalCells - 1);
    write_cell_sample(samples, idx, cell_idx, rnd, aabbMin, aabbMax, gridResolution);
}

__global__ void __launch_bounds__(256) sample_occupied_kernel(float4* __restrict__ samples, const int* __restrict__ activeCellIndices,
                                                              const int* __restrict__ numActiveCells, float3 aabbMin, float3 aabbMax,
                                                              uint3 gridResolution, int N, unsigned long long seed) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N) return;
    int totalActive = *numActiveCells;
    if (totalActive == 0) return;
    curandStatePhilox4_32_10_t state;
    curand_init(seed, idx, 0, &state);
    float4 rnd = curand_uniform4(&state);
    int listIdx = min((int)(rnd.w * totalActive), totalActive - 1);
    write_cell_sample(samples, idx, activeCellIndices[listIdx], rnd, aabbMin, aabbMax, gridResolution);
}

// sigma is never negative, so an integer max on the float bits orders it correctly.
__global__ void __launch_bounds__(256) update_tmp_grid_kernel(const float4* __restrict__ samples, const float* __restrict__ density_out,
                                                              float* __restrict__ tmpGrid, float densityBias, int N) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N) return;
    int cell_idx = __float_as_int(samples[idx].w);
    const float logit = density_out[(size_t)idx * 16];   // first output of the density network
    const float sigma = expf(fminf(logit - densityBias, 8.0f));
    atomicMax(reinterpret_cast<int*>(&tmpGrid[cell_idx]), __float_as_int(sigma));
}

// Decay + max into the master grid, and the block's partial sum of the NEW master values (fp64).
__global__ void __launch_bounds__(256) update_master_grid_kernel(const float* __restrict__ tmpGrid, float* __restrict__ masterGrid,
                                                                 float decay, int N, double* __restrict__ partial) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    float val = 0.0f;
    if (idx < N) {
        const float kept = masterGrid[idx];     // a negative entry marks a cell that is never updated
        const float fresh = tmpGrid[idx];       // this update's per-cell maximum of sigma
        val = (kept < 0.f) ? kept : fmaxf(kept * decay, fresh);
        masterGrid[idx] = val;
    }
    double s = (double)val;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    __shared__ double ws[8];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < 8; k++) t += ws[k];
        partial[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(1024) reduce_partials_kernel(const double* __restrict__ partial, int count, float* __restrict__ d_sum) {
    double s = 0.0;
    for (int i = threadIdx.x; i < count; i += blockDim.x) s += partial[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    __shared__ double ws[32];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < 32; k++) t += ws[k];
        d_sum[0] = (float)t;
    }
}

__global__ void __launch_bounds__(256) update_bits_kernel(uint32_t* __restrict__ d_occupancy_grid, const float* __restrict__ d_master_grid,
                                                          const float* __restrict__ d_sum, int total_cells, int cells_per_cascade,
                                                          int pyramid_cells_per_cascade, float min_optical_thickness, float base_voxel) {
    int cell_idx = blockIdx.x * blockDim.x + threadIdx.x;
    bool is_active = false;
    if (cell_idx < total_cells) {
        float mean_density = d_sum[0] / (float)total_cells;
        int cascade = cell_idx / cells_per_cascade;
        float cascade_thresh = (min_optical_thickness / base_voxel) / exp2f((float)cascade);
        float threshold = fminf(cascade_thresh, mean_density);
        is_active = (d_master_grid[cell_idx] > threshold);
    }
    unsigned int warp_mask = __ballot_sync(0xFFFFFFFF, is_active);
    if ((threadIdx.x & 31) == 0 && cell_idx < total_cells) {
        int cascade = cell_idx / cells_per_cascade;
        int local = cell_idx % cells_per_cascade;
        int bitpos = cascade * pyramid_cells_per_cascade + local;
        d_occupancy_grid[bitpos / 32] = warp_mask;
    }
}

// One mip level for every cascade: blockIdx.y = cascade.  in/out offsets are in bits from the cascade's start.
__global__ void __launch_bounds__(256) max_pool_kernel(uint8_t* __restrict__ grid, uint32_t cascade_stride_bytes, uint32_t in_offset_bits,
                                                       uint32_t out_offset_bits, uint3 res_out) {
    uint8_t* base = grid + (size_t)blockIdx.y * cascade_stride_bytes;
    const uint8_t* level_in = base + (in_offset_bits >> 3);
    uint32_t* level_out_32 = reinterpret_cast<uint32_t*>(base + (out_offset_bits >> 3));
    int out_idx = blockIdx.x * blockDim.x + threadIdx.x;
    int total_out_cells = res_out.x * res_out.y * res_out.z;
    bool is_occupied = false;
    if (out_idx < total_out_cells) {
        int out_x = out_idx % res_out.x;
        int out_y = (out_idx / res_out.x) % res_out.y;
        int out_z = out_idx / (res_out.x * res_out.y);
        int res_in_x = res_out.x * 2, res_in_y = res_out.y * 2;
#pragma unroll
        for (int dz = 0; dz < 2; ++dz)
            for (int dy = 0; dy < 2; ++dy)
                for (int dx = 0; dx < 2; ++dx) {
                    int in_idx = (out_z * 2 + dz) * (res_in_x * res_in_y) + (out_y * 2 + dy) * res_in_x + (out_x * 2 + dx);
                    is_occupied = is_occupied || ((level_in[in_idx >> 3] >> (in_idx & 7)) & 1);
                }
    }
    unsigned int warp_mask = __ballot_sync(0xFFFFFFFF, is_occupied);
    if ((threadIdx.x & 31) == 0 && out_idx < total_out_cells) {
        if (total_out_cells >= 32) {
            level_out_32[out_idx / 32] = warp_mask;
        } else {
            uint8_t* level_out_8 = reinterpret_cast<uint8_t*>(level_out_32);
            int num_bytes = (total_out_cells + 7) / 8;
            for (int i = 0; i < num_bytes; ++i) level_out_8[i] = (warp_mask >> (i * 8)) & 0xFF;
        }
    }
}

__global__ void __launch_bounds__(256) extract_active_kernel(const uint8_t* __restrict__ occupancyGrid, int* __restrict__ activeCellIndices,
                                                             int* __restrict__ numActiveCells, int totalCells, int cells_per_cascade,
                                                             int pyramid_cells_per_cascade) {
    int cellIdx = blockIdx.x * blockDim.x + threadIdx.x;
    bool occ = false;
    if (cellIdx < totalCells) {
        int cascade = cellIdx / cells_per_cascade;
        int local = cellIdx % cells_per_cascade;
        int bitpos = cascade * pyramid_cells_per_cascade + local;
        occ = (occupancyGrid[bitpos / 8] >> (bitpos % 8)) & 1;
    }
    // one atomic per warp: lanes take consecutive slots in lane order
    unsigned mask = __ballot_sync(0xffffffffu, occ);
    int lane = threadIdx.x & 31;
    int base = 0;
    if (lane == 0 && mask) base = atomicAdd(numActiveCells, __popc(mask));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (occ) activeCellIndices[base + __popc(mask & ((1u << lane) - 1u))] = cellIdx;
}

}  // namespace nb

using namespace nb;

static float3 f3(const float* p) { return make_float3(p[0], p[1], p[2]); }

extern "C" int nb_occ_sample_cells(const nb_scene_desc* scene, float* d_samples4, int n, int total_cells, int cell_offset, uint64_t seed,
                                   void* stream) {
    if (!scene || !d_samples4 || n < 0 || total_cells <= 0 || cell_offset < 0 || (reinterpret_cast<uintptr_t>(d_samples4) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_occ_sample_cells: null/misaligned pointer or bad counts");
    if (n == 0) return NB_OK;
    sample_cells_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((float4*)d_samples4, f3(scene->aabb_min), f3(scene->aabb_max),
                                                                           make_uint3(scene->grid_res[0], scene->grid_res[1], scene->grid_res[2]), n,
                                                                           total_cells, cell_offset, (unsigned long long)seed);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_occ_sample_occupied(const nb_scene_desc* scene, float* d_samples4, const int* d_active_cells, const int* d_num_active, int n,
                                      uint64_t seed, void* stream) {
    if (!scene || !d_samples4 || !d_active_cells || !d_num_active || n < 0 || (reinterpret_cast<uintptr_t>(d_samples4) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_occ_sample_occupied: null/misaligned pointer or bad count");
    if (n == 0) return NB_OK;
    sample_occupied_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((float4*)d_samples4, d_active_cells, d_num_active,
                                                                              f3(scene->aabb_min), f3(scene->aabb_max),
                                                                              make_uint3(scene->grid_res[0], scene->grid_res[1], scene->grid_res[2]), n,
                                                                              (unsigned long long)seed);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_occ_update_tmp_grid(const float* d_samples4, const float* d_density_out16, float* d_tmp_grid, float density_bias, int n,
                                      void* stream) {
    if (!d_samples4 || !d_density_out16 || !d_tmp_grid || n < 0) return nb_set_error(NB_ERR_INVALID, "nb_occ_update_tmp_grid: null pointer or bad count");
    if (n == 0) return NB_OK;
    update_tmp_grid_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const float4*)d_samples4, d_density_out16, d_tmp_grid, density_bias, n);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int64_t nb_occ_scratch_bytes(int total_cells) { return total_cells <= 0 ? 0 : (int64_t)((total_cells + 255) / 256) * 8; }

extern "C" int nb_occ_update_master_grid(const float* d_tmp_grid, float* d_master_grid, float decay, int total_cells, void* d_scratch,
                                         float* d_sum, void* stream) {
    if (!d_tmp_grid || !d_master_grid || !d_scratch || !d_sum || total_cells <= 0 || (reinterpret_cast<uintptr_t>(d_scratch) & 7u))
        return nb_set_error(NB_ERR_INVALID, "nb_occ_update_master_grid: null/misaligned pointer or bad count");
    int blocks = (total_cells + 255) / 256;
    update_master_grid_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(d_tmp_grid, d_master_grid, decay, total_cells, (double*)d_scratch);
    reduce_partials_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((const double*)d_scratch, blocks, d_sum);
    NB_CHECK_LAUNCH();
    g_launch_count += 2;
    return NB_OK;
}

extern "C" int nb_occ_update_bitfield(const nb_scene_desc* scene, uint8_t* d_bitfield, const float* d_master_grid, const float* d_sum,
                                      float min_optical_thickness, void* stream) {
    if (!scene || !d_bitfield || !d_master_grid || !d_sum || (reinterpret_cast<uintptr_t>(d_bitfield) & 3u))
        return nb_set_error(NB_ERR_INVALID, "nb_occ_update_bitfield: null or misaligned pointer");
    uint32_t rx = scene->grid_res[0], ry = scene->grid_res[1], rz = scene->grid_res[2];
    int G = (int)(rx * ry * rz);
    if (G % 32) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_occ_update_bitfield: cells per cascade must be a multiple of 32");
    int N = scene->num_cascades * G;
    uint32_t S = 0, x = rx, y = ry, z = rz;
    for (int l = 0; l < scene->mip_levels; l++) { S += x * y * z; x >>= 1; y >>= 1; z >>= 1; }
    if (S % 32) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_occ_update_bitfield: pyramid cells per cascade must be a multiple of 32");
    cudaStream_t st = (cudaStream_t)stream;
    float base_voxel = (scene->aabb_max[0] - scene->aabb_min[0]) / (float)rx;
    update_bits_kernel<<<(N + 255) / 256, 256, 0, st>>>((uint32_t*)d_bitfield, d_master_grid, d_sum, N, G, (int)S, min_optical_thickness, base_voxel);
    g_launch_count++;
    uint32_t in_off = 0;
    x = rx; y = ry; z = rz;
    for (int l = 0; l < scene->mip_levels - 1; l++) {
        uint32_t cells = x * y * z;
        uint3 ro = make_uint3(x / 2, y / 2, z / 2);
        uint32_t out_cells = ro.x * ro.y * ro.z;
        dim3 grid((out_cells + 255) / 256, scene->num_cascades, 1);
        max_pool_kernel<<<grid, 256, 0, st>>>(d_bitfield, S / 8, in_off, in_off + cells, ro);
        g_launch_count++;
        in_off += cells;
        x = ro.x; y = ro.y; z = ro.z;
    }
    NB_CHECK_LAUNCH();
    return NB_OK;
}

extern "C" int nb_occ_extract_active(const nb_scene_desc* scene, const uint8_t* d_bitfield, int* d_active_cells, int* d_num_active, void* stream) {
    if (!scene || !d_bitfield || !d_active_cells || !d_num_active) return nb_set_error(NB_ERR_INVALID, "nb_occ_extract_active: null pointer");
    uint32_t x = scene->grid_res[0], y = scene->grid_res[1], z = scene->grid_res[2];
    int G = (int)(x * y * z);
    int N = scene->num_cascades * G;
    uint32_t S = 0;
    for (int l = 0; l < scene->mip_levels; l++) { S += x * y * z; x >>= 1; y >>= 1; z >>= 1; }
    cudaStream_t st = (cudaStream_t)stream;
    NB_CUDA(cudaMemsetAsync(d_num_active, 0, sizeof(int), st));
    extract_active_kernel<<<(N + 255) / 256, 256, 0, st>>>(d_bitfield, d_active_cells, d_num_active, N, G, (int)S);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
