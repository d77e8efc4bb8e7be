// Rays: slab test against the outermost cascade, hierarchical DDA march over the occupancy bitfield
// (count pass and emit pass), exclusive scan of the per-ray counts and the sample-budget cutoff.
//
// Replaces compute_ray_aabb_inv_kernel (modules/NeRF/otherKernels.cu:91-154), march_rays_dda_calc_hits,
// custom_exclusive_sum, find_cutoff_ray_kernel / find_cutoff_ray_from_kernel and march_rays_dda_offset
// (modules/NeRF/processRays.cu:486-549, 626-929) and the host orchestration processRaysHitLinear /
// processRaysHitData / processRaysHitPositions (processRays.cu:931-1173).
//
// What differs from the reference: the cutoff (how many whole rays fit the sample budget), the batch's first
// sample and its sample total are written to a small device-side "plan" by the scan itself, and the emit
// kernel reads the plan from device memory.  The reference reads those numbers back to the host between
// kernels (three blocking copies per optimizer step); here the host needs them only to size the following
// launches and can read the 16-byte plan once.  The sample list itself (counts, offsets, ray ids, t,
// contracted positions, all in ray order) is the reference's, expression for expression.
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

constexpr uint32_t MAX_HITS = 1024;  // per-ray sample cap, modules/NeRF/InstantNerf.h:24

struct Scene {
    uint3 res;
    float3 aabb_min, aabb_max;
    int num_cascades, levels, spv;
};

static Scene make_scene(const nb_scene_desc* d) {
    Scene s;
    s.res = make_uint3(d->grid_res[0], d->grid_res[1], d->grid_res[2]);
    s.aabb_min = make_float3(d->aabb_min[0], d->aabb_min[1], d->aabb_min[2]);
    s.aabb_max = make_float3(d->aabb_max[0], d->aabb_max[1], d->aabb_max[2]);
    s.num_cascades = d->num_cascades; s.levels = d->mip_levels; s.spv = d->samples_per_voxel;
    return s;
}

__global__ void __launch_bounds__(256) ray_aabb_kernel(const uint32_t num_rays, const float3* __restrict__ rays_o,
                                                       const float3* __restrict__ rays_d, const float3 aabb_min, const float3 aabb_max,
                                                       const int num_cascades, float3* __restrict__ rays_d_inv,
                                                       float* __restrict__ nears, float* __restrict__ fars) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_rays) return;
    float scale = exp2f((float)(num_cascades - 1));
    float3 min_bound = make_float3(aabb_min.x * scale, aabb_min.y * scale, aabb_min.z * scale);
    float3 max_bound = make_float3(aabb_max.x * scale, aabb_max.y * scale, aabb_max.z * scale);
    float3 o = rays_o[i];
    float3 d = rays_d[i];
    if (fabsf(d.x) < 1e-8f) d.x = 1e-8f;
    if (fabsf(d.y) < 1e-8f) d.y = 1e-8f;
    if (fabsf(d.z) < 1e-8f) d.z = 1e-8f;
    float3 d_inv;
    d_inv.x = 1.0f / d.x;
    d_inv.y = 1.0f / d.y;
    d_inv.z = 1.0f / d.z;
    rays_d_inv[i] = d_inv;
    float t1x = (min_bound.x - o.x) * d_inv.x, t2x = (max_bound.x - o.x) * d_inv.x;
    if (t1x > t2x) { float tmp = t1x; t1x = t2x; t2x = tmp; }
    float t1y = (min_bound.y - o.y) * d_inv.y, t2y = (max_bound.y - o.y) * d_inv.y;
    if (t1y > t2y) { float tmp = t1y; t1y = t2y; t2y = tmp; }
    float t1z = (min_bound.z - o.z) * d_inv.z, t2z = (max_bound.z - o.z) * d_inv.z;
    if (t1z > t2z) { float tmp = t1z; t1z = t2z; t2z = tmp; }
    float t_enter = fmaxf(fmaxf(t1x, t1y), t1z);
    float t_exit = fminf(fminf(t2x, t2y), t2z);
    if (t_enter > t_exit || t_exit < 0.0f) {
        nears[i] = 0.0f;
        fars[i] = 0.0f;
    } else {
        nears[i] = fmaxf(t_enter, 0.0f);
        fars[i] = t_exit;
    }
}

// modules/NeRF/processRays.cu:11-19
__device__ __forceinline__ int get_cascade(float3 pos, float3 aabb_min, float3 aabb_max, int num_cascades) {
    float rx = fmaxf(pos.x / aabb_max.x, pos.x / aabb_min.x);
    float ry = fmaxf(pos.y / aabb_max.y, pos.y / aabb_min.y);
    float rz = fmaxf(pos.z / aabb_max.z, pos.z / aabb_min.z);
    float max_scale = fmaxf(rx, fmaxf(ry, rz));
    if (max_scale <= 1.0f) return 0;
    int cascade = (int)ceilf(log2f(max_scale));
    return max(0, min(cascade, num_cascades - 1));
}

// modules/NeRF/processRays.cu:21-46
__device__ __forceinline__ float3 contract_pos(float3 pos, float3 aabb_min, float3 aabb_max) {
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

// modules/NeRF/processRays.cu:83-93
__device__ __forceinline__ uint32_t get_mipmap_offset(uint3 base_res, int target_level) {
    uint32_t offset = 0;
    uint3 res = base_res;
    for (int l = 0; l < target_level; ++l) {
        offset += res.x * res.y * res.z;
        res.x >>= 1; res.y >>= 1; res.z >>= 1;
    }
    return offset;
}

// The DDA walk shared by the count pass (EMIT = false) and the emit pass.  One thread per ray.
template <bool EMIT>
__device__ __forceinline__ uint32_t march_ray(const Scene& sc, float3 o, float3 d, float3 d_inv, float t_min, float t_max_ray,
                                              const uint8_t* __restrict__ occupancy_grid, uint32_t ray_id, uint32_t out_base_idx,
                                              float* __restrict__ t_hits_out, uint32_t* __restrict__ ray_indices_out,
                                              float4* __restrict__ mlp_pos_vec) {
    const float3 aabb_min = sc.aabb_min, aabb_max = sc.aabb_max;
    const uint3 grid_resolution = sc.res;
    const int levelsMipmap = sc.levels;
    float3 aabb_extent = make_float3(aabb_max.x - aabb_min.x, aabb_max.y - aabb_min.y, aabb_max.z - aabb_min.z);
    int3 step = make_int3((d.x >= 0.0f) ? 1 : -1, (d.y >= 0.0f) ? 1 : -1, (d.z >= 0.0f) ? 1 : -1);
    const uint32_t total_mipmap_cells = get_mipmap_offset(grid_resolution, levelsMipmap);

    uint32_t hit_count = 0;
    float current_t = t_min;
    int current_level = levelsMipmap - 1;

    while (current_t < t_max_ray && hit_count < MAX_HITS) {
        float3 current_pos = make_float3(o.x + current_t * d.x, o.y + current_t * d.y, o.z + current_t * d.z);
        int cascade = get_cascade(current_pos, aabb_min, aabb_max, sc.num_cascades);
        float cascade_scale = exp2f((float)cascade);
        float3 c_aabb_min = make_float3(aabb_min.x * cascade_scale, aabb_min.y * cascade_scale, aabb_min.z * cascade_scale);
        float3 c_aabb_extent = make_float3(aabb_extent.x * cascade_scale, aabb_extent.y * cascade_scale, aabb_extent.z * cascade_scale);
        uint3 res_l = make_uint3(grid_resolution.x >> current_level, grid_resolution.y >> current_level, grid_resolution.z >> current_level);
        float3 voxel_size_l = make_float3(c_aabb_extent.x / res_l.x, c_aabb_extent.y / res_l.y, c_aabb_extent.z / res_l.z);
        float3 rel_pos = make_float3((current_pos.x - c_aabb_min.x) / c_aabb_extent.x, (current_pos.y - c_aabb_min.y) / c_aabb_extent.y,
                                     (current_pos.z - c_aabb_min.z) / c_aabb_extent.z);
        int3 voxel_index = make_int3(max(0, min((int)floorf(rel_pos.x * res_l.x), (int)res_l.x - 1)),
                                     max(0, min((int)floorf(rel_pos.y * res_l.y), (int)res_l.y - 1)),
                                     max(0, min((int)floorf(rel_pos.z * res_l.z), (int)res_l.z - 1)));
        uint32_t level_offset = get_mipmap_offset(grid_resolution, current_level);
        uint32_t cascade_offset = cascade * total_mipmap_cells;
        uint32_t flat_idx = cascade_offset + level_offset + voxel_index.z * (res_l.x * res_l.y) + voxel_index.y * res_l.x + voxel_index.x;
        uint32_t byte_idx = flat_idx >> 3;
        uint32_t bit_idx = flat_idx & 7;
        bool is_occupied = (occupancy_grid[byte_idx] >> bit_idx) & 1;

        float3 next_boundary = make_float3(c_aabb_min.x + (voxel_index.x + (step.x > 0 ? 1.0f : 0.0f)) * voxel_size_l.x,
                                           c_aabb_min.y + (voxel_index.y + (step.y > 0 ? 1.0f : 0.0f)) * voxel_size_l.y,
                                           c_aabb_min.z + (voxel_index.z + (step.z > 0 ? 1.0f : 0.0f)) * voxel_size_l.z);
        float3 t_max_axis = make_float3((next_boundary.x - o.x) * d_inv.x, (next_boundary.y - o.y) * d_inv.y, (next_boundary.z - o.z) * d_inv.z);
        float next_t = fminf(fminf(t_max_axis.x, t_max_axis.y), t_max_axis.z);

        if (is_occupied) {
            if (current_level > 0) {
                current_level--;
                continue;
            }
            if (!EMIT) {
                int n = sc.spv;
                int remaining = (int)MAX_HITS - (int)hit_count;
                if (n > remaining) n = remaining;
                hit_count += n;
            } else {
                const int K = sc.spv;
                float span = next_t - current_t;
                for (int k = 0; k < K; ++k) {
                    if (hit_count >= MAX_HITS) break;
                    float t_k = current_t + (k + 0.5f) / (float)K * span;
                    uint32_t write_idx = out_base_idx + hit_count;
                    t_hits_out[write_idx] = t_k;
                    ray_indices_out[write_idx] = ray_id;
                    float3 pos = make_float3(o.x + t_k * d.x, o.y + t_k * d.y, o.z + t_k * d.z);
                    pos = contract_pos(pos, aabb_min, aabb_max);
                    st_cs_v4(&mlp_pos_vec[write_idx], make_uint4(__float_as_uint(pos.x), __float_as_uint(pos.y), __float_as_uint(pos.z), 0u));
                    hit_count++;
                }
            }
        }
        current_t = fmaxf(current_t + 1e-5f, next_t + 1e-6f);
        current_level = levelsMipmap - 1;
    }
    return hit_count;
}

__global__ void __launch_bounds__(256) march_count_kernel(const __grid_constant__ Scene sc, const uint32_t num_rays,
                                                          const float3* __restrict__ rays_o, const float3* __restrict__ rays_d,
                                                          const float3* __restrict__ rays_d_inv, const float* __restrict__ nears,
                                                          const float* __restrict__ fars, const uint8_t* __restrict__ grid,
                                                          uint32_t* __restrict__ num_steps) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_rays) return;
    num_steps[i] = march_ray<false>(sc, rays_o[i], rays_d[i], rays_d_inv[i], nears[i], fars[i], grid, i, 0u, nullptr, nullptr, nullptr);
}

// plan[0] = one past the last ray of the batch (absolute index), plan[2] = first sample of the batch.
// Rays [rays_done, plan[0]) are marched; ray ids are written relative to rays_done.
__global__ void __launch_bounds__(256) march_emit_kernel(const __grid_constant__ Scene sc, const uint32_t num_rays, const uint32_t rays_done,
                                                         const float3* __restrict__ rays_o, const float3* __restrict__ rays_d,
                                                         const float3* __restrict__ rays_d_inv, const float* __restrict__ nears,
                                                         const float* __restrict__ fars, const uint8_t* __restrict__ grid,
                                                         const uint32_t* __restrict__ ray_offsets, const uint32_t* __restrict__ plan,
                                                         float* __restrict__ t_out, uint32_t* __restrict__ ray_idx_out,
                                                         float4* __restrict__ pos_out) {
    uint32_t local = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t i = local + rays_done;
    uint32_t end = min(plan[0], num_rays);
    if (i >= end) return;
    uint32_t base = plan[2];
    march_ray<true>(sc, rays_o[i], rays_d[i], rays_d_inv[i], nears[i], fars[i], grid, local, ray_offsets[i] - base, t_out, ray_idx_out, pos_out);
}

// ---- exclusive scan + cutoff --------------------------------------------------------------------------
constexpr int SCAN_BLOCK = 1024;

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t val, uint32_t* warp_sums, uint32_t& block_total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = val;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = warp_sums[lane];
        uint32_t wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        warp_sums[lane] = wi - w;  // exclusive prefix of the warps
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    block_total = warp_sums[32];
    return incl - val + warp_sums[warp];
}

__global__ void __launch_bounds__(SCAN_BLOCK) scan_blocks_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                                                 uint32_t* __restrict__ block_sums, uint32_t n) {
    __shared__ uint32_t warp_sums[33];
    uint32_t gid = blockIdx.x * SCAN_BLOCK + threadIdx.x;
    uint32_t v = gid < n ? in[gid] : 0u;
    uint32_t total;
    uint32_t ex = block_exclusive_scan(v, warp_sums, total);
    if (gid < n) out[gid] = ex;
    if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// One block: exclusive scan of the block sums in place, and the plan's initial state.
__global__ void __launch_bounds__(SCAN_BLOCK) scan_block_sums_kernel(uint32_t* __restrict__ block_sums, uint32_t num_blocks,
                                                                     uint32_t* __restrict__ plan, uint32_t rays_done) {
    __shared__ uint32_t warp_sums[33];
    uint32_t v = threadIdx.x < num_blocks ? block_sums[threadIdx.x] : 0u;
    uint32_t total;
    uint32_t ex = block_exclusive_scan(v, warp_sums, total);
    if (threadIdx.x < num_blocks) block_sums[threadIdx.x] = ex;
    if (threadIdx.x == 0) {
        plan[0] = rays_done; plan[1] = 0u; plan[2] = 0u; plan[3] = total;
    }
}

// Adds the block prefixes and marks the cutoff: the last ray whose inclusive sample count (from the batch's
// first ray) still fits the budget.  Inclusive counts never decrease, so exactly one ray is that boundary.
__global__ void __launch_bounds__(SCAN_BLOCK) scan_finish_kernel(uint32_t* __restrict__ offsets, const uint32_t* __restrict__ num_steps,
                                                                 const uint32_t* __restrict__ block_sums, uint32_t n,
                                                                 uint32_t batch_size, uint32_t* __restrict__ plan) {
    uint32_t gid = blockIdx.x * SCAN_BLOCK + threadIdx.x;
    if (gid >= n) return;
    uint32_t off = offsets[gid] + block_sums[blockIdx.x];
    offsets[gid] = off;
    uint32_t steps = num_steps[gid];
    uint32_t incl = off + steps;  // base is 0: the scan starts at ray 0
    if (incl <= batch_size) {
        bool boundary = true;
        if (gid + 1 < n) {
            // next ray's inclusive count = incl + its own count
            if (incl + num_steps[gid + 1] <= batch_size) boundary = false;
        }
        if (boundary) { plan[0] = gid + 1; plan[1] = incl; }
    }
}

__global__ void plan_init_kernel(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ num_steps, uint32_t n,
                                 uint32_t rays_done, uint32_t* __restrict__ plan) {
    plan[0] = rays_done; plan[1] = 0u;
    plan[2] = rays_done < n ? offsets[rays_done] : 0u;
    plan[3] = n > 0 ? offsets[n - 1] + num_steps[n - 1] : 0u;
}

// find_cutoff_ray_from_kernel, modules/NeRF/processRays.cu:771-799
__global__ void __launch_bounds__(256) cutoff_from_kernel(const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ num_steps,
                                                          uint32_t n, uint32_t batch_size, uint32_t rays_done, uint32_t* __restrict__ plan) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x + rays_done;
    if (i >= n) return;
    const uint32_t base = offsets[rays_done];
    uint32_t incl = offsets[i] + num_steps[i] - base;
    if (incl <= batch_size) {
        bool boundary = true;
        if (i < n - 1 && offsets[i + 1] + num_steps[i + 1] - base <= batch_size) boundary = false;
        if (boundary) { plan[0] = i + 1; plan[1] = incl; }
    }
}

}  // namespace nb

using namespace nb;

static int check_scene(const nb_scene_desc* s, const char* who) {
    if (!s) return nb_set_error(NB_ERR_INVALID, who);
    if (s->num_cascades < 1 || s->mip_levels < 1 || s->mip_levels > 8 || s->samples_per_voxel < 1)
        return nb_set_error(NB_ERR_INVALID, "scene: cascades >= 1, 1 <= mip levels <= 8, samples per voxel >= 1 required");
    for (int a = 0; a < 3; a++)
        if (s->grid_res[a] == 0 || (s->grid_res[a] >> (s->mip_levels - 1)) == 0)
            return nb_set_error(NB_ERR_INVALID, "scene: grid resolution too small for the mip levels");
    return NB_OK;
}

extern "C" int nb_ray_aabb(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, int64_t num_rays, float* d_rays_d_inv,
                           float* d_nears, float* d_fars, void* stream) {
    int rc = check_scene(scene, "nb_ray_aabb: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_rays_d_inv || !d_nears || !d_fars || num_rays < 0 || num_rays > 0x7fffffff)
        return nb_set_error(NB_ERR_INVALID, "nb_ray_aabb: null pointer or bad ray count");
    if (num_rays == 0) return NB_OK;
    Scene sc = make_scene(scene);
    ray_aabb_kernel<<<(unsigned)((num_rays + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint32_t)num_rays, (const float3*)d_rays_o, (const float3*)d_rays_d, sc.aabb_min, sc.aabb_max, sc.num_cascades, (float3*)d_rays_d_inv,
        d_nears, d_fars);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_march_count(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv,
                              const float* d_nears, const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays,
                              uint32_t* d_num_steps, void* stream) {
    int rc = check_scene(scene, "nb_march_count: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_rays_d_inv || !d_nears || !d_fars || !d_bitfield || !d_num_steps || num_rays < 0 || num_rays > 0x7fffffff)
        return nb_set_error(NB_ERR_INVALID, "nb_march_count: null pointer or bad ray count");
    if (num_rays == 0) return NB_OK;
    Scene sc = make_scene(scene);
    march_count_kernel<<<(unsigned)((num_rays + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        sc, (uint32_t)num_rays, (const float3*)d_rays_o, (const float3*)d_rays_d, (const float3*)d_rays_d_inv, d_nears, d_fars, d_bitfield,
        d_num_steps);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_march_scan(const uint32_t* d_num_steps, uint32_t* d_ray_offsets, uint32_t* d_block_sums, int64_t num_rays,
                             uint32_t batch_size, uint32_t* d_plan, void* stream) {
    if (!d_num_steps || !d_ray_offsets || !d_block_sums || !d_plan || num_rays < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_march_scan: null pointer or negative ray count");
    if (num_rays > (int64_t)SCAN_BLOCK * SCAN_BLOCK)
        return nb_set_error(NB_ERR_LIMIT, "nb_march_scan: at most 1048576 rays per chunk");
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t n = (uint32_t)num_rays;
    uint32_t blocks = (n + SCAN_BLOCK - 1) / SCAN_BLOCK;
    if (n > 0) scan_blocks_kernel<<<blocks, SCAN_BLOCK, 0, st>>>(d_num_steps, d_ray_offsets, d_block_sums, n);
    scan_block_sums_kernel<<<1, SCAN_BLOCK, 0, st>>>(d_block_sums, blocks, d_plan, 0u);
    if (n > 0) scan_finish_kernel<<<blocks, SCAN_BLOCK, 0, st>>>(d_ray_offsets, d_num_steps, d_block_sums, n, batch_size, d_plan);
    NB_CHECK_LAUNCH();
    g_launch_count += (n > 0 ? 3 : 1);
    return NB_OK;
}

extern "C" int nb_march_cutoff(const uint32_t* d_num_steps, const uint32_t* d_ray_offsets, int64_t num_rays, uint32_t rays_done,
                               uint32_t batch_size, uint32_t* d_plan, void* stream) {
    if (!d_num_steps || !d_ray_offsets || !d_plan || num_rays < 0 || num_rays > 0x7fffffff || (int64_t)rays_done > num_rays)
        return nb_set_error(NB_ERR_INVALID, "nb_march_cutoff: null pointer or bad ray range");
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t n = (uint32_t)num_rays;
    plan_init_kernel<<<1, 1, 0, st>>>(d_ray_offsets, d_num_steps, n, rays_done, d_plan);
    uint32_t left = n - rays_done;
    if (left > 0) cutoff_from_kernel<<<(left + 255) / 256, 256, 0, st>>>(d_ray_offsets, d_num_steps, n, batch_size, rays_done, d_plan);
    NB_CHECK_LAUNCH();
    g_launch_count += (left > 0 ? 2 : 1);
    return NB_OK;
}

extern "C" int nb_march_emit(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv,
                             const float* d_nears, const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays, uint32_t rays_done,
                             int64_t max_rays_in_batch, const uint32_t* d_ray_offsets, const uint32_t* d_plan, float* d_t_out,
                             uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream) {
    int rc = check_scene(scene, "nb_march_emit: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_rays_d_inv || !d_nears || !d_fars || !d_bitfield || !d_ray_offsets || !d_plan || !d_t_out ||
        !d_ray_idx_out || !d_pos4_out || num_rays < 0 || num_rays > 0x7fffffff || (int64_t)rays_done > num_rays || max_rays_in_batch < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_march_emit: null pointer or bad ray range");
    if (reinterpret_cast<uintptr_t>(d_pos4_out) & 15u) return nb_set_error(NB_ERR_INVALID, "nb_march_emit: positions must be 16-byte aligned");
    int64_t span = num_rays - rays_done;
    if (max_rays_in_batch < span) span = max_rays_in_batch;
    if (span == 0) return NB_OK;
    Scene sc = make_scene(scene);
    march_emit_kernel<<<(unsigned)((span + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        sc, (uint32_t)num_rays, rays_done, (const float3*)d_rays_o, (const float3*)d_rays_d, (const float3*)d_rays_d_inv, d_nears, d_fars,
        d_bitfield, d_ray_offsets, d_plan, d_t_out, d_ray_idx_out, (float4*)d_pos4_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
