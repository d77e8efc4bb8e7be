// Rays: slab test against the outermost cascade, the walk over the cascaded occupancy pyramid, exclusive scan of the
// per-ray sample counts and the compaction of the samples of a ray range into the field kernels' input.
//
// Replaces compute_ray_aabb_inv_kernel (modules/NeRF/otherKernels.cu:91-154), march_rays_dda_calc_hits,
// custom_exclusive_sum, find_cutoff_ray_kernel / find_cutoff_ray_from_kernel and march_rays_dda_offset
// (modules/NeRF/processRays.cu:486-549, 626-929) and the host orchestration processRaysHitLinear /
// processRaysHitData / processRaysHitPositions (processRays.cu:931-1173).
//
// The sample list (counts, offsets, ray ids, t, contracted positions, all in ray order) is the reference's, bit for
// bit; how it is produced is not:
//   * ONE walk per ray.  The reference walks every ray twice per batch (count, then emit) and, when training, walks
//     all remaining rays of the chunk again for every optimizer step.  Here the walk stores the sample distances of a
//     ray in that ray's row of a scratch matrix [ray][1024] (HBM is plentiful: 4 KB per ray) together with the count;
//     a batch is then cut out of the rows by a warp-per-ray copy that also evaluates the contracted positions.
//   * Where to cut is decided by the host from the scanned offsets, read back once per walk instead of once (the
//     reference: three times) per batch.
//   * A probe order that skips the pyramid descent inside solid regions (see walk_ray).
// The two-pass entry points (count / scan / cutoff / emit) remain for callers that want the reference's sequence.
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

constexpr uint32_t MAX_HITS = 1024;  // per-ray sample cap, modules/NeRF/InstantNerf.h:24
constexpr int MAX_MIP_LEVELS = 8;
// Hard bound on the advances of one ray.  A ray crosses at most 3 x 128 finest voxels per cascade plus its 1024 samples;
// 65536 is far beyond any walk that makes progress and only ends one that does not.
constexpr uint32_t MAX_WALK_ADVANCES = 1u << 16;

struct Scene {
    uint3 res;
    float3 aabb_min, aabb_max;
    int num_cascades, levels, spv;
    uint32_t level_offset[MAX_MIP_LEVELS];  // first cell of every pyramid level inside a cascade
    uint32_t pyramid_cells;                 // cells of one cascade's whole pyramid
    int nested;                             // every level halves the one below exactly (resolution divisible by 2^(levels-1))
};

static Scene make_scene(const nb_scene_desc* d) {
    Scene s;
    s.res = make_uint3(d->grid_res[0], d->grid_res[1], d->grid_res[2]);
    s.aabb_min = make_float3(d->aabb_min[0], d->aabb_min[1], d->aabb_min[2]);
    s.aabb_max = make_float3(d->aabb_max[0], d->aabb_max[1], d->aabb_max[2]);
    s.num_cascades = d->num_cascades; s.levels = d->mip_levels; s.spv = d->samples_per_voxel;
    uint32_t off = 0;
    uint3 r = s.res;
    for (int l = 0; l < MAX_MIP_LEVELS; l++) {
        s.level_offset[l] = off;
        if (l < s.levels) { off += r.x * r.y * r.z; r.x >>= 1; r.y >>= 1; r.z >>= 1; }
    }
    s.pyramid_cells = off;
    const uint32_t m = (1u << (s.levels - 1)) - 1u;
    s.nested = ((s.res.x & m) == 0 && (s.res.y & m) == 0 && (s.res.z & m) == 0) ? 1 : 0;
    return s;
}

__global__ void __launch_bounds__(256) ray_aabb_kernel(const uint32_t num_rays, const float3* __restrict__ rays_o,
                                                       const float3* __restrict__ rays_d, const float3 aabb_min, const float3 aabb_max,
                                                       const int num_cascades, float3* __restrict__ rays_d_inv,
                                                       float* __restrict__ nears, float* __restrict__ fars) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_rays) return;
    const float scale = exp2f((float)(num_cascades - 1));
    const float lo[3] = {aabb_min.x * scale, aabb_min.y * scale, aabb_min.z * scale};
    const float hi[3] = {aabb_max.x * scale, aabb_max.y * scale, aabb_max.z * scale};
    const float3 o3 = rays_o[i], d3 = rays_d[i];
    const float o[3] = {o3.x, o3.y, o3.z};
    float d[3] = {d3.x, d3.y, d3.z};
    float inv[3];
    float t_enter = -INFINITY, t_exit = INFINITY;
#pragma unroll
    for (int a = 0; a < 3; a++) {
        if (fabsf(d[a]) < 1e-8f) d[a] = 1e-8f;
        inv[a] = 1.0f / d[a];
        const float ta = (lo[a] - o[a]) * inv[a], tb = (hi[a] - o[a]) * inv[a];
        t_enter = fmaxf(t_enter, fminf(ta, tb));
        t_exit = fminf(t_exit, fmaxf(ta, tb));
    }
    rays_d_inv[i] = make_float3(inv[0], inv[1], inv[2]);
    const bool miss = t_enter > t_exit || t_exit < 0.0f;
    nears[i] = miss ? 0.0f : fmaxf(t_enter, 0.0f);
    fars[i] = miss ? 0.0f : t_exit;
}

// Which cascade a point belongs to: ceil(log2(largest |p| / box half-extent ratio)), modules/NeRF/processRays.cu:11-19.
__device__ __forceinline__ int get_cascade(float3 pos, float3 aabb_min, float3 aabb_max, int num_cascades) {
    const float rx = fmaxf(pos.x / aabb_max.x, pos.x / aabb_min.x);
    const float ry = fmaxf(pos.y / aabb_max.y, pos.y / aabb_min.y);
    const float rz = fmaxf(pos.z / aabb_max.z, pos.z / aabb_min.z);
    const float max_scale = fmaxf(rx, fmaxf(ry, rz));
    if (max_scale <= 1.0f) return 0;
    return max(0, min((int)ceilf(log2f(max_scale)), num_cascades - 1));
}

// The voxel of pyramid level `level` that holds the point at relative position `rel` of its cascade box: is it
// occupied, and at which ray distance does the ray leave it.
struct Probe {
    bool occupied;
    float exit_t;
};

struct RayConst {
    float3 o, d_inv;
    float3 ahead;  // 1 where the ray moves towards +axis, else 0: selects the far face of a voxel
};

__device__ __forceinline__ Probe probe_level(const Scene& sc, const RayConst& rc, const uint8_t* __restrict__ bits, int level, uint32_t cascade_base,
                                             float3 box_min, float3 box_extent, float3 rel) {
    const uint32_t rx = sc.res.x >> level, ry = sc.res.y >> level, rz = sc.res.z >> level;
    const float sx = box_extent.x / rx, sy = box_extent.y / ry, sz = box_extent.z / rz;  // voxel size
    const int vx = max(0, min((int)floorf(rel.x * rx), (int)rx - 1));
    const int vy = max(0, min((int)floorf(rel.y * ry), (int)ry - 1));
    const int vz = max(0, min((int)floorf(rel.z * rz), (int)rz - 1));
    const uint32_t cell = cascade_base + sc.level_offset[level] + vz * (rx * ry) + vy * rx + vx;
    Probe p;
    p.occupied = (bits[cell >> 3] >> (cell & 7u)) & 1u;
    const float fx = box_min.x + (vx + rc.ahead.x) * sx, fy = box_min.y + (vy + rc.ahead.y) * sy, fz = box_min.z + (vz + rc.ahead.z) * sz;
    p.exit_t = fminf(fminf((fx - rc.o.x) * rc.d_inv.x, (fy - rc.o.y) * rc.d_inv.y), (fz - rc.o.z) * rc.d_inv.z);
    return p;
}

// One ray through the occupancy pyramid.  sink(k, t) receives sample k at ray distance t; returns the sample count.
//
// The reference (march_rays_dda_calc_hits / _offset) restarts every advance at the coarsest level and descends while
// the voxel is occupied; it then either samples the occupied finest voxel or jumps to the exit of the first empty
// voxel it met.  Because a parent bit is the OR of its children, "first empty level from the top" is the same level
// whichever order the levels are looked at, so inside solid regions - where the last advance ended in an occupied
// finest voxel and the next one most likely does too - the finest level is probed first and the descent is skipped.
// That needs parent and child voxels to nest exactly (sc.nested); otherwise the reference's order is kept.
template <class Sink>
__device__ __forceinline__ uint32_t walk_ray(const Scene& sc, float3 o, float3 d, float3 d_inv, float t_begin, float t_end,
                                             const uint8_t* __restrict__ bits, Sink&& sink) {
    const float3 extent = make_float3(sc.aabb_max.x - sc.aabb_min.x, sc.aabb_max.y - sc.aabb_min.y, sc.aabb_max.z - sc.aabb_min.z);
    RayConst rc;
    rc.o = o; rc.d_inv = d_inv;
    rc.ahead = make_float3(d.x >= 0.0f ? 1.0f : 0.0f, d.y >= 0.0f ? 1.0f : 0.0f, d.z >= 0.0f ? 1.0f : 0.0f);
    const int top = sc.levels - 1;
    uint32_t count = 0;
    float t = t_begin;
    bool in_solid = false;
    uint32_t advances = 0;
    while (t < t_end && count < MAX_HITS && advances++ < MAX_WALK_ADVANCES) {
        const float3 pos = make_float3(o.x + t * d.x, o.y + t * d.y, o.z + t * d.z);
        const int cascade = get_cascade(pos, sc.aabb_min, sc.aabb_max, sc.num_cascades);
        const float cs = exp2f((float)cascade);
        const float3 box_min = make_float3(sc.aabb_min.x * cs, sc.aabb_min.y * cs, sc.aabb_min.z * cs);
        const float3 box_extent = make_float3(extent.x * cs, extent.y * cs, extent.z * cs);
        const float3 rel = make_float3((pos.x - box_min.x) / box_extent.x, (pos.y - box_min.y) / box_extent.y, (pos.z - box_min.z) / box_extent.z);
        const uint32_t cascade_base = cascade * sc.pyramid_cells;
        Probe p;
        if (in_solid && sc.nested) {
            p = probe_level(sc, rc, bits, 0, cascade_base, box_min, box_extent, rel);
            if (!p.occupied) {
                for (int l = top; l > 0; l--) {
                    const Probe q = probe_level(sc, rc, bits, l, cascade_base, box_min, box_extent, rel);
                    if (!q.occupied) { p = q; break; }
                }
            }
        } else {
            for (int l = top;; l--) {
                p = probe_level(sc, rc, bits, l, cascade_base, box_min, box_extent, rel);
                if (!p.occupied || l == 0) break;
            }
        }
        in_solid = p.occupied;
        if (p.occupied) {
            // samples_per_voxel points at the centres of equal sub-spans of [t, exit)
            const int K = sc.spv;
            const float span = p.exit_t - t;
            for (int k = 0; k < K && count < MAX_HITS; ++k) {
                sink(count, t + (k + 0.5f) / (float)K * span);
                count++;
            }
        }
        // The reference advances with exactly this expression (processRays.cu:235,733,925).  From t = 256 on the 1e-5 is
        // below half an ulp and is rounded away, and a voxel face computed a rounding error behind t (or an exit of -inf
        // from a -0.0 direction component) then leaves t where it was: the reference's loop would never end.  Where the
        // expression makes progress its value is kept bit for bit; where it does not, t moves to the next float.
        const float next = fmaxf(t + 1e-5f, p.exit_t + 1e-6f);
        t = next > t ? next : nextafterf(t, INFINITY);
    }
    return count;
}

struct CountOnly {
    __device__ __forceinline__ void operator()(uint32_t, float) const {}
};
struct RowSink {
    float* row;
    __device__ __forceinline__ void operator()(uint32_t k, float t) const { row[k] = t; }
};
// Writes a sample straight into the compacted arrays (the two-pass entry point).
struct CompactSink {
    const Scene* sc;
    float3 o, d;
    uint32_t ray_id, base;
    float* t_out;
    uint32_t* ray_out;
    float4* pos_out;
    __device__ __forceinline__ void operator()(uint32_t k, float t) const {
        const uint32_t w = base + k;
        t_out[w] = t;
        ray_out[w] = ray_id;
        const float3 p = contract_pos(make_float3(o.x + t * d.x, o.y + t * d.y, o.z + t * d.z), sc->aabb_min, sc->aabb_max);
        st_cs_v4(&pos_out[w], make_uint4(__float_as_uint(p.x), __float_as_uint(p.y), __float_as_uint(p.z), 0u));
    }
};

struct RayArrays {
    const float3* o;
    const float3* d;
    const float3* d_inv;
    const float* nears;
    const float* fars;
};

__global__ void __launch_bounds__(256) march_count_kernel(const __grid_constant__ Scene sc, const uint32_t num_rays, RayArrays r,
                                                          const uint8_t* __restrict__ bits, uint32_t* __restrict__ num_steps) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_rays) return;
    num_steps[i] = walk_ray(sc, r.o[i], r.d[i], r.d_inv[i], r.nears[i], r.fars[i], bits, CountOnly{});
}

// The single walk: sample distances of ray i into rows[i * row_stride ...], count into num_steps[i].
__global__ void __launch_bounds__(256) march_fill_kernel(const __grid_constant__ Scene sc, const uint32_t num_rays, RayArrays r,
                                                         const uint8_t* __restrict__ bits, uint32_t* __restrict__ num_steps,
                                                         float* __restrict__ rows, uint32_t row_stride) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_rays) return;
    num_steps[i] = walk_ray(sc, r.o[i], r.d[i], r.d_inv[i], r.nears[i], r.fars[i], bits, RowSink{rows + (size_t)i * row_stride});
}

// plan[0] = one past the last ray of the batch (absolute index), plan[2] = first sample of the batch.
// Rays [rays_done, plan[0]) are walked; ray ids are written relative to rays_done.
__global__ void __launch_bounds__(256) march_emit_kernel(const __grid_constant__ Scene sc, const uint32_t num_rays, const uint32_t rays_done,
                                                         RayArrays r, const uint8_t* __restrict__ bits, const uint32_t* __restrict__ ray_offsets,
                                                         const uint32_t* __restrict__ plan, float* __restrict__ t_out,
                                                         uint32_t* __restrict__ ray_idx_out, float4* __restrict__ pos_out) {
    uint32_t local = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t i = local + rays_done;
    uint32_t end = min(plan[0], num_rays);
    if (i >= end) return;
    CompactSink s{&sc, r.o[i], r.d[i], local, ray_offsets[i] - plan[2], t_out, ray_idx_out, pos_out};
    walk_ray(sc, s.o, s.d, r.d_inv[i], r.nears[i], r.fars[i], bits, s);
}

// Cuts rays [ray_begin, ray_begin + ray_count) out of the scratch rows: one warp per ray, lane k copies sample k and
// evaluates its contracted position; ray ids are relative to ray_begin, samples land at offsets[ray] - sample_base.
__global__ void __launch_bounds__(256) march_compact_kernel(const float3 aabb_min, const float3 aabb_max, const float3* __restrict__ rays_o,
                                                            const float3* __restrict__ rays_d, uint32_t ray_begin, uint32_t ray_count,
                                                            const uint32_t* __restrict__ num_steps, const uint32_t* __restrict__ offsets,
                                                            uint32_t sample_base, const float* __restrict__ rows, uint32_t row_stride,
                                                            float* __restrict__ t_out, uint32_t* __restrict__ ray_idx_out,
                                                            float4* __restrict__ pos_out) {
    const uint32_t local = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    if (local >= ray_count) return;
    const uint32_t i = ray_begin + local;
    const uint32_t count = num_steps[i];
    if (count == 0) return;
    const uint32_t dst = offsets[i] - sample_base;
    const float3 o = rays_o[i], d = rays_d[i];
    const float* row = rows + (size_t)i * row_stride;
    for (uint32_t k = lane; k < count; k += 32) {
        const float t = row[k];
        t_out[dst + k] = t;
        ray_idx_out[dst + k] = local;
        const float3 p = contract_pos(make_float3(o.x + t * d.x, o.y + t * d.y, o.z + t * d.z), aabb_min, aabb_max);
        st_cs_v4(&pos_out[dst + k], make_uint4(__float_as_uint(p.x), __float_as_uint(p.y), __float_as_uint(p.z), 0u));
    }
}

// One round of front-to-back rendering: samples [round_begin, round_begin + round_width) of every ray of
// [ray_begin, ray_begin + ray_count) that is still visible (transmittance at least 1e-4 after the rounds before) and
// has that many samples.  A block plans 256 rays (count per ray, scan, ONE atomic on the round's counter for the
// block's sample range) and its warps then copy the rays' samples out of the rows.  Sample ranges of different blocks
// land in arrival order; a ray's own samples are contiguous and in order, which is all compositing needs.
__global__ void __launch_bounds__(256) round_emit_kernel(const float3 aabb_min, const float3 aabb_max, const float3* __restrict__ rays_o,
                                                         const float3* __restrict__ rays_d, uint32_t ray_begin, uint32_t ray_count,
                                                         const uint32_t* __restrict__ num_steps, const float* __restrict__ transmittance,
                                                         uint32_t round_begin, uint32_t round_width, const float* __restrict__ rows,
                                                         uint32_t row_stride, uint32_t capacity, uint32_t* __restrict__ counter,
                                                         unsigned long long* __restrict__ emitted_total, uint32_t* __restrict__ round_off, uint32_t* __restrict__ ray_idx_out,
                                                         float4* __restrict__ pos_out) {
    __shared__ uint32_t s_warp[8], s_cnt[256], s_off[256], s_base;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t local = blockIdx.x * 256 + threadIdx.x;
    uint32_t c = 0;
    if (local < ray_count) {
        const uint32_t i = ray_begin + local;
        const uint32_t n = num_steps[i];
        const bool visible = round_begin == 0 || transmittance[i] >= 1e-4f;
        if (visible && n > round_begin) c = min(n - round_begin, round_width);
    }
    uint32_t incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t before = 0, total = 0;
#pragma unroll
    for (uint32_t w = 0; w < 8; w++) {
        const uint32_t v = s_warp[w];
        if (w < warp) before += v;
        total += v;
    }
    if (threadIdx.x == 0) {
        s_base = total ? atomicAdd(counter, total) : 0u;
        if (total && emitted_total != nullptr) atomicAdd(emitted_total, (unsigned long long)total);
    }
    s_cnt[threadIdx.x] = c;
    s_off[threadIdx.x] = before + incl - c;
    __syncthreads();
    const uint32_t base = s_base;
    if (c > 0) round_off[ray_begin + local] = base + before + incl - c;
    for (uint32_t j = warp; j < 256; j += 8) {
        const uint32_t cj = s_cnt[j];
        if (cj == 0) continue;
        const uint32_t i = ray_begin + blockIdx.x * 256 + j;
        const uint32_t dst = base + s_off[j];
        if (dst + cj > capacity) continue;  // cannot happen when the caller's bound holds; never write past the arrays
        const float3 o = rays_o[i], d = rays_d[i];
        const float* row = rows + (size_t)i * row_stride + round_begin;
        for (uint32_t k = lane; k < cj; k += 32) {
            const float t = row[k];
            ray_idx_out[dst + k] = i;
            const float3 p = contract_pos(make_float3(o.x + t * d.x, o.y + t * d.y, o.z + t * d.z), aabb_min, aabb_max);
            st_cs_v4(&pos_out[dst + k], make_uint4(__float_as_uint(p.x), __float_as_uint(p.y), __float_as_uint(p.z), 0u));
        }
    }
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
                                                                 uint32_t batch_size, uint32_t* __restrict__ plan, int write_total) {
    uint32_t gid = blockIdx.x * SCAN_BLOCK + threadIdx.x;
    if (gid >= n) return;
    uint32_t off = offsets[gid] + block_sums[blockIdx.x];
    offsets[gid] = off;
    uint32_t steps = num_steps[gid];
    if (write_total && gid == n - 1) offsets[n] = off + steps;  // offsets has n + 1 entries: the last one is the sample total
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
    if (s->num_cascades < 1 || s->mip_levels < 1 || s->mip_levels > MAX_MIP_LEVELS || s->samples_per_voxel < 1)
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
    RayArrays r{(const float3*)d_rays_o, (const float3*)d_rays_d, (const float3*)d_rays_d_inv, d_nears, d_fars};
    march_count_kernel<<<(unsigned)((num_rays + 255) / 256), 256, 0, (cudaStream_t)stream>>>(sc, (uint32_t)num_rays, r, d_bitfield, d_num_steps);
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
    if (n > 0) scan_finish_kernel<<<blocks, SCAN_BLOCK, 0, st>>>(d_ray_offsets, d_num_steps, d_block_sums, n, batch_size, d_plan, 0);
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
    RayArrays r{(const float3*)d_rays_o, (const float3*)d_rays_d, (const float3*)d_rays_d_inv, d_nears, d_fars};
    march_emit_kernel<<<(unsigned)((span + 255) / 256), 256, 0, (cudaStream_t)stream>>>(sc, (uint32_t)num_rays, rays_done, r, d_bitfield, d_ray_offsets,
                                                                                         d_plan, d_t_out, d_ray_idx_out, (float4*)d_pos4_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_march_row_stride(void) { return (int)MAX_HITS; }

extern "C" int nb_march_fill(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv,
                             const float* d_nears, const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays, uint32_t* d_num_steps,
                             float* d_t_rows, uint32_t* d_ray_offsets, uint32_t* d_block_sums, void* stream) {
    int rc = check_scene(scene, "nb_march_fill: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_rays_d_inv || !d_nears || !d_fars || !d_bitfield || !d_num_steps || !d_t_rows || !d_ray_offsets ||
        !d_block_sums || num_rays < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_march_fill: null pointer or negative ray count");
    if (num_rays > (int64_t)SCAN_BLOCK * SCAN_BLOCK) return nb_set_error(NB_ERR_LIMIT, "nb_march_fill: at most 1048576 rays per call");
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t n = (uint32_t)num_rays;
    if (n == 0) return nb_zero_async(d_ray_offsets, sizeof(uint32_t), stream);
    Scene sc = make_scene(scene);
    RayArrays r{(const float3*)d_rays_o, (const float3*)d_rays_d, (const float3*)d_rays_d_inv, d_nears, d_fars};
    march_fill_kernel<<<(n + 255) / 256, 256, 0, st>>>(sc, n, r, d_bitfield, d_num_steps, d_t_rows, MAX_HITS);
    const uint32_t blocks = (n + SCAN_BLOCK - 1) / SCAN_BLOCK;
    scan_blocks_kernel<<<blocks, SCAN_BLOCK, 0, st>>>(d_num_steps, d_ray_offsets, d_block_sums, n);
    // the plan words these kernels maintain live behind the block sums (the scratch holds 1024 + 4 words)
    scan_block_sums_kernel<<<1, SCAN_BLOCK, 0, st>>>(d_block_sums, blocks, d_block_sums + SCAN_BLOCK, 0u);
    scan_finish_kernel<<<blocks, SCAN_BLOCK, 0, st>>>(d_ray_offsets, d_num_steps, d_block_sums, n, 0xffffffffu, d_block_sums + SCAN_BLOCK, 1);
    NB_CHECK_LAUNCH();
    g_launch_count += 4;
    return NB_OK;
}

extern "C" int nb_march_compact(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, uint32_t ray_begin,
                                uint32_t ray_count, const uint32_t* d_num_steps, const uint32_t* d_ray_offsets, uint32_t sample_base,
                                const float* d_t_rows, float* d_t_out, uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream) {
    int rc = check_scene(scene, "nb_march_compact: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_num_steps || !d_ray_offsets || !d_t_rows || !d_t_out || !d_ray_idx_out || !d_pos4_out)
        return nb_set_error(NB_ERR_INVALID, "nb_march_compact: null pointer");
    if (reinterpret_cast<uintptr_t>(d_pos4_out) & 15u) return nb_set_error(NB_ERR_INVALID, "nb_march_compact: positions must be 16-byte aligned");
    if (ray_count == 0) return NB_OK;
    Scene sc = make_scene(scene);
    const uint64_t threads = (uint64_t)ray_count * 32;
    march_compact_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        sc.aabb_min, sc.aabb_max, (const float3*)d_rays_o, (const float3*)d_rays_d, ray_begin, ray_count, d_num_steps, d_ray_offsets, sample_base,
        d_t_rows, MAX_HITS, d_t_out, d_ray_idx_out, (float4*)d_pos4_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_march_round_emit(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, uint32_t ray_begin,
                                   uint32_t ray_count, const uint32_t* d_num_steps, const float* d_transmittance, uint32_t round_begin,
                                   uint32_t round_width, const float* d_t_rows, uint32_t capacity, uint32_t* d_counter,
                                   uint64_t* d_emitted_total, uint32_t* d_round_offsets, uint32_t* d_ray_idx_out, float* d_pos4_out,
                                   void* stream) {
    int rc = check_scene(scene, "nb_march_round_emit: null scene");
    if (rc) return rc;
    if (!d_rays_o || !d_rays_d || !d_num_steps || !d_t_rows || !d_counter || !d_round_offsets || !d_ray_idx_out || !d_pos4_out ||
        (round_begin > 0 && !d_transmittance))
        return nb_set_error(NB_ERR_INVALID, "nb_march_round_emit: null pointer");
    if (round_width == 0 || round_begin >= (uint32_t)MAX_HITS)
        return nb_set_error(NB_ERR_INVALID, "nb_march_round_emit: the round must lie inside a row");
    if (reinterpret_cast<uintptr_t>(d_pos4_out) & 15u)
        return nb_set_error(NB_ERR_INVALID, "nb_march_round_emit: positions must be 16-byte aligned");
    if (ray_count == 0) return NB_OK;
    Scene sc = make_scene(scene);
    round_emit_kernel<<<(ray_count + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
        sc.aabb_min, sc.aabb_max, (const float3*)d_rays_o, (const float3*)d_rays_d, ray_begin, ray_count, d_num_steps, d_transmittance, round_begin,
        round_width, d_t_rows, MAX_HITS, capacity, d_counter, (unsigned long long*)d_emitted_total, d_round_offsets, d_ray_idx_out,
        (float4*)d_pos4_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
