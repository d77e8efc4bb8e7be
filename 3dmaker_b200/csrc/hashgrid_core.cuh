// Device pieces of the multiresolution hash grid shared by the stand-alone and the fused kernels: level geometry,
// corner indices and weights of one (point, level), the fixed-order trilinear blend and the CTA-wide encode of a
// 128-point tile into shared memory.  Arithmetic follows modules/TinyMLP/networkFusionHashtable.cu:62-70,111-222.
#pragma once

#include <atomic>

#include "mlp_core.cuh"

namespace nb {

extern std::atomic<int> g_pair_ops;   // nb_set_tuning("pair_ops", ...)
extern std::atomic<int> g_run_merge;  // nb_set_tuning("scatter_run_merge", ...)
extern std::atomic<int> g_grad_table_half;        // nb_set_tuning("grad_table_half", ...)
extern std::atomic<int> g_grad_table_scale_log2;  // nb_set_tuning("grad_table_scale_log2", ...)
inline float grad_table_scale() { return g_grad_table_half.load() ? (float)(1u << g_grad_table_scale_log2.load()) : 1.0f; }

struct GridParams {
    int L, T, dls;
    int ls;        // entries between the starts of consecutive levels in the table and its gradient: T for a whole grid,
                   // ranks * T for the view of the levels one rank owns (level_view)
    int run_merge; // > 0: the gradient scatter sums runs of consecutive samples in one cell before reducing, in warps that
                   // have at most this many runs (merging costs about 300 instructions per warp and level)
    int pair_ops;  // non-zero: the two x-neighbours of a corner pair that share an aligned slot pair move as one access
    int grad_half; // non-zero: the table gradient is one __half2 per entry (4 bytes), every contribution multiplied by
    float grad_scale;  // grad_scale before it is rounded to fp16; zero: two floats per entry, unscaled
    float scales[NB_MAX_LEVELS];   // forward (encode) resolutions
    float sscales[NB_MAX_LEVELS];  // resolutions of the gradient scatter
};

inline GridParams make_params(const nb_grid_desc* d) {
    GridParams p;
    p.L = d->num_levels; p.T = d->table_size; p.ls = d->table_size; p.dls = d->dense_level_start; p.pair_ops = g_pair_ops.load(); p.run_merge = g_run_merge.load();
    p.grad_half = g_grad_table_half.load() != 0; p.grad_scale = grad_table_scale();
    for (int i = 0; i < NB_MAX_LEVELS; i++) { p.scales[i] = d->scales[i]; p.sscales[i] = d->scatter_scales[i]; }
    return p;
}

// The grid as the owner of levels rank, rank + ranks, rank + 2 ranks, ... sees it: those levels renumbered 0, 1, ...,
// resolutions picked accordingly, consecutive levels ranks * T entries apart.  Pointers into the table or its gradient
// that go with this view start at level `rank` (first_level_offset entries into the array).  Dense levels stay a prefix
// because resolutions grow with the level.
inline GridParams level_view(const GridParams& whole, int rank, int ranks) {
    GridParams p = whole;
    p.L = whole.L / ranks;
    p.ls = whole.T * ranks;
    p.dls = 0;
    for (int k = 0; k < p.L; k++) {
        const int l = rank + k * ranks;
        p.scales[k] = whole.scales[l]; p.sscales[k] = whole.sscales[l];
        if (l < whole.dls) p.dls = k + 1;
    }
    return p;
}

__device__ __forceinline__ uint32_t hash_coords(int cx, int cy, int cz, int T) {
    return ((static_cast<uint32_t>(cx) * 1U) ^ (static_cast<uint32_t>(cy) * 2654435761U) ^
            (static_cast<uint32_t>(cz) * 805459861U)) & static_cast<uint32_t>(T - 1);
}
__device__ __forceinline__ uint32_t dense_index(int cx, int cy, int cz, int N_l) {
    return cx + cy * (N_l + 1) + cz * (N_l + 1) * (N_l + 1);
}

struct Corners {
    uint32_t idx[8];  // entry index inside the level (pairs of features), corner order 000,100,010,110,001,101,011,111
    float wx1, wy1, wz1;
    uint32_t cell;    // the low corner (x0 | y0 << 10 | z0 << 20) when the level has fewer than 1024 cells per axis, else ~0
};

// BWD_CLAMP = false: low corner clamped to [0, N_l] (forward); true: to [0, N_l - 1] (backward).
template <bool BWD_CLAMP>
__device__ __forceinline__ void corners_of(float px, float py, float pz, float scale, bool dense, int T, Corners& c) {
    int N_l = __float2int_rd(scale);
    float x_l = px * scale, y_l = py * scale, z_l = pz * scale;
    int x0 = __float2int_rd(x_l), y0 = __float2int_rd(y_l), z0 = __float2int_rd(z_l);
    const int hi = BWD_CLAMP ? N_l - 1 : N_l;
    x0 = max(0, min(x0, hi)); y0 = max(0, min(y0, hi)); z0 = max(0, min(z0, hi));
    int x1 = min(x0 + 1, N_l), y1 = min(y0 + 1, N_l), z1 = min(z0 + 1, N_l);
    c.cell = (N_l < 1024) ? ((uint32_t)x0 | ((uint32_t)y0 << 10) | ((uint32_t)z0 << 20)) : 0xffffffffu;
    c.wx1 = 1.0f - x_l + floorf(x_l);
    c.wy1 = 1.0f - y_l + floorf(y_l);
    c.wz1 = 1.0f - z_l + floorf(z_l);
    if (dense) {
        c.idx[0] = dense_index(x0, y0, z0, N_l); c.idx[1] = dense_index(x1, y0, z0, N_l);
        c.idx[2] = dense_index(x0, y1, z0, N_l); c.idx[3] = dense_index(x1, y1, z0, N_l);
        c.idx[4] = dense_index(x0, y0, z1, N_l); c.idx[5] = dense_index(x1, y0, z1, N_l);
        c.idx[6] = dense_index(x0, y1, z1, N_l); c.idx[7] = dense_index(x1, y1, z1, N_l);
    } else {
        c.idx[0] = hash_coords(x0, y0, z0, T); c.idx[1] = hash_coords(x1, y0, z0, T);
        c.idx[2] = hash_coords(x0, y1, z0, T); c.idx[3] = hash_coords(x1, y1, z0, T);
        c.idx[4] = hash_coords(x0, y0, z1, T); c.idx[5] = hash_coords(x1, y0, z1, T);
        c.idx[6] = hash_coords(x0, y1, z1, T); c.idx[7] = hash_coords(x1, y1, z1, T);
    }
}

__device__ __forceinline__ void corner_weights(const Corners& c, float (&w)[8]) {
    const float wx1 = c.wx1, wy1 = c.wy1, wz1 = c.wz1;
    w[0] = wx1 * wy1 * wz1;                   w[1] = (1 - wx1) * wy1 * wz1;
    w[2] = wx1 * (1 - wy1) * wz1;             w[3] = (1 - wx1) * (1 - wy1) * wz1;
    w[4] = wx1 * wy1 * (1 - wz1);             w[5] = (1 - wx1) * wy1 * (1 - wz1);
    w[6] = wx1 * (1 - wy1) * (1 - wz1);       w[7] = (1 - wx1) * (1 - wy1) * (1 - wz1);
}

// The 8 corner entries (feature pairs) of one level.  Corners 2j and 2j+1 differ in x only; whenever their indices
// differ in the lowest bit only (every even x0 on a hashed level, since the x prime is 1; every even low index on a
// dense level) both sit in one aligned 8-byte slot pair and are fetched with one load.
__device__ __forceinline__ void gather_corners(const uint32_t* __restrict__ tl, const Corners& c, bool pair_ops, uint32_t (&f)[8]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t a = c.idx[2 * j], b = c.idx[2 * j + 1];
        if (pair_ops && ((a ^ b) == 1u)) {
            uint2 v = __ldg(reinterpret_cast<const uint2*>(tl + (a & ~1u)));
            const bool a_hi = (a & 1u) != 0;
            f[2 * j] = a_hi ? v.y : v.x;
            f[2 * j + 1] = a_hi ? v.x : v.y;
        } else {
            f[2 * j] = __ldg(tl + a);
            f[2 * j + 1] = __ldg(tl + b);
        }
    }
}

// Fixed-order blend of the reference (networkFusionHashtable.cu:185-201), both features.
__device__ __forceinline__ uint32_t blend(const uint32_t (&f)[8], const float (&w)[8]) {
    float2 v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = unpack_half2(f[k]);
    float rx = v[7].x * w[7], ry = v[7].y * w[7];
#pragma unroll
    for (int k = 6; k >= 0; k--) {
        rx = __fmaf_rn(v[k].x, w[k], rx);
        ry = __fmaf_rn(v[k].y, w[k], ry);
    }
    return pack_half2(rx, ry);
}

// Encodes the CTA's 128 points into the shared tile: tile[r][2l .. 2l+1].
template <int TILE_STRIDE>
__device__ __forceinline__ void encode_tile(const GridParams& gp, const float* __restrict__ pos4, const uint32_t* __restrict__ table2,
                                            int64_t row_base, int64_t n, __half* tile, int tid) {
    const int r = tid & (TILE_ROWS - 1);
    const int half_sel = tid >> 7;  // 0 or 1: which half of the levels
    const int lpt = gp.L >> 1;      // levels per thread
    const int64_t row = row_base + r;
    if (row < n) {
        float4 p = ld_nc_f4(pos4 + row * 4);
        for (int li = 0; li < lpt; li += 2) {
            const int la = half_sel * lpt + li, lb = la + 1;
            const bool has_b = (li + 1) < lpt;
            Corners ca, cb;
            corners_of<false>(p.x, p.y, p.z, gp.scales[la], la < gp.dls, gp.T, ca);
            corners_of<false>(p.x, p.y, p.z, gp.scales[has_b ? lb : la], (has_b ? lb : la) < gp.dls, gp.T, cb);
            const uint32_t* ta = table2 + (size_t)la * gp.ls;
            const uint32_t* tb = table2 + (size_t)(has_b ? lb : la) * gp.ls;
            uint32_t fa[8], fb[8];
            gather_corners(ta, ca, gp.pair_ops != 0, fa);
            gather_corners(tb, cb, gp.pair_ops != 0, fb);
            float wa[8], wb[8];
            corner_weights(ca, wa);
            corner_weights(cb, wb);
            *reinterpret_cast<uint32_t*>(&tile[r * TILE_STRIDE + 2 * la]) = blend(fa, wa);
            if (has_b) *reinterpret_cast<uint32_t*>(&tile[r * TILE_STRIDE + 2 * lb]) = blend(fb, wb);
        }
    } else {
        for (int li = 0; li < lpt; li++)
            *reinterpret_cast<uint32_t*>(&tile[r * TILE_STRIDE + 2 * (half_sel * lpt + li)]) = 0u;
    }
}

// The 8 reductions of one (sample, level): v[2k], v[2k+1] = the two features' contributions to corner k.
__device__ __forceinline__ void reduce_corners(const Corners& c, const float (&v)[16], bool pair_ops, float* __restrict__ base) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t a = c.idx[2 * j], b = c.idx[2 * j + 1];
        if (pair_ops && ((a ^ b) == 1u)) {
            // x-neighbours in one aligned slot pair: one 16-byte reduction instead of two 8-byte ones
            const bool a_hi = (a & 1u) != 0;
            red_add_v4(base + (size_t)(a & ~1u) * 2, a_hi ? v[4 * j + 2] : v[4 * j], a_hi ? v[4 * j + 3] : v[4 * j + 1],
                       a_hi ? v[4 * j] : v[4 * j + 2], a_hi ? v[4 * j + 1] : v[4 * j + 3]);
        } else {
            red_add_v2(base + (size_t)a * 2, v[4 * j], v[4 * j + 1]);
            red_add_v2(base + (size_t)b * 2, v[4 * j + 2], v[4 * j + 3]);
        }
    }
}

// The same into the half-precision table (one 4-byte entry per corner), contributions scaled before rounding.
__device__ __forceinline__ void reduce_corners_half(const Corners& c, const float (&v)[16], bool pair_ops, float s, uint32_t* __restrict__ base) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t a = c.idx[2 * j], b = c.idx[2 * j + 1];
        const uint32_t va = pack_half2(v[4 * j] * s, v[4 * j + 1] * s), vb = pack_half2(v[4 * j + 2] * s, v[4 * j + 3] * s);
        if (pair_ops && ((a ^ b) == 1u)) {
            const bool a_hi = (a & 1u) != 0;
            red_add_h2x2(base + (a & ~1u), a_hi ? vb : va, a_hi ? va : vb);
        } else {
            red_add_h2(base + a, va);
            red_add_h2(base + b, vb);
        }
    }
}

// Adds the gradient of one level (feature pair g) of the warp's 32 samples to the fp32 table gradient: 8 corner
// entries per sample.  Backward clamp and scatter resolution as hashTableScatter_Backward
// (networkFusionBackwardHashtable.cu:797-900).  ALL 32 LANES MUST CALL; lanes without a sample pass active = false.
//
// Samples arrive in ray order, and on the coarser levels a ray stays inside one cell for many consecutive samples.
// Lanes that follow each other in the same cell form a run; when the warp has few runs their 16 contributions are
// summed across the run with shuffles and only the run's first lane issues reductions (the reference merges equal
// addresses inside a warp on its dense levels for the same reason, networkFusionBackwardHashtable.cu:843-887).
// Scattered positions (most lanes in different cells) take the direct path.
// sink(c, v) adds v[2k], v[2k+1] to corner k's entry.
template <class Sink>
__device__ __forceinline__ void scatter_runs(const GridParams& gp, const Corners& c, float2 g, bool active, int lane, Sink&& sink) {
    float w[8];
    corner_weights(c, w);
    active = active && (g.x != 0.f || g.y != 0.f);
    // inactive lanes and levels too fine for a cell key never merge: a key no other lane has
    const uint32_t key = (active && c.cell != 0xffffffffu) ? c.cell : (0xc0000000u | (uint32_t)lane);
    const uint32_t below = __shfl_up_sync(0xffffffffu, key, 1);
    const bool head = lane == 0 || key != below;
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    float v[16];
#pragma unroll
    for (int k = 0; k < 8; k++) { v[2 * k] = g.x * w[k]; v[2 * k + 1] = g.y * w[k]; }
    if (__popc(heads) > gp.run_merge) {
        if (active) sink(c, v);
        return;
    }
    const int run = __popc(heads & (0xffffffffu >> (31 - lane)));  // index of this lane's run
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int other = __shfl_down_sync(0xffffffffu, run, o);
        const bool same = (lane + o < 32) && other == run;
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const float n = __shfl_down_sync(0xffffffffu, v[k], o);
            if (same) v[k] += n;
        }
    }
    if (head && active) sink(c, v);
}

template <class Sink>
__device__ __forceinline__ void scatter_level_runs(const GridParams& gp, int level, float px, float py, float pz, float2 g, bool active, int lane,
                                                   Sink&& sink) {
    Corners c;
    corners_of<true>(px, py, pz, gp.sscales[level], level < gp.dls, gp.T, c);
    scatter_runs(gp, c, g, active, lane, sink);
}

// GRAD_HALF is a compile-time choice (kernels exist in both forms and the launchers pick by gp.grad_half): the scatter
// is unrolled over 16 levels inside the field kernels and a run-time branch here doubles that code.
template <bool GRAD_HALF = false>
__device__ __forceinline__ void scatter_level_warp(const GridParams& gp, int level, float px, float py, float pz, float2 g, bool active,
                                                   float* __restrict__ grads, int lane) {
    const bool pair_ops = gp.pair_ops != 0;
    if constexpr (GRAD_HALF) {
        uint32_t* base = reinterpret_cast<uint32_t*>(grads) + (size_t)level * gp.ls;
        const float s = gp.grad_scale;
        scatter_level_runs(gp, level, px, py, pz, g, active, lane,
                           [&](const Corners& c, const float (&v)[16]) { reduce_corners_half(c, v, pair_ops, s, base); });
    } else {
        float* base = grads + (size_t)level * gp.ls * 2;
        scatter_level_runs(gp, level, px, py, pz, g, active, lane, [&](const Corners& c, const float (&v)[16]) { reduce_corners(c, v, pair_ops, base); });
    }
}

// ---- coarse levels from shared memory ------------------------------------------------------------------------------
// When the samples a CTA works on lie close together, the corners they touch on a coarse level form a small box of the
// level's grid.  The CTA then copies that box into shared memory once (forward) or accumulates into it and adds it to the
// table gradient once (backward) instead of going to L2 eight times per sample and level.  Which levels are staged is
// decided per group of tiles from the bounding box of the group's positions: levels 0, 1, ... as long as their boxes fit
// the capacity.  Works for any sample order; nb_sample_order makes the boxes small.
struct StagePlan {
    int count;                                  // levels [0, count) are staged
    int ox[NB_MAX_LEVELS], oy[NB_MAX_LEVELS], oz[NB_MAX_LEVELS];   // lowest corner of the box, in corner coordinates
    int w[NB_MAX_LEVELS], wh[NB_MAX_LEVELS], whd[NB_MAX_LEVELS];   // extent in x, x * y, x * y * z (= entries)
    int h[NB_MAX_LEVELS], d[NB_MAX_LEVELS];                        // extent in y and z
    int base[NB_MAX_LEVELS];                    // first entry of the level in the staging array
};

// Low / high corner coordinates and interpolation weights of a point on one level (the arithmetic of corners_of).
struct CornerBox {
    int x0, y0, z0, x1, y1, z1, N_l;
    float wx1, wy1, wz1;
};

template <bool BWD_CLAMP>
__device__ __forceinline__ void corner_box(float px, float py, float pz, float scale, CornerBox& b) {
    const int N_l = __float2int_rd(scale);
    const float x_l = px * scale, y_l = py * scale, z_l = pz * scale;
    const int hi = BWD_CLAMP ? N_l - 1 : N_l;
    b.N_l = N_l;
    b.x0 = max(0, min(__float2int_rd(x_l), hi)); b.y0 = max(0, min(__float2int_rd(y_l), hi)); b.z0 = max(0, min(__float2int_rd(z_l), hi));
    b.x1 = min(b.x0 + 1, N_l); b.y1 = min(b.y0 + 1, N_l); b.z1 = min(b.z0 + 1, N_l);
    b.wx1 = 1.0f - x_l + floorf(x_l);
    b.wy1 = 1.0f - y_l + floorf(y_l);
    b.wz1 = 1.0f - z_l + floorf(z_l);
}

// Entry index of corner (x, y, z) inside its level.
__device__ __forceinline__ uint32_t level_index(int x, int y, int z, int N_l, bool dense, int T) {
    return dense ? dense_index(x, y, z, N_l) : hash_coords(x, y, z, T);
}

__device__ __forceinline__ void corners_from_box(const CornerBox& b, bool dense, int T, Corners& c) {
    c.wx1 = b.wx1; c.wy1 = b.wy1; c.wz1 = b.wz1;
    c.cell = (b.N_l < 1024) ? ((uint32_t)b.x0 | ((uint32_t)b.y0 << 10) | ((uint32_t)b.z0 << 20)) : 0xffffffffu;
#pragma unroll
    for (int k = 0; k < 8; k++) c.idx[k] = level_index((k & 1) ? b.x1 : b.x0, (k & 2) ? b.y1 : b.y0, (k & 4) ? b.z1 : b.z0, b.N_l, dense, T);
}

// True when all 8 corners of the point lie inside the staged box of the level; loc[k] = their places in the staging array.
__device__ __forceinline__ bool staged_corners(const StagePlan& pl, int level, const CornerBox& b, int (&loc)[8]) {
    const int lx0 = b.x0 - pl.ox[level], ly0 = b.y0 - pl.oy[level], lz0 = b.z0 - pl.oz[level];
    const int lx1 = b.x1 - pl.ox[level], ly1 = b.y1 - pl.oy[level], lz1 = b.z1 - pl.oz[level];
    const int w = pl.w[level], wh = pl.wh[level], h = pl.h[level], d = pl.d[level];
    if (lx0 < 0 || ly0 < 0 || lz0 < 0 || lx1 >= w || ly1 >= h || lz1 >= d) return false;
#pragma unroll
    for (int k = 0; k < 8; k++) loc[k] = pl.base[level] + ((k & 1) ? lx1 : lx0) + ((k & 2) ? ly1 : ly0) * w + ((k & 4) ? lz1 : lz0) * wh;
    return true;
}

// Block-wide: bounding box of the positions of rows [row_first, row_first + rows) (through perm when given), then the
// staging plan of levels 0, 1, ... while their boxes fit `capacity` entries.  s_box: 6 floats of shared memory.
// All THREADS threads of the group must call (tid = 0 .. THREADS - 1, whole warps); `barrier()` synchronises exactly
// them; ends with a barrier.  BWD_CLAMP selects the backward's clamp and resolutions.
template <bool BWD_CLAMP, int THREADS, class Barrier>
__device__ __forceinline__ void plan_stage(const GridParams& gp, const float* __restrict__ pos4, const uint32_t* __restrict__ perm,
                                           int64_t row_first, int rows, int64_t n, int capacity, int max_levels, float* s_box, StagePlan& pl,
                                           int tid, Barrier&& barrier) {
    float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
    for (int r = tid; r < rows; r += THREADS) {
        const int64_t row = row_first + r;
        if (row < n) {
            const int64_t s = perm ? (int64_t)perm[row] : row;
            const float4 p = ld_nc_f4(pos4 + s * 4);
            lo[0] = fminf(lo[0], p.x); lo[1] = fminf(lo[1], p.y); lo[2] = fminf(lo[2], p.z);
            hi[0] = fmaxf(hi[0], p.x); hi[1] = fmaxf(hi[1], p.y); hi[2] = fmaxf(hi[2], p.z);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; a++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[a] = fminf(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], o));
            hi[a] = fmaxf(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], o));
        }
    if (tid < 6) s_box[tid] = tid < 3 ? INFINITY : -INFINITY;
    barrier();
    if ((tid & 31) == 0) {
        // float min / max through the integer atomics: order-preserving for non-negative values, and a box that comes out
        // too large (negative or non-finite coordinates) only means fewer levels are staged
#pragma unroll
        for (int a = 0; a < 3; a++) {
            atomicMin(reinterpret_cast<int*>(&s_box[a]), __float_as_int(fmaxf(lo[a], 0.0f)));
            atomicMax(reinterpret_cast<int*>(&s_box[3 + a]), __float_as_int(fmaxf(hi[a], 0.0f)));
        }
    }
    barrier();
    if (tid < gp.L && tid < max_levels) {
        const int l = tid;
        const float scale = BWD_CLAMP ? gp.sscales[l] : gp.scales[l];
        CornerBox a, b;
        corner_box<BWD_CLAMP>(s_box[0], s_box[1], s_box[2], scale, a);
        corner_box<BWD_CLAMP>(s_box[3], s_box[4], s_box[5], scale, b);
        pl.ox[l] = a.x0; pl.oy[l] = a.y0; pl.oz[l] = a.z0;
        const int w = b.x1 - a.x0 + 1, h = b.y1 - a.y0 + 1, d = b.z1 - a.z0 + 1;
        const bool sane = w > 0 && h > 0 && d > 0 && w <= 1024 && h <= 1024 && d <= 1024;
        pl.w[l] = sane ? w : 1; pl.wh[l] = sane ? w * h : 1; pl.h[l] = sane ? h : 1; pl.d[l] = sane ? d : 1;
        pl.whd[l] = (sane && (int64_t)w * h * d <= capacity) ? w * h * d : capacity + 1;
    }
    barrier();
    if (tid == 0) {
        int used = 0, count = 0;
        const int top = min(gp.L, max_levels);
        while (count < top && used + pl.whd[count] <= capacity) { pl.base[count] = used; used += pl.whd[count]; count++; }
        pl.count = count;
    }
    barrier();
}

// Host side of the stand-alone scatter (hashgrid.cu): levels [level_begin, level_end) from a gradient matrix whose
// rows are denc_stride halves apart.  scatter_shared_levels = how many leading levels of a launch over n samples go
// through the shared-memory accumulation kernel.
int scatter_shared_levels(const GridParams& gp, int64_t n);
int scatter_launch(const GridParams& gp, const float* d_pos4, const __half* d_denc, int denc_stride, int64_t n, float* d_table_grads,
                   int level_begin, int level_end, cudaStream_t st);
// The same for the owner of some levels of a level-partitioned grid (level_partition.cu): `view` = level_view of the
// grid, samples of all ranks from the gathered position slots, gradients from the received pieces.
int scatter_launch_pieces(const GridParams& view, const float* d_pos_all, const uint32_t* d_pieces, int ranks, int own, int64_t cap,
                          float* d_table_grads_view, cudaStream_t st);

// Coalesced write of the encoded tile (128 x 2L halves) to global memory.
template <int TILE_STRIDE>
__device__ __forceinline__ void store_enc_tile(const __half* tile, __half* __restrict__ enc_out, int L, int64_t row_base, int64_t n,
                                               int tid) {
    const int cpr = (2 * L) / 8;
    for (int c = tid; c < TILE_ROWS * cpr; c += CTA_THREADS) {
        int r = c / cpr, c8 = c % cpr;
        if (row_base + r < n) {
            uint4 v = *reinterpret_cast<const uint4*>(&tile[r * TILE_STRIDE + c8 * 8]);
            st_cs_v4(&enc_out[(row_base + r) * (2 * L) + c8 * 8], v);
        }
    }
}

}  // namespace nb
