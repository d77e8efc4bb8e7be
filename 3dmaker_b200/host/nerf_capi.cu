// C handle API over the InstantNerf host class, for hosts that cannot include C++ headers (the Python test and
// benchmark harness binds it with ctypes).  Every function catches C++ exceptions and turns them into a status
// plus nb_last_error().
#include <cstring>
#include <exception>

#include "../csrc/common.cuh"
#include "InstantNerf.h"

static_assert(sizeof(nb_nerf_options) == sizeof(NerfOptions), "nb_nerf_options must mirror NerfOptions byte for byte");

struct nb_nerf {
    InstantNerf impl;
};

#define NB_GUARD(body)                                              \
    try {                                                           \
        body;                                                       \
        return NB_OK;                                               \
    } catch (const std::exception& e) {                             \
        return nb_set_error(NB_ERR_CUDA, e.what());                 \
    } catch (...) {                                                 \
        return nb_set_error(NB_ERR_CUDA, "unknown C++ exception"); \
    }

extern "C" int nb_nerf_default_options(nb_nerf_options* out) {
    if (!out) return nb_set_error(NB_ERR_INVALID, "nb_nerf_default_options: null pointer");
    NerfOptions d;
    std::memcpy(out, &d, sizeof(NerfOptions));
    return NB_OK;
}

extern "C" nb_nerf* nb_nerf_create(const nb_nerf_options* options, int memory_mode) {
    if (!options) { nb_set_error(NB_ERR_INVALID, "nb_nerf_create: null options"); return nullptr; }
    nb_nerf* h = nullptr;
    try {
        h = new nb_nerf();
        NerfOptions o;
        std::memcpy(&o, options, sizeof(NerfOptions));
        h->impl.init(o, memory_mode == 1 ? INFERENCE : TRAINING);
        return h;
    } catch (const std::exception& e) {
        nb_set_error(NB_ERR_CUDA, e.what());
    } catch (...) {
        nb_set_error(NB_ERR_CUDA, "unknown C++ exception");
    }
    delete h;
    return nullptr;
}

extern "C" void nb_nerf_destroy(nb_nerf* h) { delete h; }

extern "C" int nb_nerf_train_rays(nb_nerf* h, const float* d_rays_o, const float* d_rays_d, const float* d_rays_depth, const float* d_rays_sigma,
                                  const float* d_rgb_true, uint32_t num_rays, int* step_count, uint32_t* hit_counts, float* d_rgb_out, void* stream) {
    if (!h || !d_rays_o || !d_rays_d || !step_count) return nb_set_error(NB_ERR_INVALID, "nb_nerf_train_rays: null pointer");
    NB_GUARD(h->impl.trainWithRaysHit((const float3*)d_rays_o, (const float3*)d_rays_d, d_rays_depth, d_rays_sigma, d_rgb_true, num_rays, *step_count,
                                      hit_counts, d_rgb_out, (cudaStream_t)stream))
}

extern "C" int nb_nerf_render(nb_nerf* h, const float* d_rays_o, const float* d_rays_d, uint32_t num_rays, float* d_rgb_out, void* stream) {
    if (!h || !d_rays_o || !d_rays_d) return nb_set_error(NB_ERR_INVALID, "nb_nerf_render: null pointer");
    NB_GUARD(h->impl.renderImageHit((const float3*)d_rays_o, (const float3*)d_rays_d, num_rays, d_rgb_out, (cudaStream_t)stream))
}

extern "C" int nb_nerf_set_learning_rate(nb_nerf* h, float lr) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setLearningRate(lr);
    return NB_OK;
}

extern "C" int nb_nerf_set_bg_color(nb_nerf* h, float r, float g, float b) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setBgColor(make_float3(r, g, b));
    return NB_OK;
}

extern "C" int nb_nerf_set_profiling(nb_nerf* h, int on) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setProfiling(on != 0);
    return NB_OK;
}

extern "C" int nb_nerf_set_memory_mode(nb_nerf* h, int memory_mode) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    NB_GUARD(h->impl.setMemoryMode(memory_mode == 1 ? INFERENCE : TRAINING))
}

extern "C" int nb_nerf_set_global_ray_scale(nb_nerf* h, uint32_t scale) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setGlobalRayScale(scale);
    return NB_OK;
}

extern "C" int nb_nerf_set_single_step(nb_nerf* h, int on) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setSingleStep(on != 0);
    return NB_OK;
}

extern "C" int nb_nerf_set_steps_per_call(nb_nerf* h, int steps) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setStepsPerCall(steps);
    return NB_OK;
}

extern "C" int nb_nerf_set_optimizer_shard(nb_nerf* h, uint32_t rank, uint32_t world, nb_param_sync_fn fn, void* user) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (world > 1 && !fn) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_optimizer_shard: a parameter-sync callback is required");
    NB_GUARD(h->impl.setOptimizerShard(rank, world, [fn, user](half* p, int64_t count, cudaStream_t st) { fn(user, p, count, st); }))
}

extern "C" int nb_nerf_set_peer_exchange(nb_nerf* h, uint32_t rank, uint32_t world, const float* const* peer_grads, void* const* peer_w_h,
                                         nb_barrier_fn fn, void* user) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (world > 1 && (!peer_grads || !peer_w_h || !fn)) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_peer_exchange: peer pointers and a barrier are required");
    std::vector<const float*> g;
    std::vector<void*> p;
    for (uint32_t r = 0; world > 1 && r < world; r++) { g.push_back(peer_grads[r]); p.push_back(peer_w_h[r]); }
    NB_GUARD(h->impl.setPeerExchange(rank, world, g, p, [fn, user](cudaStream_t st) { fn(user, st); }))
}

extern "C" int nb_nerf_set_level_partition(nb_nerf* h, uint32_t rank, uint32_t world, nb_block_fn gather, nb_block_fn exchange, nb_grad_sync_fn reduce,
                                           void* user) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (world > 1 && (!gather || !exchange || !reduce)) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_level_partition: the three collectives are required");
    if (world <= 1) { NB_GUARD(h->impl.setLevelPartition(0, 1, nullptr, nullptr, nullptr)) }
    NB_GUARD(h->impl.setLevelPartition(
        rank, world, [gather, user](const void* s, void* r, int64_t bytes, cudaStream_t st) { gather(user, s, r, bytes, st); },
        [exchange, user](const void* s, void* r, int64_t bytes, cudaStream_t st) { exchange(user, s, r, bytes, st); },
        [reduce, user](float* g, int64_t count, cudaStream_t st) { reduce(user, g, count, st); }))
}

extern "C" int nb_nerf_set_occupancy_shard(nb_nerf* h, uint32_t rank, uint32_t world, nb_grad_sync_fn reduce_max, void* user) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (world <= 1) { NB_GUARD(h->impl.setOccupancyShard(0, 1, nullptr)) }
    if (!reduce_max) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_occupancy_shard: a MAX all-reduce is required");
    NB_GUARD(h->impl.setOccupancyShard(rank, world, [reduce_max, user](float* g, int64_t count, cudaStream_t st) { reduce_max(user, g, count, st); }))
}

extern "C" int nb_nerf_sync_levels(nb_nerf* h, int master, void* stream) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    NB_GUARD(h->impl.syncLevels((cudaStream_t)stream, master != 0))
}

extern "C" int nb_nerf_set_hit_counts_capacity(nb_nerf* h, uint32_t capacity) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setHitCountsCapacity(capacity);
    return NB_OK;
}

extern "C" int nb_nerf_set_fused_field(nb_nerf* h, int on) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    return h->impl.setFusedField(on != 0) ? 1 : 0;
}

extern "C" int nb_nerf_set_render_rounds(nb_nerf* h, int on) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    h->impl.setRenderRounds(on != 0);
    return h->impl.renderRounds() ? 1 : 0;
}

extern "C" int nb_nerf_last_render_samples(nb_nerf* h, uint64_t* samples) {
    if (!h || !samples) return nb_set_error(NB_ERR_INVALID, "nb_nerf_last_render_samples: null pointer");
    NB_GUARD(*samples = h->impl.lastRenderSamples())
}

extern "C" int nb_nerf_set_grad_sync(nb_nerf* h, nb_grad_sync_fn fn, void* user) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (!fn) h->impl.setGradSync(nullptr);
    else h->impl.setGradSync([fn, user](float* g, int64_t count, cudaStream_t s) { fn(user, g, count, (void*)s); });
    return NB_OK;
}

extern "C" int nb_nerf_set_grad_buffer(nb_nerf* h, float* d_grads, int64_t count) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    nb::ParamArena& a = h->impl.arena();
    if (d_grads && count < a.total) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_grad_buffer: the buffer is smaller than the parameter arena");
    if (reinterpret_cast<uintptr_t>(d_grads) & 15u) return nb_set_error(NB_ERR_INVALID, "nb_nerf_set_grad_buffer: the buffer must be 16-byte aligned");
    NB_GUARD(a.set_external_grad(d_grads))
}

extern "C" int nb_nerf_get_arena(nb_nerf* h, nb_nerf_arena_view* out) {
    if (!h || !out) return nb_set_error(NB_ERR_INVALID, "nb_nerf_get_arena: null pointer");
    nb::ParamArena& a = h->impl.arena();
    out->w = a.W(); out->w_h = a.Wh(); out->g = a.training ? a.G() : nullptr; out->m = a.training ? a.M() : nullptr;
    out->v = a.training ? a.V() : nullptr;
    out->total = a.total; out->sparse_count = a.sparse_count;
    out->density_weight_offset = h->impl.densityNetwork()->weightOffset(); out->density_bias_offset = h->impl.densityNetwork()->biasOffset();
    out->color_weight_offset = h->impl.colorNetwork()->weightOffset(); out->color_bias_offset = h->impl.colorNetwork()->biasOffset();
    out->density_weight_count = h->impl.densityNetwork()->weightCount(); out->density_bias_count = h->impl.densityNetwork()->biasCount();
    out->color_weight_count = h->impl.colorNetwork()->weightCount(); out->color_bias_count = h->impl.colorNetwork()->biasCount();
    return NB_OK;
}

extern "C" int nb_nerf_load_params(nb_nerf* h, const float* hash, const float* density_w, const float* density_b, const float* color_w,
                                   const float* color_b) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    NB_GUARD({
        if (hash) h->impl.densityNetwork()->loadHashgrid(hash);
        if (density_w && density_b) h->impl.densityNetwork()->loadWeights(density_w, density_b);
        if (color_w && color_b) h->impl.colorNetwork()->loadWeights(color_w, color_b);
    })
}

extern "C" int nb_nerf_occupancy(nb_nerf* h, uint8_t** d_bitfield, int64_t* bitfield_bytes, float** d_master_grid) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    if (d_bitfield) *d_bitfield = h->impl.occupancyGridMutable();
    if (bitfield_bytes) *bitfield_bytes = (int64_t)h->impl.occupancyBytes();
    if (d_master_grid) *d_master_grid = h->impl.masterOccupancyGrid();
    return NB_OK;
}

extern "C" int nb_nerf_rebuild_occupancy(nb_nerf* h, void* stream) {
    if (!h) return nb_set_error(NB_ERR_INVALID, "null handle");
    NB_GUARD(h->impl.rebuildOccupancy((cudaStream_t)stream))
}

extern "C" int nb_nerf_get_step_view(nb_nerf* h, nb_nerf_step_view* out) {
    if (!h || !out) return nb_set_error(NB_ERR_INVALID, "nb_nerf_get_step_view: null pointer");
    InstantNerf::StepView v = h->impl.stepView();
    out->num_steps = v.num_steps; out->ray_offsets = v.ray_offsets; out->ray_indices = v.ray_indices; out->t_sorted = v.t_sorted;
    out->positions = v.positions; out->density_out = v.density_out; out->sigma = v.sigma; out->color_out = v.color_out;
    out->render_rgb = v.render_rgb; out->phi = v.phi; out->dw = v.dw; out->weight_sum = v.weight_sum; out->tmp_dsigma = v.tmp_dsigma;
    out->color_in = v.color_in; out->color_grad = v.color_grad; out->density_grad = v.density_grad;
    out->last_total_hits = h->impl.lastTotalHits(); out->train_steps = h->impl.trainSteps();
    out->logit_stride = v.logit_stride; out->color_stride = v.color_stride; out->rays_consumed = h->impl.lastRaysConsumed(); out->sample_base = v.sample_base;
    return NB_OK;
}

extern "C" int nb_nerf_phase_times(nb_nerf* h, double* out_ms12, int64_t* steps) {
    if (!h || !out_ms12) return nb_set_error(NB_ERR_INVALID, "nb_nerf_phase_times: null pointer");
    const NerfPhaseTimes& t = h->impl.phaseTimes();
    const double v[12] = {t.march, t.occupancy, t.densityFwd, t.shGather, t.colorFwd, t.compositing, t.lossGrad, t.colorBwd, t.densityGrad, t.densityBwd,
                          t.scatter, t.optimizer};
    std::memcpy(out_ms12, v, sizeof(v));
    if (steps) *steps = t.steps;
    return NB_OK;
}

extern "C" int nb_nerf_save(nb_nerf* h, const char* path) {
    if (!h || !path) return nb_set_error(NB_ERR_INVALID, "nb_nerf_save: null pointer");
    NB_GUARD(h->impl.save(path))
}

extern "C" int nb_nerf_load(nb_nerf* h, const char* path) {
    if (!h || !path) return nb_set_error(NB_ERR_INVALID, "nb_nerf_load: null pointer");
    NB_GUARD(h->impl.load(path))
}
