// InstantNerf over the C ABI.  Step and frame orchestration follow the reference
// (modules/NeRF/InstantNerf.cu:150-339 set-up, :359-583 training, :713-864 rendering, :1009-1204 occupancy,
// :1206-1352 file format) with these deliberate differences:
//   * the networks run forward ONCE per step (the reference runs an inference pass for the rendered colour and a
//     second, activation-saving pass for backward; both compute the same values);
//   * the cutoff / sample total of a batch come back in one 16-byte pinned read (the reference blocks three times);
//   * the colour network's padded [n][8] output and gradient are consumed in place (no pad / un-pad kernels);
//   * both networks share one parameter arena: one gradient buffer, one Adam launch, MLP gradients zeroed by it;
//   * batches are not padded to 16 rows (the kernels take any count).
#include "InstantNerf.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <fstream>

using nb::throw_on_cuda;
using nb::throw_on_error;

static int pyramidCellsPerCascade(uint3 res, int levels) {
    int s = 0;
    for (int i = 0; i < levels; i++) {
        s += res.x * res.y * res.z;
        res = make_uint3(res.x / 2, res.y / 2, res.z / 2);
    }
    return s;
}

InstantNerf::~InstantNerf() {
    delete m_colorMLP;
    delete m_densityMLP;
    if (h_plan) cudaFreeHost(h_plan);
    for (WalkSet& w : m_walk) {
        if (w.h_offsets) cudaFreeHost(w.h_offsets);
        if (w.done) cudaEventDestroy(w.done);
        for (cudaEvent_t e : w.freed) if (e) cudaEventDestroy(e);
    }
    for (cudaEvent_t e : m_batchDone) if (e) cudaEventDestroy(e);
    for (cudaStream_t st : m_batchStream) if (st) cudaStreamDestroy(st);
    if (m_raysReady) cudaEventDestroy(m_raysReady);
    if (m_walkStream) cudaStreamDestroy(m_walkStream);
}

nb_scene_desc InstantNerf::scene() const {
    nb_scene_desc s;
    s.grid_res[0] = m_opts.gridResolution.x; s.grid_res[1] = m_opts.gridResolution.y; s.grid_res[2] = m_opts.gridResolution.z;
    s.aabb_min[0] = m_opts.aabbMin.x; s.aabb_min[1] = m_opts.aabbMin.y; s.aabb_min[2] = m_opts.aabbMin.z;
    s.aabb_max[0] = m_opts.aabbMax.x; s.aabb_max[1] = m_opts.aabbMax.y; s.aabb_max[2] = m_opts.aabbMax.z;
    s.num_cascades = m_opts.numCascades; s.mip_levels = m_opts.levelsMipmap; s.samples_per_voxel = m_opts.samplesPerVoxel;
    return s;
}

template <class F>
void InstantNerf::timed(cudaStream_t stream, double& acc, F&& f) {
    if (!m_opts.isProfiling) { f(); return; }
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    cudaEventRecord(a, stream);
    f();
    cudaEventRecord(b, stream);
    cudaEventSynchronize(b);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    acc += ms;
    cudaEventDestroy(a); cudaEventDestroy(b);
}

void InstantNerf::printStats() {
    const NerfPhaseTimes& t = m_times;
    double n = t.steps > 0 ? (double)t.steps : 1.0;
    std::printf("[InstantNerf] %ld steps, mean ms per step: march %.3f occupancy %.3f density fwd %.3f SH %.3f colour fwd %.3f "
                "compositing %.3f loss grad %.3f colour bwd %.3f density grad %.3f density bwd %.3f scatter %.3f optimizer %.3f\n",
                t.steps, t.march / n, t.occupancy / n, t.densityFwd / n, t.shGather / n, t.colorFwd / n, t.compositing / n, t.lossGrad / n,
                t.colorBwd / n, t.densityGrad / n, t.densityBwd / n, t.scatter / n, t.optimizer / n);
}

void InstantNerf::resetStats() { m_times = NerfPhaseTimes(); }

void InstantNerf::init(const NerfOptions& opts, MemoryMode memMode) {
    if (opts.featuresPerLevel != 2) throw std::runtime_error("InstantNerf: featuresPerLevel must be 2");
    if (opts.numLevels * opts.featuresPerLevel != 32) throw std::runtime_error("InstantNerf: the colour network expects 16 levels x 2 features");
    m_opts = opts;
    m_memMode = memMode;
    delete m_colorMLP; m_colorMLP = nullptr;
    delete m_densityMLP; m_densityMLP = nullptr;

    const int G = opts.gridResolution.x * opts.gridResolution.y * opts.gridResolution.z;
    const int S = pyramidCellsPerCascade(opts.gridResolution, opts.levelsMipmap);
    d_occupancyGrid.allocate((size_t)(opts.numCascades * S + 7) / 8, true);
    d_masterOccupancyGrid.allocate((size_t)opts.numCascades * G * sizeof(float), true);

    MLPGridOptions densityOpts;
    densityOpts.vectorDim = 4;
    densityOpts.hiddenDim = opts.densityHiddenDim;
    densityOpts.outputDim = 16;
    densityOpts.numLayers = opts.densityNumLayers;
    densityOpts.activationType = ACT_RELU;
    densityOpts.tableSize = opts.hashTableSize;
    densityOpts.numLevels = opts.numLevels;
    densityOpts.b = opts.growthFactor;
    densityOpts.lowestSize = opts.baseResolution;
    densityOpts.featuresLevel = opts.featuresPerLevel;

    MLPOption colorOpts;
    colorOpts.inputDim = 32;
    colorOpts.hiddenDim = opts.colorHiddenDim;
    colorOpts.outputDim = 3;
    colorOpts.numLayers = opts.colorNumLayers;
    colorOpts.activationType = ACT_RELU;
    colorOpts.outputActivation = OUT_ACT_SIGMOID;

    // one arena: [hash table | density W, b | colour W, b]
    const int64_t nHash = TinyMLPHashGrid::hashCount(densityOpts);
    const int64_t nDensity = TinyMLPHashGrid::mlpParamCount(densityOpts);
    const int64_t nColor = TinyMLP::paramCount(colorOpts);
    m_arena.allocate(nHash + nDensity + nColor, nHash, true);
    // The networks keep no per-object batch buffers here (maxBatch 1): every activation buffer of the step belongs
    // to this class, so that one forward serves compositing and backward.  Seeds as the reference's defaults (42).
    m_densityMLP = new TinyMLPHashGrid(densityOpts, 1, 1, 42, false, &m_arena, 0, nHash);
    m_colorMLP = new TinyMLP(colorOpts, 1, 1, 42, false, &m_arena, nHash + nDensity);

    if (!h_plan) throw_on_cuda(cudaMallocHost(&h_plan, 4 * sizeof(uint32_t)), "pinned plan");
    m_renderinit = true;
    m_trainSteps = 0;
    m_optSteps = 0;
    initRenderBuffers();
    earlyOccupancyGridUpdate();
}

void InstantNerf::initRenderBuffers() {
    if (!m_renderinit) { std::fprintf(stderr, "[InstantNerf] Error: init() must be called before initRenderBuffers()\n"); return; }
    if (m_opts.rayChunkSize % 16 != 0) { std::fprintf(stderr, "[InstantNerf] Error: rayChunkSize must be a multiple of 16"); return; }
    const size_t R = (size_t)m_opts.rayChunkSize;
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const size_t N = (size_t)m_opts.numCascades * G;
    const bool training = (m_memMode == TRAINING);
    const size_t B = (size_t)(training ? m_opts.batchSize : m_opts.renderBatchSize) + 16;
    const nb_mlp_desc& dd = m_densityMLP->desc();
    const nb_mlp_desc& cd = m_colorMLP->desc();

    d_rays_d_inv.allocate(R * 3 * sizeof(float)); d_nears.allocate(R * sizeof(float)); d_fars.allocate(R * sizeof(float));
    if (R > (size_t)1 << 20) throw std::runtime_error("rayChunkSize above 1048576 is not supported");
    d_block_sums.allocate((1024 + 4) * sizeof(uint32_t)); d_plan.allocate(4 * sizeof(uint32_t), true);
    for (WalkSet& w : m_walk) {
        w.num_steps.allocate(R * sizeof(uint32_t)); w.offsets.allocate((R + 1) * sizeof(uint32_t));
        // sample distances of every ray of a chunk, one row per ray (see nb_march_fill)
        w.rows.allocate(R * (size_t)nb_march_row_stride() * sizeof(float));
        if (w.capacity < R + 1) {
            if (w.h_offsets) cudaFreeHost(w.h_offsets);
            throw_on_cuda(cudaMallocHost(&w.h_offsets, (R + 1) * sizeof(uint32_t)), "pinned offsets");
            w.capacity = R + 1;
        }
        if (!w.done) throw_on_cuda(cudaEventCreateWithFlags(&w.done, cudaEventDisableTiming), "walk event");
        for (cudaEvent_t& e : w.freed) if (!e) throw_on_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "walk event");
    }
    for (cudaEvent_t& e : m_batchDone) if (!e) throw_on_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "batch event");
    for (cudaStream_t& st : m_batchStream) if (!st) throw_on_cuda(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "batch stream");
    if (!m_raysReady) throw_on_cuda(cudaEventCreateWithFlags(&m_raysReady, cudaEventDisableTiming), "walk event");
    if (!m_walkStream) throw_on_cuda(cudaStreamCreateWithFlags(&m_walkStream, cudaStreamNonBlocking), "walk stream");
    d_round_off.allocate(R * sizeof(uint32_t)); d_transmittance.allocate(R * sizeof(float)); d_composited.allocate(R * 4 * sizeof(float));
    d_round_counters.allocate(kRoundCounters * sizeof(uint32_t), true); d_render_samples.allocate(sizeof(uint64_t), true);
    d_render_rgb.allocate(R * 3 * sizeof(float)); d_render_depth.allocate(R * sizeof(float)); d_phi.allocate(R * 3 * sizeof(float));
    d_weight_sum.allocate(R * sizeof(float));

    d_positions.allocate((B + 1) * 4 * sizeof(float));   // + the slot's count element of a level-partitioned step
    d_ray_indices.allocate(B * sizeof(uint32_t)); d_t_sorted.allocate(B * sizeof(float));
    d_positions2.allocate(B * 4 * sizeof(float)); d_ray_indices2.allocate(B * sizeof(uint32_t)); d_t_sorted2.allocate(B * sizeof(float));
    d_sigma2.allocate(B * sizeof(float)); d_color_out2.allocate(B * 4 * sizeof(float));
    d_density_out.allocate(std::max(B, (size_t)G + 16) * 16 * sizeof(float));
    d_sigma.allocate(B * sizeof(float)); d_color_in.allocate(B * 32 * sizeof(half)); d_color_out.allocate(B * 8 * sizeof(float));
    if (training) {
        m_arena.enable_training();
        d_enc.allocate(B * dd.input_dim * sizeof(half));
        d_density_acts.allocate(B * dd.hidden_dim * sizeof(half) * std::max(1, dd.num_layers - 1));
        d_color_acts.allocate(B * cd.hidden_dim * sizeof(half) * std::max(1, cd.num_layers - 1));
        d_color_grad.allocate(B * 8 * sizeof(half)); d_color_dx.allocate(B * 32 * sizeof(half)); d_density_grad.allocate(B * 16 * sizeof(half));
        d_denc.allocate(B * dd.input_dim * sizeof(half)); d_tmpsigma.allocate(B * sizeof(float)); d_dw.allocate(B * sizeof(float));
    } else {
        d_enc.release(); d_density_acts.release(); d_color_acts.release(); d_color_grad.release(); d_color_dx.release();
        d_density_grad.release(); d_denc.release(); d_tmpsigma.release(); d_dw.release();
    }
    d_occ_samples.allocate(((size_t)G + 16) * 4 * sizeof(float)); d_tmp_grid.allocate(N * sizeof(float), true); d_sum.allocate(sizeof(float), true);
    d_occ_scratch.allocate((size_t)nb_occ_scratch_bytes((int)N) + 8); d_active_cells.allocate(N * sizeof(int)); d_num_active.allocate(sizeof(int), true);
    m_traininit = true;
    setFusedField(true);
}

void InstantNerf::freeBuffers() { m_traininit = false; }

void InstantNerf::setMemoryMode(MemoryMode mode) {
    if (!m_traininit) return;
    if (m_memMode == mode) return;
    if (m_opts.renderBatchSize == m_opts.batchSize && !m_opts.legacyRenderFlag) return;
    m_memMode = mode;
    initRenderBuffers();
}

// Shared tail of both occupancy updates: decay into the master grid (+ its sum), threshold into level-0 bits,
// OR-pool the pyramid.  InstantNerf.cu:1081-1104 / :1147-1170.
void InstantNerf::finishOccupancyUpdate(cudaStream_t stream) {
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const int N = m_opts.numCascades * G;
    nb_scene_desc sc = scene();
    throw_on_error(nb_occ_update_master_grid(d_tmp_grid.as<float>(), d_masterOccupancyGrid.as<float>(), m_opts.decayValue, N,
                                             d_occ_scratch.as<void>(), d_sum.as<float>(), stream), "occupancy: master grid");
    throw_on_error(nb_occ_update_bitfield(&sc, d_occupancyGrid.as<uint8_t>(), d_masterOccupancyGrid.as<float>(), d_sum.as<float>(),
                                          m_opts.minDensityThreshold, stream), "occupancy: bitfield");
}

// One jittered sample in every cell of every cascade.  InstantNerf.cu:1108-1171.
void InstantNerf::earlyOccupancyGridUpdate(cudaStream_t stream) {
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const int N = m_opts.numCascades * G;
    nb_scene_desc sc = scene();
    throw_on_error(nb_zero_async(d_tmp_grid.as<float>(), (int64_t)N * sizeof(float), stream), "occupancy: clear");
    for (int c = 0; c < m_opts.numCascades; ++c) {
        throw_on_error(nb_occ_sample_cells(&sc, d_occ_samples.as<float>(), G, G, c * G, (uint64_t)m_trainSteps + (uint64_t)c, stream),
                       "occupancy: sample");
        occupancyDensity(G, stream);
    }
    if (m_occWorld > 1) m_occReduceMax(d_tmp_grid.as<float>(), (int64_t)N, stream);
    finishOccupancyUpdate(stream);
}

// Density of the sampled points [0, count) of d_occ_samples and the per-cell maximum; with the update split over ranks
// only this rank's contiguous share of the points (16-point granules keep every pointer aligned).
void InstantNerf::occupancyDensity(int count, cudaStream_t stream) {
    TinyMLPHashGrid* d = m_densityMLP;
    int lo = 0, hi = count;
    if (m_occWorld > 1) {
        const int64_t granules = ((int64_t)count + 15) / 16;
        lo = (int)std::min<int64_t>(count, granules * m_occRank / m_occWorld * 16);
        hi = (int)std::min<int64_t>(count, granules * (m_occRank + 1) / m_occWorld * 16);
    }
    if (hi <= lo) return;
    const float* samples = d_occ_samples.as<float>() + (size_t)lo * 4;
    float* out = d_density_out.as<float>() + (size_t)lo * 16;
    throw_on_error(nb_grid_mlp_forward(&d->grid(), &d->desc(), samples, m_arena.Wh(d->hashOffset()), m_arena.Wh(d->weightOffset()),
                                       m_arena.W(d->biasOffset()), hi - lo, out, nullptr, nullptr, stream), "occupancy: density");
    throw_on_error(nb_occ_update_tmp_grid(samples, out, d_tmp_grid.as<float>(), m_opts.densityBias, hi - lo, stream), "occupancy: cell maximum");
}

void InstantNerf::setOccupancyShard(uint32_t rank, uint32_t world, GradSync reduceMax) {
    if (world <= 1) { m_occRank = 0; m_occWorld = 1; m_occReduceMax = GradSync(); return; }
    if (rank >= world || !reduceMax) throw std::runtime_error("setOccupancyShard: rank below world and a MAX all-reduce are required");
    m_occRank = rank; m_occWorld = world; m_occReduceMax = std::move(reduceMax);
}

// Half a grid's worth of samples, half of them inside currently occupied cells.  InstantNerf.cu:1009-1106.
void InstantNerf::lateOccupancyGridUpdate(cudaStream_t stream) {
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const int N = m_opts.numCascades * G;
    nb_scene_desc sc = scene();
    throw_on_error(nb_zero_async(d_tmp_grid.as<float>(), (int64_t)N * sizeof(float), stream), "occupancy: clear");
    throw_on_error(nb_occ_extract_active(&sc, d_occupancyGrid.as<uint8_t>(), d_active_cells.as<int>(), d_num_active.as<int>(), stream),
                   "occupancy: active cells");
    const int chunks = m_opts.numCascades;
    const int perChunk = (N / 2) / chunks;
    const int occPerChunk = perChunk / 2;
    const int uniPerChunk = perChunk - occPerChunk;
    for (int ch = 0; ch < chunks; ++ch) {
        uint64_t seedBase = (uint64_t)m_trainSteps * (2ULL * chunks) + 2ULL * ch;
        throw_on_error(nb_occ_sample_occupied(&sc, d_occ_samples.as<float>(), d_active_cells.as<int>(), d_num_active.as<int>(), occPerChunk, seedBase,
                                              stream), "occupancy: sample occupied");
        throw_on_error(nb_occ_sample_cells(&sc, d_occ_samples.as<float>() + (size_t)occPerChunk * 4, uniPerChunk, N, 0, seedBase + 1ULL, stream),
                       "occupancy: sample uniform");
        occupancyDensity(occPerChunk + uniPerChunk, stream);
    }
    if (m_occWorld > 1) m_occReduceMax(d_tmp_grid.as<float>(), (int64_t)N, stream);
    finishOccupancyUpdate(stream);
}

InstantNerf::StepView InstantNerf::stepView() const {
    StepView v;
    v.num_steps = m_walk[0].num_steps.as<uint32_t>() + m_lastStepFirstRay; v.ray_offsets = m_walk[0].offsets.as<uint32_t>() + m_lastStepFirstRay;
    v.ray_indices = d_ray_indices.as<uint32_t>(); v.sample_base = m_lastSampleBase;
    v.t_sorted = d_t_sorted.as<float>(); v.positions = d_positions.as<float>(); v.density_out = d_density_out.as<float>();
    v.sigma = d_sigma.as<float>(); v.color_out = d_color_out.as<float>(); v.render_rgb = d_render_rgb.as<float>(); v.phi = d_phi.as<float>();
    v.dw = d_dw.as<float>(); v.weight_sum = d_weight_sum.as<float>(); v.tmp_dsigma = d_tmpsigma.as<float>();
    v.color_in = d_color_in.as<half>(); v.color_grad = d_color_grad.as<half>(); v.density_grad = d_density_grad.as<half>();
    v.logit_stride = m_fused ? 1 : 16;
    v.color_stride = m_fused ? 4 : 8;
    return v;
}

bool InstantNerf::setFusedField(bool on) {
    m_fused = on && m_densityMLP && m_colorMLP && nb_field_supported(&m_densityMLP->grid(), &m_densityMLP->desc(), &m_colorMLP->desc());
    return m_fused;
}

// Walks rays [first, first + count) once (slab test, occupancy walk into the scratch rows, scan) and brings the
// scanned offsets to the host: offsets[i] = first sample of ray first + i, offsets[count] = sample total.  There are
// two sets of walk buffers so that a renderer can have the next chunk walked while it still cuts batches out of the
// current one; wait = false only enqueues (the set's event marks the read-back), finishWalk() waits for it.
void InstantNerf::walkRays(const float3* d_rays_o, const float3* d_rays_d, uint32_t first, uint32_t count, cudaStream_t stream, int set, bool wait) {
    nb_scene_desc sc = scene();
    WalkSet& w = m_walk[set];
    const float* o = reinterpret_cast<const float*>(d_rays_o + first);
    const float* d = reinterpret_cast<const float*>(d_rays_d + first);
    throw_on_error(nb_ray_aabb(&sc, o, d, count, d_rays_d_inv.as<float>(), d_nears.as<float>(), d_fars.as<float>(), stream), "ray/box");
    throw_on_error(nb_march_fill(&sc, o, d, d_rays_d_inv.as<float>(), d_nears.as<float>(), d_fars.as<float>(), d_occupancyGrid.as<uint8_t>(), count,
                                 w.num_steps.as<uint32_t>(), w.rows.as<float>(), w.offsets.as<uint32_t>(), d_block_sums.as<uint32_t>(), stream),
                   "march: walk");
    throw_on_cuda(cudaMemcpyAsync(w.h_offsets, w.offsets.as<uint32_t>(), ((size_t)count + 1) * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream),
                  "march: offsets");
    throw_on_cuda(cudaEventRecord(w.done, stream), "march: offsets");
    if (wait) finishWalk(set);
}

void InstantNerf::finishWalk(int set) { throw_on_cuda(cudaEventSynchronize(m_walk[set].done), "march: offsets"); }

// Last ray e >= begin of a walked window of `count` rays such that the samples of rays [begin, e) fit `budget`.
static uint32_t cutRays(const uint32_t* offsets, uint32_t begin, uint32_t count, uint32_t budget) {
    const uint64_t limit = (uint64_t)offsets[begin] + budget;
    const uint32_t* e = std::upper_bound(offsets + begin + 1, offsets + count + 1, limit, [](uint64_t v, uint32_t x) { return v < x; });
    return (uint32_t)(e - offsets) - 1;
}

void InstantNerf::trainWithRaysHit(const float3* d_rays_o, const float3* d_rays_d, const float* d_rays_depth, const float* d_rays_sigma,
                                   const float* d_rgb_true, uint32_t numRays, int& trainStepCount, uint32_t* hitCounts, float* d_rgb_out,
                                   cudaStream_t stream) {
    if (!m_traininit) { std::fprintf(stderr, "[InstantNerf] Error: init() must be called before trainWithRaysHit()\n"); return; }
    if (m_memMode != TRAINING || !m_arena.training) throw std::runtime_error("trainWithRaysHit called while in inference mode!");
    nb_scene_desc sc = scene();
    TinyMLPHashGrid* dn = m_densityMLP;
    TinyMLP* cn = m_colorMLP;
    const float bg[3] = {m_opts.bgColor.x, m_opts.bgColor.y, m_opts.bgColor.z};
    const uint32_t budget = (uint32_t)m_opts.batchSize;
    uint32_t raysDone = 0;
    int i = 0;
    auto recordHits = [&](uint32_t hits) {
        if (hitCounts != nullptr && (m_hitCountsCapacity == 0 || (uint32_t)i < m_hitCountsCapacity)) hitCounts[i] = hits;
    };
    // The reference walks the rays left in the chunk again for every optimizer step (InstantNerf.cu:386-407).  The
    // walk only depends on the rays and the occupancy bits, so one walk serves every step until the bits change
    // (every 16th step) or the walked window runs out while rays remain beyond it.
    uint32_t winFirst = 0, winCount = 0;
    bool walked = false;
    // m_stepsPerCall > 0 (data parallelism): exactly that many optimizer steps, hence gradient exchanges, per call on
    // every rank - rays left over after the last step stay untrained, and a rank that has used up its rays earlier
    // runs the remaining steps with no samples (it still joins the exchange and applies the common update).
    while (m_stepsPerCall > 0 ? i < m_stepsPerCall : raysDone < numRays) {
        if (raysDone >= numRays) {
            recordHits(0);
            m_lastTotalHits = 0;
            if (m_trainSteps % 16 == 0) {
                if (m_partWorld > 1) syncLevels(stream);
                timed(stream, m_times.occupancy, [&]() {
                    if (m_trainSteps < 256) earlyOccupancyGridUpdate(stream);
                    else lateOccupancyGridUpdate(stream);
                });
            }
            if (m_partWorld > 1) {
                // no samples of its own, but this rank's levels are needed for everybody else's: it joins every exchange
                partitionedForward(nullptr, 0, m_fused ? 4 : 8, stream);
                partitionedBackward(nullptr, 0, stream);
            }
            if (m_gradSync) m_gradSync(m_arena.G(0), m_arena.total, stream);
            optimizerStep(stream);
            trainStepCount++; m_trainSteps++; m_times.steps++; i++;
            continue;
        }
        uint32_t begin = 0, end = 0;
        timed(stream, m_times.march, [&]() {
            for (;;) {
                if (!walked) {
                    winFirst = raysDone;
                    winCount = std::min<uint32_t>((uint32_t)m_opts.rayChunkSize, numRays - raysDone);
                    walkRays(d_rays_o, d_rays_d, winFirst, winCount, stream, 0, true);
                    walked = true;
                }
                begin = raysDone - winFirst;
                end = cutRays(m_walk[0].h_offsets, begin, winCount, budget);
                // budget not exhausted by what is left of the window, but the window does not reach the last ray:
                // the reference's chunk would start at raysDone and reach further, so walk again from here
                if (end == winCount && begin > 0 && winFirst + winCount < numRays) { walked = false; continue; }
                break;
            }
        });
        const uint32_t currentChunkRays = end - begin;
        const uint32_t totalHits = m_walk[0].h_offsets[end] - m_walk[0].h_offsets[begin];
        const uint32_t sampleBase = m_walk[0].h_offsets[begin];
        if (currentChunkRays == 0) {
            std::fprintf(stderr, "Error: Batch size is too small to fit even a single ray! Increase batchSize.\n");
            // With a fixed number of steps per call every rank must still reach each gradient exchange: leaving here would
            // strand the other ranks in their collective.  The ray that does not fit is dropped and the loop goes on.
            if (m_stepsPerCall > 0) { raysDone++; m_lastRaysConsumed = raysDone; continue; }
            return;
        }
        const float* chunk_o = reinterpret_cast<const float*>(d_rays_o + raysDone);
        const float* chunk_d = reinterpret_cast<const float*>(d_rays_d + raysDone);
        const float* chunk_depth = d_rays_depth ? d_rays_depth + raysDone : nullptr;
        const float* chunk_sigma = d_rays_sigma ? d_rays_sigma + raysDone : nullptr;
        const uint32_t* steps_b = m_walk[0].num_steps.as<uint32_t>() + begin;
        const uint32_t* offs_b = m_walk[0].offsets.as<uint32_t>() + begin;
        if (totalHits > 0) {
            timed(stream, m_times.march, [&]() {
                throw_on_error(nb_march_compact(&sc, reinterpret_cast<const float*>(d_rays_o + winFirst), reinterpret_cast<const float*>(d_rays_d + winFirst),
                                                begin, currentChunkRays, m_walk[0].num_steps.as<uint32_t>(), m_walk[0].offsets.as<uint32_t>(), sampleBase,
                                                m_walk[0].rows.as<float>(), d_t_sorted.as<float>(), d_ray_indices.as<uint32_t>(), d_positions.as<float>(),
                                                stream), "march: compact");
            });
        }
        recordHits(totalHits);
        m_lastTotalHits = totalHits;
        m_lastStepFirstRay = begin;
        m_lastSampleBase = sampleBase;
        const int64_t n = totalHits;

        // occupancy schedule of the reference: every 16 steps, all cells for the first 256 steps (InstantNerf.cu:488-494).
        // It only reads the parameters, which do not change before the optimizer below; the walk above used the old bits,
        // as the reference's march of this step does, and the next step walks again.
        if (m_trainSteps % 16 == 0) {
            if (m_partWorld > 1) syncLevels(stream);     // the density queries of the update read every level
            timed(stream, m_times.occupancy, [&]() {
                if (m_trainSteps < 256) earlyOccupancyGridUpdate(stream);
                else lateOccupancyGridUpdate(stream);
            });
            walked = false;
        }

        const int logitStride = m_fused ? 1 : 16, colorStride = m_fused ? 4 : 8;
        if (m_partWorld > 1) {
            partitionedForward(chunk_d, n, colorStride, stream);
        } else if (n > 0 && m_fused) {
            timed(stream, m_times.densityFwd, [&]() {
                throw_on_error(nb_field_forward(&dn->grid(), &dn->desc(), &cn->desc(), d_positions.as<float>(), m_arena.Wh(dn->hashOffset()), chunk_d,
                                                d_ray_indices.as<uint32_t>(), 0, m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()),
                                                m_arena.Wh(cn->weightOffset()), m_arena.W(cn->biasOffset()), n, m_opts.densityBias, d_enc.as<half>(),
                                                d_sigma.as<float>(), d_density_out.as<float>(), d_color_out.as<float>(), colorStride, stream),
                               "field forward");
            });
        } else if (n > 0) {
            timed(stream, m_times.densityFwd, [&]() {
                throw_on_error(nb_grid_mlp_forward(&dn->grid(), &dn->desc(), d_positions.as<float>(), m_arena.Wh(dn->hashOffset()),
                                                   m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()), n, d_density_out.as<float>(),
                                                   d_enc.as<half>(), d_density_acts.as<half>(), stream), "density forward");
            });
            timed(stream, m_times.shGather, [&]() {
                throw_on_error(nb_sh_gather(chunk_d, d_ray_indices.as<uint32_t>(), 0, n, m_opts.densityBias, d_density_out.as<float>(),
                                            d_color_in.as<half>(), d_sigma.as<float>(), stream), "SH gather");
            });
            timed(stream, m_times.colorFwd, [&]() {
                throw_on_error(nb_mlp_forward(&cn->desc(), d_color_in.as<half>(), m_arena.Wh(cn->weightOffset()), m_arena.W(cn->biasOffset()), n,
                                              d_color_out.as<float>(), d_color_acts.as<half>(), stream), "colour forward");
            });
        }
        timed(stream, m_times.compositing, [&]() {
            throw_on_error(nb_composite_train(currentChunkRays, sampleBase, offs_b, steps_b, d_t_sorted.as<float>(), d_sigma.as<float>(), chunk_depth,
                                              chunk_sigma, d_color_out.as<float>(), colorStride,
                                              d_rgb_true ? d_rgb_true + (size_t)raysDone * 3 : nullptr, d_render_rgb.as<float>(),
                                              d_render_depth.as<float>(), d_phi.as<float>(), d_dw.as<float>(), d_weight_sum.as<float>(),
                                              m_opts.lambdaDist, m_opts.lambdaDepth, bg, stream), "compositing");
        });
        if (d_rgb_out != nullptr)
            throw_on_cuda(cudaMemcpyAsync(d_rgb_out + (size_t)raysDone * 3, d_render_rgb.as<float>(), (size_t)currentChunkRays * 3 * sizeof(float),
                                          cudaMemcpyDeviceToDevice, stream), "rgb out");
        if (n > 0) {
            timed(stream, m_times.lossGrad, [&]() {
                throw_on_error(nb_color_grad(currentChunkRays, sampleBase, steps_b, offs_b, d_t_sorted.as<float>(), d_density_out.as<float>(),
                                             logitStride, d_color_out.as<float>(), colorStride, d_phi.as<float>(), d_render_rgb.as<float>(),
                                             d_dw.as<float>(), d_weight_sum.as<float>(), d_color_grad.as<half>(), 8, d_tmpsigma.as<float>(),
                                             m_opts.lossScale, m_opts.densityBias, numRays * m_rayScale, stream), "loss gradients");
            });
            if (m_partWorld > 1) {
                // below, outside this block: every rank takes part in the exchange whether or not it has samples
            } else if (m_fused) {
                timed(stream, m_times.colorBwd, [&]() {
                    throw_on_error(nb_field_backward(&dn->desc(), &cn->desc(), d_enc.as<half>(), chunk_d, d_ray_indices.as<uint32_t>(), 0,
                                                     m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()), m_arena.Wh(cn->weightOffset()),
                                                     m_arena.W(cn->biasOffset()), n, d_color_grad.as<half>(), d_tmpsigma.as<float>(),
                                                     m_arena.G(dn->weightOffset()), m_arena.G(dn->biasOffset()), m_arena.G(cn->weightOffset()),
                                                     m_arena.G(cn->biasOffset()), d_denc.as<half>(), &dn->grid(), d_positions.as<float>(),
                                                     m_arena.G(dn->hashOffset()), stream), "field backward");
                });
            } else {
                timed(stream, m_times.colorBwd, [&]() {
                    throw_on_error(nb_mlp_backward(&cn->desc(), d_color_grad.as<half>(), m_arena.Wh(cn->weightOffset()), d_color_in.as<half>(),
                                                   d_color_acts.as<half>(), n, m_arena.G(cn->weightOffset()), m_arena.G(cn->biasOffset()),
                                                   d_color_dx.as<half>(), stream), "colour backward");
                });
                timed(stream, m_times.densityGrad, [&]() {
                    throw_on_error(nb_density_grad(n, d_tmpsigma.as<float>(), d_color_dx.as<half>(), d_density_grad.as<half>(), stream), "density gradient");
                });
                timed(stream, m_times.densityBwd, [&]() {
                    throw_on_error(nb_mlp_backward(&dn->desc(), d_density_grad.as<half>(), m_arena.Wh(dn->weightOffset()), d_enc.as<half>(),
                                                   d_density_acts.as<half>(), n, m_arena.G(dn->weightOffset()), m_arena.G(dn->biasOffset()),
                                                   d_denc.as<half>(), stream), "density backward");
                });
                timed(stream, m_times.scatter, [&]() {
                    throw_on_error(nb_hash_scatter_backward(&dn->grid(), d_positions.as<float>(), d_denc.as<half>(), n, m_arena.G(dn->hashOffset()), stream),
                                   "gradient scatter");
                });
            }
        }
        if (m_partWorld > 1) partitionedBackward(chunk_d, n, stream);
        if (m_gradSync) m_gradSync(m_arena.G(0), m_arena.total, stream);
        optimizerStep(stream);
        trainStepCount++;
        m_trainSteps++;
        m_times.steps++;
        raysDone += currentChunkRays;
        i++;
        m_lastRaysConsumed = raysDone;
    }
}

void InstantNerf::setOptimizerShard(uint32_t rank, uint32_t world, ParamSync sync) {
    if (world <= 1) { m_shardRank = 0; m_shardWorld = 1; m_paramSync = ParamSync(); return; }
    if (rank >= world) throw std::runtime_error("setOptimizerShard: rank must be below the number of ranks");
    if (m_arena.sparse_count % (4 * (int64_t)world) != 0) throw std::runtime_error("setOptimizerShard: the hash table does not split into 16-byte aligned slices");
    m_shardRank = rank; m_shardWorld = world; m_paramSync = std::move(sync);
}

void InstantNerf::setPeerExchange(uint32_t rank, uint32_t world, const std::vector<const float*>& peerGrads, const std::vector<void*>& peerParamsH,
                                  RankBarrier barrier) {
    if (world <= 1) { m_peerGrads.clear(); m_peerParamsH.clear(); m_rankBarrier = RankBarrier(); m_shardRank = 0; m_shardWorld = 1; return; }
    if (rank >= world || peerGrads.size() != world || peerParamsH.size() != world || !barrier)
        throw std::runtime_error("setPeerExchange: one gradient and one parameter pointer per rank and a barrier are required");
    if (m_arena.sparse_count % (4 * (int64_t)world) != 0) throw std::runtime_error("setPeerExchange: the hash table does not split into 16-byte aligned slices");
    if (peerGrads[rank] != m_arena.G(0) || peerParamsH[rank] != (void*)m_arena.Wh(0))
        throw std::runtime_error("setPeerExchange: this rank's own entries must be its own arenas");
    m_peerGrads = peerGrads; m_peerParamsH = peerParamsH; m_rankBarrier = std::move(barrier);
    m_shardRank = rank; m_shardWorld = world;
    m_paramSync = ParamSync();
}

void InstantNerf::setLevelPartition(uint32_t rank, uint32_t world, BlockGather gather, BlockExchange exchange, GradSync reduce) {
    if (world <= 1) {
        m_partRank = 0; m_partWorld = 1; m_partGather = BlockGather(); m_partExchange = BlockExchange(); m_partReduce = GradSync();
        d_pos_all.release(); d_pieces_send.release(); d_pieces_recv.release();
        return;
    }
    const int levels = m_densityMLP->grid().num_levels;
    if (rank >= world || levels % (int)world != 0) throw std::runtime_error("setLevelPartition: rank below world, world a divisor of the number of levels");
    if (!gather || !exchange || !reduce) throw std::runtime_error("setLevelPartition: the three collectives are required");
    if (!m_fused) throw std::runtime_error("setLevelPartition: needs the fused field kernels");
    if (m_shardWorld > 1 || !m_peerGrads.empty()) throw std::runtime_error("setLevelPartition: not together with a replicated-table exchange");
    if (m_arena.sparse_count != (int64_t)levels * m_densityMLP->grid().table_size * 2) throw std::runtime_error("setLevelPartition: unexpected table layout");
    const size_t B = (size_t)m_opts.batchSize;
    d_pos_all.allocate((size_t)world * (B + 1) * 4 * sizeof(float));
    d_pieces_send.allocate((size_t)levels * B * sizeof(uint32_t));
    d_pieces_recv.allocate((size_t)levels * B * sizeof(uint32_t));
    m_partRank = rank; m_partWorld = world;
    m_partGather = std::move(gather); m_partExchange = std::move(exchange); m_partReduce = std::move(reduce);
}

// Owned levels -> every rank, level block by level block: levels k * world ... (k + 1) * world - 1 are contiguous in the
// arena and this rank's level is block `rank` of them, which is the in-place form of an all-gather.
void InstantNerf::syncLevels(cudaStream_t stream, bool master) {
    if (m_partWorld <= 1) return;
    const int levels = m_densityMLP->grid().num_levels;
    const int64_t level = m_arena.sparse_count / levels;
    for (int k = 0; k < levels / (int)m_partWorld; k++) {
        const int64_t block = (int64_t)k * m_partWorld * level, mine = block + (int64_t)m_partRank * level;
        m_partGather(m_arena.Wh(mine), m_arena.Wh(block), level * (int64_t)sizeof(half), stream);
        if (master) m_partGather(m_arena.W(mine), m_arena.W(block), level * (int64_t)sizeof(float), stream);
    }
}

// Forward of a level-partitioned step: positions to everybody, the owned levels encoded for everybody's samples, pieces
// to the samples' ranks, networks from the received pieces.  Runs on every rank in every step, with or without samples.
void InstantNerf::partitionedForward(const float* chunk_d, int64_t n, int colorStride, cudaStream_t stream) {
    TinyMLPHashGrid* dn = m_densityMLP;
    TinyMLP* cn = m_colorMLP;
    const int64_t B = (int64_t)m_opts.batchSize;
    const int world = (int)m_partWorld, rank = (int)m_partRank;
    // phase times in this mode: shGather = positions to everybody, colorFwd = encoding of the owned levels, densityGrad =
    // the two exchanges of pieces, densityFwd / colorBwd = the networks, scatter = the owners' scatter
    timed(stream, m_times.shGather, [&]() {
        throw_on_error(nb_part_stamp_count(d_positions.as<float>(), B, n, stream), "partition: count");
        m_partGather(d_positions.as<float>(), d_pos_all.as<float>(), (B + 1) * 4 * (int64_t)sizeof(float), stream);
    });
    timed(stream, m_times.colorFwd, [&]() {
        throw_on_error(nb_part_encode(&dn->grid(), world, rank, B, d_pos_all.as<float>(), m_arena.Wh(dn->hashOffset()), d_pieces_send.as<void>(), stream),
                       "partition: encode");
    });
    const int64_t piece = (int64_t)(dn->grid().num_levels / world) * B * (int64_t)sizeof(uint32_t);
    timed(stream, m_times.densityGrad, [&]() { m_partExchange(d_pieces_send.as<void>(), d_pieces_recv.as<void>(), piece, stream); });
    if (n > 0) timed(stream, m_times.densityFwd, [&]() {
        throw_on_error(nb_part_field_forward(&dn->grid(), &dn->desc(), &cn->desc(), world, B, d_pieces_recv.as<void>(), chunk_d, d_ray_indices.as<uint32_t>(), 0,
                                             m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()), m_arena.Wh(cn->weightOffset()),
                                             m_arena.W(cn->biasOffset()), n, m_opts.densityBias, d_enc.as<half>(), d_sigma.as<float>(),
                                             d_density_out.as<float>(), d_color_out.as<float>(), colorStride, stream), "partition: field forward");
    });
}

// Backward: the networks' gradients and dL/d(encoding) of this rank's samples, the latter packed by owner, exchanged, and
// scattered by every owner into its levels for everybody's samples (positions still in d_pos_all from the forward).
void InstantNerf::partitionedBackward(const float* chunk_d, int64_t n, cudaStream_t stream) {
    TinyMLPHashGrid* dn = m_densityMLP;
    TinyMLP* cn = m_colorMLP;
    const int64_t B = (int64_t)m_opts.batchSize;
    const int world = (int)m_partWorld, rank = (int)m_partRank;
    // the backward writes dL/d(encoding) straight into the pieces (rows behind n stay as they are: receivers go by the count)
    if (n > 0) timed(stream, m_times.colorBwd, [&]() {
        throw_on_error(nb_part_field_backward(&dn->desc(), &cn->desc(), world, B, d_enc.as<half>(), chunk_d, d_ray_indices.as<uint32_t>(), 0,
                                              m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()), m_arena.Wh(cn->weightOffset()),
                                              m_arena.W(cn->biasOffset()), n, d_color_grad.as<half>(), d_tmpsigma.as<float>(),
                                              m_arena.G(dn->weightOffset()), m_arena.G(dn->biasOffset()), m_arena.G(cn->weightOffset()),
                                              m_arena.G(cn->biasOffset()), d_pieces_send.as<void>(), stream), "partition: field backward");
    });
    const int64_t piece = (int64_t)(dn->grid().num_levels / world) * B * (int64_t)sizeof(uint32_t);
    timed(stream, m_times.densityGrad, [&]() { m_partExchange(d_pieces_send.as<void>(), d_pieces_recv.as<void>(), piece, stream); });
    timed(stream, m_times.scatter, [&]() {
        throw_on_error(nb_part_scatter(&dn->grid(), world, rank, B, d_pos_all.as<float>(), d_pieces_recv.as<void>(), m_arena.G(dn->hashOffset()), stream),
                       "partition: scatter");
    });
}

void InstantNerf::optimizerStep(cudaStream_t stream) {
    timed(stream, m_times.optimizer, [&]() {
        if (m_optSteps < 50000) m_optSteps++;
        float bc1 = 1.0f - std::pow(m_opts.beta1, (float)m_optSteps);
        float bc2 = 1.0f - std::pow(m_opts.beta2, (float)m_optSteps);
        if (!m_peerGrads.empty()) {
            m_rankBarrier(stream);     // every rank's backward has finished: the gradients may be read
            throw_on_error(nb_adam_step_peer(m_arena.W(0), m_arena.M(0), m_arena.V(0), m_peerGrads.data(), m_peerParamsH.data(), (int)m_shardRank,
                                             (int)m_shardWorld, m_arena.sparse_count, m_arena.total, m_opts.learningRate, m_opts.beta1, m_opts.beta2,
                                             m_opts.epsilon, bc1, bc2, 1.0f / m_opts.lossScale, stream), "optimizer (peer)");
            m_rankBarrier(stream);     // every rank has stored its slice everywhere and read what it needed of this gradient
            throw_on_error(nb_zero_async(m_arena.G(0), m_arena.total * (int64_t)sizeof(float), stream), "optimizer: clear");
            return;
        }
        if (m_partWorld > 1) {
            // owned levels of the table, then the networks on the gradient summed over the ranks
            const int64_t H = m_arena.sparse_count, level = H / m_densityMLP->grid().num_levels;
            if (m_partReduce) m_partReduce(m_arena.G(H), m_arena.total - H, stream);
            int grad_half_part = 0;
            nb_get_tuning("grad_table_half", &grad_half_part);
            for (int64_t l = m_partRank; l < m_densityMLP->grid().num_levels; l += m_partWorld) {
                const int64_t off = l * level;
                // with the half-precision table the level's gradient sits at half the byte offset
                float* g = grad_half_part ? reinterpret_cast<float*>(reinterpret_cast<half*>(m_arena.G(0)) + off) : m_arena.G(off);
                throw_on_error(nb_adam_step(m_arena.W(off), m_arena.Wh(off), g, m_arena.M(off), m_arena.V(off), level, level, m_opts.learningRate,
                                            m_opts.beta1, m_opts.beta2, m_opts.epsilon, bc1, bc2, 1.0f / m_opts.lossScale, 1, stream),
                               "optimizer (owned level)");
            }
            throw_on_error(nb_adam_step(m_arena.W(H), m_arena.Wh(H), m_arena.G(H), m_arena.M(H), m_arena.V(H), 0, m_arena.total - H, m_opts.learningRate,
                                        m_opts.beta1, m_opts.beta2, m_opts.epsilon, bc1, bc2, 1.0f / m_opts.lossScale, 1, stream),
                           "optimizer (networks)");
            return;
        }
        int grad_half = 0;
        nb_get_tuning("grad_table_half", &grad_half);
        if (grad_half && (m_gradSync || m_shardWorld > 1))
            throw std::runtime_error("optimizer: the half-precision gradient table cannot be exchanged as one fp32 array; use setPeerExchange");
        auto adam = [&](int64_t off, int64_t sparse, int64_t count, const char* what) {
            throw_on_error(nb_adam_step(m_arena.W(off), m_arena.Wh(off), m_arena.G(off), m_arena.M(off), m_arena.V(off), sparse, count,
                                        m_opts.learningRate, m_opts.beta1, m_opts.beta2, m_opts.epsilon, bc1, bc2, 1.0f / m_opts.lossScale, 1, stream),
                           what);
        };
        if (m_shardWorld <= 1) { adam(0, m_arena.sparse_count, m_arena.total, "optimizer"); return; }
        const int64_t H = m_arena.sparse_count, shard = H / m_shardWorld, lo = (int64_t)m_shardRank * shard, hi = lo + shard;
        adam(lo, shard, shard, "optimizer (table slice)");
        adam(H, 0, m_arena.total - H, "optimizer (networks)");
        // the other slices still hold this rank's own unreduced gradient
        if (lo > 0) throw_on_error(nb_zero_async(m_arena.G(0), lo * (int64_t)sizeof(float), stream), "optimizer: clear");
        if (hi < H) throw_on_error(nb_zero_async(m_arena.G(hi), (H - hi) * (int64_t)sizeof(float), stream), "optimizer: clear");
        if (m_paramSync) m_paramSync(m_arena.Wh(0), H, stream);
    });
}

// One walked chunk rendered front to back in rounds of samples per ray.  Round r covers samples [b_r, b_r + w_r) of
// every ray that still has samples there and is not yet opaque; which rays those are is decided on the device
// (nb_march_round_emit), the host only bounds each launch: a ray with n samples reaches round r when n > b_r, and a
// round over k such rays holds at most k * w_r samples.  Ray ranges are cut at 1024-ray blocks so that this bound fits
// the sample arrays (a single block that does not fit is cut ray by ray).
void InstantNerf::renderChunkRounds(const WalkSet& w, const float* chunk_o, const float* chunk_d, uint32_t chunkRays, uint32_t capacity,
                                    float* rgb_dst, cudaStream_t stream) {
    static constexpr int kRounds = 7;
    static constexpr uint32_t kBegin[kRounds] = {0, 16, 32, 64, 128, 256, 512};
    static constexpr uint32_t kWidth[kRounds] = {16, 16, 32, 64, 128, 256, 512};
    static_assert(kBegin[kRounds - 1] + kWidth[kRounds - 1] == 1024, "the rounds cover a whole row");
    constexpr uint32_t BLOCK = 1024;
    nb_scene_desc sc = scene();
    TinyMLPHashGrid* dn = m_densityMLP;
    TinyMLP* cn = m_colorMLP;
    const float bg[3] = {m_opts.bgColor.x, m_opts.bgColor.y, m_opts.bgColor.z};
    const uint32_t* off = w.h_offsets;
    const uint32_t numBlocks = (chunkRays + BLOCK - 1) / BLOCK;
    // m_roundRays[block * kRounds + r] = rays of the block with more than kBegin[r] samples
    m_roundRays.assign((size_t)numBlocks * kRounds, 0u);
    uint32_t reach[kRounds] = {0, 0, 0, 0, 0, 0, 0};
    for (uint32_t b = 0; b < numBlocks; b++) {
        uint32_t hist[kRounds + 1] = {0, 0, 0, 0, 0, 0, 0, 0};  // by the number of rounds a ray reaches
        const uint32_t end = std::min(chunkRays, (b + 1) * BLOCK);
        for (uint32_t i = b * BLOCK; i < end; i++) {
            const uint32_t n = off[i + 1] - off[i];
            // n in (0, 16] reaches 1 round, (16, 32] 2, (32, 64] 3, ... (512, 1024] 7
            const uint32_t rounds = n == 0 ? 0u : (n <= 16 ? 1u : std::min<uint32_t>(kRounds, 29u - (uint32_t)__builtin_clz(n - 1)));
            hist[rounds]++;
        }
        uint32_t rays = 0;
        for (int r = kRounds - 1; r >= 0; r--) {
            rays += hist[r + 1];
            m_roundRays[(size_t)b * kRounds + r] = rays;
            reach[r] += rays;
        }
    }
    int slot = kRoundCounters;  // forces the first clear
    auto takeCounters = [&](int count) -> uint32_t* {
        if (slot + count > kRoundCounters) {
            throw_on_cuda(cudaMemsetAsync(d_round_counters.as<uint32_t>(), 0, kRoundCounters * sizeof(uint32_t), stream), "round counters");
            slot = 0;
        }
        uint32_t* c = d_round_counters.as<uint32_t>() + slot;
        slot += count;
        return c;
    };
    auto blockBound = [&](uint32_t b, int r) { return (uint64_t)m_roundRays[(size_t)b * kRounds + r] * kWidth[r]; };
    auto fieldOn = [&](uint64_t bound, const uint32_t* counter) {
        throw_on_error(nb_field_forward_counted(&dn->grid(), &dn->desc(), &cn->desc(), d_positions.as<float>(), m_arena.Wh(dn->hashOffset()), chunk_d,
                                                d_ray_indices.as<uint32_t>(), 0, m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()),
                                                m_arena.Wh(cn->weightOffset()), m_arena.W(cn->biasOffset()), (int64_t)bound, counter,
                                                m_opts.densityBias, d_sigma.as<float>(), d_color_out.as<float>(), 4, stream), "field inference");
    };
    // The usual case: every 1024-ray block fits the sample arrays in every round.  Then the chunk is cut into ray ranges
    // that fit in EVERY round and each range runs all its rounds in a row, the compositing kernel of a round copying the
    // next round's samples out as it goes: two launches per round.
    bool everyBlockFits = true;
    for (uint32_t b = 0; b < numBlocks && everyBlockFits; b++)
        for (int r = 0; r < kRounds; r++) everyBlockFits = everyBlockFits && blockBound(b, r) <= capacity;
    if (everyBlockFits) {
        uint32_t b0 = 0;
        while (b0 < numBlocks) {
            uint64_t sum[kRounds] = {0, 0, 0, 0, 0, 0, 0};
            uint32_t b1 = b0;
            while (b1 < numBlocks) {
                bool ok = true;
                for (int r = 0; r < kRounds; r++) ok = ok && sum[r] + blockBound(b1, r) <= capacity;
                if (!ok) break;
                for (int r = 0; r < kRounds; r++) sum[r] += blockBound(b1, r);
                b1++;
            }
            const uint32_t begin = b0 * BLOCK, end = std::min(chunkRays, b1 * BLOCK);
            int last = 0;
            for (int r = 0; r < kRounds; r++) if (sum[r] > 0) last = r;
            uint32_t* counters = takeCounters(last + 1);
            throw_on_error(nb_march_round_emit(&sc, chunk_o, chunk_d, begin, end - begin, w.num_steps.as<uint32_t>(), d_transmittance.as<float>(),
                                               kBegin[0], kWidth[0], w.rows.as<float>(), capacity, counters, d_render_samples.as<uint64_t>(),
                                               d_round_off.as<uint32_t>(), d_ray_indices.as<uint32_t>(), d_positions.as<float>(), stream),
                           "march: round");
            for (int r = 0; r <= last; r++) {
                if (sum[r] > 0) fieldOn(sum[r], counters + r);
                const bool more = r < last;
                throw_on_error(nb_composite_round(begin, end - begin, w.num_steps.as<uint32_t>(), d_round_off.as<uint32_t>(), w.rows.as<float>(),
                                                  kBegin[r], kWidth[r], d_sigma.as<float>(), d_color_out.as<float>(), 4, d_transmittance.as<float>(),
                                                  d_composited.as<float>(), rgb_dst, d_render_depth.as<float>(), bg, more ? kWidth[r + 1] : 0u, &sc,
                                                  chunk_o, chunk_d, capacity, more ? counters + r + 1 : nullptr,
                                                  d_render_samples.as<uint64_t>(), d_ray_indices.as<uint32_t>(), d_positions.as<float>(), stream),
                               "compositing");
            }
            b0 = b1;
        }
        return;
    }
    // Otherwise (sample arrays smaller than one round of 1024 rays): round by round, ranges cut per round, each with a
    // copy-out launch of its own.
    auto launchRange = [&](int r, uint32_t begin, uint32_t end, uint64_t bound) {
        if (r > 0 && bound == 0) return;  // nobody reaches the round; round 0 still writes the background
        uint32_t* counter = takeCounters(1);
        throw_on_error(nb_march_round_emit(&sc, chunk_o, chunk_d, begin, end - begin, w.num_steps.as<uint32_t>(), d_transmittance.as<float>(),
                                           kBegin[r], kWidth[r], w.rows.as<float>(), capacity, counter, d_render_samples.as<uint64_t>(),
                                           d_round_off.as<uint32_t>(),
                                           d_ray_indices.as<uint32_t>(), d_positions.as<float>(), stream), "march: round");
        if (bound > 0) fieldOn(bound, counter);
        throw_on_error(nb_composite_round(begin, end - begin, w.num_steps.as<uint32_t>(), d_round_off.as<uint32_t>(), w.rows.as<float>(), kBegin[r],
                                          kWidth[r], d_sigma.as<float>(), d_color_out.as<float>(), 4, d_transmittance.as<float>(),
                                          d_composited.as<float>(), rgb_dst, d_render_depth.as<float>(), bg, 0u, nullptr, nullptr, nullptr, 0u,
                                          nullptr, nullptr, nullptr, nullptr, stream), "compositing");
    };
    for (int r = 0; r < kRounds; r++) {
        if (r > 0 && reach[r] == 0) break;  // round 0 always runs: it writes the background of rays without samples
        uint32_t rangeBegin = 0;
        uint64_t bound = 0;
        for (uint32_t b = 0; b < numBlocks; b++) {
            const uint32_t blockBegin = b * BLOCK, blockEnd = std::min(chunkRays, (b + 1) * BLOCK);
            const uint64_t blockBound = (uint64_t)m_roundRays[(size_t)b * kRounds + r] * kWidth[r];
            if (blockBound > capacity) {
                // a block that alone exceeds the arrays: flush what is pending, then cut this block ray by ray
                if (blockBegin > rangeBegin) launchRange(r, rangeBegin, blockBegin, bound);
                uint32_t begin = blockBegin;
                uint64_t acc = 0;
                for (uint32_t i = blockBegin; i < blockEnd; i++) {
                    const uint32_t n = off[i + 1] - off[i];
                    const uint32_t c = n > kBegin[r] ? std::min(n - kBegin[r], kWidth[r]) : 0u;
                    if (c > capacity) throw std::runtime_error("renderImageHit: the sample batch is too small for one round of one ray");
                    if (acc + c > capacity) { launchRange(r, begin, i, acc); begin = i; acc = 0; }
                    acc += c;
                }
                launchRange(r, begin, blockEnd, acc);
                rangeBegin = blockEnd; bound = 0;
                continue;
            }
            if (bound + blockBound > capacity) {
                launchRange(r, rangeBegin, blockBegin, bound);
                rangeBegin = blockBegin; bound = 0;
            }
            bound += blockBound;
        }
        if (rangeBegin < chunkRays) launchRange(r, rangeBegin, chunkRays, bound);
    }
}

void InstantNerf::renderImageHit(const float3* d_rays_o, const float3* d_rays_d, uint32_t numRays, float* d_rgb_out, cudaStream_t stream) {
    if (!m_traininit) { std::fprintf(stderr, "[InstantNerf] Error: init() must be called before renderImageHit()\n"); return; }
    nb_scene_desc sc = scene();
    TinyMLPHashGrid* dn = m_densityMLP;
    TinyMLP* cn = m_colorMLP;
    const float bg[3] = {m_opts.bgColor.x, m_opts.bgColor.y, m_opts.bgColor.z};
    const uint32_t hitBatch = (uint32_t)((m_memMode == INFERENCE) ? m_opts.renderBatchSize : m_opts.batchSize);
    // Chunks are walked one ahead, on the walk stream: while the host waits for chunk k's offsets and cuts its batches, and
    // while the field kernels of chunk k run, the device is already walking chunk k + 1.  Events order the two streams:
    // a walk starts once the caller's rays are there and the batches that read its buffer set are through; the batches
    // of a chunk start once its walk has finished.
    const uint32_t chunk = (uint32_t)m_opts.rayChunkSize;
    const uint32_t numChunks = (numRays + chunk - 1) / chunk;
    m_renderSamplesHost = 0;
    throw_on_cuda(cudaMemsetAsync(d_render_samples.as<uint64_t>(), 0, sizeof(uint64_t), stream), "render statistics");
    throw_on_cuda(cudaEventRecord(m_raysReady, stream), "walk event");
    throw_on_cuda(cudaStreamWaitEvent(m_walkStream, m_raysReady, 0), "walk event");
    // Sample batches alternate between two streams (each with its own sample arrays) when they write disjoint parts of the
    // caller's frame; the caller's stream joins them at the end.  The kernel-by-kernel sequence and rendering in rounds
    // stay on the caller's stream.
    const bool alternate = m_fused && !renderRounds() && d_rgb_out != nullptr;
    uint32_t batchIndex = 0;
    if (alternate)
        for (cudaStream_t bs : m_batchStream) throw_on_cuda(cudaStreamWaitEvent(bs, m_raysReady, 0), "batch event");
    auto joinBatches = [&]() {
        if (!alternate) return;
        for (int lane = 0; lane < 2; lane++) {
            throw_on_cuda(cudaEventRecord(m_batchDone[lane], m_batchStream[lane]), "batch event");
            throw_on_cuda(cudaStreamWaitEvent(stream, m_batchDone[lane], 0), "batch event");
        }
    };
    if (numChunks > 0) walkRays(d_rays_o, d_rays_d, 0, std::min(chunk, numRays), m_walkStream, 0, false);
    for (uint32_t k = 0; k < numChunks; k++) {
        const uint32_t ray_offset = k * chunk;
        const uint32_t chunkRays = std::min<uint32_t>(chunk, numRays - ray_offset);
        const int set = (int)(k & 1);
        if (k + 1 < numChunks) {
            if (k >= 1)  // batches of chunk k - 1 (an event never recorded counts as reached)
                for (cudaEvent_t e : m_walk[set ^ 1].freed) throw_on_cuda(cudaStreamWaitEvent(m_walkStream, e, 0), "walk event");
            walkRays(d_rays_o, d_rays_d, ray_offset + chunk, std::min(chunk, numRays - ray_offset - chunk), m_walkStream, set ^ 1, false);
        }
        finishWalk(set);
        const WalkSet& w = m_walk[set];
        const float* chunk_o = reinterpret_cast<const float*>(d_rays_o + ray_offset);
        const float* chunk_d = reinterpret_cast<const float*>(d_rays_d + ray_offset);
        if (renderRounds()) {
            throw_on_cuda(cudaStreamWaitEvent(stream, m_walk[set].done, 0), "walk event");
            renderChunkRounds(w, chunk_o, chunk_d, chunkRays, hitBatch, d_rgb_out != nullptr ? d_rgb_out + (size_t)ray_offset * 3 : d_render_rgb.as<float>(),
                              stream);
            throw_on_cuda(cudaEventRecord(m_walk[set].freed[0], stream), "walk event");
            continue;
        }
        uint32_t raysDone = 0;
        bool laneUsed[2] = {false, false};
        while (raysDone < chunkRays) {
            const uint32_t next = cutRays(w.h_offsets, raysDone, chunkRays, hitBatch);
            if (next <= raysDone) {
                std::fprintf(stderr, "Error: Batch size is too small to fit even a single ray! Increase batchSize.\n");
                if (k + 1 < numChunks) cudaStreamWaitEvent(stream, m_walk[set ^ 1].done, 0);  // leave no walk behind the caller's stream
                joinBatches();
                return;
            }
            const uint32_t crrRays = next - raysDone;
            const uint32_t base = w.h_offsets[raysDone];
            const int64_t n = w.h_offsets[next] - base;
            m_renderSamplesHost += (uint64_t)n;
            const int lane = alternate ? (int)(batchIndex++ & 1u) : 0;
            cudaStream_t ls = alternate ? m_batchStream[lane] : stream;
            if (!laneUsed[lane]) {
                throw_on_cuda(cudaStreamWaitEvent(ls, m_walk[set].done, 0), "walk event");
                laneUsed[lane] = true;
            }
            float* positions = lane ? d_positions2.as<float>() : d_positions.as<float>();
            uint32_t* rayIdx = lane ? d_ray_indices2.as<uint32_t>() : d_ray_indices.as<uint32_t>();
            float* tSorted = lane ? d_t_sorted2.as<float>() : d_t_sorted.as<float>();
            float* sigma = lane ? d_sigma2.as<float>() : d_sigma.as<float>();
            float* colorOut = lane ? d_color_out2.as<float>() : d_color_out.as<float>();
            if (n > 0) {
                throw_on_error(nb_march_compact(&sc, chunk_o, chunk_d, raysDone, crrRays, w.num_steps.as<uint32_t>(), w.offsets.as<uint32_t>(), base,
                                                w.rows.as<float>(), tSorted, rayIdx, positions, ls), "march: compact");
                if (m_fused) {
                    throw_on_error(nb_field_forward(&dn->grid(), &dn->desc(), &cn->desc(), positions, m_arena.Wh(dn->hashOffset()),
                                                    chunk_d + (size_t)raysDone * 3, rayIdx, 0, m_arena.Wh(dn->weightOffset()),
                                                    m_arena.W(dn->biasOffset()), m_arena.Wh(cn->weightOffset()), m_arena.W(cn->biasOffset()), n,
                                                    m_opts.densityBias, nullptr, sigma, nullptr, colorOut, 4, ls), "field inference");
                } else {
                    throw_on_error(nb_grid_mlp_forward(&dn->grid(), &dn->desc(), positions, m_arena.Wh(dn->hashOffset()),
                                                       m_arena.Wh(dn->weightOffset()), m_arena.W(dn->biasOffset()), n, d_density_out.as<float>(), nullptr,
                                                       nullptr, ls), "density inference");
                    throw_on_error(nb_sh_gather(chunk_d + (size_t)raysDone * 3, rayIdx, 0, n, m_opts.densityBias, d_density_out.as<float>(),
                                                d_color_in.as<half>(), sigma, ls), "SH gather");
                    throw_on_error(nb_mlp_forward(&cn->desc(), d_color_in.as<half>(), m_arena.Wh(cn->weightOffset()), m_arena.W(cn->biasOffset()), n,
                                                  colorOut, nullptr, ls), "colour inference");
                }
            }
            // composited straight into the caller's frame when there is one
            float* rgb_dst = d_rgb_out != nullptr ? d_rgb_out + (size_t)(ray_offset + raysDone) * 3 : d_render_rgb.as<float>();
            throw_on_error(nb_composite_infer(crrRays, base, raysDone, w.offsets.as<uint32_t>(), w.num_steps.as<uint32_t>() + raysDone, tSorted, sigma,
                                              colorOut, m_fused ? 4 : 8, nullptr, rgb_dst, d_render_depth.as<float>() + raysDone, nullptr, bg, ls),
                           "compositing");
            raysDone += crrRays;
        }
        for (int lane = 0; lane < 2; lane++)
            if (laneUsed[lane]) throw_on_cuda(cudaEventRecord(m_walk[set].freed[lane], alternate ? m_batchStream[lane] : stream), "walk event");
    }
    joinBatches();
}

uint64_t InstantNerf::lastRenderSamples() {
    uint64_t emitted = 0;
    if (d_render_samples.bytes() >= sizeof(uint64_t))
        throw_on_cuda(cudaMemcpy(&emitted, d_render_samples.as<uint64_t>(), sizeof(uint64_t), cudaMemcpyDeviceToHost), "render statistics");
    return emitted + m_renderSamplesHost;
}

// .inerf: "INERF1", raw NerfOptions, fp32 hash table, density W then b, colour W then b (sized for a 16-wide colour
// output as the reference does, the tail beyond the real 8 outputs is zero), fp32 master occupancy grid, bitfield.
// modules/NeRF/InstantNerf.cu:1206-1352.
static void mlp_counts(int in, int hid, int out, int layers, int& w, int& b) {
    w = b = 0;
    for (int l = 0; l < layers; l++) {
        int in_d = (l == 0) ? in : hid, out_d = (l == layers - 1) ? out : hid;
        w += in_d * out_d; b += out_d;
    }
}

void InstantNerf::save(const std::string& filename) {
    if (!m_renderinit) throw std::runtime_error("InstantNerf not initialized, cannot save.");
    std::ofstream out(filename, std::ios::binary);
    if (!out.is_open()) throw std::runtime_error("Cannot open file for saving: " + filename);
    const char magic[6] = {'I', 'N', 'E', 'R', 'F', '1'};
    out.write(magic, 6);
    out.write(reinterpret_cast<const char*>(&m_opts), sizeof(NerfOptions));
    const size_t nHash = (size_t)m_opts.numLevels * m_opts.hashTableSize * m_opts.featuresPerLevel;
    std::vector<float> h(nHash);
    m_densityMLP->saveHashgrid(h.data());
    out.write(reinterpret_cast<const char*>(h.data()), (std::streamsize)(nHash * sizeof(float)));
    int dw, db, cw, cb;
    mlp_counts(m_opts.numLevels * m_opts.featuresPerLevel, m_opts.densityHiddenDim, 16, m_opts.densityNumLayers, dw, db);
    mlp_counts(32, m_opts.colorHiddenDim, 16, m_opts.colorNumLayers, cw, cb);
    std::vector<float> w((size_t)std::max<int64_t>(dw, m_densityMLP->weightCount()), 0.f), b((size_t)std::max<int64_t>(db, m_densityMLP->biasCount()), 0.f);
    m_densityMLP->saveWeights(w.data(), b.data());
    out.write(reinterpret_cast<const char*>(w.data()), dw * sizeof(float));
    out.write(reinterpret_cast<const char*>(b.data()), db * sizeof(float));
    w.assign((size_t)std::max<int64_t>(cw, m_colorMLP->weightCount()), 0.f); b.assign((size_t)std::max<int64_t>(cb, m_colorMLP->biasCount()), 0.f);
    m_colorMLP->saveWeights(w.data(), b.data());
    out.write(reinterpret_cast<const char*>(w.data()), cw * sizeof(float));
    out.write(reinterpret_cast<const char*>(b.data()), cb * sizeof(float));
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const size_t N = (size_t)m_opts.numCascades * G;
    std::vector<float> master(N);
    throw_on_cuda(cudaMemcpy(master.data(), d_masterOccupancyGrid.as<float>(), N * sizeof(float), cudaMemcpyDeviceToHost), "save: master grid");
    out.write(reinterpret_cast<const char*>(master.data()), (std::streamsize)(N * sizeof(float)));
    std::vector<uint8_t> bits(d_occupancyGrid.bytes());
    throw_on_cuda(cudaMemcpy(bits.data(), d_occupancyGrid.as<uint8_t>(), bits.size(), cudaMemcpyDeviceToHost), "save: bitfield");
    out.write(reinterpret_cast<const char*>(bits.data()), (std::streamsize)bits.size());
}

void InstantNerf::load(const std::string& filename) {
    std::ifstream in(filename, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Cannot open file for loading: " + filename);
    char magic[6];
    in.read(magic, 6);
    if (std::string(magic, 6) != "INERF1") throw std::runtime_error("Invalid INERF file format");
    NerfOptions loaded;
    in.read(reinterpret_cast<char*>(&loaded), sizeof(NerfOptions));
    init(loaded);
    const size_t nHash = (size_t)m_opts.numLevels * m_opts.hashTableSize * m_opts.featuresPerLevel;
    std::vector<float> h(nHash);
    in.read(reinterpret_cast<char*>(h.data()), (std::streamsize)(nHash * sizeof(float)));
    m_densityMLP->loadHashgrid(h.data());
    int dw, db, cw, cb;
    mlp_counts(m_opts.numLevels * m_opts.featuresPerLevel, m_opts.densityHiddenDim, 16, m_opts.densityNumLayers, dw, db);
    mlp_counts(32, m_opts.colorHiddenDim, 16, m_opts.colorNumLayers, cw, cb);
    std::vector<float> w((size_t)std::max<int64_t>(dw, m_densityMLP->weightCount()), 0.f), b((size_t)std::max<int64_t>(db, m_densityMLP->biasCount()), 0.f);
    in.read(reinterpret_cast<char*>(w.data()), dw * sizeof(float));
    in.read(reinterpret_cast<char*>(b.data()), db * sizeof(float));
    m_densityMLP->loadWeights(w.data(), b.data());
    w.assign((size_t)std::max<int64_t>(cw, m_colorMLP->weightCount()), 0.f); b.assign((size_t)std::max<int64_t>(cb, m_colorMLP->biasCount()), 0.f);
    in.read(reinterpret_cast<char*>(w.data()), cw * sizeof(float));
    in.read(reinterpret_cast<char*>(b.data()), cb * sizeof(float));
    m_colorMLP->loadWeights(w.data(), b.data());
    const int G = m_opts.gridResolution.x * m_opts.gridResolution.y * m_opts.gridResolution.z;
    const size_t N = (size_t)m_opts.numCascades * G;
    std::vector<float> master(N);
    in.read(reinterpret_cast<char*>(master.data()), (std::streamsize)(N * sizeof(float)));
    std::vector<uint8_t> bits(d_occupancyGrid.bytes());
    in.read(reinterpret_cast<char*>(bits.data()), (std::streamsize)bits.size());
    if (!in) throw std::runtime_error("INERF file truncated: " + filename);
    throw_on_cuda(cudaMemcpy(d_masterOccupancyGrid.as<float>(), master.data(), N * sizeof(float), cudaMemcpyHostToDevice), "load: master grid");
    throw_on_cuda(cudaMemcpy(d_occupancyGrid.as<uint8_t>(), bits.data(), bits.size(), cudaMemcpyHostToDevice), "load: bitfield");
}
