// Scene engine: owns the occupancy grid, both networks (in ONE parameter arena) and all scratch buffers, and
// runs the optimizer step and the frame render.  Source-compatible with the reference's InstantNerf
// (modules/NeRF/InstantNerf.h:35-76 NerfOptions, :279-334 class): same option struct (field order is part of
// the .inerf file format), same public methods and argument meaning.
//
// What differs underneath (see InstantNerf.cu): one forward pass per step instead of two, one 16-byte read-back
// per step instead of three, no pad/unpad copies between the networks, one Adam launch for everything, and a
// hook between backward and optimizer for the data-parallel gradient all-reduce.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include "TinyMLPHashGrid.h"

#define MAX_HITS 1024  // per-ray sample cap

// Programs written against the reference's InstantNerf.h use this macro for their own CUDA calls; as there
// (modules/NeRF/InstantNerf.h:13-22) a failed call prints where it happened and throws std::runtime_error.
#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                                                                  \
    do {                                                                                                  \
        cudaError_t nb_cuda_check_status_ = (call);                                                       \
        if (nb_cuda_check_status_ != cudaSuccess) {                                                       \
            std::fprintf(stderr, "CUDA error at %s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(nb_cuda_check_status_)); \
            throw std::runtime_error(cudaGetErrorString(nb_cuda_check_status_));                          \
        }                                                                                                 \
    } while (0)
#endif

enum MemoryMode { TRAINING, INFERENCE };

struct NerfOptions {
    uint3 gridResolution = make_uint3(128, 128, 128);
    float3 aabbMin = make_float3(-1.0f, -1.0f, -1.0f);
    float3 aabbMax = make_float3(1.0f, 1.0f, 1.0f);
    int levelsMipmap = 4;
    int numCascades = 1;
    int samplesPerVoxel = 1;

    int densityHiddenDim = 64;
    int densityNumLayers = 2;

    int colorHiddenDim = 64;
    int colorNumLayers = 2;

    int hashTableSize = 1 << 19;
    int numLevels = 16;
    float growthFactor = 1.3819f;
    int baseResolution = 16;
    int featuresPerLevel = 2;

    int renderBatchSize = 2048 * 1024;
    int batchSize = 256 * 1024;
    int rayChunkSize = 256 * 1024;

    float lambdaDepth = 0.02882f;
    float lambdaDist = 0.0362781f;
    float learningRate = 1e-3f;
    float beta1 = 0.9f;
    float beta2 = 0.999f;
    float epsilon = 1e-8f;
    float lossScale = 1.0f;

    float3 bgColor = make_float3(1.0f, 1.0f, 1.0f);
    float minDensityThreshold = 0.01;
    float decayValue = 0.95f;
    float densityBias = 1.0f;

    bool legacyRenderFlag = false;
    bool isProfiling = false;
};

// Per-phase device time of the last training steps / rendered frames (milliseconds, summed), filled when
// NerfOptions.isProfiling is set.  Plays the role of the reference's GPUStats (InstantNerf.h:128-277).
struct NerfPhaseTimes {
    double march = 0, occupancy = 0, densityFwd = 0, shGather = 0, colorFwd = 0, compositing = 0, lossGrad = 0, colorBwd = 0,
           densityGrad = 0, densityBwd = 0, scatter = 0, optimizer = 0;
    long steps = 0;
};

class InstantNerf {
public:
    InstantNerf() = default;
    ~InstantNerf();
    InstantNerf(const InstantNerf&) = delete;
    InstantNerf& operator=(const InstantNerf&) = delete;

    void init(const NerfOptions& opts, MemoryMode memMode = TRAINING);
    void printStats();
    void resetStats();
    void setLearningRate(float lr) { m_opts.learningRate = lr; }
    void setBgColor(float3 c) { m_opts.bgColor = c; }
    void setProfiling(bool p) { m_opts.isProfiling = p; }
    void setMemoryMode(MemoryMode mode);

    // One optimizer step per batch of whole rays that fits batchSize samples, until all numRays are consumed.
    // d_rays_depth / d_rays_sigma (depth priors) and d_rgb_out / hitCounts may be null.
    void trainWithRaysHit(const float3* d_rays_o, const float3* d_rays_d, const float* d_rays_depth, const float* d_rays_sigma,
                          const float* d_rgb_true, uint32_t numRays, int& trainStepCount, uint32_t* hitCounts, float* d_rgb_out,
                          cudaStream_t stream);
    void renderImageHit(const float3* d_rays_o, const float3* d_rays_d, uint32_t numRays, float* d_rgb_out, cudaStream_t stream);
    // The reference keeps an older sparse-layout renderer under this name; here it is the same path as renderImageHit.
    void renderImage(const float3* d_rays_o, const float3* d_rays_d, uint32_t numRays, float* d_rgb_out = nullptr, cudaStream_t stream = 0) {
        renderImageHit(d_rays_o, d_rays_d, numRays, d_rgb_out, stream);
    }

    const NerfOptions& options() const { return m_opts; }
    const uint8_t* occupancyGrid() { return d_occupancyGrid.as<uint8_t>(); }
    size_t occupancyBytes() { return d_occupancyGrid.bytes(); }

    void save(const std::string& filename);
    void load(const std::string& filename);

    // ---- additions (not in the reference) -------------------------------------------------------------
    // Called on the gradient arena between backward and the optimizer of every step (data-parallel all-reduce).
    using GradSync = std::function<void(float* d_grads, int64_t count, cudaStream_t stream)>;
    void setGradSync(GradSync fn) { m_gradSync = std::move(fn); }
    // Data parallelism with the hash table's optimizer state used shard-wise: of the table's `sparse_count` elements this
    // rank updates slice [rank, rank + 1) * sparse_count / world only (the gradient-sync callback is expected to leave
    // the SUMMED gradient of that slice there, e.g. by a reduce-scatter in place), every rank updates the small dense tail
    // (network weights), the rest of the table gradient is cleared, and `sync` then runs on the fp16 parameter copy - an
    // all-gather of the slices, so that every rank's forward reads identical parameters.  The fp32 master copy, m and v of a
    // slice are current on its owner only.  world <= 1 restores the whole-arena update.
    using ParamSync = std::function<void(half* d_params_h, int64_t sparse_count, cudaStream_t stream)>;
    void setOptimizerShard(uint32_t rank, uint32_t world, ParamSync sync);
    // Data parallelism with ONE kernel for reduce-scatter + optimizer + all-gather (nb_adam_step_peer): peerGrads[r] /
    // peerParamsH[r] are rank r's gradient arena and fp16 parameter arena as THIS process can address them (entry `rank`:
    // this engine's own), `barrier` meets all ranks on the given stream.  Per step: barrier, the kernel on this rank's
    // slice of the table, barrier, this rank's gradient arena cleared.  The gradient-sync callback is not used in this
    // mode.  world <= 1 switches back.
    using RankBarrier = std::function<void(cudaStream_t stream)>;
    void setPeerExchange(uint32_t rank, uint32_t world, const std::vector<const float*>& peerGrads, const std::vector<void*>& peerParamsH,
                         RankBarrier barrier);
    // Data parallelism with the table PARTITIONED BY LEVEL instead of replicated (csrc/level_partition.cu): rank r of
    // `world` owns levels r, r + world, ...; per step the ranks exchange sample positions (one all-gather), encodings (one
    // all-to-all) and encoding gradients (one all-to-all back), 128 bytes per sample in all, and nothing of the table;
    // every rank updates its own levels and, after `reduce` has summed the small dense tail of the gradient arena over the
    // ranks, the network weights.  Needs the fused field kernels; world must divide the number of levels.
    //   gather(send, recv, bytes, stream):   recv = the ranks' `bytes`-sized blocks one after the other (all-gather)
    //   exchange(send, recv, bytes, stream): block q of send goes to rank q, block r of recv comes from rank r (all-to-all)
    // Between steps the levels a rank does not own go stale in its copy of the table; syncLevels() brings every rank's
    // copy up to date (fp16 forward copy; with `master` also the fp32 copy) and runs by itself before occupancy updates.
    // Call it before rendering, saving or comparing replicas.  world <= 1 switches back.
    // Data parallelism: the density queries of an occupancy update (the only heavy part of it) are split over the ranks -
    // rank r evaluates slice r of every batch of sampled cells - and `reduceMax` (an all-reduce with MAX over the ranks)
    // runs on the per-cell maxima before they are folded into the grid.  A maximum does not depend on the order, so
    // every rank ends with the bits a single GPU computes.  world <= 1 switches back.
    void setOccupancyShard(uint32_t rank, uint32_t world, GradSync reduceMax);
    using BlockGather = std::function<void(const void* d_send, void* d_recv, int64_t bytes, cudaStream_t stream)>;
    using BlockExchange = std::function<void(const void* d_send, void* d_recv, int64_t bytes, cudaStream_t stream)>;
    void setLevelPartition(uint32_t rank, uint32_t world, BlockGather gather, BlockExchange exchange, GradSync reduce);
    void syncLevels(cudaStream_t stream, bool master = false);
    bool levelPartitioned() const { return m_partWorld > 1; }
    // Loss gradients are normalised by numRays * scale (the global ray count when ranks split a batch).
    void setGlobalRayScale(uint32_t scale) { m_rayScale = scale ? scale : 1u; }
    // One kernel each way for the whole field (encode + both networks) instead of the reference's kernel sequence;
    // on by default when the network shapes allow it.  Returns the mode now in effect.
    bool setFusedField(bool on);
    bool fusedField() const { return m_fused; }
    // Rendering in rounds of samples per ray (16, 16, 32, 64, ...): rays are not evaluated behind the point where their
    // transmittance has dropped below 1e-4, which the reference's compositing never reaches either.  Pays when surfaces
    // hide much of what the occupancy grid keeps (about half the samples of a many-object scene) and costs a few
    // launches per chunk when they do not, so it is off by default; needs the fused field kernels.  When off, every
    // sample of every ray is evaluated as in the reference.
    void setRenderRounds(bool on) { m_renderRounds = on; }
    bool renderRounds() const { return m_renderRounds && m_fused; }
    // samples the field was evaluated on during the last renderImageHit call (waits for the device)
    uint64_t lastRenderSamples();
    nb::ParamArena& arena() { return m_arena; }
    TinyMLPHashGrid* densityNetwork() { return m_densityMLP; }
    TinyMLP* colorNetwork() { return m_colorMLP; }
    uint8_t* occupancyGridMutable() { return d_occupancyGrid.as<uint8_t>(); }
    float* masterOccupancyGrid() { return d_masterOccupancyGrid.as<float>(); }
    void rebuildOccupancy(cudaStream_t stream = 0) { earlyOccupancyGridUpdate(stream); }
    int trainSteps() const { return m_trainSteps; }
    uint32_t lastTotalHits() const { return m_lastTotalHits; }
    // Data parallelism: exactly k optimizer steps (hence k gradient exchanges) per trainWithRaysHit call on every rank;
    // rays left after the k-th step stay untrained, a rank that runs out of rays earlier steps with no samples.
    // k = 0 restores the reference's loop (as many steps as the rays need).
    void setStepsPerCall(int k) { m_stepsPerCall = k > 0 ? k : 0; }
    void setSingleStep(bool on) { m_stepsPerCall = on ? 1 : 0; }
    // Entries the caller's hitCounts array holds (0 = unbounded, as the reference writes it): steps beyond it are not recorded.
    void setHitCountsCapacity(uint32_t n) { m_hitCountsCapacity = n; }
    uint32_t lastRaysConsumed() const { return m_lastRaysConsumed; }
    const NerfPhaseTimes& phaseTimes() const { return m_times; }
    // Buffers of the last step, for parity tests (valid until the next call).
    struct StepView {
        const uint32_t *num_steps, *ray_offsets, *ray_indices;
        const float *t_sorted, *positions, *density_out, *sigma, *color_out, *render_rgb, *phi, *dw, *weight_sum, *tmp_dsigma;
        const half *color_in, *color_grad, *density_grad;
        int logit_stride;  // density_out[i * logit_stride] = raw logit 0 of sample i (16: full density output rows)
        int color_stride;  // floats between colour rows
        uint32_t sample_base;  // ray_offsets[r] - sample_base = first sample of the step's ray r in the sample arrays
    };
    StepView stepView() const;

private:
    void initRenderBuffers();
    void freeBuffers();
    void earlyOccupancyGridUpdate(cudaStream_t stream = 0);
    void lateOccupancyGridUpdate(cudaStream_t stream = 0);
    void finishOccupancyUpdate(cudaStream_t stream);
    void optimizerStep(cudaStream_t stream);
    void walkRays(const float3* d_rays_o, const float3* d_rays_d, uint32_t first, uint32_t count, cudaStream_t stream, int set, bool wait);
    void finishWalk(int set);
    nb_scene_desc scene() const;
    template <class F> void timed(cudaStream_t stream, double& acc, F&& f);

    NerfOptions m_opts;
    MemoryMode m_memMode = TRAINING;
    nb::ParamArena m_arena;
    TinyMLP* m_colorMLP = nullptr;
    TinyMLPHashGrid* m_densityMLP = nullptr;
    GradSync m_gradSync;
    ParamSync m_paramSync;
    RankBarrier m_rankBarrier;
    std::vector<const float*> m_peerGrads;
    std::vector<void*> m_peerParamsH;
    uint32_t m_shardRank = 0, m_shardWorld = 1;
    // level partition: position slots of all ranks, pieces to send and received
    uint32_t m_partRank = 0, m_partWorld = 1;
    BlockGather m_partGather;
    BlockExchange m_partExchange;
    GradSync m_partReduce;
    nb::DeviceMem d_pos_all, d_pieces_send, d_pieces_recv;
    uint32_t m_occRank = 0, m_occWorld = 1;
    GradSync m_occReduceMax;
    void occupancyDensity(int count, cudaStream_t stream);   // density + per-cell maximum of d_occ_samples[0, count), this rank's slice
    void partitionedForward(const float* chunk_d, int64_t n, int colorStride, cudaStream_t stream);
    void partitionedBackward(const float* chunk_d, int64_t n, cudaStream_t stream);
    uint32_t m_rayScale = 1;
    bool m_fused = false;
    bool m_renderRounds = false;
    NerfPhaseTimes m_times;

    nb::DeviceMem d_occupancyGrid, d_masterOccupancyGrid;
    // per ray chunk
    nb::DeviceMem d_rays_d_inv, d_nears, d_fars, d_block_sums, d_plan, d_render_rgb, d_render_depth, d_phi,
        d_weight_sum;
    // per sample batch
    nb::DeviceMem d_positions, d_ray_indices, d_t_sorted, d_density_out, d_sigma, d_color_in, d_color_out, d_color_acts, d_enc, d_density_acts,
        d_color_grad, d_color_dx, d_density_grad, d_denc, d_tmpsigma, d_dw;
    // occupancy
    nb::DeviceMem d_occ_samples, d_tmp_grid, d_sum, d_occ_scratch, d_active_cells, d_num_active;
    uint32_t* h_plan = nullptr;  // pinned, 4 words
    // buffers of one occupancy walk over a ray chunk; two sets so that rendering can walk ahead
    struct WalkSet {
        nb::DeviceMem num_steps, offsets, rows;
        uint32_t* h_offsets = nullptr;  // pinned: scanned sample offsets of the walked rays (+ total)
        size_t capacity = 0;
        cudaEvent_t done = nullptr;   // the walk into this set has finished (recorded on the stream that walked)
        cudaEvent_t freed[2] = {nullptr, nullptr};  // per batch stream: the batches that read this set are through
    };
    WalkSet m_walk[2];
    // Rendering walks on a stream of its own: the walk keeps one thread per ray busy with dependent probes and fills a
    // fraction of the machine, so it runs beside the field kernels of the chunk before instead of in front of them.
    cudaStream_t m_walkStream = nullptr;
    cudaEvent_t m_raysReady = nullptr;
    // Sample batches of a frame alternate between two streams with a set of sample arrays each, so that the small kernels
    // and the tail of one batch overlap the field kernel of the next.  Set 0 = the arrays training uses.
    cudaStream_t m_batchStream[2] = {nullptr, nullptr};
    cudaEvent_t m_batchDone[2] = {nullptr, nullptr};
    nb::DeviceMem d_positions2, d_ray_indices2, d_t_sorted2, d_sigma2, d_color_out2;
    // rendering in rounds: per ray of the chunk its place in the round's sample arrays, transmittance and colour so far;
    // one sample counter per (round, ray range), zeroed per chunk
    nb::DeviceMem d_round_off, d_transmittance, d_composited, d_round_counters, d_render_samples;
    uint64_t m_renderSamplesHost = 0;  // the part of the count the host knows (every sample, when not in rounds)
    std::vector<uint32_t> m_roundRays;  // host scratch: per 1024-ray block and round, the rays that reach the round
    static constexpr int kRoundCounters = 64;
    void renderChunkRounds(const WalkSet& w, const float* chunk_o, const float* chunk_d, uint32_t chunkRays, uint32_t capacity, float* rgb_dst,
                           cudaStream_t stream);
    uint32_t m_lastStepFirstRay = 0, m_lastSampleBase = 0;

    bool m_traininit = false;
    bool m_renderinit = false;
    int m_trainSteps = 0;
    int m_optSteps = 0;  // Adam step counter (capped at 50000 for the bias corrections)
    uint32_t m_lastTotalHits = 0;
    uint32_t m_lastRaysConsumed = 0;
    int m_stepsPerCall = 0;
    uint32_t m_hitCountsCapacity = 0;
};
