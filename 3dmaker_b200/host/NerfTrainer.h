// Training / rendering facade, source-compatible with the reference's INerfTrainer where the hot path is
// concerned (modules/NeRF/NerfTrainer.h:9-112): same config and stats structs, cosine learning-rate schedule,
// chunk loop, orbit camera, PSNR, .inerf + scene footer files.
//
// The reference feeds the loop from its DataLoader (image files through pinned host memory), which is outside
// this library.  Rays come from a RaySource instead: a callback that fills device buffers with the next chunk of
// rays and target colours.  loadDataset() therefore reports that dataset loading is not part of the library.
#pragma once

#include <functional>
#include <random>

#include "InstantNerf.h"

struct Vec3 { float x, y, z; };

struct Image {
    int width = 0, height = 0;
    std::vector<float> rgb;
};

struct TrainStats {
    int step = 0;
    int targetSteps = 0;
    float loss = 0.0f;
    float psnr = 0.0f;
    float lr = 0.0f;
    float epochs = 0.0f;
    float msPerStep = 0.0f;
    float etaSeconds = 0.0f;
};

struct NerfConfig {
    float lambdaDepth = 0.01f;
    float lambdaDist = 0.1f;
    int numCascades = 0;
    float minDensityThreshold = 0.01f;
    int sampleK = 1;
    int batchSize = 256 * 1024;
    int renderBatchSize = 256 * 1024;
    float depthFraction = 12.5f / 100.0f;
    bool shouldValidate = false;

    float maxLR = 1e-2f;
    float minLR = 1e-3f;
    int annealSteps = 0;
};

class INerfTrainer {
public:
    // Fills d_rays_o / d_rays_d (float3 per ray) and d_rgb_true (3 floats per ray) with `count` rays starting at
    // `cursor` of the epoch identified by `epochSeed`, composited over `bg`, on `stream`.
    using RaySource = std::function<void(uint32_t cursor, uint32_t count, uint32_t epochSeed, float3 bg, float3* d_rays_o, float3* d_rays_d,
                                         float* d_rgb_true, cudaStream_t stream)>;

    INerfTrainer() = default;
    ~INerfTrainer();
    INerfTrainer(const INerfTrainer&) = delete;
    INerfTrainer& operator=(const INerfTrainer&) = delete;

    void init(const NerfConfig& config);
    void loadDataset(const std::string& path);  // throws: image datasets are outside this library, use setRaySource
    // Replaces loadDataset for synthetic or externally loaded data (no counterpart in the reference).
    void setRaySource(RaySource source, uint32_t totalRays, Vec3 sceneUp = {0.0f, 1.0f, 0.0f}, bool randomBackground = true);
    // A posed image set already in device memory (decoding image files stays outside the library): training rays are
    // drawn from it by nb_fetch_ray_chunk exactly as DataLoader::fetchRayChunk draws them (PCG pick, hold-out of every 8th
    // image when the config asks for validation, depth-prior slots), and validate() / renderTrainView() work as in the
    // reference.  The set's device buffers must outlive the trainer.  No counterpart in the reference, where
    // loadDataset() produces the same state from files.
    void setImageSet(const nb_image_set& set, Vec3 sceneUp = {0.0f, 1.0f, 0.0f}, bool randomBackground = true);
    // Hold-out PSNR over every 8th image, white background (NerfTrainer.cu:378-409); 0 without an image set.
    float validate();
    // Frame `index` of the image set re-rendered from its own pose (NerfTrainer.cu:368-376).
    Image renderTrainView(int index, int width = 0, int height = 0);
    // Data-parallel training (no counterpart in the reference, which is single-GPU): one process per GPU, each with its own
    // INerfTrainer on the same ray source.  A chunk of the ray source becomes the GLOBAL batch: rank r fetches and trains
    // rays [r * chunk / world, (r + 1) * chunk / world) of it, loss gradients are normalised by the global ray count, every
    // rank takes exactly stepsPerChunk optimizer steps per chunk, and `sync` (e.g. ncclAllReduce(sum) in place on the
    // caller's communicator and the given stream) runs on the flat gradient arena between backward and Adam of each.
    // world == 1 restores single-process training.  Call after init() and before training.
    void setDataParallel(InstantNerf::GradSync sync, uint32_t rank, uint32_t world, int stepsPerChunk = 1);
    // Lets a caller override what init() derives (AABB, network sizes, ...) before the model is built.
    NerfOptions& options() { return m_masterConfig; }

    void train(int maxSteps, int maxEpochs = 0);
    void beginTraining(int totalSteps);
    TrainStats trainSteps(int nSteps);
    bool isTrainingDone() const { return m_targetSteps > 0 && m_globalStep >= m_targetSteps; }
    const std::vector<float>& lossHistory() const { return m_lossHistory; }
    int step() const { return m_globalStep; }
    int targetSteps() const { return m_targetSteps; }
    float epochs() const { return (m_total_rays > 0) ? (float)(m_raysSeen / (double)m_total_rays) : 0.0f; }
    float msPerStep() const { return (float)m_emaMsPerStep; }

    void save(const std::string& path);
    void load(const std::string& path);

    Vec3 sceneCenter() const { return m_sceneCenter; }
    Vec3 sceneUp() const { return m_sceneUp; }

    Image renderOrbit(float azimuthDeg, float elevationDeg, float radius, float fovDeg = 50.0f, int width = 800, int height = 800);
    // Camera-to-world of the orbit camera, row-major 3x4 (the matrix renderOrbit builds, NerfTrainer.cu:330-366).
    void orbitCamera(float azimuthDeg, float elevationDeg, float radius, float c2w[12]) const;
    // Renders pixels [firstPixel, firstPixel + count) of the frame into d_rgb_out (device, 3 floats per pixel).
    void renderPixels(const float c2w[12], float focal, int width, int height, int64_t firstPixel, int64_t count, float* d_rgb_out,
                      cudaStream_t stream = 0);
    InstantNerf* engine() { return m_nerf; }

private:
    void buildModel();
    float trainOneChunk(bool computeLoss);
    float currentLR() const;
    void ensureChunkBuffers();

    NerfConfig m_config;
    NerfOptions m_masterConfig;
    InstantNerf* m_nerf = nullptr;
    RaySource m_source;
    nb_image_set m_imageSet{};
    bool m_hasImageSet = false;
    uint32_t m_holdoutEvery = 0;
    nb::DeviceMem m_d_prior_depth, m_d_prior_sigma;
    bool m_randomBg = true;
    uint32_t m_total_rays = 0;
    uint32_t m_dpRank = 0, m_dpWorld = 1;

    Vec3 m_sceneCenter = {0.0f, 0.0f, 0.0f};
    Vec3 m_sceneUp = {0.0f, 1.0f, 0.0f};
    float m_sceneScale = 1.0f;
    float m_cameraAngleX = 0.0f;

    int m_globalStep = 0;
    int m_targetSteps = 0;
    uint32_t m_rayCursor = 0;
    uint32_t m_epochSeed = 0;
    std::vector<float> m_lossHistory;
    double m_raysSeen = 0.0;
    double m_emaMsPerStep = 0.0;

    nb::DeviceMem m_d_loss, m_d_chunkRgb, m_d_rays_o, m_d_rays_d, m_d_rgb_true, m_d_frame_o, m_d_frame_d;

    std::mt19937 m_rng{42};
    std::uniform_real_distribution<float> m_dist{0.0f, 1.0f};
    std::uniform_int_distribution<uint32_t> m_seed_dist{0u, 0xFFFFFFFFu};
};
