// INerfTrainer facade.  Follows modules/NeRF/NerfTrainer.cu: defaults of init() (:49-95), cosine learning rate
// (:131-135), one chunk = fetch rays, train, optional MSE read-back (:137-179), stats (:190-225), .inerf plus the
// 36-byte "SCN1" scene footer (:266-300), orbit camera and frame render (:302-366).
#include "NerfTrainer.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <fstream>
#include <iostream>

using nb::throw_on_cuda;
using nb::throw_on_error;

static constexpr float kPI = 3.14159265358979323846f;

void INerfTrainer::init(const NerfConfig& config) {
    m_config = config;
    NerfOptions& opts = m_masterConfig;
    opts.gridResolution = make_uint3(128, 128, 128);
    opts.aabbMin = make_float3(-1.5f, -1.5f, -1.5f);
    opts.aabbMax = make_float3(1.5f, 1.5f, 1.5f);
    opts.levelsMipmap = 4;
    opts.numCascades = (config.numCascades > 0) ? config.numCascades : 1;
    opts.samplesPerVoxel = config.sampleK;
    opts.densityHiddenDim = 64; opts.densityNumLayers = 2;
    opts.colorHiddenDim = 32; opts.colorNumLayers = 3;
    opts.hashTableSize = 1 << 19; opts.numLevels = 16; opts.growthFactor = 1.3819f; opts.baseResolution = 16; opts.featuresPerLevel = 2;
    opts.renderBatchSize = config.renderBatchSize;
    opts.batchSize = config.batchSize;
    opts.rayChunkSize = config.batchSize / 4;
    opts.lambdaDepth = config.lambdaDepth; opts.lambdaDist = config.lambdaDist;
    opts.learningRate = config.maxLR;
    opts.beta1 = 0.9f; opts.beta2 = 0.999f; opts.epsilon = 1e-8f;
    opts.lossScale = 128.0f;
    opts.bgColor = make_float3(1.0f, 1.0f, 1.0f);
    opts.minDensityThreshold = config.minDensityThreshold;
    opts.decayValue = 0.95f;
    opts.densityBias = 0.0f;
    opts.legacyRenderFlag = false;
    opts.isProfiling = false;
    m_d_loss.allocate(sizeof(float), true);
}

INerfTrainer::~INerfTrainer() { delete m_nerf; }

void INerfTrainer::buildModel() {
    if (m_nerf) return;
    m_nerf = new InstantNerf();
    m_nerf->init(m_masterConfig, TRAINING);
}

void INerfTrainer::ensureChunkBuffers() {
    size_t R = (size_t)m_masterConfig.rayChunkSize;
    if (m_d_rays_o.bytes() >= R * 3 * sizeof(float)) return;
    m_d_rays_o.allocate(R * 3 * sizeof(float)); m_d_rays_d.allocate(R * 3 * sizeof(float)); m_d_rgb_true.allocate(R * 3 * sizeof(float));
    m_d_chunkRgb.allocate(R * 3 * sizeof(float));
}

void INerfTrainer::loadDataset(const std::string& path) {
    throw std::runtime_error("INerfTrainer::loadDataset(" + path + "): image datasets are outside this library; feed rays with setRaySource()");
}

void INerfTrainer::setRaySource(RaySource source, uint32_t totalRays, Vec3 sceneUp, bool randomBackground) {
    m_source = std::move(source);
    m_total_rays = totalRays;
    m_sceneUp = sceneUp;
    m_randomBg = randomBackground;
    buildModel();
    ensureChunkBuffers();
    m_globalStep = 0;
    m_rayCursor = 0;
    m_lossHistory.clear();
}

void INerfTrainer::setImageSet(const nb_image_set& set, Vec3 sceneUp, bool randomBackground) {
    if (!set.d_images_rgba || !set.d_transforms || set.num_images <= 0 || set.width <= 0 || set.height <= 0)
        throw std::runtime_error("setImageSet: empty image set");
    m_imageSet = set;
    m_imageSet.dense_fraction = (set.num_records > 0) ? m_config.depthFraction : 0.0f;
    m_hasImageSet = true;
    m_holdoutEvery = m_config.shouldValidate ? 8u : 0u;   // NerfTrainer.cu:88
    m_cameraAngleX = 2.0f * atanf(0.5f * set.width / set.focal);
    const uint64_t total = (uint64_t)set.num_images * set.width * set.height;
    if (total > 0x7fffffffu) throw std::runtime_error("setImageSet: more than 2^31 - 1 pixels");
    RaySource src = [this](uint32_t cursor, uint32_t count, uint32_t epochSeed, float3 bg, float3* d_o, float3* d_d, float* d_rgb, cudaStream_t st) {
        const float bgc[3] = {bg.x, bg.y, bg.z};
        if (m_d_prior_depth.bytes() < count * sizeof(float)) { m_d_prior_depth.allocate(count * sizeof(float)); m_d_prior_sigma.allocate(count * sizeof(float)); }
        throw_on_error(nb_fetch_ray_chunk(&m_imageSet, (int)cursor, (int)count, epochSeed, 1, bgc, (int)m_holdoutEvery, reinterpret_cast<float*>(d_o),
                                          reinterpret_cast<float*>(d_d), d_rgb, m_d_prior_depth.as<float>(), m_d_prior_sigma.as<float>(), st),
                       "ray fetch");
    };
    setRaySource(std::move(src), (uint32_t)total, sceneUp, randomBackground);
}

float INerfTrainer::validate() {
    if (!m_nerf || !m_hasImageSet) return 0.0f;
    const int HOLDOUT = 8;
    const int pixels = m_imageSet.width * m_imageSet.height;
    const int tile = (int)m_masterConfig.rayChunkSize;
    ensureChunkBuffers();
    m_nerf->setMemoryMode(INFERENCE);
    const float white[3] = {1.0f, 1.0f, 1.0f};
    m_nerf->setBgColor(make_float3(1.0f, 1.0f, 1.0f));
    throw_on_error(nb_zero_async(m_d_loss.as<float>(), sizeof(float), 0), "loss reset");
    long long totalPixels = 0;
    for (int i = 0; i < m_imageSet.num_images; i += HOLDOUT) {
        for (int off = 0; off < pixels; off += tile) {
            const int count = std::min(tile, pixels - off);
            throw_on_error(nb_fetch_ray_chunk(&m_imageSet, i * pixels + off, count, 0u, 0, white, 0, m_d_rays_o.as<float>(), m_d_rays_d.as<float>(),
                                              m_d_rgb_true.as<float>(), nullptr, nullptr, 0), "ray fetch");
            m_nerf->renderImageHit(m_d_rays_o.as<float3>(), m_d_rays_d.as<float3>(), (uint32_t)count, m_d_chunkRgb.as<float>(), 0);
            throw_on_error(nb_mse_rays(m_d_chunkRgb.as<float>(), m_d_rgb_true.as<float>(), m_d_loss.as<float>(), count, 0), "validation error");
            totalPixels += count;
        }
    }
    float h_loss = 0.0f;
    throw_on_cuda(cudaMemcpy(&h_loss, m_d_loss.as<float>(), sizeof(float), cudaMemcpyDeviceToHost), "validation loss");
    const float mse = h_loss / (float)std::max(1LL, totalPixels);
    return -10.0f * log10f(fmaxf(mse, 1e-8f));
}

Image INerfTrainer::renderTrainView(int index, int width, int height) {
    Image img;
    if (!m_nerf || !m_hasImageSet || index < 0 || index >= m_imageSet.num_images) return img;
    if (width <= 0) width = m_imageSet.width;
    if (height <= 0) height = m_imageSet.height;
    float m16[16];
    throw_on_cuda(cudaMemcpy(m16, m_imageSet.d_transforms + (size_t)index * 16, sizeof(m16), cudaMemcpyDeviceToHost), "frame pose");
    float c2w[12];
    for (int r = 0; r < 3; r++)
        for (int c = 0; c < 4; c++) c2w[4 * r + c] = m16[4 * r + c];
    const float focal = 0.5f * width / tanf(0.5f * m_cameraAngleX);
    img.width = width; img.height = height;
    img.rgb.assign((size_t)width * height * 3, 0.0f);
    nb::DeviceMem d_rgb;
    d_rgb.allocate(img.rgb.size() * sizeof(float));
    renderPixels(c2w, focal, width, height, 0, (int64_t)width * height, d_rgb.as<float>(), 0);
    throw_on_cuda(cudaDeviceSynchronize(), "renderTrainView");
    throw_on_cuda(cudaMemcpy(img.rgb.data(), d_rgb.as<float>(), img.rgb.size() * sizeof(float), cudaMemcpyDeviceToHost), "renderTrainView");
    return img;
}

float INerfTrainer::currentLR() const {
    int anneal = (m_config.annealSteps > 0) ? m_config.annealSteps : std::max(1, m_targetSteps);
    float progress = fminf((float)m_globalStep / (float)anneal, 1.0f);
    return m_config.minLR + 0.5f * (m_config.maxLR - m_config.minLR) * (1.0f + cosf(kPI * progress));
}

float INerfTrainer::trainOneChunk(bool computeLoss) {
    const uint32_t rayChunk = (uint32_t)m_masterConfig.rayChunkSize;
    if (m_rayCursor >= m_total_rays) m_rayCursor = 0;
    if (m_rayCursor == 0) m_epochSeed = m_seed_dist(m_rng);
    int chunkSize = (int)std::min(rayChunk, m_total_rays - m_rayCursor);

    m_nerf->setLearningRate(currentLR());
    m_nerf->setMemoryMode(TRAINING);
    float3 bg = m_masterConfig.bgColor;
    if (m_randomBg) bg = make_float3(m_dist(m_rng), m_dist(m_rng), m_dist(m_rng));  // random-background augmentation
    m_nerf->setBgColor(bg);

    m_source(m_rayCursor, (uint32_t)chunkSize, m_epochSeed, bg, m_d_rays_o.as<float3>(), m_d_rays_d.as<float3>(), m_d_rgb_true.as<float>(), 0);
    if (computeLoss) throw_on_error(nb_zero_async(m_d_loss.as<float>(), sizeof(float), 0), "loss reset");

    const bool priors = m_hasImageSet && m_imageSet.num_records > 0;
    m_nerf->trainWithRaysHit(m_d_rays_o.as<float3>(), m_d_rays_d.as<float3>(), priors ? m_d_prior_depth.as<float>() : nullptr,
                             priors ? m_d_prior_sigma.as<float>() : nullptr, m_d_rgb_true.as<float>(), (uint32_t)chunkSize,
                             m_globalStep, nullptr, computeLoss ? m_d_chunkRgb.as<float>() : nullptr, 0);
    m_rayCursor += chunkSize;
    m_raysSeen += chunkSize;
    if (!computeLoss) return -1.0f;
    throw_on_error(nb_mse_rays(m_d_chunkRgb.as<float>(), m_d_rgb_true.as<float>(), m_d_loss.as<float>(), chunkSize, 0), "chunk MSE");
    float h_loss = 0.0f;
    throw_on_cuda(cudaMemcpy(&h_loss, m_d_loss.as<float>(), sizeof(float), cudaMemcpyDeviceToHost), "chunk MSE");
    return h_loss / std::max(1, chunkSize);
}

void INerfTrainer::beginTraining(int totalSteps) {
    m_targetSteps = std::max(1, totalSteps);
    m_globalStep = 0;
    m_rayCursor = 0;
    m_raysSeen = 0.0;
    m_emaMsPerStep = 0.0;
    m_lossHistory.clear();
}

TrainStats INerfTrainer::trainSteps(int nSteps) {
    TrainStats s;
    if (!m_nerf || !m_source || m_total_rays == 0) return s;
    if (m_targetSteps == 0) beginTraining(20000);
    int target = std::min(m_globalStep + std::max(1, nSteps), m_targetSteps);
    int startStep = m_globalStep;
    auto t0 = std::chrono::high_resolution_clock::now();
    float mse = -1.0f;
    bool first = true;
    while (m_globalStep < target) {
        float chunkMse = trainOneChunk(first);
        if (chunkMse > 0.0f) mse = chunkMse;
        first = false;
    }
    throw_on_cuda(cudaDeviceSynchronize(), "trainSteps");
    auto t1 = std::chrono::high_resolution_clock::now();
    int stepsDone = m_globalStep - startStep;
    if (stepsDone > 0) {
        double msPerStep = std::chrono::duration<double, std::milli>(t1 - t0).count() / stepsDone;
        m_emaMsPerStep = (m_emaMsPerStep > 0.0) ? (0.70 * m_emaMsPerStep + 0.30 * msPerStep) : msPerStep;
    }
    if (mse > 0.0f) m_lossHistory.push_back(mse);
    int remaining = std::max(0, m_targetSteps - m_globalStep);
    s.step = m_globalStep;
    s.targetSteps = m_targetSteps;
    s.loss = (mse > 0.0f) ? mse : (m_lossHistory.empty() ? 0.0f : m_lossHistory.back());
    s.psnr = (s.loss > 0.0f) ? -10.0f * log10f(fmaxf(s.loss, 1e-8f)) : 0.0f;
    s.lr = currentLR();
    s.epochs = epochs();
    s.msPerStep = (float)m_emaMsPerStep;
    s.etaSeconds = (float)(m_emaMsPerStep * remaining / 1000.0);
    return s;
}

void INerfTrainer::train(int maxSteps, int maxEpochs) {
    (void)maxEpochs;
    if (!m_nerf || !m_source || m_total_rays == 0) {
        std::cerr << "[INerfTrainer] train() called before a ray source was set." << std::endl;
        return;
    }
    beginTraining(maxSteps);
    int tick = std::max(1, maxSteps / 100);
    while (!isTrainingDone()) {
        TrainStats s = trainSteps(tick);
        std::printf("\r%d/%d steps | epoch %.2f | %.2f ms/step | ETA %.0f s | PSNR %.1f   ", s.step, s.targetSteps, s.epochs, s.msPerStep,
                    s.etaSeconds, s.psnr);
        std::fflush(stdout);
    }
    std::printf("\n");
}

static const char kSceneMagic[4] = {'S', 'C', 'N', '1'};
static const std::streamoff kSceneFooterBytes = 4 + 8 * (std::streamoff)sizeof(float);

void INerfTrainer::save(const std::string& path) {
    if (!m_nerf) return;
    m_nerf->save(path);
    std::ofstream out(path, std::ios::binary | std::ios::app);
    if (!out) return;
    float buf[8] = {m_sceneCenter.x, m_sceneCenter.y, m_sceneCenter.z, m_sceneUp.x, m_sceneUp.y, m_sceneUp.z, m_sceneScale, m_cameraAngleX};
    out.write(kSceneMagic, 4);
    out.write(reinterpret_cast<const char*>(buf), sizeof(buf));
}

void INerfTrainer::load(const std::string& path) {
    buildModel();
    m_nerf->load(path);
    m_masterConfig = m_nerf->options();
    std::ifstream in(path, std::ios::binary | std::ios::ate);
    if (!in) return;
    std::streamoff size = in.tellg();
    if (size < kSceneFooterBytes) return;
    in.seekg(size - kSceneFooterBytes, std::ios::beg);
    char magic[4];
    in.read(magic, 4);
    if (std::string(magic, 4) != std::string(kSceneMagic, 4)) return;
    float buf[8];
    in.read(reinterpret_cast<char*>(buf), sizeof(buf));
    m_sceneCenter = {buf[0], buf[1], buf[2]};
    m_sceneUp = {buf[3], buf[4], buf[5]};
    m_sceneScale = buf[6];
    m_cameraAngleX = buf[7];
}

static inline float3 cross3(float3 a, float3 b) { return make_float3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
static inline float3 normalize3(float3 v) {
    float l = sqrtf(v.x * v.x + v.y * v.y + v.z * v.z);
    return l > 0 ? make_float3(v.x / l, v.y / l, v.z / l) : v;
}

void INerfTrainer::orbitCamera(float azimuthDeg, float elevationDeg, float radius, float c2w[12]) const {
    float3 center = make_float3(m_sceneCenter.x, m_sceneCenter.y, m_sceneCenter.z);
    float3 up = normalize3(make_float3(m_sceneUp.x, m_sceneUp.y, m_sceneUp.z));
    float3 ref = (fabsf(up.y) < 0.9f) ? make_float3(0, 1, 0) : make_float3(1, 0, 0);
    float3 a = normalize3(cross3(up, ref));
    float3 b = cross3(up, a);
    float az = azimuthDeg * kPI / 180.0f, el = elevationDeg * kPI / 180.0f;
    float3 planar = make_float3(cosf(az) * a.x + sinf(az) * b.x, cosf(az) * a.y + sinf(az) * b.y, cosf(az) * a.z + sinf(az) * b.z);
    float3 dir = make_float3(cosf(el) * planar.x + sinf(el) * up.x, cosf(el) * planar.y + sinf(el) * up.y, cosf(el) * planar.z + sinf(el) * up.z);
    float3 eye = make_float3(center.x + radius * dir.x, center.y + radius * dir.y, center.z + radius * dir.z);
    float3 f = normalize3(make_float3(center.x - eye.x, center.y - eye.y, center.z - eye.z));
    float3 r = normalize3(cross3(f, up));
    float3 u = cross3(r, f);
    const float m[12] = {r.x, u.x, -f.x, eye.x, r.y, u.y, -f.y, eye.y, r.z, u.z, -f.z, eye.z};
    for (int i = 0; i < 12; i++) c2w[i] = m[i];
}

void INerfTrainer::renderPixels(const float c2w[12], float focal, int width, int height, int64_t firstPixel, int64_t count, float* d_rgb_out,
                                cudaStream_t stream) {
    if (!m_nerf) throw std::runtime_error("renderPixels called before the model exists");
    size_t need = (size_t)count * 3 * sizeof(float);
    if (m_d_frame_o.bytes() < need) { m_d_frame_o.allocate(need); m_d_frame_d.allocate(need); }  // kept between frames
    throw_on_error(nb_generate_rays(width, height, focal, c2w, firstPixel, count, m_d_frame_o.as<float>(), m_d_frame_d.as<float>(), stream),
                   "ray generation");
    m_nerf->setMemoryMode(INFERENCE);
    m_nerf->renderImageHit(m_d_frame_o.as<float3>(), m_d_frame_d.as<float3>(), (uint32_t)count, d_rgb_out, stream);
}

Image INerfTrainer::renderOrbit(float azimuthDeg, float elevationDeg, float radius, float fovDeg, int width, int height) {
    Image img;
    if (!m_nerf || width <= 0 || height <= 0) return img;
    img.width = width; img.height = height;
    img.rgb.assign((size_t)width * height * 3, 0.0f);
    float c2w[12];
    orbitCamera(azimuthDeg, elevationDeg, radius, c2w);
    float focal = 0.5f * width / tanf(0.5f * fovDeg * kPI / 180.0f);
    nb::DeviceMem d_rgb;
    d_rgb.allocate(img.rgb.size() * sizeof(float));
    renderPixels(c2w, focal, width, height, 0, (int64_t)width * height, d_rgb.as<float>(), 0);
    throw_on_cuda(cudaDeviceSynchronize(), "renderOrbit");
    throw_on_cuda(cudaMemcpy(img.rgb.data(), d_rgb.as<float>(), img.rgb.size() * sizeof(float), cudaMemcpyDeviceToHost), "renderOrbit");
    return img;
}
