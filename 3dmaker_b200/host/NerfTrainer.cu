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

// Learning rate of the step about to run: half a cosine from maxLR down to minLR over the anneal span (annealSteps, or
// the whole run when that is 0), minLR from there on.  Schedule of the reference's currentLR (NerfTrainer.cu:131-135).
namespace {
struct CosineDecay {
    float high, low;
    int span;
    float at(int step) const {
        const float x = (span > 0 && step < span) ? (float)step / (float)span : 1.0f;
        return low + (high - low) * 0.5f * (1.0f + cosf(kPI * x));
    }
};
}  // namespace

float INerfTrainer::currentLR() const {
    const CosineDecay lr{m_config.maxLR, m_config.minLR, m_config.annealSteps > 0 ? m_config.annealSteps : std::max(1, m_targetSteps)};
    return lr.at(m_globalStep);
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

    // Data parallel: the chunk is the GLOBAL ray batch of these steps; this rank fetches and trains its contiguous share.
    uint32_t first = m_rayCursor;
    const uint32_t globalChunk = (uint32_t)chunkSize;
    if (m_dpWorld > 1) {
        first += (uint32_t)((uint64_t)globalChunk * m_dpRank / m_dpWorld);
        chunkSize = (int)((uint64_t)globalChunk * (m_dpRank + 1) / m_dpWorld - (uint64_t)globalChunk * m_dpRank / m_dpWorld);
    }
    m_source(first, (uint32_t)chunkSize, m_epochSeed, bg, m_d_rays_o.as<float3>(), m_d_rays_d.as<float3>(), m_d_rgb_true.as<float>(), 0);
    if (computeLoss) throw_on_error(nb_zero_async(m_d_loss.as<float>(), sizeof(float), 0), "loss reset");

    const bool priors = m_hasImageSet && m_imageSet.num_records > 0;
    m_nerf->trainWithRaysHit(m_d_rays_o.as<float3>(), m_d_rays_d.as<float3>(), priors ? m_d_prior_depth.as<float>() : nullptr,
                             priors ? m_d_prior_sigma.as<float>() : nullptr, m_d_rgb_true.as<float>(), (uint32_t)chunkSize,
                             m_globalStep, nullptr, computeLoss ? m_d_chunkRgb.as<float>() : nullptr, 0);
    m_rayCursor += globalChunk;
    m_raysSeen += globalChunk;
    if (!computeLoss) return -1.0f;
    throw_on_error(nb_mse_rays(m_d_chunkRgb.as<float>(), m_d_rgb_true.as<float>(), m_d_loss.as<float>(), chunkSize, 0), "chunk MSE");
    float h_loss = 0.0f;
    throw_on_cuda(cudaMemcpy(&h_loss, m_d_loss.as<float>(), sizeof(float), cudaMemcpyDeviceToHost), "chunk MSE");
    return h_loss / std::max(1, chunkSize);
}

void INerfTrainer::setDataParallel(InstantNerf::GradSync sync, uint32_t rank, uint32_t world, int stepsPerChunk) {
    if (world == 0 || rank >= world) throw std::runtime_error("setDataParallel: rank must be below the number of ranks");
    buildModel();
    m_dpRank = rank; m_dpWorld = world;
    m_nerf->setGlobalRayScale(world);
    m_nerf->setGradSync(world > 1 ? std::move(sync) : InstantNerf::GradSync());
    // the same number of optimizer steps, hence gradient exchanges, per chunk on every rank
    m_nerf->setStepsPerCall(world > 1 ? std::max(1, stepsPerChunk) : 0);
}

// ---- run bookkeeping ---------------------------------------------------------------------------------------------
// The C handle API counts optimizer steps inside the engine (trainWithRaysHit advances m_globalStep through its
// reference argument); what the facade adds is the target, the ray cursor, the pace estimate and the loss history.

void INerfTrainer::beginTraining(int totalSteps) {
    m_lossHistory.clear();
    m_raysSeen = 0.0;
    m_emaMsPerStep = 0.0;
    m_rayCursor = 0;
    m_globalStep = 0;
    m_targetSteps = totalSteps < 1 ? 1 : totalSteps;
}

// Blends a new ms-per-step measurement into the running pace: 30 % new, 70 % history (the weights of the reference's
// progress estimate, NerfTrainer.cu:208-211); the first measurement is taken as it is.
static double blendPace(double pace, double measuredMs) { return pace > 0.0 ? pace + 0.30 * (measuredMs - pace) : measuredMs; }

TrainStats INerfTrainer::trainSteps(int nSteps) {
    TrainStats report;
    if (m_nerf == nullptr || !m_source || m_total_rays == 0) return report;
    if (m_targetSteps == 0) beginTraining(20000);

    using Clock = std::chrono::steady_clock;
    const int stopAt = std::min(m_targetSteps, m_globalStep + std::max(nSteps, 1));
    const int before = m_globalStep;
    const Clock::time_point began = Clock::now();
    // only the first chunk of a tick pays for the MSE read-back (NerfTrainer.cu:173-178)
    float tickMse = -1.0f;
    for (bool measure = true; m_globalStep < stopAt; measure = false) {
        const float v = trainOneChunk(measure);
        if (v > 0.0f) tickMse = v;
    }
    throw_on_cuda(cudaDeviceSynchronize(), "trainSteps");
    const double elapsedMs = std::chrono::duration<double, std::milli>(Clock::now() - began).count();
    if (m_globalStep > before) m_emaMsPerStep = blendPace(m_emaMsPerStep, elapsedMs / (m_globalStep - before));
    if (tickMse > 0.0f) m_lossHistory.push_back(tickMse);

    report.loss = tickMse > 0.0f ? tickMse : (m_lossHistory.empty() ? 0.0f : m_lossHistory.back());
    report.psnr = report.loss > 0.0f ? -10.0f * log10f(fmaxf(report.loss, 1e-8f)) : 0.0f;
    report.step = m_globalStep;
    report.targetSteps = m_targetSteps;
    report.lr = currentLR();
    report.epochs = epochs();
    report.msPerStep = (float)m_emaMsPerStep;
    report.etaSeconds = (float)(m_emaMsPerStep * 1e-3 * std::max(m_targetSteps - m_globalStep, 0));
    return report;
}

void INerfTrainer::train(int maxSteps, int /*maxEpochs*/) {
    if (m_nerf == nullptr || !m_source || m_total_rays == 0) {
        std::cerr << "[INerfTrainer] train() called before a ray source was set." << std::endl;
        return;
    }
    beginTraining(maxSteps);
    // a hundred progress lines per run
    for (const int stride = std::max(maxSteps / 100, 1); !isTrainingDone();) {
        const TrainStats r = trainSteps(stride);
        std::printf("\r%d/%d steps | epoch %.2f | %.2f ms/step | ETA %.0f s | PSNR %.1f   ", r.step, r.targetSteps, r.epochs, r.msPerStep,
                    r.etaSeconds, r.psnr);
        std::fflush(stdout);
    }
    std::printf("\n");
}

// ---- scene footer ------------------------------------------------------------------------------------------------
// 36 bytes behind the .inerf payload: "SCN1", then centre xyz, up xyz, scale, horizontal field of view (radians), all
// fp32 - the record the reference appends and looks for at the end of the file (NerfTrainer.cu:266-300).
namespace {
struct SceneFooter {
    char tag[4];
    float centre[3], up[3], scale, fovX;
};
static_assert(sizeof(SceneFooter) == 36, "the scene footer is 36 bytes on disk");
const char kFooterTag[4] = {'S', 'C', 'N', '1'};

bool readFooter(const std::string& path, SceneFooter& f) {
    std::ifstream in(path, std::ios::binary);
    if (!in) return false;
    in.seekg(0, std::ios::end);
    const std::streamoff bytes = in.tellg();
    if (bytes < (std::streamoff)sizeof(SceneFooter)) return false;
    in.seekg(bytes - (std::streamoff)sizeof(SceneFooter));
    in.read(reinterpret_cast<char*>(&f), sizeof(SceneFooter));
    return bool(in) && std::equal(f.tag, f.tag + 4, kFooterTag);
}
}  // namespace

void INerfTrainer::save(const std::string& path) {
    if (m_nerf == nullptr) return;
    m_nerf->save(path);
    SceneFooter f;
    std::copy(kFooterTag, kFooterTag + 4, f.tag);
    f.centre[0] = m_sceneCenter.x; f.centre[1] = m_sceneCenter.y; f.centre[2] = m_sceneCenter.z;
    f.up[0] = m_sceneUp.x; f.up[1] = m_sceneUp.y; f.up[2] = m_sceneUp.z;
    f.scale = m_sceneScale;
    f.fovX = m_cameraAngleX;
    std::ofstream out(path, std::ios::binary | std::ios::app);
    if (out) out.write(reinterpret_cast<const char*>(&f), sizeof(SceneFooter));
}

void INerfTrainer::load(const std::string& path) {
    buildModel();
    m_nerf->load(path);
    m_masterConfig = m_nerf->options();
    SceneFooter f;
    if (!readFooter(path, f)) return;   // a bare .inerf file: keep the current scene frame
    m_sceneCenter = {f.centre[0], f.centre[1], f.centre[2]};
    m_sceneUp = {f.up[0], f.up[1], f.up[2]};
    m_sceneScale = f.scale;
    m_cameraAngleX = f.fovX;
}

// ---- orbit camera ------------------------------------------------------------------------------------------------
namespace {
struct V3 {
    float v[3];
    float operator[](int i) const { return v[i]; }
};
V3 cross(const V3& a, const V3& b) { return {{a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]}}; }
V3 unit(const V3& a) {
    const float len = sqrtf(a[0] * a[0] + a[1] * a[1] + a[2] * a[2]);
    return len > 0.0f ? V3{{a[0] / len, a[1] / len, a[2] / len}} : a;
}
V3 mix2(float s, const V3& a, float t, const V3& b) { return {{s * a[0] + t * b[0], s * a[1] + t * b[1], s * a[2] + t * b[2]}}; }
}  // namespace

// Camera on a sphere of `radius` around the scene centre, looking at it: azimuth turns in the plane perpendicular to the
// scene's up vector, elevation lifts towards it.  Row-major 3x4 with columns right, up, backward, eye - the matrix
// renderOrbit of the reference builds (NerfTrainer.cu:330-366).
void INerfTrainer::orbitCamera(float azimuthDeg, float elevationDeg, float radius, float c2w[12]) const {
    const V3 centre{{m_sceneCenter.x, m_sceneCenter.y, m_sceneCenter.z}};
    const V3 up = unit(V3{{m_sceneUp.x, m_sceneUp.y, m_sceneUp.z}});
    // two unit vectors spanning the horizontal plane; the helper axis avoids one parallel to up
    const V3 helper = fabsf(up[1]) < 0.9f ? V3{{0.f, 1.f, 0.f}} : V3{{1.f, 0.f, 0.f}};
    const V3 e0 = unit(cross(up, helper));
    const V3 e1 = cross(up, e0);
    const float az = azimuthDeg * (kPI / 180.0f), el = elevationDeg * (kPI / 180.0f);
    const V3 outward = mix2(cosf(el), mix2(cosf(az), e0, sinf(az), e1), sinf(el), up);
    const V3 eye = mix2(1.0f, centre, radius, outward);
    const V3 forward = unit(mix2(1.0f, centre, -1.0f, eye));
    const V3 right = unit(cross(forward, up));
    const V3 camUp = cross(right, forward);
    for (int row = 0; row < 3; row++) {
        c2w[4 * row + 0] = right[row];
        c2w[4 * row + 1] = camUp[row];
        c2w[4 * row + 2] = -forward[row];
        c2w[4 * row + 3] = eye[row];
    }
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
