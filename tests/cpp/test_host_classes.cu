// Contract test of the C++ host classes (GPU).  Same style as the reference's own checks
// (modules/TinyMLP/tests_kernels/testModes.cu: EXPECT_THROW macros, [SUCCESS]/[FAILED] lines), but the process
// exit code is the number of failures so a test runner can rely on it.
#include <cmath>
#include <cstdio>
#include <utility>
#include <vector>

#include "../../3dmaker_b200/host/NerfTrainer.h"

static int g_fail = 0;
#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) { std::printf("[FAILED] %s:%d %s\n", __FILE__, __LINE__, #cond); g_fail++; } \
    } while (0)
#define EXPECT_THROW(stmt)                                                 \
    do {                                                                   \
        bool thrown_ = false;                                              \
        try { stmt; } catch (const std::exception&) { thrown_ = true; }    \
        if (!thrown_) { std::printf("[FAILED] %s:%d no exception from %s\n", __FILE__, __LINE__, #stmt); g_fail++; } \
    } while (0)
#define EXPECT_NO_THROW(stmt)                                              \
    do {                                                                   \
        try { stmt; } catch (const std::exception& e) { std::printf("[FAILED] %s:%d %s threw %s\n", __FILE__, __LINE__, #stmt, e.what()); g_fail++; } \
    } while (0)

static void test_tinymlp_modes() {
    MLPOption opt{32, 64, 3, 3, ACT_RELU, OUT_ACT_SIGMOID};
    const int B = 1000;
    TinyMLP mlp(opt, B, 0, 42, /*isTraining=*/false);
    half *in, *tgt, *dx; float* out;
    cudaMalloc(&in, B * 32 * sizeof(half)); cudaMalloc(&tgt, B * 3 * sizeof(half)); cudaMalloc(&dx, B * 32 * sizeof(half));
    cudaMalloc(&out, B * 3 * sizeof(float));
    cudaMemset(in, 0, B * 32 * sizeof(half)); cudaMemset(tgt, 0, B * 3 * sizeof(half));
    EXPECT_THROW(mlp.zero_grad());
    EXPECT_THROW(mlp.forward(in, out, B));
    EXPECT_THROW(mlp.calculate_loss_and_grad(tgt, B));
    EXPECT_THROW(mlp.backward(B));
    EXPECT_THROW(mlp.backward(dx, B));
    EXPECT_THROW(mlp.step());
    EXPECT_NO_THROW(mlp.inference(in, out, B));
    mlp.switchToTrainingMode();
    EXPECT_NO_THROW(mlp.zero_grad());
    EXPECT_NO_THROW(mlp.forward(in, out, B));
    EXPECT_THROW(mlp.forward(in, out, B + 1));  // beyond maxBatchSize
    float loss = -1.f;
    EXPECT_NO_THROW(loss = mlp.calculate_loss_and_grad(tgt, B, 128.0f, true));
    CHECK(loss > 0.0f && loss < 1.0f);          // sigmoid outputs against zero targets
    EXPECT_NO_THROW(mlp.backward(dx, B));
    EXPECT_NO_THROW(mlp.step(1e-2f, 0.9f, 0.99f, 1e-15f, 128.0f));
    // the step lowers the loss on the same batch
    mlp.zero_grad(); mlp.forward(in, out, B);
    float loss2 = mlp.calculate_loss_and_grad(tgt, B, 128.0f, true);
    CHECK(loss2 < loss);
    // weights survive a file round trip
    std::vector<float> w(TinyMLP::paramCount(opt)), b(w.size()), w2(w.size()), b2(w.size());
    mlp.saveWeights(w.data(), b.data());
    mlp.saveWeights("/tmp/nb_tinymlp.bin");
    TinyMLP other(opt, B, 0, 7, false);
    other.loadWeights("/tmp/nb_tinymlp.bin");
    other.saveWeights(w2.data(), b2.data());
    bool same = true;
    for (int64_t i = 0; i < mlp.weightCount(); i++) same = same && (w[i] == w2[i]);
    CHECK(same);
    MLPOption bad = opt; bad.hiddenDim = 32; bad.numLayers = 2;
    TinyMLP mismatch(bad, B, 0, 7, false);
    EXPECT_THROW(mismatch.loadWeights("/tmp/nb_tinymlp.bin"));
    EXPECT_THROW(mismatch.loadWeights("/nonexistent/file.bin"));
    mlp.switchToInferenceMode();
    EXPECT_THROW(mlp.step());
    cudaFree(in); cudaFree(tgt); cudaFree(dx); cudaFree(out);
    std::printf("[SUCCESS?] TinyMLP mode contract, %d failures so far\n", g_fail);
}

static void test_hashgrid_modes() {
    MLPGridOptions g{3, 64, 16, 2, ACT_RELU, 1 << 14, 16, 1.3819f, 16, 2};
    const int B = 777;
    MLPGridOptions bad = g; bad.vectorDim = 5;
    EXPECT_THROW(TinyMLPHashGrid(bad, B));
    bad = g; bad.featuresLevel = 4;
    EXPECT_THROW(TinyMLPHashGrid(bad, B));
    TinyMLPHashGrid net(g, B, 0, 42, false);
    float *pos, *out; half* grad;
    cudaMalloc(&pos, B * 3 * sizeof(float)); cudaMalloc(&out, B * 16 * sizeof(float)); cudaMalloc(&grad, B * 16 * sizeof(half));
    std::vector<float> hp(B * 3);
    for (size_t i = 0; i < hp.size(); i++) hp[i] = (float)((i * 2654435761u) % 1000) / 1000.0f;
    cudaMemcpy(pos, hp.data(), hp.size() * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemset(grad, 0, B * 16 * sizeof(half));
    EXPECT_THROW(net.zero_grad());
    EXPECT_THROW(net.forward(pos, out, B));
    EXPECT_THROW(net.backward(grad, B));
    EXPECT_THROW(net.step());
    EXPECT_NO_THROW(net.inference(pos, out, B));
    std::vector<float> o1(B * 16), o2(B * 16);
    cudaMemcpy(o1.data(), out, o1.size() * sizeof(float), cudaMemcpyDeviceToHost);
    net.switchToTrainingMode();
    EXPECT_NO_THROW(net.zero_grad());
    EXPECT_NO_THROW(net.forward(pos, out, B));
    cudaMemcpy(o2.data(), out, o2.size() * sizeof(float), cudaMemcpyDeviceToHost);
    bool same = true;
    for (size_t i = 0; i < o1.size(); i++) same = same && (o1[i] == o2[i]);
    CHECK(same);                                 // training and inference forward agree bit for bit
    EXPECT_NO_THROW(net.backward(grad, B));
    EXPECT_NO_THROW(net.step());
    EXPECT_THROW(net.forward(pos, out, B + 1));
    CHECK(net.getSplitScatter());
    cudaFree(pos); cudaFree(out); cudaFree(grad);
    std::printf("[SUCCESS?] TinyMLPHashGrid mode contract, %d failures so far\n", g_fail);
}

// A facade run on rays of one fixed camera whose target colour is constant, in the manner of the reference's
// modules/NeRF/test_kernels/test_training.cu.
static void test_trainer_facade() {
    INerfTrainer trainer;
    NerfConfig cfg;
    cfg.batchSize = 1 << 16; cfg.renderBatchSize = 1 << 16; cfg.lambdaDist = 0.0f;
    trainer.init(cfg);
    EXPECT_THROW(trainer.loadDataset("/nonexistent"));
    NerfOptions& o = trainer.options();
    o.gridResolution = make_uint3(32, 32, 32); o.levelsMipmap = 3; o.hashTableSize = 1 << 14;
    o.aabbMin = make_float3(-0.5f, -0.5f, -0.5f); o.aabbMax = make_float3(0.5f, 0.5f, 0.5f);
    const int W = 64, H = 64;
    float c2w[12];
    trainer.orbitCamera(30.0f, 10.0f, 1.5f, c2w);
    CHECK(std::fabs(std::sqrt(c2w[3] * c2w[3] + c2w[7] * c2w[7] + c2w[11] * c2w[11]) - 1.5f) < 1e-5f);
    const float focal = 0.5f * W / std::tan(0.5f * 50.0f * 3.14159265f / 180.0f);
    std::vector<float> target((size_t)W * H * 3);
    for (size_t i = 0; i < target.size(); i += 3) { target[i] = 0.8f; target[i + 1] = 0.3f; target[i + 2] = 0.1f; }
    auto source = [&](uint32_t cursor, uint32_t count, uint32_t, float3, float3* d_o, float3* d_d, float* d_rgb, cudaStream_t s) {
        nb_generate_rays(W, H, focal, c2w, cursor, count, (float*)d_o, (float*)d_d, s);
        cudaMemcpyAsync(d_rgb, target.data() + (size_t)cursor * 3, (size_t)count * 3 * sizeof(float), cudaMemcpyHostToDevice, s);
    };
    EXPECT_NO_THROW(trainer.setRaySource(source, W * H, Vec3{0, 1, 0}, /*randomBackground=*/false));
    trainer.beginTraining(60);
    TrainStats first = trainer.trainSteps(5);
    TrainStats last = first;
    while (!trainer.isTrainingDone()) last = trainer.trainSteps(5);
    CHECK(first.loss > 0.0f && last.loss < 0.5f * first.loss);
    CHECK(last.step == 60 && last.lr < cfg.maxLR && last.lr >= cfg.minLR - 1e-6f);
    Image img = trainer.renderOrbit(30.0f, 10.0f, 1.5f, 50.0f, W, H);
    CHECK(img.width == W && img.height == H && img.rgb.size() == (size_t)W * H * 3);
    double mse = 0;
    for (size_t i = 0; i < img.rgb.size(); i++) mse += (img.rgb[i] - target[i]) * (img.rgb[i] - target[i]);
    mse /= img.rgb.size();
    std::printf("facade: loss %.5f -> %.5f, rendered MSE %.5f\n", first.loss, last.loss, mse);
    CHECK(mse < 0.6 * first.loss);             // the rendered frame reflects the training progress
    EXPECT_NO_THROW(trainer.save("/tmp/nb_trainer.inerf"));
    INerfTrainer again;
    again.init(cfg);
    EXPECT_NO_THROW(again.load("/tmp/nb_trainer.inerf"));
    Image img2 = again.renderOrbit(30.0f, 10.0f, 1.5f, 50.0f, W, H);
    bool same = img2.rgb.size() == img.rgb.size();
    for (size_t i = 0; same && i < img.rgb.size(); i++) same = (img.rgb[i] == img2.rgb[i]);
    CHECK(same);
    std::printf("[SUCCESS?] INerfTrainer facade, %d failures so far\n", g_fail);
}

// An image set in device memory as the source of training rays, hold-out validation and train-view rendering.
static void test_trainer_image_set() {
    INerfTrainer trainer;
    NerfConfig cfg;
    cfg.batchSize = 1 << 16; cfg.renderBatchSize = 1 << 16; cfg.lambdaDist = 0.0f; cfg.shouldValidate = true;
    trainer.init(cfg);
    CHECK(trainer.validate() == 0.0f);                       // no image set yet
    NerfOptions& o = trainer.options();
    o.gridResolution = make_uint3(32, 32, 32); o.levelsMipmap = 3; o.hashTableSize = 1 << 14;
    o.aabbMin = make_float3(-0.5f, -0.5f, -0.5f); o.aabbMax = make_float3(0.5f, 0.5f, 0.5f);
    const int N = 16, W = 48, H = 48;
    std::vector<uint8_t> rgba((size_t)N * W * H * 4);
    for (size_t i = 0; i < rgba.size(); i += 4) { rgba[i] = 204; rgba[i + 1] = 77; rgba[i + 2] = 26; rgba[i + 3] = 255; }
    std::vector<float> poses((size_t)N * 16, 0.0f);
    for (int i = 0; i < N; i++) {
        float c2w[12];
        trainer.orbitCamera(22.5f * i, 15.0f, 1.5f, c2w);
        for (int k = 0; k < 12; k++) poses[(size_t)i * 16 + k] = c2w[k];
        poses[(size_t)i * 16 + 15] = 1.0f;
    }
    uint8_t* d_rgba = nullptr; float* d_poses = nullptr;
    cudaMalloc(&d_rgba, rgba.size()); cudaMalloc(&d_poses, poses.size() * sizeof(float));
    cudaMemcpy(d_rgba, rgba.data(), rgba.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_poses, poses.data(), poses.size() * sizeof(float), cudaMemcpyHostToDevice);
    nb_image_set set{};
    set.d_images_rgba = d_rgba; set.d_transforms = d_poses; set.num_images = N; set.width = W; set.height = H;
    set.focal = 0.5f * W / std::tan(0.5f * 50.0f * 3.14159265f / 180.0f);
    nb_image_set empty{};
    EXPECT_THROW(trainer.setImageSet(empty));
    EXPECT_NO_THROW(trainer.setImageSet(set, Vec3{0, 1, 0}, /*randomBackground=*/false));
    const float before = trainer.validate();
    trainer.beginTraining(80);
    while (!trainer.isTrainingDone()) trainer.trainSteps(10);
    const float after = trainer.validate();
    std::printf("image set: hold-out PSNR %.2f dB -> %.2f dB\n", before, after);
    CHECK(after > before + 3.0f && after > 9.0f);   // 80 steps of a 2^14-entry model: enough to see the hold-out error fall
    Image view = trainer.renderTrainView(3);
    CHECK(view.width == W && view.height == H && view.rgb.size() == (size_t)W * H * 3);
    Image small = trainer.renderTrainView(3, 24, 24);
    CHECK(small.width == 24 && small.rgb.size() == (size_t)24 * 24 * 3);
    CHECK(trainer.renderTrainView(N).rgb.empty());
    cudaFree(d_rgba); cudaFree(d_poses);
    std::printf("[SUCCESS?] INerfTrainer image set, %d failures so far\n", g_fail);
}

// The facade's data-parallel entry seen from one rank of two: the ray source is asked for this rank's half of every
// chunk, the exchange callback runs exactly stepsPerChunk times per chunk on the whole gradient arena, and the cursor
// advances by the global chunk.
static void test_trainer_data_parallel_contract() {
    INerfTrainer trainer;
    NerfConfig cfg;
    cfg.batchSize = 1 << 14; cfg.renderBatchSize = 1 << 14; cfg.lambdaDist = 0.0f;
    trainer.init(cfg);
    NerfOptions& o = trainer.options();
    o.gridResolution = make_uint3(32, 32, 32); o.levelsMipmap = 3; o.hashTableSize = 1 << 14;
    o.aabbMin = make_float3(-0.5f, -0.5f, -0.5f); o.aabbMax = make_float3(0.5f, 0.5f, 0.5f);
    const int W = 128, H = 128;                      // 16384 rays = four chunks of batchSize / 4
    float c2w[12];
    trainer.orbitCamera(30.0f, 10.0f, 1.5f, c2w);
    const float focal = 0.5f * W / std::tan(0.5f * 50.0f * 3.14159265f / 180.0f);
    std::vector<std::pair<uint32_t, uint32_t>> asked;
    auto source = [&](uint32_t cursor, uint32_t count, uint32_t, float3, float3* d_o, float3* d_d, float* d_rgb, cudaStream_t s) {
        asked.push_back({cursor, count});
        nb_generate_rays(W, H, focal, c2w, cursor, count, (float*)d_o, (float*)d_d, s);
        cudaMemsetAsync(d_rgb, 0, (size_t)count * 3 * sizeof(float), s);
    };
    int exchanges = 0;
    int64_t seenCount = 0;
    EXPECT_THROW(trainer.setDataParallel([](float*, int64_t, cudaStream_t) {}, 2, 2));
    EXPECT_NO_THROW(trainer.setDataParallel([&](float* g, int64_t count, cudaStream_t) { exchanges += (g != nullptr); seenCount = count; },
                                            /*rank=*/1, /*world=*/2, /*stepsPerChunk=*/3));
    EXPECT_NO_THROW(trainer.setRaySource(source, W * H, Vec3{0, 1, 0}, false));
    trainer.beginTraining(6);
    TrainStats st = trainer.trainSteps(6);
    const uint32_t chunk = (uint32_t)o.rayChunkSize;
    CHECK(st.step == 6 && exchanges == 6);
    CHECK(seenCount == trainer.engine()->arena().total);
    CHECK(asked.size() == 2 && asked[0].first == chunk / 2 && asked[0].second == chunk / 2 && asked[1].first == chunk + chunk / 2);
    std::printf("[SUCCESS?] INerfTrainer data-parallel contract, %d failures so far\n", g_fail);
}

int main() {
    test_tinymlp_modes();
    test_hashgrid_modes();
    test_trainer_facade();
    test_trainer_image_set();
    test_trainer_data_parallel_contract();
    std::printf(g_fail == 0 ? "[SUCCESS] all host-class checks passed\n" : "[FAILED] %d checks failed\n", g_fail);
    return g_fail;
}
