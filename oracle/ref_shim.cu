// TEST INFRASTRUCTURE: C wrappers around the reference's own classes and kernels, compiled together with the
// reference sources (where they lie under the reference tree) into oracle/_ref/libref3dmaker.so by
// oracle/build_ref.py.  The parity tests load that library next to libnerf_b200.so and run both on the same
// device buffers; bench.py --impl reference times it.  Nothing here is part of the product.
//
// The reference's InstantNerf.cu textually includes otherKernels.cu, and most kernels have no launcher of their
// own, so this file includes InstantNerf.cu to reach them.  `private` is opened up only to let the tests inject
// parameters into, and read scratch buffers out of, the reference's InstantNerf.
#define private public
#include "InstantNerf.cu"
#undef private

#include <cstring>

extern "C" {

// ---- field: hash-grid network + colour network driven the way InstantNerf::trainWithRaysHit drives them, on
// explicit samples (modules/NeRF/InstantNerf.cu:506-571 without the ray-dependent loss) -----------------------
struct RefField {
    TinyMLPHashGrid* density;
    TinyMLP* color;
    int maxBatch;
    float* d_density_out;   // [n][16]
    half* d_color_in;       // [n][32]
    float* d_sigma;         // [n]
    float* d_color_out;     // [n][3]
    half* d_color_dx;       // [n][32]
    half* d_density_grad;   // [n][16]
    float* d_zero_dsigma;   // [n] zeros
    uint32_t* d_ray_idx;    // identity
};

void* ref_field_create(int numLevels, int tableSize, int lowestSize, float b, int densityHidden, int densityLayers, int colorHidden,
                       int colorLayers, int maxBatch) {
    RefField* f = new RefField();
    MLPGridOptions g;
    g.vectorDim = 4; g.hiddenDim = densityHidden; g.outputDim = 16; g.numLayers = densityLayers; g.activationType = ACT_RELU;
    g.tableSize = tableSize; g.numLevels = numLevels; g.b = b; g.lowestSize = lowestSize; g.featuresLevel = 2;
    f->density = new TinyMLPHashGrid(g, maxBatch, maxBatch);
    MLPOption c;
    c.inputDim = 32; c.hiddenDim = colorHidden; c.outputDim = 3; c.numLayers = colorLayers; c.activationType = ACT_RELU;
    c.outputActivation = OUT_ACT_SIGMOID;
    f->color = new TinyMLP(c, maxBatch, maxBatch);
    f->maxBatch = maxBatch;
    size_t n = (size_t)maxBatch;
    cudaMalloc(&f->d_density_out, n * 16 * sizeof(float));
    cudaMalloc(&f->d_color_in, n * 32 * sizeof(half));
    cudaMalloc(&f->d_sigma, n * sizeof(float));
    cudaMalloc(&f->d_color_out, n * 3 * sizeof(float));
    cudaMalloc(&f->d_color_dx, n * 32 * sizeof(half));
    cudaMalloc(&f->d_density_grad, n * 16 * sizeof(half));
    cudaMalloc(&f->d_zero_dsigma, n * sizeof(float));
    cudaMemset(f->d_zero_dsigma, 0, n * sizeof(float));
    cudaMalloc(&f->d_ray_idx, n * sizeof(uint32_t));
    std::vector<uint32_t> idx(n);
    for (size_t i = 0; i < n; i++) idx[i] = (uint32_t)i;
    cudaMemcpy(f->d_ray_idx, idx.data(), n * sizeof(uint32_t), cudaMemcpyHostToDevice);
    return f;
}

void ref_field_destroy(void* h) {
    RefField* f = (RefField*)h;
    if (!f) return;
    delete f->density; delete f->color;
    cudaFree(f->d_density_out); cudaFree(f->d_color_in); cudaFree(f->d_sigma); cudaFree(f->d_color_out); cudaFree(f->d_color_dx);
    cudaFree(f->d_density_grad); cudaFree(f->d_zero_dsigma); cudaFree(f->d_ray_idx);
    delete f;
}

void ref_field_load(void* h, const float* hash, const float* dW, const float* db, const float* cW, const float* cb) {
    RefField* f = (RefField*)h;
    if (hash) f->density->loadHashgrid(hash);
    if (dW && db) f->density->loadWeights(dW, db);
    if (cW && cb) f->color->loadWeights(cW, cb);
}

void ref_field_save(void* h, float* hash, float* dW, float* db, float* cW, float* cb) {
    RefField* f = (RefField*)h;
    cudaDeviceSynchronize();
    if (hash) f->density->saveHashgrid(hash);
    if (dW && db) f->density->saveWeights(dW, db);
    if (cW && cb) f->color->saveWeights(cW, cb);
}

// zero_grad + forward + loss + both backward passes, no optimizer: leaves the gradients in place for comparison.
void ref_field_forward_backward(void* h, const float* d_pos4, const float* d_dirs3, const half* d_target_h3, int n, float densityBias,
                                float lossScale, cudaStream_t stream);
float* ref_field_hash_grads(void* h) { return ((RefField*)h)->density->d_hashtable_grads; }
// gradient of one layer: net 0 = density, 1 = colour; what 0 = weights, 1 = biases
float* ref_field_layer_grads(void* h, int net, int layer, int what) {
    RefField* f = (RefField*)h;
    float** arr = net == 0 ? (what == 0 ? f->density->d_w_grad : f->density->d_b_grad) : (what == 0 ? f->color->d_w_grad : f->color->d_b_grad);
    float* p = nullptr;
    cudaMemcpy(&p, arr + layer, sizeof(float*), cudaMemcpyDeviceToHost);
    return p;
}
// Saved activation `index` of the grid network after a forward: 0 = the encoded features [n][32] fp16
// (networkFusionHashtable.cu:553-569), 1.. = hidden layers.
void* ref_field_grid_activation(void* h, int index) {
    half* p = nullptr;
    cudaMemcpy(&p, ((RefField*)h)->density->d_activations + index, sizeof(half*), cudaMemcpyDeviceToHost);
    return p;
}
float* ref_field_density_out(void* h) { return ((RefField*)h)->d_density_out; }
float* ref_field_color_out(void* h) { return ((RefField*)h)->d_color_out; }
void* ref_field_color_in(void* h) { return ((RefField*)h)->d_color_in; }

// Forward of both networks on n samples (activation-saving variants), as the training loop runs them.
void ref_field_forward(void* h, const float* d_pos4, const float* d_dirs3, int n, float densityBias, cudaStream_t stream) {
    RefField* f = (RefField*)h;
    f->density->forward(d_pos4, f->d_density_out, n, stream);
    compute_SH_gather<<<(n + 255) / 256, 256, 0, stream>>>((const float3*)d_dirs3, f->d_ray_idx, 0, n, densityBias, f->d_density_out, f->d_color_in,
                                                           f->d_sigma);
    f->color->forward(f->d_color_in, f->d_color_out, n, stream);
}

// One whole optimizer step on explicit samples with the MSE loss of TinyMLP::calculate_loss_and_grad:
// zero_grad, forward, loss, colour backward (dX), density gradient, grid backward (+ scatter), both Adam steps.
// d_target_h3: fp16 [n][3].  Returns nothing; read parameters back with ref_field_save.
void ref_field_train_step(void* h, const float* d_pos4, const float* d_dirs3, const half* d_target_h3, int n, float densityBias, float lossScale,
                          float lr, float beta1, float beta2, float eps, cudaStream_t stream) {
    RefField* f = (RefField*)h;
    f->density->zero_grad(stream);
    f->color->zero_grad(stream);
    ref_field_forward(h, d_pos4, d_dirs3, n, densityBias, stream);
    f->color->calculate_loss_and_grad(d_target_h3, n, lossScale, false, stream);
    f->color->backward(f->d_color_dx, n, stream);
    compute_density_grad<<<(n + 255) / 256, 256, 0, stream>>>(n, f->d_zero_dsigma, f->d_color_dx, f->d_density_grad);
    f->density->backward(f->d_density_grad, n, stream);
    f->color->step(lr, beta1, beta2, eps, lossScale, stream);
    f->density->step(lr, beta1, beta2, eps, lossScale, stream);
}

// The optimizer alone, on whatever the gradient buffers hold (tests write a known gradient there first):
// TinyMLP::step and TinyMLPHashGrid::step (TinyMLP.cu:379-404, TinyMLPHashGrid.cu:379-392).
void ref_field_step(void* h, float lossScale, float lr, float beta1, float beta2, float eps, cudaStream_t stream) {
    RefField* f = (RefField*)h;
    f->color->step(lr, beta1, beta2, eps, lossScale, stream);
    f->density->step(lr, beta1, beta2, eps, lossScale, stream);
}

void ref_field_forward_backward(void* h, const float* d_pos4, const float* d_dirs3, const half* d_target_h3, int n, float densityBias,
                                float lossScale, cudaStream_t stream) {
    RefField* f = (RefField*)h;
    f->density->zero_grad(stream);
    f->color->zero_grad(stream);
    ref_field_forward(h, d_pos4, d_dirs3, n, densityBias, stream);
    f->color->calculate_loss_and_grad(d_target_h3, n, lossScale, false, stream);
    f->color->backward(f->d_color_dx, n, stream);
    compute_density_grad<<<(n + 255) / 256, 256, 0, stream>>>(n, f->d_zero_dsigma, f->d_color_dx, f->d_density_grad);
    f->density->backward(f->d_density_grad, n, stream);
}

// ---- scene engine -------------------------------------------------------------------------------------
void* ref_nerf_create(const void* options_bytes, int memory_mode) {
    NerfOptions o;
    std::memcpy(&o, options_bytes, sizeof(NerfOptions));
    InstantNerf* n = new InstantNerf();
    n->init(o, memory_mode == 1 ? INFERENCE : TRAINING);
    return n;
}
int ref_nerf_options_size() { return (int)sizeof(NerfOptions); }
void ref_nerf_destroy(void* h) { delete (InstantNerf*)h; }

void ref_nerf_load_params(void* h, const float* hash, const float* dW, const float* db, const float* cW, const float* cb) {
    InstantNerf* n = (InstantNerf*)h;
    if (hash) n->m_densityMLP->loadHashgrid(hash);
    if (dW && db) n->m_densityMLP->loadWeights(dW, db);
    if (cW && cb) n->m_colorMLP->loadWeights(cW, cb);
}
void ref_nerf_save_params(void* h, float* hash, float* dW, float* db, float* cW, float* cb) {
    InstantNerf* n = (InstantNerf*)h;
    cudaDeviceSynchronize();
    if (hash) n->m_densityMLP->saveHashgrid(hash);
    if (dW && db) n->m_densityMLP->saveWeights(dW, db);
    if (cW && cb) n->m_colorMLP->saveWeights(cW, cb);
}
void ref_nerf_rebuild_occupancy(void* h) {
    InstantNerf* n = (InstantNerf*)h;
    n->earlyOccupancyGridUpdate(0);
    cudaDeviceSynchronize();
}
void ref_nerf_set_train_steps(void* h, int steps) { ((InstantNerf*)h)->m_trainSteps = steps; }
uint8_t* ref_nerf_bitfield(void* h, long* bytes) {
    InstantNerf* n = (InstantNerf*)h;
    if (bytes) *bytes = (long)n->d_occupancyGrid.size();
    return n->d_occupancyGrid.data();
}
float* ref_nerf_master_grid(void* h) { return ((InstantNerf*)h)->d_masterOccupancyGrid.data(); }

// d_depth / d_sigma: per-ray depth priors.  The reference offsets these pointers by the rays already consumed
// before testing them for null (InstantNerf.cu:383-384), so callers must pass real buffers (depth -1 = prior off).
int ref_nerf_train(void* h, const float* d_rays_o, const float* d_rays_d, const float* d_depth, const float* d_sigma, const float* d_rgb_true,
                   unsigned numRays, float* d_rgb_out, unsigned* hitCounts, cudaStream_t stream) {
    InstantNerf* n = (InstantNerf*)h;
    int steps = 0;
    n->trainWithRaysHit((const float3*)d_rays_o, (const float3*)d_rays_d, d_depth, d_sigma, d_rgb_true, numRays, steps, hitCounts, d_rgb_out, stream);
    return steps;
}
void ref_nerf_render(void* h, const float* d_rays_o, const float* d_rays_d, unsigned numRays, float* d_rgb_out, cudaStream_t stream) {
    ((InstantNerf*)h)->renderImageHit((const float3*)d_rays_o, (const float3*)d_rays_d, numRays, d_rgb_out, stream);
}
// InstantNerf::save / load, the .inerf file (InstantNerf.cu:1206-1352).  0 on success, 1 when the reference threw.
int ref_nerf_save(void* h, const char* path) {
    try { ((InstantNerf*)h)->save(path); } catch (const std::exception& e) { std::fprintf(stderr, "ref_nerf_save: %s\n", e.what()); return 1; }
    return 0;
}
int ref_nerf_load(void* h, const char* path) {
    try { ((InstantNerf*)h)->load(path); } catch (const std::exception& e) { std::fprintf(stderr, "ref_nerf_load: %s\n", e.what()); return 1; }
    return 0;
}
void ref_nerf_set_learning_rate(void* h, float lr) { ((InstantNerf*)h)->setLearningRate(lr); }
void ref_nerf_set_memory_mode(void* h, int mode) { ((InstantNerf*)h)->setMemoryMode(mode == 1 ? INFERENCE : TRAINING); }

// scratch buffers of the last step, by name index (parity tests)
void* ref_nerf_buffer(void* h, int which) {
    RenderingBuffers& b = ((InstantNerf*)h)->m_render_buffers;
    switch (which) {
        case 0: return b.d_num_steps.data();
        case 1: return b.d_ray_offsets.data();
        case 2: return b.d_ray_indices.data();
        case 3: return b.d_t_sorted.data();
        case 4: return b.d_mlp_positions.data();
        case 5: return b.d_density_out.data();
        case 6: return b.d_density_sigma.data();
        case 7: return b.d_color_output.data();
        case 8: return b.d_render_rgb_chunk.data();
        case 9: return b.d_phi_chunk.data();
        case 10: return b.d_dw_out.data();
        case 11: return b.d_weight_sum.data();
        case 12: return b.d_tmpsigma.data();
        case 13: return b.d_custom_color_grad.data();
        case 14: return b.d_custom_density_grad.data();
        case 15: return b.d_nears_chunk.data();
        case 16: return b.d_fars_chunk.data();
        case 17: return b.d_rays_d_inv_chunk.data();
        default: return nullptr;
    }
}

// ---- single kernels ------------------------------------------------------------------------------------
void ref_ray_aabb(unsigned numRays, const float* o, const float* d, const float* aabbMin3, const float* aabbMax3, int numCascades, float* dInv,
                  float* nears, float* fars, cudaStream_t stream) {
    compute_ray_aabb_inv_kernel<<<(numRays + 255) / 256, 256, 0, stream>>>(numRays, (const float3*)o, (const float3*)d,
                                                                         make_float3(aabbMin3[0], aabbMin3[1], aabbMin3[2]),
                                                                         make_float3(aabbMax3[0], aabbMax3[1], aabbMax3[2]), numCascades, (float3*)dInv,
                                                                         nears, fars);
}

// processRaysHitLinear (modules/NeRF/processRays.cu:931-1040): returns the rays that fit, *totalHits their samples.
int ref_process_rays_hit_linear(unsigned numRays, const float* o, const float* d, const float* dInv, const float* nears, const float* fars,
                                const uint8_t* grid, const unsigned* res3, const float* aabbMin3, const float* aabbMax3, int numCascades,
                                int mipLevels, int spv, int batchSize, unsigned* totalHits, unsigned* d_active, unsigned* d_num_steps,
                                unsigned* d_ray_offsets, float* d_pos4, unsigned* d_ray_idx, float* d_t, unsigned* d_block_sums, cudaStream_t stream) {
    return processRaysHitLinear(numRays, (const float3*)o, (const float3*)d, (const float3*)dInv, nears, fars, grid,
                                make_uint3(res3[0], res3[1], res3[2]), make_float3(aabbMin3[0], aabbMin3[1], aabbMin3[2]),
                                make_float3(aabbMax3[0], aabbMax3[1], aabbMax3[2]), numCascades, mipLevels, spv, batchSize, totalHits, d_active,
                                d_num_steps, d_ray_offsets, d_pos4, d_ray_idx, d_t, d_block_sums, stream);
}

void ref_volume_rendering(unsigned numRays, const unsigned* offsets, const unsigned* steps, const float* t, const float* sigma, const float* rgb3,
                          const float* rgbTrue, float* outRgb, float* outDepth, float* phi, float* dw, float* wsum, float lambdaDist,
                          float lambdaDepth, const float* bg3, unsigned base, unsigned raysDone, cudaStream_t stream) {
    launchVolumeRendering(numRays, offsets, steps, t, sigma, nullptr, nullptr, rgb3, rgbTrue, outRgb, outDepth, phi, dw, wsum, lambdaDist, lambdaDepth,
                          make_float3(bg3[0], bg3[1], bg3[2]), base, raysDone, stream);
}

// The same launcher with per-ray depth priors (depth < 0 = no prior for that ray), compositing.cu:108-111,157-159,183-189.
void ref_volume_rendering_priors(unsigned numRays, const unsigned* offsets, const unsigned* steps, const float* t, const float* sigma,
                                 const float* depthPrior, const float* sigmaPrior, const float* rgb3, const float* rgbTrue, float* outRgb,
                                 float* outDepth, float* phi, float* dw, float* wsum, float lambdaDist, float lambdaDepth, const float* bg3,
                                 cudaStream_t stream) {
    launchVolumeRendering(numRays, offsets, steps, t, sigma, depthPrior, sigmaPrior, rgb3, rgbTrue, outRgb, outDepth, phi, dw, wsum, lambdaDist,
                          lambdaDepth, make_float3(bg3[0], bg3[1], bg3[2]), 0, 0, stream);
}

void ref_color_grad(unsigned numRays, const unsigned* steps, const unsigned* offsets, const float* t, const float* densityOut16, const float* colorOut3,
                    const float* phi, const float* finalRgb, const float* dw, const float* wsum, half* colorGrad3, float* dsigma, float lossScale,
                    float densityBias, unsigned totalRays, cudaStream_t stream) {
    compute_color_grad<<<(numRays + 255) / 256, 256, 0, stream>>>(numRays, 0, steps, offsets, t, densityOut16, colorOut3, phi, finalRgb, dw, wsum,
                                                                  colorGrad3, dsigma, lossScale, densityBias, totalRays);
}

void ref_sample_aabb(float* samples4, const float* aabbMin3, const float* aabbMax3, const unsigned* res3, int N, int totalCells, int cellOffset,
                     unsigned long long seed, cudaStream_t stream) {
    sampleAABB<<<(N + 255) / 256, 256, 0, stream>>>(samples4, make_float3(aabbMin3[0], aabbMin3[1], aabbMin3[2]),
                                                    make_float3(aabbMax3[0], aabbMax3[1], aabbMax3[2]), make_uint3(res3[0], res3[1], res3[2]), N,
                                                    totalCells, cellOffset, seed);
}

}  // extern "C"
