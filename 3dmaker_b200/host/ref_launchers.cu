// The reference's own extern "C" launcher names, as thin adapters over the arena ABI of include/nerf_b200.h.
//
// The reference's classes and test programs reach their kernels through these functions (modules/TinyMLP/TinyMLP.h:
// 158-263, TinyMLPHashGrid.h:172-256, modules/NeRF/InstantNerf.h:385-568).  A program that calls them directly - not
// through TinyMLP / TinyMLPHashGrid / InstantNerf, which this library replaces as whole classes - links against
// libnerf_b200.so unchanged.  What the adapters have to bridge:
//   * per-layer weights, biases and gradients arrive as DEVICE arrays of device pointers.  The pointers are read back on
//     every call (a blocking copy of a few words: an address is no identity, arrays are freed and others allocated in
//     their place) and the layers are copied into one flat scratch block per call, which is what the arena kernels take;
//   * void returns: a failure is printed to stderr (the reference's launchers print or silently return).
// Provided: the inference launchers of both networks, the loss, the three optimizers and zero-grad, the ray march
// (count + scan + cutoff + emit with the reference's three read-backs folded into one) and volume rendering.  The
// activation-saving forward and the backward launchers hand per-layer ACTIVATION arrays around; they are not provided:
// a caller at that level uses nb_mlp_forward / nb_mlp_backward / nb_grid_mlp_forward with flat buffers instead.
#include <algorithm>
#include <cstdio>
#include <map>
#include <mutex>
#include <vector>

#include "TinyMLPHashGrid.h"

namespace {

void report(int rc, const char* what) {
    if (rc != NB_OK) std::fprintf(stderr, "[libnerf_b200] %s: %s\n", what, nb_last_error());
}

// Host copy of a device array of `count` device pointers (null entries when the copy fails).
template <class T>
std::vector<T*> pointer_array(T** d_array, int count) {
    std::vector<T*> host((size_t)std::max(count, 0), nullptr);
    if (d_array == nullptr || count <= 0) return host;
    if (cudaMemcpy(host.data(), d_array, sizeof(T*) * (size_t)count, cudaMemcpyDeviceToHost) != cudaSuccess) host.assign((size_t)count, nullptr);
    return host;
}

// Flat scratch block per (device, purpose); grows, never shrinks.
struct Scratch {
    nb::DeviceMem mem;
    void* get(size_t bytes) {
        if (mem.bytes() < bytes) mem.allocate(bytes);
        return mem.as<void>();
    }
};
Scratch& scratch(int which) {
    static Scratch s[8];
    return s[which];
}

nb_mlp_desc desc_of(const MLPOption& o) {
    nb_mlp_desc d;
    d.input_dim = o.inputDim; d.hidden_dim = o.hiddenDim; d.output_dim = o.outputDim; d.num_layers = o.numLayers;
    d.output_activation = o.outputActivation;
    return d;
}

void layer_dims(const nb_mlp_desc& d, int l, int& in, int& out) {
    in = l == 0 ? d.input_dim : d.hidden_dim;
    out = l == d.num_layers - 1 ? d.output_dim : d.hidden_dim;
}

// Copies the layers' weights (fp16) and biases (fp32) back to back into scratch; returns false on a failed copy.
bool gather_network(const nb_mlp_desc& d, half** d_weights_array, float** d_biases_array, half*& flat_w, float*& flat_b, cudaStream_t st) {
    const auto W = pointer_array(d_weights_array, d.num_layers);
    const auto B = pointer_array(d_biases_array, d.num_layers);
    size_t nw = 0, nb_ = 0;
    for (int l = 0; l < d.num_layers; l++) { int i, o; layer_dims(d, l, i, o); nw += (size_t)i * o; nb_ += (size_t)o; }
    flat_w = (half*)scratch(0).get(nw * sizeof(half) + 64);
    flat_b = (float*)scratch(1).get(nb_ * sizeof(float) + 64);
    size_t ow = 0, ob = 0;
    for (int l = 0; l < d.num_layers; l++) {
        int i, o;
        layer_dims(d, l, i, o);
        if (!W[l] || !B[l]) return false;
        if (cudaMemcpyAsync(flat_w + ow, W[l], (size_t)i * o * sizeof(half), cudaMemcpyDeviceToDevice, st) != cudaSuccess) return false;
        if (cudaMemcpyAsync(flat_b + ob, B[l], (size_t)o * sizeof(float), cudaMemcpyDeviceToDevice, st) != cudaSuccess) return false;
        ow += (size_t)i * o; ob += (size_t)o;
    }
    return true;
}

}  // namespace

// ---- TinyMLP.h ------------------------------------------------------------------------------------------------------
extern "C" void launchNetworkFusionKernel(MLPOption* opt, half* d_inputs, half** d_weights_array, float** d_biases_array, float* d_outputs,
                                          int batchSize, cudaStream_t stream) {
    nb_mlp_desc d = desc_of(*opt);
    half* w; float* b;
    if (!gather_network(d, d_weights_array, d_biases_array, w, b, stream)) { std::fprintf(stderr, "[libnerf_b200] launchNetworkFusionKernel: bad layer pointers\n"); return; }
    report(nb_mlp_forward(&d, d_inputs, w, b, batchSize, d_outputs, nullptr, stream), "launchNetworkFusionKernel");
}

extern "C" void launchMSELossGrad(const float* predictions, const half* targets, half* dLoss_out, float* total_loss, int batchSize, int paddedDim,
                                  int validDim, float loss_scale, cudaStream_t stream, int outputActivation) {
    report(nb_mse_loss_grad(predictions, targets, dLoss_out, total_loss, batchSize, paddedDim, validDim, loss_scale, outputActivation, stream),
           "launchMSELossGrad");
}

extern "C" void launchZeroGradients(MLPOption* opt, float** w_grads, float** b_grads, cudaStream_t stream) {
    nb_mlp_desc d = desc_of(*opt);
    const auto W = pointer_array(w_grads, d.num_layers);
    const auto B = pointer_array(b_grads, d.num_layers);
    for (int l = 0; l < d.num_layers; l++) {
        int i, o;
        layer_dims(d, l, i, o);
        if (!W[l] || !B[l]) { std::fprintf(stderr, "[libnerf_b200] launchZeroGradients: bad layer pointers\n"); return; }
        report(nb_zero_async(W[l], (int64_t)i * o * sizeof(float), stream), "launchZeroGradients");
        report(nb_zero_async(B[l], (int64_t)o * sizeof(float), stream), "launchZeroGradients");
    }
}

// Dense Adam of one kind of parameter, layer by layer.  The fp16 copy of a layer goes to fwd[l] when given, else to scratch.
static void adam_layers(const nb_mlp_desc& d, bool weights, float** master, half** fwd, float** grads, float** m, float** v, float lr, float beta1,
                        float beta2, float epsilon, float bc1, float bc2, float inv_loss_scale, cudaStream_t stream, const char* who) {
    const auto P = pointer_array(master, d.num_layers);
    const auto G = pointer_array(grads, d.num_layers);
    const auto M = pointer_array(m, d.num_layers);
    const auto V = pointer_array(v, d.num_layers);
    const std::vector<half*> F = pointer_array(fwd, fwd ? d.num_layers : 0);
    for (int l = 0; l < d.num_layers; l++) {
        int i, o;
        layer_dims(d, l, i, o);
        const int64_t count = weights ? (int64_t)i * o : (int64_t)o;
        void* wh = fwd ? (void*)F[l] : scratch(2).get((size_t)count * sizeof(half) + 64);
        if (!P[l] || !G[l] || !M[l] || !V[l] || !wh) { std::fprintf(stderr, "[libnerf_b200] %s: bad layer pointers\n", who); return; }
        // the reference's dense optimizers leave the gradient in place (zero-grad is a launch of its own)
        report(nb_adam_step(P[l], wh, G[l], M[l], V[l], 0, count, lr, beta1, beta2, epsilon, bc1, bc2, inv_loss_scale, 0, stream), who);
    }
}

extern "C" void launchAdamWeightsOptim(MLPOption* opt, float** master_weights, half** fwd_weights, float** gradients, float** m, float** v, float lr,
                                       float beta1, float beta2, float epsilon, float bias_correction1, float bias_correction2,
                                       float inv_loss_scale, cudaStream_t stream) {
    adam_layers(desc_of(*opt), true, master_weights, fwd_weights, gradients, m, v, lr, beta1, beta2, epsilon, bias_correction1, bias_correction2,
                inv_loss_scale, stream, "launchAdamWeightsOptim");
}

extern "C" void launchAdamBiasOptim(MLPOption* opt, float** biases, float** gradients, float** m, float** v, float lr, float beta1, float beta2,
                                    float epsilon, float bias_correction1, float bias_correction2, float inv_loss_scale, cudaStream_t stream) {
    adam_layers(desc_of(*opt), false, biases, nullptr, gradients, m, v, lr, beta1, beta2, epsilon, bias_correction1, bias_correction2, inv_loss_scale,
                stream, "launchAdamBiasOptim");
}

// ---- TinyMLPHashGrid.h ------------------------------------------------------------------------------------------------
extern "C" void launchNetworkFusionHashTableKernel(MLPGridOptions* opt, half* d_hashtable, float* d_inputs, half** d_weights_array,
                                                   float** d_biases_array, float* d_outputs, int batchSize, cudaStream_t stream) {
    // grid geometry per (levels, table size, base resolution, growth); the set-up runs a kernel and waits once per geometry
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, float>, nb_grid_desc> grids;
    nb_grid_desc g;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto key = std::make_tuple(opt->numLevels, opt->tableSize, opt->lowestSize, opt->b);
        auto it = grids.find(key);
        if (it == grids.end()) {
            nb_grid_desc fresh;
            int rc = nb_grid_setup(&fresh, opt->numLevels, opt->tableSize, opt->lowestSize, opt->b, stream);
            if (rc != NB_OK) { report(rc, "launchNetworkFusionHashTableKernel"); return; }
            it = grids.emplace(key, fresh).first;
        }
        g = it->second;
    }
    if (opt->vectorDim != 4) { std::fprintf(stderr, "[libnerf_b200] launchNetworkFusionHashTableKernel: positions must be float4 (vectorDim 4)\n"); return; }
    nb_mlp_desc d;
    d.input_dim = opt->numLevels * opt->featuresLevel; d.hidden_dim = opt->hiddenDim; d.output_dim = opt->outputDim; d.num_layers = opt->numLayers;
    d.output_activation = 0;
    half* w; float* b;
    if (!gather_network(d, d_weights_array, d_biases_array, w, b, stream)) { std::fprintf(stderr, "[libnerf_b200] launchNetworkFusionHashTableKernel: bad layer pointers\n"); return; }
    report(nb_grid_mlp_forward(&g, &d, d_inputs, d_hashtable, w, b, batchSize, d_outputs, nullptr, nullptr, stream), "launchNetworkFusionHashTableKernel");
}

extern "C" void launchAdamHashGridOptim(MLPGridOptions* opt, float* master_hash, half* fwd_hash, float* gradients, float* m, float* v, float lr,
                                        float beta1, float beta2, float epsilon, float bias_correction1, float bias_correction2,
                                        float inv_loss_scale, cudaStream_t stream) {
    const int64_t count = (int64_t)opt->numLevels * opt->tableSize * opt->featuresLevel;
    report(nb_adam_step(master_hash, fwd_hash, gradients, m, v, count, count, lr, beta1, beta2, epsilon, bias_correction1, bias_correction2,
                        inv_loss_scale, 0, stream), "launchAdamHashGridOptim");
}

// ---- InstantNerf.h ------------------------------------------------------------------------------------------------------
static nb_scene_desc scene_of(uint3 res, float3 lo, float3 hi, int cascades, int levels, int spv) {
    nb_scene_desc s;
    s.grid_res[0] = res.x; s.grid_res[1] = res.y; s.grid_res[2] = res.z;
    s.aabb_min[0] = lo.x; s.aabb_min[1] = lo.y; s.aabb_min[2] = lo.z;
    s.aabb_max[0] = hi.x; s.aabb_max[1] = hi.y; s.aabb_max[2] = hi.z;
    s.num_cascades = cascades; s.mip_levels = levels; s.samples_per_voxel = spv;
    return s;
}

// Count, scan, cutoff from ray 0, emit.  Returns the rays that fit `batchSize` samples, *totalHits their samples; the
// reference blocks three times on the way (processRays.cu:979-1013), this once.
extern "C" int processRaysHitLinear(const uint32_t num_rays, const float3* rays_o, const float3* rays_d, const float3* rays_d_inv, const float* nears,
                                    const float* fars, const uint8_t* occupancy_grid, const uint3 grid_resolution, const float3 aabb_min,
                                    const float3 aabb_max, const int numCascades, const int mipmapLevels, const int samplesPerVoxel,
                                    const int batchSize, uint32_t* totalHits, uint32_t* d_active_rays_count, uint32_t* d_num_steps,
                                    uint32_t* d_ray_offsets, float* d_mlp_positions_batch, uint32_t* d_ray_indices, float* d_t_sorted,
                                    uint32_t* d_block_sums, cudaStream_t stream) {
    nb_scene_desc sc = scene_of(grid_resolution, aabb_min, aabb_max, numCascades, mipmapLevels, samplesPerVoxel);
    uint32_t* d_plan = (uint32_t*)scratch(3).get(64);
    const float* o = reinterpret_cast<const float*>(rays_o);
    const float* d = reinterpret_cast<const float*>(rays_d);
    const float* di = reinterpret_cast<const float*>(rays_d_inv);
    int rc = nb_march_count(&sc, o, d, di, nears, fars, occupancy_grid, num_rays, d_num_steps, stream);
    if (rc == NB_OK) rc = nb_march_scan(d_num_steps, d_ray_offsets, d_block_sums, num_rays, (uint32_t)batchSize, d_plan, stream);
    uint32_t plan[4] = {0, 0, 0, 0};
    if (rc == NB_OK && cudaMemcpyAsync(plan, d_plan, sizeof(plan), cudaMemcpyDeviceToHost, stream) != cudaSuccess) rc = NB_ERR_CUDA;
    if (rc == NB_OK && cudaStreamSynchronize(stream) != cudaSuccess) rc = NB_ERR_CUDA;
    if (rc == NB_OK && plan[0] > 0)
        rc = nb_march_emit(&sc, o, d, di, nears, fars, occupancy_grid, num_rays, 0, plan[0], d_ray_offsets, d_plan, d_t_sorted, d_ray_indices,
                           d_mlp_positions_batch, stream);
    if (rc == NB_OK && d_active_rays_count != nullptr &&
        cudaMemcpyAsync(d_active_rays_count, d_plan, sizeof(uint32_t), cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        rc = NB_ERR_CUDA;
    if (rc != NB_OK) { report(rc, "processRaysHitLinear"); if (totalHits) *totalHits = 0; return 0; }
    if (totalHits) *totalHits = plan[1];
    return (int)plan[0];
}

extern "C" void launchVolumeRendering(const uint32_t num_rays, const uint32_t* d_ray_offsets, const uint32_t* d_num_steps, const float* d_t_sorted,
                                      const float* d_density_sigma, const float* d_depth_chunk, const float* d_sigma_chunk, const float* d_rgb_output,
                                      const float* d_rgb_true, float* d_render_rgb, float* d_render_depth, float* d_phi_out, float* d_dw_out,
                                      float* d_weight_sum, float lambda_dist, float lambda_depth, float3 bg_color, uint32_t base, uint32_t raysDone,
                                      cudaStream_t stream) {
    const float bg[3] = {bg_color.x, bg_color.y, bg_color.z};
    if (d_dw_out == nullptr) {
        report(nb_composite_infer(num_rays, base, raysDone, d_ray_offsets, d_num_steps, d_t_sorted, d_density_sigma, d_rgb_output, 3, d_rgb_true,
                                  d_render_rgb, d_render_depth, d_phi_out, bg, stream), "launchVolumeRendering");
    } else {
        // the reference's training kernel takes the offsets as they are and ignores base / raysDone (compositing.cu:241-261)
        report(nb_composite_train(num_rays, 0, d_ray_offsets, d_num_steps, d_t_sorted, d_density_sigma, d_depth_chunk, d_sigma_chunk,
                                  d_rgb_output, 3, d_rgb_true, d_render_rgb, d_render_depth, d_phi_out, d_dw_out, d_weight_sum, lambda_dist,
                                  lambda_depth, bg, stream), "launchVolumeRendering");
    }
}
