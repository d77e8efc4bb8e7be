// Front-to-back volume compositing (inference and training variants), the distortion loss terms and the
// per-sample loss gradients.
//
// Replaces render_rays_kernel and render_rays_distortion_kernel (modules/NeRF/compositing.cu:5-213, launcher
// launchVolumeRendering :215-279) and compute_color_grad (modules/NeRF/otherKernels.cu:303-409).
// One thread per ray, samples of a ray contiguous in ray order, exactly the reference's arithmetic.
// Colour buffers carry a row stride so the colour network's padded [n][8] output and gradient are used in
// place (the reference un-pads to [n][3] and pads back with two extra kernels, TinyMLP.cu:276-284,361-367).
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__global__ void __launch_bounds__(256) render_rays_kernel(const uint32_t num_rays, const uint32_t base, const uint32_t raysDone,
                                                          const uint32_t* __restrict__ ray_offsets, const uint32_t* __restrict__ num_steps,
                                                          const float* __restrict__ t_sorted, const float* __restrict__ density_sigma,
                                                          const float* __restrict__ rgb_output, const int rgb_stride,
                                                          const float* __restrict__ rgb_true, float* __restrict__ final_rgb,
                                                          float* __restrict__ final_depth, float* __restrict__ phi_out, float3 bg_color) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= num_rays) return;
    uint32_t offset = ray_offsets[r + raysDone] - base;
    uint32_t count = num_steps[r];
    float T = 1.0f;
    float r_c = 0.0f, g_c = 0.0f, b_c = 0.0f;
    float depth = 0.0f;
    for (uint32_t i = 0; i < count; ++i) {
        uint32_t idx = offset + i;
        float t = t_sorted[idx];
        float delta_t = 0.0f;
        if (i < count - 1) delta_t = t_sorted[idx + 1] - t;
        else delta_t = 1e-3f;
        if (delta_t < 0.0f) delta_t = 0.0f;
        float sigma = density_sigma[idx];
        float alpha = 1.0f - expf(-sigma * delta_t);
        float weight = alpha * T;
        r_c += weight * rgb_output[(size_t)idx * rgb_stride + 0];
        g_c += weight * rgb_output[(size_t)idx * rgb_stride + 1];
        b_c += weight * rgb_output[(size_t)idx * rgb_stride + 2];
        depth += weight * t;
        T *= (1.0f - alpha);
        if (T < 1e-4f) break;
    }
    r_c += T * bg_color.x;
    g_c += T * bg_color.y;
    b_c += T * bg_color.z;
    final_rgb[r * 3 + 0] = r_c;
    final_rgb[r * 3 + 1] = g_c;
    final_rgb[r * 3 + 2] = b_c;
    if (final_depth != nullptr) final_depth[r] = depth;
    if (rgb_true != nullptr && phi_out != nullptr) {
        phi_out[r * 3 + 0] = 2.0f * (r_c - rgb_true[r * 3 + 0]);
        phi_out[r * 3 + 1] = 2.0f * (g_c - rgb_true[r * 3 + 1]);
        phi_out[r * 3 + 2] = 2.0f * (b_c - rgb_true[r * 3 + 2]);
    }
}

__device__ __forceinline__ float disparity_warp(float t, float t_near, float inv_g_range) {
    return (1.0f - t_near / fmaxf(t, 1e-4f)) * inv_g_range;
}

__global__ void __launch_bounds__(256) render_rays_distortion_kernel(
    const uint32_t num_rays, const uint32_t* __restrict__ ray_offsets, const uint32_t* __restrict__ num_steps,
    const float* __restrict__ t_sorted, const float* __restrict__ density_sigma, const float* __restrict__ depth_chunk,
    const float* __restrict__ sigma_chunk, const float* __restrict__ rgb_output, const int rgb_stride, const float* __restrict__ rgb_true,
    float* __restrict__ final_rgb, float* __restrict__ final_depth, float* __restrict__ phi_out, float* __restrict__ dw_out,
    float* __restrict__ weight_sum, float lambda_dist, float lambda_depth, float3 bg_color) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= num_rays) return;
    uint32_t offset = ray_offsets[r];
    uint32_t count = num_steps[r];
    float d_prior = depth_chunk ? depth_chunk[r] : -1.0f;
    float sigma_prior = sigma_chunk ? sigma_chunk[r] : -1.0f;
    float depth_weight_loss = (d_prior >= 0) ? lambda_depth : 0.0f;
    float t_near = (count > 0) ? fmaxf(t_sorted[offset], 1e-4f) : 1.0f;
    float t_far_ray = (count > 0) ? t_sorted[offset + count - 1] : 1.0f;
    float g_far = 1.0f - t_near / fmaxf(t_far_ray, t_near + 1e-4f);
    float inv_g_range = (g_far > 1e-6f) ? (1.0f / g_far) : 0.0f;
    float T = 1.0f;
    float r_c = 0.0f, g_c = 0.0f, b_c = 0.0f;
    float depth = 0.0f;
    float c = 2.0f / 3;
    float dw_global_sum = 0.0f, dwm_global_sum = 0.0f, dw_sum = 0.0f, dwm_sum = 0.0f, depth_loss_sum = 0.0f;
    for (uint32_t i = 0; i < count; i++) {
        uint32_t idx = offset + i;
        float t = t_sorted[idx];
        float t_next = (i < count - 1) ? t_sorted[idx + 1] : (t + 1e-3f);
        float delta_t = t_next - t;
        if (delta_t < 0.0f) { delta_t = 0.0f; t_next = t; }
        float s = disparity_warp(t, t_near, inv_g_range);
        float s_next = disparity_warp(t_next, t_near, inv_g_range);
        float m = 0.5f * (s + s_next);
        float sigma = density_sigma[idx];
        float alpha = 1.0f - expf(-sigma * delta_t);
        float weight = alpha * T;
        r_c += weight * rgb_output[(size_t)idx * rgb_stride + 0];
        g_c += weight * rgb_output[(size_t)idx * rgb_stride + 1];
        b_c += weight * rgb_output[(size_t)idx * rgb_stride + 2];
        depth += weight * t;
        T *= (1.0f - alpha);
        dw_global_sum += weight;
        dwm_global_sum += weight * m;
        float tx = (t - d_prior) / sigma_prior;
        float depthWeight = expf(-0.5f * tx * tx) * delta_t;
        depth_loss_sum += depthWeight;
        dw_out[idx] = weight;
    }
    depth_loss_sum = 1.0f / fmaxf(depth_loss_sum, 1e-8f);
    float weight_g_sum = 0.0f;
    for (uint32_t i = 0; i < count; i++) {
        uint32_t idx = offset + i;
        float t = t_sorted[idx];
        float t_next = (i < count - 1) ? t_sorted[idx + 1] : (t + 1e-3f);
        float delta_t = t_next - t;
        if (delta_t < 0.0f) { delta_t = 0.0f; t_next = t; }
        float s = disparity_warp(t, t_near, inv_g_range);
        float s_next = disparity_warp(t_next, t_near, inv_g_range);
        float m = 0.5f * (s + s_next);
        float delta_s = s_next - s;
        if (delta_s < 0.0f) delta_s = 0.0f;
        float crrWeight = dw_out[idx];
        float tx = (t - d_prior) / sigma_prior;
        float depthWeight = expf(-0.5f * tx * tx) * delta_t * depth_loss_sum;
        float depthLoss = -depthWeight * (1.0f / fmaxf(crrWeight, 1e-6));
        float dl_bilinear = m * (2 * dw_sum - dw_global_sum) + (dwm_global_sum - 2 * dwm_sum);
        dw_out[idx] = lambda_dist * (2 * (dl_bilinear) + c * crrWeight * delta_s) + depth_weight_loss * depthLoss;
        weight_g_sum += crrWeight * (lambda_dist * (2 * (dl_bilinear) + c * crrWeight * delta_s) + depth_weight_loss * depthLoss);
        dw_sum += crrWeight;
        dwm_sum += crrWeight * m;
    }
    weight_sum[r] = weight_g_sum;
    r_c += T * bg_color.x;
    g_c += T * bg_color.y;
    b_c += T * bg_color.z;
    final_rgb[r * 3 + 0] = r_c;
    final_rgb[r * 3 + 1] = g_c;
    final_rgb[r * 3 + 2] = b_c;
    if (final_depth != nullptr) final_depth[r] = depth;
    if (rgb_true != nullptr && phi_out != nullptr) {
        phi_out[r * 3 + 0] = 2.0f * (r_c - rgb_true[r * 3 + 0]);
        phi_out[r * 3 + 1] = 2.0f * (g_c - rgb_true[r * 3 + 1]);
        phi_out[r * 3 + 2] = 2.0f * (b_c - rgb_true[r * 3 + 2]);
    }
}

// GRAD8: the gradient row is 8 halves wide (16-byte store, channels 3..7 zero); otherwise 3 halves.
template <bool GRAD8>
__global__ void __launch_bounds__(256) color_grad_kernel(const uint32_t numRays, const uint32_t* __restrict__ num_steps,
                                                         const uint32_t* __restrict__ ray_offsets, const float* __restrict__ t_sorted,
                                                         const float* __restrict__ density_mlp_out, const int logit_stride,
                                                         const float* __restrict__ color_mlp_out, const int color_stride, const float* __restrict__ phi_chunk,
                                                         const float* __restrict__ final_rgb, const float* __restrict__ dw_out,
                                                         const float* __restrict__ weight_sum, __half* __restrict__ custom_color_grad,
                                                         float* __restrict__ tmp_dsigma, float loss_scale, const float densityBias,
                                                         const uint32_t totalRaysBatch) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= numRays) return;
    float currentT = 1.0f;
    float3 currentRgb = make_float3(0.0f, 0.0f, 0.0f);
    float currentWeightG = 0.0f;
    uint32_t rayIdx = ray_offsets[idx];
    float crrWeightGSum = weight_sum[idx];
    uint32_t maxDepth = num_steps[idx];
    float phi_r = phi_chunk[idx * 3], phi_g = phi_chunk[idx * 3 + 1], phi_b = phi_chunk[idx * 3 + 2];
    float final_r = final_rgb[idx * 3], final_g = final_rgb[idx * 3 + 1], final_b = final_rgb[idx * 3 + 2];
    float delta_t;
    for (int depth_idx = 0; depth_idx < maxDepth; depth_idx++) {
        uint32_t i = rayIdx + depth_idx;
        float t_current = t_sorted[i];
        if (depth_idx == maxDepth - 1) delta_t = 1e-3f;
        else delta_t = fmaxf(t_sorted[i + 1] - t_current, 0.0f);
        float sigma = expf(fminf(density_mlp_out[(size_t)i * logit_stride] - densityBias, 8.0f));
        float alpha = 1.0f - expf(-sigma * delta_t);
        float weight = currentT * alpha;
        float c_r = color_mlp_out[(size_t)i * color_stride + 0];
        float c_g = color_mlp_out[(size_t)i * color_stride + 1];
        float c_b = color_mlp_out[(size_t)i * color_stride + 2];
        currentRgb.x += weight * c_r;
        currentRgb.y += weight * c_g;
        currentRgb.z += weight * c_b;
        float batch_scale = 1.0f / (float)totalRaysBatch;
        float cg_r = phi_r * weight * c_r * (1.0f - c_r) * loss_scale * batch_scale;
        float cg_g = phi_g * weight * c_g * (1.0f - c_g) * loss_scale * batch_scale;
        float cg_b = phi_b * weight * c_b * (1.0f - c_b) * loss_scale * batch_scale;
        cg_r = fmaxf(-65504.0f, fminf(65504.0f, cg_r));
        cg_g = fmaxf(-65504.0f, fminf(65504.0f, cg_g));
        cg_b = fmaxf(-65504.0f, fminf(65504.0f, cg_b));
        if (cg_r != cg_r || cg_g != cg_g || cg_b != cg_b) { cg_r = 0.0f; cg_g = 0.0f; cg_b = 0.0f; }
        if (GRAD8) {
            uint4 v = make_uint4(pack_half2(cg_r, cg_g), pack_half2(cg_b, 0.0f), 0u, 0u);
            *reinterpret_cast<uint4*>(custom_color_grad + (size_t)i * 8) = v;
        } else {
            custom_color_grad[(size_t)i * 3 + 0] = __float2half(cg_r);
            custom_color_grad[(size_t)i * 3 + 1] = __float2half(cg_g);
            custom_color_grad[(size_t)i * 3 + 2] = __float2half(cg_b);
        }
        float suff_r = final_r - currentRgb.x;
        float suff_g = final_g - currentRgb.y;
        float suff_b = final_b - currentRgb.z;
        float ds_r = currentT * c_r * (1.0f - alpha) - suff_r;
        float ds_g = currentT * c_g * (1.0f - alpha) - suff_g;
        float ds_b = currentT * c_b * (1.0f - alpha) - suff_b;
        float g_i = dw_out[i];
        currentWeightG += weight * g_i;
        float suffix_weight = crrWeightGSum - currentWeightG;
        float d_sigma_i = delta_t * (ds_r * phi_r + ds_g * phi_g + ds_b * phi_b);
        d_sigma_i += delta_t * (g_i * currentT * (1.0f - alpha) - suffix_weight);
        float ds = d_sigma_i * sigma * loss_scale * batch_scale;
        ds = fmaxf(-65504.0f, fminf(65504.0f, ds));
        if (ds != ds) ds = 0.0f;
        tmp_dsigma[i] = ds;
        currentT = currentT * (1.0f - alpha);
    }
}

}  // namespace nb

using namespace nb;

extern "C" int nb_composite_infer(int64_t num_rays, uint32_t base, uint32_t rays_done, const uint32_t* d_ray_offsets,
                                  const uint32_t* d_num_steps, const float* d_t_sorted, const float* d_sigma, const float* d_rgb,
                                  int rgb_stride, const float* d_rgb_true, float* d_final_rgb, float* d_final_depth, float* d_phi,
                                  const float* bg_color3, void* stream) {
    if (!d_ray_offsets || !d_num_steps || !d_t_sorted || !d_sigma || !d_rgb || !d_final_rgb || !bg_color3 || num_rays < 0 ||
        num_rays > 0x7fffffff || rgb_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_infer: null pointer, bad ray count or rgb stride < 3");
    if (num_rays == 0) return NB_OK;
    render_rays_kernel<<<(unsigned)((num_rays + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint32_t)num_rays, base, rays_done, d_ray_offsets, d_num_steps, d_t_sorted, d_sigma, d_rgb, rgb_stride, d_rgb_true, d_final_rgb,
        d_final_depth, d_phi, make_float3(bg_color3[0], bg_color3[1], bg_color3[2]));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_composite_train(int64_t num_rays, const uint32_t* d_ray_offsets, const uint32_t* d_num_steps, const float* d_t_sorted,
                                  const float* d_sigma, const float* d_depth_prior, const float* d_sigma_prior, const float* d_rgb,
                                  int rgb_stride, const float* d_rgb_true, float* d_final_rgb, float* d_final_depth, float* d_phi,
                                  float* d_dw_out, float* d_weight_sum, float lambda_dist, float lambda_depth, const float* bg_color3,
                                  void* stream) {
    if (!d_ray_offsets || !d_num_steps || !d_t_sorted || !d_sigma || !d_rgb || !d_final_rgb || !d_dw_out || !d_weight_sum || !bg_color3 ||
        num_rays < 0 || num_rays > 0x7fffffff || rgb_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_train: null pointer, bad ray count or rgb stride < 3");
    if (num_rays == 0) return NB_OK;
    render_rays_distortion_kernel<<<(unsigned)((num_rays + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint32_t)num_rays, d_ray_offsets, d_num_steps, d_t_sorted, d_sigma, d_depth_prior, d_sigma_prior, d_rgb, rgb_stride, d_rgb_true,
        d_final_rgb, d_final_depth, d_phi, d_dw_out, d_weight_sum, lambda_dist, lambda_depth,
        make_float3(bg_color3[0], bg_color3[1], bg_color3[2]));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_color_grad(int64_t num_rays, const uint32_t* d_num_steps, const uint32_t* d_ray_offsets, const float* d_t_sorted,
                             const float* d_logit0, int logit_stride, const float* d_color_out, int color_stride, const float* d_phi,
                             const float* d_final_rgb, const float* d_dw_out, const float* d_weight_sum, void* d_color_grad_h,
                             int grad_stride, float* d_tmp_dsigma, float loss_scale, float density_bias, uint32_t total_rays_batch,
                             void* stream) {
    if (!d_num_steps || !d_ray_offsets || !d_t_sorted || !d_logit0 || logit_stride < 1 || !d_color_out || !d_phi || !d_final_rgb || !d_dw_out ||
        !d_weight_sum || !d_color_grad_h || !d_tmp_dsigma || num_rays < 0 || num_rays > 0x7fffffff || color_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_color_grad: null pointer, bad ray count or colour stride < 3");
    if (grad_stride != 3 && grad_stride != 8) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_color_grad: gradient row stride must be 3 or 8 halves");
    if (grad_stride == 8 && (reinterpret_cast<uintptr_t>(d_color_grad_h) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_color_grad: 8-wide gradient rows must be 16-byte aligned");
    if (total_rays_batch == 0) return nb_set_error(NB_ERR_INVALID, "nb_color_grad: total_rays_batch must be positive");
    if (num_rays == 0) return NB_OK;
    unsigned grid = (unsigned)((num_rays + 255) / 256);
    if (grad_stride == 8)
        color_grad_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((uint32_t)num_rays, d_num_steps, d_ray_offsets, d_t_sorted, d_logit0, logit_stride,
                                                                        d_color_out, color_stride, d_phi, d_final_rgb, d_dw_out, d_weight_sum,
                                                                        (__half*)d_color_grad_h, d_tmp_dsigma, loss_scale, density_bias,
                                                                        total_rays_batch);
    else
        color_grad_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((uint32_t)num_rays, d_num_steps, d_ray_offsets, d_t_sorted, d_logit0, logit_stride,
                                                                         d_color_out, color_stride, d_phi, d_final_rgb, d_dw_out, d_weight_sum,
                                                                         (__half*)d_color_grad_h, d_tmp_dsigma, loss_scale, density_bias,
                                                                         total_rays_batch);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
