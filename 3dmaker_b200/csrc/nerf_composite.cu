// Front-to-back volume compositing (inference and training variants), the distortion loss terms and the
// per-sample loss gradients.
//
// Replaces render_rays_kernel and render_rays_distortion_kernel (modules/NeRF/compositing.cu:5-213, launcher
// launchVolumeRendering :215-279) and compute_color_grad (modules/NeRF/otherKernels.cu:303-409).
//
// The reference gives every ray to one thread that walks the ray's samples in a loop: neighbouring lanes read
// addresses a whole ray apart and the loop is a chain of dependent loads, exponentials and multiplies.  Here a WARP
// owns a ray and lane k owns sample k of the current 32-sample window, so loads are contiguous and everything that
// the reference carries from sample to sample - transmittance, accumulated colour, the distortion loss's prefix
// sums, the suffix terms of the gradients - becomes a warp scan with a carry between windows:
//     T_i      = prod_{j<i} (1 - alpha_j)                       exclusive product scan
//     W_<i     = sum_{j<i} w_j ,  WM_<i = sum_{j<i} w_j m_j      exclusive sum scans (distortion loss)
//     C_<=i    = sum_{j<=i} w_j c_j , G_<=i = sum_{j<=i} w_j g_j   inclusive sum scans (gradient suffix terms)
// The formulas are the reference's; sums are associated differently, so results agree to fp32 rounding, not bitwise.
// Colour buffers carry a row stride so the colour network's padded output and gradient are used in place (the
// reference un-pads to [n][3] and pads back with two extra kernels, TinyMLP.cu:276-284,361-367).
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}
__device__ __forceinline__ float warp_incl_sum(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float n = __shfl_up_sync(FULL, v, o);
        if (lane >= o) v += n;
    }
    return v;
}
__device__ __forceinline__ float warp_incl_prod(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float n = __shfl_up_sync(FULL, v, o);
        if (lane >= o) v *= n;
    }
    return v;
}
// value of the lane below (identity for lane 0): turns an inclusive scan into an exclusive one
__device__ __forceinline__ float from_lane_below(float incl, int lane, float identity) {
    float n = __shfl_up_sync(FULL, incl, 1);
    return lane == 0 ? identity : n;
}

// Sample i of a ray with `count` samples starting at `first`: distance, distance of the next sample, interval clamped
// at zero.  The last sample has no successor and gets a 1e-3 interval: as the literal where NOMINAL_LAST (the
// inference and gradient kernels of the reference), as (t + 1e-3) - t otherwise (its training kernel) - the two differ
// in the last bits and each kernel keeps its own form.
struct Interval {
    float t, t_next, dt;
};
template <bool NOMINAL_LAST>
__device__ __forceinline__ Interval load_interval(const float* __restrict__ t_sorted, uint32_t first, uint32_t i, uint32_t count) {
    Interval v;
    v.t = t_sorted[first + i];
    v.t_next = (i + 1 < count) ? t_sorted[first + i + 1] : v.t + 1e-3f;
    v.dt = (NOMINAL_LAST && i + 1 >= count) ? 1e-3f : v.t_next - v.t;
    if (v.dt < 0.0f) { v.dt = 0.0f; v.t_next = v.t; }
    return v;
}

// ---------------------------------------------------------------------------------------------------------
// inference: colour and depth of a ray, stopping once the transmittance has dropped below 1e-4
// ---------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) composite_infer_kernel(const uint32_t num_rays, const uint32_t sample_base,
                                                              const uint32_t* __restrict__ ray_offsets, const uint32_t* __restrict__ num_steps,
                                                              const float* __restrict__ t_sorted, const float* __restrict__ sigma_in,
                                                              const float* __restrict__ rgb_in, const int rgb_stride,
                                                              const float* __restrict__ rgb_true, float* __restrict__ final_rgb,
                                                              float* __restrict__ final_depth, float* __restrict__ phi_out, float3 bg) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= num_rays) return;
    const uint32_t first = ray_offsets[r] - sample_base;
    const uint32_t count = num_steps[r];
    float T = 1.0f;  // transmittance in front of the current window
    float cr = 0.f, cg = 0.f, cb = 0.f, depth = 0.f;
    for (uint32_t w0 = 0; w0 < count; w0 += 32) {
        const uint32_t i = w0 + lane;
        const bool valid = i < count;
        float alpha = 0.f, t = 0.f;
        if (valid) {
            Interval iv = load_interval<true>(t_sorted, first, i, count);
            t = iv.t;
            alpha = 1.0f - expf(-sigma_in[first + i] * iv.dt);
        }
        const float incl = warp_incl_prod(1.0f - alpha, lane);
        const float T_before = T * from_lane_below(incl, lane, 1.0f);
        // the reference leaves its loop after the first sample that takes T below 1e-4: sample i counts exactly when
        // the transmittance in front of it is still at least 1e-4
        const bool live = valid && T_before >= 1e-4f;
        if (live) {
            const float w = alpha * T_before;
            const float* c = rgb_in + (size_t)(first + i) * rgb_stride;
            cr += w * c[0]; cg += w * c[1]; cb += w * c[2];
            depth += w * t;
        }
        const unsigned live_mask = __ballot_sync(FULL, live);
        const int last = 31 - __clz((int)live_mask);            // live_mask != 0: lane 0 of a window is live or the loop ended
        const float T_after_last = __shfl_sync(FULL, T * incl, last);
        T = T_after_last;
        if (live_mask != __ballot_sync(FULL, valid) || T < 1e-4f) break;
    }
    cr = warp_sum(cr); cg = warp_sum(cg); cb = warp_sum(cb); depth = warp_sum(depth);
    if (lane == 0) {
        cr += T * bg.x; cg += T * bg.y; cb += T * bg.z;
        final_rgb[r * 3 + 0] = cr; final_rgb[r * 3 + 1] = cg; final_rgb[r * 3 + 2] = cb;
        if (final_depth != nullptr) final_depth[r] = depth;
        if (rgb_true != nullptr && phi_out != nullptr) {
            phi_out[r * 3 + 0] = 2.0f * (cr - rgb_true[r * 3 + 0]);
            phi_out[r * 3 + 1] = 2.0f * (cg - rgb_true[r * 3 + 1]);
            phi_out[r * 3 + 2] = 2.0f * (cb - rgb_true[r * 3 + 2]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// inference in rounds: the same front-to-back sum, cut into rounds of samples so that rays whose transmittance has
// dropped below 1e-4 are not evaluated any further (the samples the reference's loop never reaches contribute
// nothing to it either).  State per ray between rounds: transmittance and (r, g, b, depth) composited so far.
// ---------------------------------------------------------------------------------------------------------
// When next_width > 0 the kernel also copies out the NEXT round (samples [round_begin + round_width, ... + next_width)) of
// the rays that are still visible after this one: a block's eight rays take one range of the next round's counter and
// each warp writes its ray's ids and contracted positions there - what round_emit_kernel does in a launch of its own.
__global__ void __launch_bounds__(256) composite_round_kernel(const uint32_t ray_begin, const uint32_t ray_count,
                                                              const uint32_t* __restrict__ num_steps, uint32_t* __restrict__ round_off,
                                                              const float* __restrict__ rows, const uint32_t row_stride,
                                                              const uint32_t round_begin, const uint32_t round_width,
                                                              const float* __restrict__ sigma_in, const float* __restrict__ rgb_in,
                                                              const int rgb_stride, float* __restrict__ transmittance,
                                                              float4* __restrict__ composited, float* __restrict__ final_rgb,
                                                              float* __restrict__ final_depth, float3 bg, const uint32_t next_width,
                                                              const float3 aabb_min, const float3 aabb_max, const float3* __restrict__ rays_o,
                                                              const float3* __restrict__ rays_d, const uint32_t capacity,
                                                              uint32_t* __restrict__ next_counter, unsigned long long* __restrict__ emitted_total,
                                                              uint32_t* __restrict__ ray_idx_out, float4* __restrict__ pos_out) {
    __shared__ uint32_t s_next[8], s_base;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t local = blockIdx.x * 8 + warp;
    const int lane = threadIdx.x & 31;
    const bool in_range = local < ray_count;
    const uint32_t r = ray_begin + local;
    const uint32_t n = in_range ? num_steps[r] : 0u;
    float T = 0.0f;
    if (in_range) T = round_begin == 0 ? 1.0f : transmittance[r];
    const bool active = in_range && T >= 1e-4f && n > round_begin;  // the predicate this round was planned with
    if (in_range && !active && round_begin == 0 && lane == 0) {
        final_rgb[r * 3 + 0] = bg.x; final_rgb[r * 3 + 1] = bg.y; final_rgb[r * 3 + 2] = bg.z;
        if (final_depth != nullptr) final_depth[r] = 0.0f;
    }
    const float* row = rows + (size_t)r * row_stride;
    if (active) {
        const uint32_t count = min(n - round_begin, round_width);
        const uint32_t first = round_off[r];
        float cr = 0.f, cg = 0.f, cb = 0.f, depth = 0.f;
        for (uint32_t w0 = 0; w0 < count; w0 += 32) {
            const uint32_t i = w0 + lane;
            const bool valid = i < count;
            float alpha = 0.f, t = 0.f;
            if (valid) {
                const uint32_t k = round_begin + i;  // index of the sample in its ray
                t = row[k];
                float dt = (k + 1 < n) ? row[k + 1] - t : 1e-3f;
                if (dt < 0.0f) dt = 0.0f;
                alpha = 1.0f - expf(-sigma_in[first + i] * dt);
            }
            const float incl = warp_incl_prod(1.0f - alpha, lane);
            const float T_before = T * from_lane_below(incl, lane, 1.0f);
            const bool live = valid && T_before >= 1e-4f;
            if (live) {
                const float w = alpha * T_before;
                const float* c = rgb_in + (size_t)(first + i) * rgb_stride;
                cr += w * c[0]; cg += w * c[1]; cb += w * c[2];
                depth += w * t;
            }
            const unsigned live_mask = __ballot_sync(FULL, live);
            const int last = 31 - __clz((int)live_mask);
            T = __shfl_sync(FULL, T * incl, last);
            if (live_mask != __ballot_sync(FULL, valid) || T < 1e-4f) break;
        }
        cr = warp_sum(cr); cg = warp_sum(cg); cb = warp_sum(cb); depth = warp_sum(depth);
        if (lane == 0) {
            float4 acc = round_begin == 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : composited[r];
            acc.x += cr; acc.y += cg; acc.z += cb; acc.w += depth;
            composited[r] = acc;
            transmittance[r] = T;
            final_rgb[r * 3 + 0] = acc.x + T * bg.x; final_rgb[r * 3 + 1] = acc.y + T * bg.y; final_rgb[r * 3 + 2] = acc.z + T * bg.z;
            if (final_depth != nullptr) final_depth[r] = acc.w;
        }
    }
    if (next_width == 0) return;  // the same for the whole grid
    const uint32_t next_begin = round_begin + round_width;
    const uint32_t c_next = (active && T >= 1e-4f && n > next_begin) ? min(n - next_begin, next_width) : 0u;
    if (lane == 0) s_next[warp] = c_next;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t total = 0;
#pragma unroll
        for (int w = 0; w < 8; w++) total += s_next[w];
        s_base = total ? atomicAdd(next_counter, total) : 0u;
        if (total && emitted_total != nullptr) atomicAdd(emitted_total, (unsigned long long)total);
    }
    __syncthreads();
    if (c_next == 0) return;
    uint32_t dst = s_base;
    for (uint32_t w = 0; w < warp; w++) dst += s_next[w];
    if (dst + c_next > capacity) return;  // cannot happen when the caller's bound holds; never write past the arrays
    if (lane == 0) round_off[r] = dst;
    const float3 o = rays_o[r], d = rays_d[r];
    for (uint32_t k = lane; k < c_next; k += 32) {
        const float t = row[next_begin + k];
        ray_idx_out[dst + k] = r;
        const float3 p = contract_pos(make_float3(o.x + t * d.x, o.y + t * d.y, o.z + t * d.z), aabb_min, aabb_max);
        st_cs_v4(&pos_out[dst + k], make_uint4(__float_as_uint(p.x), __float_as_uint(p.y), __float_as_uint(p.z), 0u));
    }
}

// ---------------------------------------------------------------------------------------------------------
// training: colour, depth, dL/dw of the distortion (and depth-prior) loss per sample, sum_i w_i dL/dw_i per ray
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float disparity_warp(float t, float t_near, float inv_g_range) {
    return (1.0f - t_near / fmaxf(t, 1e-4f)) * inv_g_range;
}

__global__ void __launch_bounds__(256) composite_train_kernel(
    const uint32_t num_rays, const uint32_t sample_base, const uint32_t* __restrict__ ray_offsets, const uint32_t* __restrict__ num_steps,
    const float* __restrict__ t_sorted, const float* __restrict__ sigma_in, const float* __restrict__ depth_prior,
    const float* __restrict__ sigma_prior_in, const float* __restrict__ rgb_in, const int rgb_stride, const float* __restrict__ rgb_true,
    float* __restrict__ final_rgb, float* __restrict__ final_depth, float* __restrict__ phi_out, float* __restrict__ dw_out,
    float* __restrict__ weight_sum, float lambda_dist, float lambda_depth, float3 bg) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= num_rays) return;
    const uint32_t first = ray_offsets[r] - sample_base;
    const uint32_t count = num_steps[r];
    const float d_prior = depth_prior ? depth_prior[r] : -1.0f;
    const float s_prior = sigma_prior_in ? sigma_prior_in[r] : -1.0f;
    const float depth_lambda = (d_prior >= 0) ? lambda_depth : 0.0f;
    // normalised disparity s(t) = (1 - t_near / t) / g_far over the ray's own sample range
    const float t_near = (count > 0) ? fmaxf(t_sorted[first], 1e-4f) : 1.0f;
    const float t_far = (count > 0) ? t_sorted[first + count - 1] : 1.0f;
    const float g_far = 1.0f - t_near / fmaxf(t_far, t_near + 1e-4f);
    const float inv_g = (g_far > 1e-6f) ? (1.0f / g_far) : 0.0f;

    // pass 1: weights (staged in dw_out), colour, depth, W = sum w, WM = sum w m, depth-prior normaliser
    float T = 1.0f;
    float cr = 0.f, cg = 0.f, cb = 0.f, depth = 0.f, W = 0.f, WM = 0.f, DN = 0.f;
    float w_keep = 0.f;  // this lane's weight when the ray fits one window (the common case): pass 2 skips the re-read
    for (uint32_t w0 = 0; w0 < count; w0 += 32) {
        const uint32_t i = w0 + lane;
        const bool valid = i < count;
        float alpha = 0.f, t = 0.f, m = 0.f, dterm = 0.f;
        if (valid) {
            Interval iv = load_interval<false>(t_sorted, first, i, count);
            t = iv.t;
            m = 0.5f * (disparity_warp(iv.t, t_near, inv_g) + disparity_warp(iv.t_next, t_near, inv_g));
            alpha = 1.0f - expf(-sigma_in[first + i] * iv.dt);
            const float tx = (iv.t - d_prior) / s_prior;
            dterm = expf(-0.5f * tx * tx) * iv.dt;
        }
        const float incl = warp_incl_prod(1.0f - alpha, lane);
        const float w = alpha * (T * from_lane_below(incl, lane, 1.0f));
        if (valid) {
            const float* c = rgb_in + (size_t)(first + i) * rgb_stride;
            cr += w * c[0]; cg += w * c[1]; cb += w * c[2];
            depth += w * t; W += w; WM += w * m; DN += dterm;
            dw_out[first + i] = w;
        }
        w_keep = w;
        T *= __shfl_sync(FULL, incl, 31);
    }
    cr = warp_sum(cr); cg = warp_sum(cg); cb = warp_sum(cb); depth = warp_sum(depth);
    W = warp_sum(W); WM = warp_sum(WM); DN = warp_sum(DN);
    const float depth_norm = 1.0f / fmaxf(DN, 1e-8f);

    // pass 2: dL/dw_i = lambda (2 (m_i (2 W_<i - W) + (WM - 2 WM_<i)) + (2/3) w_i ds_i) + depth term
    float W_lt = 0.f, WM_lt = 0.f, wg = 0.f;
    const float two_thirds = 2.0f / 3;
    for (uint32_t w0 = 0; w0 < count; w0 += 32) {
        const uint32_t i = w0 + lane;
        const bool valid = i < count;
        float w = 0.f, m = 0.f, ds = 0.f, dloss = 0.f;
        if (valid) {
            Interval iv = load_interval<false>(t_sorted, first, i, count);
            const float s = disparity_warp(iv.t, t_near, inv_g), s_next = disparity_warp(iv.t_next, t_near, inv_g);
            m = 0.5f * (s + s_next);
            ds = fmaxf(s_next - s, 0.0f);
            w = (count <= 32) ? w_keep : dw_out[first + i];
            const float tx = (iv.t - d_prior) / s_prior;
            dloss = -(expf(-0.5f * tx * tx) * iv.dt * depth_norm) * (1.0f / fmaxf(w, 1e-6));
        }
        const float w_incl = warp_incl_sum(w, lane), wm_incl = warp_incl_sum(w * m, lane);
        const float w_before = W_lt + (w_incl - w), wm_before = WM_lt + (wm_incl - w * m);
        if (valid) {
            const float bilinear = m * (2 * w_before - W) + (WM - 2 * wm_before);
            const float g = lambda_dist * (2 * bilinear + two_thirds * w * ds) + depth_lambda * dloss;
            dw_out[first + i] = g;
            wg += w * g;
        }
        W_lt += __shfl_sync(FULL, w_incl, 31);
        WM_lt += __shfl_sync(FULL, wm_incl, 31);
    }
    wg = warp_sum(wg);
    if (lane == 0) {
        weight_sum[r] = wg;
        cr += T * bg.x; cg += T * bg.y; cb += T * bg.z;
        final_rgb[r * 3 + 0] = cr; final_rgb[r * 3 + 1] = cg; final_rgb[r * 3 + 2] = cb;
        if (final_depth != nullptr) final_depth[r] = depth;
        if (rgb_true != nullptr && phi_out != nullptr) {
            phi_out[r * 3 + 0] = 2.0f * (cr - rgb_true[r * 3 + 0]);
            phi_out[r * 3 + 1] = 2.0f * (cg - rgb_true[r * 3 + 1]);
            phi_out[r * 3 + 2] = 2.0f * (cb - rgb_true[r * 3 + 2]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// loss gradients per sample: dL/d(colour pre-activation) in fp16 and dL/d(logit 0) through sigma
// ---------------------------------------------------------------------------------------------------------
// GRAD8: the gradient row is 8 halves wide (16-byte store, channels 3..7 zero); otherwise 3 halves.
template <bool GRAD8>
__global__ void __launch_bounds__(256) loss_grad_kernel(const uint32_t num_rays, const uint32_t sample_base, const uint32_t* __restrict__ num_steps,
                                                        const uint32_t* __restrict__ ray_offsets, const float* __restrict__ t_sorted,
                                                        const float* __restrict__ logit0, const int logit_stride,
                                                        const float* __restrict__ rgb_in, const int rgb_stride, const float* __restrict__ phi_in,
                                                        const float* __restrict__ final_rgb, const float* __restrict__ dw_in,
                                                        const float* __restrict__ weight_sum, __half* __restrict__ color_grad,
                                                        float* __restrict__ dsigma_out, float loss_scale, const float density_bias,
                                                        const uint32_t total_rays) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= num_rays) return;
    const uint32_t first = ray_offsets[r] - sample_base;
    const uint32_t count = num_steps[r];
    const float wg_total = weight_sum[r];
    const float phi_r = phi_in[r * 3], phi_g = phi_in[r * 3 + 1], phi_b = phi_in[r * 3 + 2];
    const float fin_r = final_rgb[r * 3], fin_g = final_rgb[r * 3 + 1], fin_b = final_rgb[r * 3 + 2];
    const float scale = loss_scale * (1.0f / (float)total_rays);
    float T = 1.0f, acc_r = 0.f, acc_g = 0.f, acc_b = 0.f, acc_wg = 0.f;  // carries: everything up to the current window
    for (uint32_t w0 = 0; w0 < count; w0 += 32) {
        const uint32_t i = w0 + lane;
        const bool valid = i < count;
        float alpha = 0.f, sigma = 0.f, dt = 0.f, c_r = 0.f, c_g = 0.f, c_b = 0.f, g = 0.f;
        if (valid) {
            Interval iv = load_interval<true>(t_sorted, first, i, count);
            dt = iv.dt;
            sigma = expf(fminf(logit0[(size_t)(first + i) * logit_stride] - density_bias, 8.0f));
            alpha = 1.0f - expf(-sigma * dt);
            const float* c = rgb_in + (size_t)(first + i) * rgb_stride;
            c_r = c[0]; c_g = c[1]; c_b = c[2];
            g = dw_in[first + i];
        }
        const float incl = warp_incl_prod(1.0f - alpha, lane);
        const float T_before = T * from_lane_below(incl, lane, 1.0f);
        const float w = T_before * alpha;
        // colour composited up to and including this sample, and the same for w g
        const float cum_r = acc_r + warp_incl_sum(w * c_r, lane), cum_g = acc_g + warp_incl_sum(w * c_g, lane);
        const float cum_b = acc_b + warp_incl_sum(w * c_b, lane), cum_wg = acc_wg + warp_incl_sum(w * g, lane);
        if (valid) {
            float gr = phi_r * w * c_r * (1.0f - c_r) * scale, gg = phi_g * w * c_g * (1.0f - c_g) * scale, gb = phi_b * w * c_b * (1.0f - c_b) * scale;
            gr = fmaxf(-65504.0f, fminf(65504.0f, gr)); gg = fmaxf(-65504.0f, fminf(65504.0f, gg)); gb = fmaxf(-65504.0f, fminf(65504.0f, gb));
            if (gr != gr || gg != gg || gb != gb) { gr = 0.0f; gg = 0.0f; gb = 0.0f; }
            if (GRAD8) {
                *reinterpret_cast<uint4*>(color_grad + (size_t)(first + i) * 8) = make_uint4(pack_half2(gr, gg), pack_half2(gb, 0.0f), 0u, 0u);
            } else {
                __half* o = color_grad + (size_t)(first + i) * 3;
                o[0] = __float2half(gr); o[1] = __float2half(gg); o[2] = __float2half(gb);
            }
            // d/d sigma_i of the colour loss: this sample's own term minus everything composited behind it
            const float keep = T_before * (1.0f - alpha);
            const float ds_r = keep * c_r - (fin_r - cum_r), ds_g = keep * c_g - (fin_g - cum_g), ds_b = keep * c_b - (fin_b - cum_b);
            float d = dt * (ds_r * phi_r + ds_g * phi_g + ds_b * phi_b);
            // ... and of the distortion / depth loss through the weights
            d += dt * (g * keep - (wg_total - cum_wg));
            d = d * sigma * scale;
            d = fmaxf(-65504.0f, fminf(65504.0f, d));
            if (d != d) d = 0.0f;
            dsigma_out[first + i] = d;
        }
        T *= __shfl_sync(FULL, incl, 31);
        acc_r = __shfl_sync(FULL, cum_r, 31); acc_g = __shfl_sync(FULL, cum_g, 31);
        acc_b = __shfl_sync(FULL, cum_b, 31); acc_wg = __shfl_sync(FULL, cum_wg, 31);
    }
}

}  // namespace nb

using namespace nb;

static unsigned warp_grid(int64_t rays) { return (unsigned)((rays * 32 + 255) / 256); }

extern "C" int nb_composite_infer(int64_t num_rays, uint32_t base, uint32_t rays_done, const uint32_t* d_ray_offsets,
                                  const uint32_t* d_num_steps, const float* d_t_sorted, const float* d_sigma, const float* d_rgb,
                                  int rgb_stride, const float* d_rgb_true, float* d_final_rgb, float* d_final_depth, float* d_phi,
                                  const float* bg_color3, void* stream) {
    if (!d_ray_offsets || !d_num_steps || !d_t_sorted || !d_sigma || !d_rgb || !d_final_rgb || !bg_color3 || num_rays < 0 ||
        num_rays > 0x3ffffff || rgb_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_infer: null pointer, bad ray count or rgb stride < 3");
    if (num_rays == 0) return NB_OK;
    composite_infer_kernel<<<warp_grid(num_rays), 256, 0, (cudaStream_t)stream>>>(
        (uint32_t)num_rays, base, d_ray_offsets + rays_done, d_num_steps, d_t_sorted, d_sigma, d_rgb, rgb_stride, d_rgb_true, d_final_rgb,
        d_final_depth, d_phi, make_float3(bg_color3[0], bg_color3[1], bg_color3[2]));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_composite_train(int64_t num_rays, uint32_t sample_base, const uint32_t* d_ray_offsets, const uint32_t* d_num_steps,
                                  const float* d_t_sorted, const float* d_sigma, const float* d_depth_prior, const float* d_sigma_prior,
                                  const float* d_rgb, int rgb_stride, const float* d_rgb_true, float* d_final_rgb, float* d_final_depth,
                                  float* d_phi, float* d_dw_out, float* d_weight_sum, float lambda_dist, float lambda_depth,
                                  const float* bg_color3, void* stream) {
    if (!d_ray_offsets || !d_num_steps || !d_t_sorted || !d_sigma || !d_rgb || !d_final_rgb || !d_dw_out || !d_weight_sum || !bg_color3 ||
        num_rays < 0 || num_rays > 0x3ffffff || rgb_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_train: null pointer, bad ray count or rgb stride < 3");
    if (num_rays == 0) return NB_OK;
    composite_train_kernel<<<warp_grid(num_rays), 256, 0, (cudaStream_t)stream>>>(
        (uint32_t)num_rays, sample_base, d_ray_offsets, d_num_steps, d_t_sorted, d_sigma, d_depth_prior, d_sigma_prior, d_rgb, rgb_stride,
        d_rgb_true, d_final_rgb, d_final_depth, d_phi, d_dw_out, d_weight_sum, lambda_dist, lambda_depth,
        make_float3(bg_color3[0], bg_color3[1], bg_color3[2]));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_color_grad(int64_t num_rays, uint32_t sample_base, const uint32_t* d_num_steps, const uint32_t* d_ray_offsets,
                             const float* d_t_sorted, const float* d_logit0, int logit_stride, const float* d_color_out, int color_stride,
                             const float* d_phi, const float* d_final_rgb, const float* d_dw_out, const float* d_weight_sum,
                             void* d_color_grad_h, int grad_stride, float* d_tmp_dsigma, float loss_scale, float density_bias,
                             uint32_t total_rays_batch, void* stream) {
    if (!d_num_steps || !d_ray_offsets || !d_t_sorted || !d_logit0 || logit_stride < 1 || !d_color_out || !d_phi || !d_final_rgb || !d_dw_out ||
        !d_weight_sum || !d_color_grad_h || !d_tmp_dsigma || num_rays < 0 || num_rays > 0x3ffffff || color_stride < 3)
        return nb_set_error(NB_ERR_INVALID, "nb_color_grad: null pointer, bad ray count or colour stride < 3");
    if (grad_stride != 3 && grad_stride != 8) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_color_grad: gradient row stride must be 3 or 8 halves");
    if (grad_stride == 8 && (reinterpret_cast<uintptr_t>(d_color_grad_h) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_color_grad: 8-wide gradient rows must be 16-byte aligned");
    if (total_rays_batch == 0) return nb_set_error(NB_ERR_INVALID, "nb_color_grad: total_rays_batch must be positive");
    if (num_rays == 0) return NB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (grad_stride == 8)
        loss_grad_kernel<true><<<warp_grid(num_rays), 256, 0, st>>>((uint32_t)num_rays, sample_base, d_num_steps, d_ray_offsets, d_t_sorted, d_logit0,
                                                                    logit_stride, d_color_out, color_stride, d_phi, d_final_rgb, d_dw_out,
                                                                    d_weight_sum, (__half*)d_color_grad_h, d_tmp_dsigma, loss_scale, density_bias,
                                                                    total_rays_batch);
    else
        loss_grad_kernel<false><<<warp_grid(num_rays), 256, 0, st>>>((uint32_t)num_rays, sample_base, d_num_steps, d_ray_offsets, d_t_sorted, d_logit0,
                                                                     logit_stride, d_color_out, color_stride, d_phi, d_final_rgb, d_dw_out,
                                                                     d_weight_sum, (__half*)d_color_grad_h, d_tmp_dsigma, loss_scale, density_bias,
                                                                     total_rays_batch);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_composite_round(uint32_t ray_begin, uint32_t ray_count, const uint32_t* d_num_steps, uint32_t* d_round_offsets,
                                  const float* d_t_rows, uint32_t round_begin, uint32_t round_width, const float* d_sigma, const float* d_rgb,
                                  int rgb_stride, float* d_transmittance, float* d_composited4, float* d_final_rgb, float* d_final_depth,
                                  const float* bg_color3, uint32_t next_width, const nb_scene_desc* scene, const float* d_rays_o,
                                  const float* d_rays_d, uint32_t capacity, uint32_t* d_next_counter, uint64_t* d_emitted_total,
                                  uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream) {
    if (!d_num_steps || !d_round_offsets || !d_t_rows || !d_sigma || !d_rgb || !d_transmittance || !d_composited4 || !d_final_rgb ||
        !bg_color3 || rgb_stride < 3 || round_width == 0)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_round: null pointer, empty round or rgb stride < 3");
    if (reinterpret_cast<uintptr_t>(d_composited4) & 15u)
        return nb_set_error(NB_ERR_INVALID, "nb_composite_round: the composited state must be 16-byte aligned");
    if (ray_count > 0x3ffffffu) return nb_set_error(NB_ERR_INVALID, "nb_composite_round: too many rays");
    float3 lo = make_float3(0.f, 0.f, 0.f), hi = make_float3(1.f, 1.f, 1.f);
    if (next_width > 0) {
        if (!scene || !d_rays_o || !d_rays_d || !d_next_counter || !d_ray_idx_out || !d_pos4_out)
            return nb_set_error(NB_ERR_INVALID, "nb_composite_round: the next round's copy-out needs the scene, the rays, a counter and the sample arrays");
        if (reinterpret_cast<uintptr_t>(d_pos4_out) & 15u)
            return nb_set_error(NB_ERR_INVALID, "nb_composite_round: positions must be 16-byte aligned");
        if ((uint64_t)round_begin + round_width >= (uint64_t)nb_march_row_stride())
            return nb_set_error(NB_ERR_INVALID, "nb_composite_round: the next round must lie inside a row");
        lo = make_float3(scene->aabb_min[0], scene->aabb_min[1], scene->aabb_min[2]);
        hi = make_float3(scene->aabb_max[0], scene->aabb_max[1], scene->aabb_max[2]);
    }
    if (ray_count == 0) return NB_OK;
    composite_round_kernel<<<warp_grid(ray_count), 256, 0, (cudaStream_t)stream>>>(
        ray_begin, ray_count, d_num_steps, d_round_offsets, d_t_rows, (uint32_t)nb_march_row_stride(), round_begin, round_width, d_sigma, d_rgb,
        rgb_stride, d_transmittance, (float4*)d_composited4, d_final_rgb, d_final_depth, make_float3(bg_color3[0], bg_color3[1], bg_color3[2]),
        next_width, lo, hi, (const float3*)d_rays_o, (const float3*)d_rays_d, capacity, d_next_counter, (unsigned long long*)d_emitted_total,
        d_ray_idx_out, (float4*)d_pos4_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
