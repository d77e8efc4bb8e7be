// Per-sample glue between the density and the colour network.
//
// nb_sh_gather replaces compute_SH_gather (modules/NeRF/otherKernels.cu:156-273): clamps the 16 density
// logits to +-64 (NaN -> 0), sigma = expf(min(logit0 - bias, 8)), evaluates the 16 real spherical
// harmonics of the sample's ray direction and packs logits ++ SH as the colour network's fp16 input.
// nb_density_grad replaces compute_density_grad (otherKernels.cu:497-562).
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__device__ __forceinline__ float sanitize_logit(float v) {
    v = fmaxf(-64.0f, fminf(64.0f, v));
    return (v != v) ? 0.0f : v;
}

__global__ void __launch_bounds__(256) sh_gather_kernel(const float* __restrict__ dirs3, const uint32_t* __restrict__ ray_indices,
                                                        int64_t offset, int64_t n, float density_bias,
                                                        const float* __restrict__ density_out, __half* __restrict__ color_in,
                                                        float* __restrict__ sigma_out) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float* dp = dirs3 + 3 * (int64_t)ray_indices[idx + offset];
    float x = dp[0], y = dp[1], z = dp[2];
    float x2 = x * x, y2 = y * y, z2 = z * z;
    float sh[16];
    sh[0] = 0.28209479f;
    sh[1] = -0.48860251f * y;
    sh[2] = 0.48860251f * z;
    sh[3] = -0.48860251f * x;
    sh[4] = 1.09254843f * x * y;
    sh[5] = -1.09254843f * y * z;
    sh[6] = 0.31539156f * (3.0f * z2 - 1.0f);
    sh[7] = -1.09254843f * x * z;
    sh[8] = 0.54627421f * (x2 - y2);
    sh[9] = -0.59004359f * y * (3.0f * x2 - y2);
    sh[10] = 2.89061144f * x * y * z;
    sh[11] = -0.45704580f * y * (5.0f * z2 - 1.0f);
    sh[12] = 0.37317633f * z * (5.0f * z2 - 3.0f);
    sh[13] = -0.45704580f * x * (5.0f * z2 - 1.0f);
    sh[14] = 1.44530572f * z * (x2 - y2);
    sh[15] = -0.59004359f * x * (x2 - 3.0f * y2);

    const float4* dv = reinterpret_cast<const float4*>(density_out + idx * 16);
    float lg[16];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        float4 v = dv[q];
        lg[4 * q + 0] = sanitize_logit(v.x); lg[4 * q + 1] = sanitize_logit(v.y);
        lg[4 * q + 2] = sanitize_logit(v.z); lg[4 * q + 3] = sanitize_logit(v.w);
    }
    sigma_out[idx] = expf(fminf(lg[0] - density_bias, 8.0f));
    uint4* dst = reinterpret_cast<uint4*>(color_in + idx * 32);
    uint4 o;
    o = make_uint4(pack_half2(lg[0], lg[1]), pack_half2(lg[2], lg[3]), pack_half2(lg[4], lg[5]), pack_half2(lg[6], lg[7]));
    st_cs_v4(&dst[0], o);
    o = make_uint4(pack_half2(lg[8], lg[9]), pack_half2(lg[10], lg[11]), pack_half2(lg[12], lg[13]), pack_half2(lg[14], lg[15]));
    st_cs_v4(&dst[1], o);
    o = make_uint4(pack_half2(sh[0], sh[1]), pack_half2(sh[2], sh[3]), pack_half2(sh[4], sh[5]), pack_half2(sh[6], sh[7]));
    st_cs_v4(&dst[2], o);
    o = make_uint4(pack_half2(sh[8], sh[9]), pack_half2(sh[10], sh[11]), pack_half2(sh[12], sh[13]), pack_half2(sh[14], sh[15]));
    st_cs_v4(&dst[3], o);
}

__device__ __forceinline__ uint32_t sanitize_pair(uint32_t v, float add_lo) {
    float2 f = unpack_half2(v);
    f.x += add_lo;
    f.x = fmaxf(-65504.0f, fminf(65504.0f, f.x));
    if (f.x != f.x) f.x = 0.0f;
    f.y = fmaxf(-65504.0f, fminf(65504.0f, f.y));
    if (f.y != f.y) f.y = 0.0f;
    return pack_half2(f.x, f.y);
}

__global__ void __launch_bounds__(256) density_grad_kernel(int64_t n, const float* __restrict__ tmp_dsigma,
                                                           const __half* __restrict__ color_dx, __half* __restrict__ density_grad) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint4* src = reinterpret_cast<const uint4*>(color_dx + i * 32);
    uint4 a = src[0], b = src[1];
    float ds = tmp_dsigma != nullptr ? tmp_dsigma[i] : 0.0f;
    a.x = sanitize_pair(a.x, ds); a.y = sanitize_pair(a.y, 0.f); a.z = sanitize_pair(a.z, 0.f); a.w = sanitize_pair(a.w, 0.f);
    b.x = sanitize_pair(b.x, 0.f); b.y = sanitize_pair(b.y, 0.f); b.z = sanitize_pair(b.z, 0.f); b.w = sanitize_pair(b.w, 0.f);
    uint4* dst = reinterpret_cast<uint4*>(density_grad + i * 16);
    st_cs_v4(&dst[0], a);
    st_cs_v4(&dst[1], b);
}

// Pinhole rays of a camera-to-world matrix, pixel (first_pixel + idx).  generate_custom_rays_kernel,
// modules/NeRF/NerfTrainer.cu:25-47; the pixel offset lets ranks render disjoint tile ranges of one frame.
// tile == 0: pixels [first_pixel, first_pixel + count).  tile > 0: ray i belongs to the (i / tile)-th of the tiles
// first_tile, first_tile + tile_stride, ... (tile pixels each) - the tiles one rank of a pixel-sharded frame renders.
__global__ void __launch_bounds__(256) generate_rays_kernel(int width, int height, float focal, float c00, float c01, float c02, float c03,
                                                            float c10, float c11, float c12, float c13, float c20, float c21, float c22,
                                                            float c23, int64_t first_pixel, int64_t count, int64_t tile, int64_t tile_stride,
                                                            float3* __restrict__ rays_o, float3* __restrict__ rays_d) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    int64_t idx = first_pixel + i;
    if (tile > 0) idx = (first_pixel + (i / tile) * tile_stride) * tile + i % tile;  // first_pixel holds the first tile here
    int px = (int)(idx % width);
    int py = (int)(idx / width);
    float dx = (px - width * 0.5f) / focal;
    float dy = -(py - height * 0.5f) / focal;
    float dz = -1.0f;
    float inv = rsqrtf(dx * dx + dy * dy + dz * dz);
    dx *= inv; dy *= inv; dz *= inv;
    rays_o[i] = make_float3(c03, c13, c23);
    rays_d[i] = make_float3(c00 * dx + c01 * dy + c02 * dz, c10 * dx + c11 * dy + c12 * dz, c20 * dx + c21 * dy + c22 * dz);
}

// Sum over rays of the mean squared colour error (mse_kernel, modules/NeRF/NerfTrainer.cu:15-23), one atomic per block.
__global__ void __launch_bounds__(256) mse_rays_kernel(const float* __restrict__ pred, const float* __restrict__ target,
                                                       float* __restrict__ loss_out, int64_t n) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    float v = 0.f;
    if (idx < n) {
        float r = pred[idx * 3 + 0] - target[idx * 3 + 0];
        float g = pred[idx * 3 + 1] - target[idx * 3 + 1];
        float b = pred[idx * 3 + 2] - target[idx * 3 + 2];
        v = (r * r + g * g + b * b) / 3.0f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    __shared__ float ws[8];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int k = 0; k < 8; k++) s += ws[k];
        atomicAdd(loss_out, s);
    }
}

// Samples as they travel from the host - position float3, target colour three halves - into the layouts the field
// kernels read: position float4 (w = 0), target eight halves (3 valid, 5 zero).  One thread per sample.
__global__ void __launch_bounds__(256) unpack_samples_kernel(const float* __restrict__ pos3, const __half* __restrict__ tgt3, int64_t n,
                                                             float4* __restrict__ pos4, uint4* __restrict__ tgt8) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (pos4 != nullptr) pos4[i] = make_float4(pos3[3 * i], pos3[3 * i + 1], pos3[3 * i + 2], 0.0f);
    if (tgt8 != nullptr) {
        const unsigned short* t = reinterpret_cast<const unsigned short*>(tgt3) + 3 * i;
        tgt8[i] = make_uint4((uint32_t)t[0] | ((uint32_t)t[1] << 16), (uint32_t)t[2], 0u, 0u);
    }
}

// Frame assembly of pixel-sharded rendering: pixel p of the frame belongs to tile p / tile, which rank (tile index %
// ranks) rendered as its (tile index / ranks)-th tile; blocks holds every rank's tiles back to back, rows_per_rank
// pixels per rank.  One float per thread (3 per pixel), coalesced on the frame side and within a tile on the block side.
__global__ void __launch_bounds__(256) undeal_tiles_kernel(const float* __restrict__ blocks, int ranks, int64_t rows_per_rank, int64_t tile,
                                                           int64_t num_pixels, float* __restrict__ frame) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_pixels * 3) return;
    const int64_t p = i / 3, c = i - 3 * p;
    const int64_t t = p / tile, within = p - t * tile;
    const int64_t rank = t % ranks, slot = t / ranks;
    frame[i] = blocks[(rank * rows_per_rank + slot * tile + within) * 3 + c];
}

}  // namespace nb

using namespace nb;

extern "C" int nb_undeal_tiles(const float* d_blocks, int ranks, int64_t rows_per_rank, int64_t tile, int64_t num_pixels, float* d_frame,
                               void* stream) {
    if (!d_blocks || !d_frame || ranks <= 0 || tile <= 0 || num_pixels < 0 || rows_per_rank < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_undeal_tiles: null pointer or bad tiling");
    const int64_t tiles = (num_pixels + tile - 1) / tile;
    if (((tiles + ranks - 1) / ranks) * tile > rows_per_rank)
        return nb_set_error(NB_ERR_INVALID, "nb_undeal_tiles: rows_per_rank is smaller than a rank's share of the frame");
    if (num_pixels == 0) return NB_OK;
    undeal_tiles_kernel<<<(unsigned)((num_pixels * 3 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_blocks, ranks, rows_per_rank, tile, num_pixels,
                                                                                                    d_frame);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_unpack_samples(const float* d_pos3, const void* d_target3_h, int64_t n, float* d_pos4, void* d_target8_h, void* stream) {
    if (n < 0 || (d_pos4 != nullptr && d_pos3 == nullptr) || (d_target8_h != nullptr && d_target3_h == nullptr))
        return nb_set_error(NB_ERR_INVALID, "nb_unpack_samples: an output without its input, or a negative count");
    if ((reinterpret_cast<uintptr_t>(d_pos4) & 15u) || (reinterpret_cast<uintptr_t>(d_target8_h) & 15u) || (reinterpret_cast<uintptr_t>(d_target3_h) & 1u) ||
        (reinterpret_cast<uintptr_t>(d_pos3) & 3u))
        return nb_set_error(NB_ERR_INVALID, "nb_unpack_samples: misaligned device pointer");
    if (n == 0 || (d_pos4 == nullptr && d_target8_h == nullptr)) return NB_OK;
    unpack_samples_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_pos3, (const __half*)d_target3_h, n, (float4*)d_pos4,
                                                                                         (uint4*)d_target8_h);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_generate_rays(int width, int height, float focal, const float* c2w_3x4, int64_t first_pixel, int64_t count, float* d_rays_o,
                                float* d_rays_d, void* stream) {
    if (!c2w_3x4 || !d_rays_o || !d_rays_d || width <= 0 || height <= 0 || first_pixel < 0 || count < 0 ||
        first_pixel + count > (int64_t)width * height || !(focal > 0.f))
        return nb_set_error(NB_ERR_INVALID, "nb_generate_rays: null pointer or pixel range outside the frame");
    if (count == 0) return NB_OK;
    const float* c = c2w_3x4;
    generate_rays_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>(width, height, focal, c[0], c[1], c[2], c[3], c[4], c[5],
                                                                                            c[6], c[7], c[8], c[9], c[10], c[11], first_pixel,
                                                                                            count, 0, 0, (float3*)d_rays_o, (float3*)d_rays_d);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_generate_rays_tiled(int width, int height, float focal, const float* c2w_3x4, int64_t tile, int64_t first_tile,
                                      int64_t tile_stride, int64_t count, float* d_rays_o, float* d_rays_d, void* stream) {
    if (!c2w_3x4 || !d_rays_o || !d_rays_d || width <= 0 || height <= 0 || tile <= 0 || first_tile < 0 || tile_stride <= 0 || count < 0 ||
        !(focal > 0.f))
        return nb_set_error(NB_ERR_INVALID, "nb_generate_rays_tiled: null pointer or bad tiling");
    if (count == 0) return NB_OK;
    // the last ray's pixel must lie inside the frame
    const int64_t last = count - 1;
    if ((first_tile + (last / tile) * tile_stride) * tile + last % tile >= (int64_t)width * height)
        return nb_set_error(NB_ERR_INVALID, "nb_generate_rays_tiled: the tiles reach past the frame");
    const float* c = c2w_3x4;
    generate_rays_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>(width, height, focal, c[0], c[1], c[2], c[3], c[4], c[5],
                                                                                            c[6], c[7], c[8], c[9], c[10], c[11], first_tile,
                                                                                            count, tile, tile_stride, (float3*)d_rays_o,
                                                                                            (float3*)d_rays_d);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_mse_rays(const float* d_pred3, const float* d_target3, float* d_loss_sum, int64_t n, void* stream) {
    if (!d_pred3 || !d_target3 || !d_loss_sum || n < 0) return nb_set_error(NB_ERR_INVALID, "nb_mse_rays: null pointer or negative count");
    if (n == 0) return NB_OK;
    mse_rays_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_pred3, d_target3, d_loss_sum, n);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_sh_gather(const float* d_dirs3, const uint32_t* d_ray_indices, int64_t offset, int64_t n, float density_bias,
                            const float* d_density_out, void* d_color_in_h, float* d_sigma, void* stream) {
    if (!d_dirs3 || !d_ray_indices || !d_density_out || !d_color_in_h || !d_sigma || n < 0 || offset < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_sh_gather: null pointer or negative count");
    if ((reinterpret_cast<uintptr_t>(d_density_out) & 15u) || (reinterpret_cast<uintptr_t>(d_color_in_h) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_sh_gather: density output and colour input must be 16-byte aligned");
    if (n == 0) return NB_OK;
    sh_gather_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_dirs3, d_ray_indices, offset, n, density_bias,
                                                                                    d_density_out, (__half*)d_color_in_h, d_sigma);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_density_grad(int64_t n, const float* d_tmp_dsigma, const void* d_color_dx_h, void* d_density_grad_h, void* stream) {
    if (!d_color_dx_h || !d_density_grad_h || n < 0) return nb_set_error(NB_ERR_INVALID, "nb_density_grad: null pointer or negative count");
    if ((reinterpret_cast<uintptr_t>(d_color_dx_h) & 15u) || (reinterpret_cast<uintptr_t>(d_density_grad_h) & 15u))
        return nb_set_error(NB_ERR_INVALID, "nb_density_grad: buffers must be 16-byte aligned");
    if (n == 0) return NB_OK;
    density_grad_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(n, d_tmp_dsigma, (const __half*)d_color_dx_h,
                                                                                       (__half*)d_density_grad_h);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
