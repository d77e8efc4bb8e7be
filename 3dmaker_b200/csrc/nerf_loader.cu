// Training / validation ray batches from an image set resident in HBM.
//
// Replaces fetchRayChunkStreamingKernel and DataLoader::fetchRayChunk (modules/NeRF/DataLoader.cu:542-690): per output
// slot a PCG hash picks an image (never a held-out one when hold-out is on) and a pixel, or slots walk the pixels in
// order; an optional fraction of the slots is redirected to depth-prior records; the pinhole ray of the pixel is
// generated from the image's camera-to-world matrix and the RGBA pixel is blended over the background colour.
// The reference keeps the images in pinned host memory mapped into the device and reads them over PCIe in this
// kernel; here the set is a device buffer (180 GB of HBM hold tens of thousands of 800 x 800 RGBA frames), so a
// training step no longer waits for the bus.  The selection arithmetic is integer and identical slot for slot.
#include <atomic>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

// PCG output function on a 32-bit LCG state (the RXS-M-XS variant the reference uses, DataLoader.cu:542-546)
__host__ __device__ inline uint32_t pcg_hash(uint32_t input) {
    const uint32_t state = input * 747796405u + 2891336453u;
    const uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}

struct LoaderArgs {
    int offset, size, total_rays;
    uint32_t seed;
    int randomize;
    int width, height;
    float focal;
    const float* transforms;      // [images][16] row-major camera-to-world
    const uint8_t* images_rgba;   // [images][height][width][4]
    float3* rays_o;
    float3* rays_d;
    float* rgb;                   // [size][3]
    float* prior_depth;           // [size], -1 where the slot is a plain colour ray (nullable)
    float* prior_sigma;           // nullable
    const int* rec_frame;         // depth-prior records (nullable when num_records == 0)
    const float *rec_u, *rec_v, *rec_depth, *rec_sigma;
    uint32_t num_records;
    float dense_fraction, uv_scale_x, uv_scale_y;
    float3 bg;
    int holdout_every;
};

__global__ void __launch_bounds__(256) fetch_ray_chunk_kernel(const LoaderArgs a) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.size) return;
    const int pixels = a.width * a.height;
    uint32_t pick;  // index of the chosen pixel in the whole set
    if (a.randomize) {
        const uint32_t rnd = pcg_hash((uint32_t)(a.offset + idx) + a.seed);
        pick = rnd % (uint32_t)a.total_rays;
        if (a.holdout_every >= 2) {
            // images 0, N, 2N, ... are held out: draw among the others, then a pixel from a second hash
            const int num_imgs = a.total_rays / pixels;
            const int num_train = num_imgs - (num_imgs + a.holdout_every - 1) / a.holdout_every;
            if (num_train >= 1) {
                const int slot = (int)(rnd % (uint32_t)num_train);
                const int img = (slot / (a.holdout_every - 1)) * a.holdout_every + slot % (a.holdout_every - 1) + 1;
                pick = (uint32_t)img * (uint32_t)pixels + pcg_hash(rnd) % (uint32_t)pixels;
            }
        }
    } else {
        pick = (uint32_t)(a.offset + idx) % (uint32_t)a.total_rays;
    }
    int img = (int)(pick / (uint32_t)pixels);
    const int pix = (int)(pick % (uint32_t)pixels);
    float px = (float)(pix % a.width), py = (float)(pix / a.width);

    // depth-prior slots: with probability dense_fraction the slot becomes a ray through a prior's keypoint
    float out_depth = -1.0f, out_sigma = -1.0f;
    if (a.randomize && a.dense_fraction > 0.0f && a.num_records > 0) {
        const uint32_t hsel = pcg_hash((uint32_t)(idx + 0x9E3779B9u) ^ (a.seed * 2654435761u));
        if (hsel * (1.0f / 4294967296.0f) < a.dense_fraction) {
            const uint32_t r = pcg_hash(hsel) % a.num_records;
            const int f = a.rec_frame[r];
            if (!(a.holdout_every >= 2 && (f % a.holdout_every == 0))) {
                img = f;
                px = a.rec_u[r] * a.uv_scale_x;
                py = a.rec_v[r] * a.uv_scale_y;
                out_depth = a.rec_depth[r];
                out_sigma = a.rec_sigma[r];
                const int xi = min(max((int)(px + 0.5f), 0), a.width - 1), yi = min(max((int)(py + 0.5f), 0), a.height - 1);
                pick = (uint32_t)img * (uint32_t)pixels + (uint32_t)(yi * a.width + xi);
            }
        }
    }

    float dx = (px - a.width * 0.5f) / a.focal, dy = -(py - a.height * 0.5f) / a.focal, dz = -1.0f;
    const float inv = rsqrtf(dx * dx + dy * dy + dz * dz);
    dx *= inv; dy *= inv; dz *= inv;
    const float* m = a.transforms + (size_t)img * 16;
    a.rays_o[idx] = make_float3(m[3], m[7], m[11]);
    a.rays_d[idx] = make_float3(m[0] * dx + m[1] * dy + m[2] * dz, m[4] * dx + m[5] * dy + m[6] * dz, m[8] * dx + m[9] * dy + m[10] * dz);

    const uchar4 c = *reinterpret_cast<const uchar4*>(a.images_rgba + (size_t)pick * 4);
    const float fa = c.w / 255.0f;
    a.rgb[idx * 3 + 0] = (c.x / 255.0f) * fa + a.bg.x * (1.0f - fa);
    a.rgb[idx * 3 + 1] = (c.y / 255.0f) * fa + a.bg.y * (1.0f - fa);
    a.rgb[idx * 3 + 2] = (c.z / 255.0f) * fa + a.bg.z * (1.0f - fa);
    if (a.prior_depth != nullptr) a.prior_depth[idx] = out_depth;
    if (a.prior_sigma != nullptr) a.prior_sigma[idx] = out_sigma;
}

}  // namespace nb

extern "C" int nb_fetch_ray_chunk(const nb_image_set* set, int offset, int size, uint32_t seed, int randomize, const float* bg_color3,
                                  int holdout_every, float* d_rays_o, float* d_rays_d, float* d_rgb, float* d_prior_depth,
                                  float* d_prior_sigma, void* stream) {
    if (!set || !set->d_images_rgba || !set->d_transforms || !bg_color3 || !d_rays_o || !d_rays_d || !d_rgb)
        return nb_set_error(NB_ERR_INVALID, "nb_fetch_ray_chunk: null pointer");
    if (set->width <= 0 || set->height <= 0 || set->num_images <= 0 || !(set->focal > 0.0f) || size < 0 || offset < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_fetch_ray_chunk: bad image set geometry or chunk range");
    const int64_t total = (int64_t)set->num_images * set->width * set->height;
    if (total > 0x7fffffffLL) return nb_set_error(NB_ERR_LIMIT, "nb_fetch_ray_chunk: more than 2^31 - 1 pixels in the set");
    if (set->num_records > 0 && (!set->d_rec_frame || !set->d_rec_u || !set->d_rec_v || !set->d_rec_depth || !set->d_rec_sigma))
        return nb_set_error(NB_ERR_INVALID, "nb_fetch_ray_chunk: depth-prior records incomplete");
    if (reinterpret_cast<uintptr_t>(set->d_images_rgba) & 3u) return nb_set_error(NB_ERR_INVALID, "nb_fetch_ray_chunk: images must be 4-byte aligned");
    if (size == 0) return NB_OK;
    nb::LoaderArgs a{};
    a.offset = offset; a.size = size; a.total_rays = (int)total; a.seed = seed; a.randomize = randomize;
    a.width = set->width; a.height = set->height; a.focal = set->focal;
    a.transforms = set->d_transforms; a.images_rgba = set->d_images_rgba;
    a.rays_o = (float3*)d_rays_o; a.rays_d = (float3*)d_rays_d; a.rgb = d_rgb; a.prior_depth = d_prior_depth; a.prior_sigma = d_prior_sigma;
    a.rec_frame = set->d_rec_frame; a.rec_u = set->d_rec_u; a.rec_v = set->d_rec_v; a.rec_depth = set->d_rec_depth; a.rec_sigma = set->d_rec_sigma;
    a.num_records = set->num_records; a.dense_fraction = set->dense_fraction;
    a.uv_scale_x = set->prior_width > 0 ? (float)set->width / (float)set->prior_width : 1.0f;
    a.uv_scale_y = set->prior_height > 0 ? (float)set->height / (float)set->prior_height : 1.0f;
    a.bg = make_float3(bg_color3[0], bg_color3[1], bg_color3[2]);
    a.holdout_every = holdout_every;
    nb::fetch_ray_chunk_kernel<<<(unsigned)((size + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a);
    NB_CHECK_LAUNCH();
    nb::g_launch_count++;
    return NB_OK;
}
