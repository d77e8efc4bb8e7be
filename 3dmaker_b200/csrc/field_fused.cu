// The whole radiance field in two kernels.
//
// field_forward_kernel : positions -> hash encode -> density MLP -> clamp + SH -> colour MLP -> (sigma, logit, rgb)
// field_backward_kernel: (dL/drgb pre-sigmoid, dL/dsigma*sigma) -> colour MLP backward -> density-output gradient
//                        -> density MLP backward -> dL/d(encoding), with dW / db of both networks
//
// They replace, for the training and rendering loops of InstantNerf (modules/NeRF/InstantNerf.cu:436-459,506-561),
// the chain TinyMLPHashGrid::forward -> compute_SH_gather -> TinyMLP::forward and TinyMLP::backward ->
// compute_density_grad -> TinyMLPHashGrid::backward's network half.  Per sample the unfused chain moves about
// 1.2 KB through HBM (density output, colour input, three saved hidden activations, dX, ...); here the forward
// writes 64 B of encoded features (the only thing worth saving: it cost 128 gathers) plus 24 B of results, and
// the backward re-derives every activation from those 64 B inside the CTA.  Hidden activations never leave the
// SM in either direction; weights of both networks stay in shared memory.
//
// Arithmetic is the same as in the unfused kernels (same fp16 rounding points), so the two paths agree to the
// last bit of every fp16 intermediate; only the fp32 summation order of dW differs.
#include <atomic>

#include "hashgrid_core.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__device__ __forceinline__ float sanitize_logit_f(float v) {
    v = fmaxf(-64.0f, fminf(64.0f, v));
    return (v != v) ? 0.0f : v;
}

// The four SH coefficients (bands 0..3, constants of modules/NeRF/otherKernels.cu:182-200) that lane column-pair t
// needs: indices 2t, 2t+1 (lo) and 8+2t, 9+2t (hi).
__device__ __forceinline__ void sh_quad(float x, float y, float z, int t, float& lo0, float& lo1, float& hi0, float& hi1) {
    float x2 = x * x, y2 = y * y, z2 = z * z;
    float sh0 = 0.28209479f;
    float sh1 = -0.48860251f * y;
    float sh2 = 0.48860251f * z;
    float sh3 = -0.48860251f * x;
    float sh4 = 1.09254843f * x * y;
    float sh5 = -1.09254843f * y * z;
    float sh6 = 0.31539156f * (3.0f * z2 - 1.0f);
    float sh7 = -1.09254843f * x * z;
    float sh8 = 0.54627421f * (x2 - y2);
    float sh9 = -0.59004359f * y * (3.0f * x2 - y2);
    float sh10 = 2.89061144f * x * y * z;
    float sh11 = -0.45704580f * y * (5.0f * z2 - 1.0f);
    float sh12 = 0.37317633f * z * (5.0f * z2 - 3.0f);
    float sh13 = -0.45704580f * x * (5.0f * z2 - 1.0f);
    float sh14 = 1.44530572f * z * (x2 - y2);
    float sh15 = -0.59004359f * x * (x2 - 3.0f * y2);
    lo0 = t == 0 ? sh0 : (t == 1 ? sh2 : (t == 2 ? sh4 : sh6));
    lo1 = t == 0 ? sh1 : (t == 1 ? sh3 : (t == 2 ? sh5 : sh7));
    hi0 = t == 0 ? sh8 : (t == 1 ? sh10 : (t == 2 ? sh12 : sh14));
    hi1 = t == 0 ? sh9 : (t == 1 ? sh11 : (t == 2 ? sh13 : sh15));
}

struct FieldIO {
    const float* pos4;        // [n] float4
    const uint32_t* table2;   // fp16 feature pairs
    const float* dirs3;       // float3 per ray
    const uint32_t* ray_idx;  // sample -> ray (nullable: sample i uses direction i)
    int64_t ray_idx_offset;
    const __half* Wd; const float* bd;  // density network
    const __half* Wc; const float* bc;  // colour network
    int64_t n;
    float density_bias;
};

// Colour-network input fragments of the warp's 16 rows from the density output fragments (16 logits) and the
// ray directions: k chunk 0 = clamped logits, k chunk 1 = SH.  Also hands back sigma / raw logit of the rows
// (valid in lanes with t == 0).
__device__ __forceinline__ void build_color_input(const float (&dout)[2][4], const FieldIO& io, int64_t row0, int lane, uint32_t (&a)[2][4],
                                                  float& raw0, float& raw1) {
    const int g = lane >> 2, t = lane & 3;
    raw0 = dout[0][0]; raw1 = dout[0][2];  // column 0 of rows g and g+8 (lanes with t == 0)
    a[0][0] = pack_half2(sanitize_logit_f(dout[0][0]), sanitize_logit_f(dout[0][1]));
    a[0][1] = pack_half2(sanitize_logit_f(dout[0][2]), sanitize_logit_f(dout[0][3]));
    a[0][2] = pack_half2(sanitize_logit_f(dout[1][0]), sanitize_logit_f(dout[1][1]));
    a[0][3] = pack_half2(sanitize_logit_f(dout[1][2]), sanitize_logit_f(dout[1][3]));
    float lo0, lo1, hi0, hi1;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        int64_t r = row0 + g + 8 * h;
        if (r >= io.n) r = io.n - 1;
        int64_t ray = io.ray_idx ? (int64_t)io.ray_idx[r + io.ray_idx_offset] : r;
        const float* dp = io.dirs3 + 3 * ray;
        sh_quad(dp[0], dp[1], dp[2], t, lo0, lo1, hi0, hi1);
        a[1][h] = pack_half2(lo0, lo1);
        a[1][2 + h] = pack_half2(hi0, hi1);
    }
}

template <class DS, class CS>
struct FieldSmem {
    static constexpr int ENC_STRIDE = DS::K0 + 8;
    static constexpr size_t fwd_bytes() {
        return (size_t)DS::SW_TOTAL * 2 + (size_t)CS::SW_TOTAL * 2 + (size_t)(DS::B_TOTAL + CS::B_TOTAL) * 4 + (size_t)TILE_ROWS * ENC_STRIDE * 2;
    }
};

template <class DS, class CS>
__global__ void __launch_bounds__(CTA_THREADS) field_forward_kernel(const __grid_constant__ GridParams gp, FieldIO io, __half* __restrict__ enc_save,
                                                                    float* __restrict__ sigma_out, float* __restrict__ logit_out,
                                                                    float* __restrict__ rgb_out, int rgb_stride) {
    static_assert(DS::OUT == 16 && CS::K0 == 32, "the colour network takes 16 density features and 16 SH coefficients");
    using FS = FieldSmem<DS, CS>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sWd = reinterpret_cast<__half*>(smem_raw);
    __half* sWc = sWd + DS::SW_TOTAL;
    float* sBd = reinterpret_cast<float*>(sWc + CS::SW_TOTAL);
    float* sBc = sBd + DS::B_TOTAL;
    __half* tile = reinterpret_cast<__half*>(sBc + CS::B_TOTAL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    load_weights_to_smem<DS>(io.Wd, io.bd, sWd, sBd, tid);
    load_weights_to_smem<CS>(io.Wc, io.bc, sWc, sBc, tid);
    cp_async_commit();
    const int64_t row_base = (int64_t)blockIdx.x * TILE_ROWS;
    encode_tile<FS::ENC_STRIDE>(gp, io.pos4, io.table2, row_base, io.n, tile, tid);
    cp_async_wait_all();
    __syncthreads();
    if (enc_save != nullptr) store_enc_tile<FS::ENC_STRIDE>(tile, enc_save, gp.L, row_base, io.n, tid);

    const int64_t row0 = row_base + warp * 16;
    if (row0 >= io.n) return;
    // density network, output kept in registers
    uint32_t a[DS::K0 / 16][4];
#pragma unroll
    for (int kc = 0; kc < DS::K0 / 16; kc++) {
        int q = lane >> 3, r = lane & 7;
        ldmatrix_x4(a[kc], &tile[(warp * 16 + r + (q & 1) * 8) * FS::ENC_STRIDE + 16 * kc + (q >> 1) * 8]);
    }
    FwdCtx dx{};
    dx.sW = sWd; dx.sBias = sBd; dx.row0 = row0; dx.n = io.n; dx.lane = lane;
    float dout[2][4];
    forward_layers<DS, 0, 0, true>(a, dx, dout);
    // clamp, sigma, SH -> colour input fragments
    uint32_t ca[2][4];
    float raw0, raw1;
    build_color_input(dout, io, row0, lane, ca, raw0, raw1);
    if (t == 0) {
        int64_t r0 = row0 + g, r1 = r0 + 8;
        if (r0 < io.n) {
            if (logit_out) logit_out[r0] = raw0;
            if (sigma_out) sigma_out[r0] = expf(fminf(sanitize_logit_f(raw0) - io.density_bias, 8.0f));
        }
        if (r1 < io.n) {
            if (logit_out) logit_out[r1] = raw1;
            if (sigma_out) sigma_out[r1] = expf(fminf(sanitize_logit_f(raw1) - io.density_bias, 8.0f));
        }
    }
    // colour network, sigmoid output, rgb (+ the padding column) written rgb_stride floats apart
    FwdCtx cx{};
    cx.sW = sWc; cx.sBias = sBc; cx.row0 = row0; cx.n = io.n; cx.lane = lane;
    cx.out = rgb_out; cx.out_stride = rgb_stride; cx.out_valid = rgb_stride < 8 ? 4 : 8;
    forward_layers<CS, 0, 1, false>(ca, cx);
}

}  // namespace nb
