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
#include <algorithm>
#include <atomic>

#include "hashgrid_core.cuh"
#include "field_backward_tc.cuh"

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
    const uint32_t* count;  // nullable: sample count known only on the device (at most n)
};

// Colour-network input fragments of the warp's 16 rows from the density output fragments (16 logits) and the
// ray directions: k chunk 0 = clamped logits, k chunk 1 = SH.  Also hands back sigma / raw logit of the rows
// (valid in lanes with t == 0).
// perm (nullable): row r of the tile order is sample perm[r].
__device__ __forceinline__ void build_color_input(const float (&dout)[2][4], const FieldIO& io, int64_t row0, int lane, uint32_t (&a)[2][4],
                                                  float& raw0, float& raw1, const uint32_t* __restrict__ perm = nullptr) {
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
        if (perm != nullptr) r = (int64_t)perm[r];
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

// MSE loss against per-sample target colours, taken in the forward's epilogue (the arithmetic of mse_loss_grad_kernel,
// optim.cu, on the colour the kernel has in registers): grad[n][8] fp16 = dL/d(colour pre-activation) x loss scale,
// total += sum of squared differences.
struct FieldLossIO {
    const __half* target;   // [n][8] fp16, columns >= 3 ignored
    __half* grad;           // [n][8] fp16
    float* total;           // nullable
    float grad_scale;       // 2 / (n * 3) * loss scale
};

// The encoding of this rank's samples as the level owners delivered it (level_partition.cu): piece q holds the levels
// q, q + ranks, ... of every sample, level-major, `cap` samples per level.
struct FieldPiecesIO {
    const uint32_t* pieces;
    int ranks;
    int64_t cap;
};

// tile[r][2l .. 2l+1] = level l of row row_base + r, taken from the pieces (zero behind the last sample)
template <int TILE_STRIDE>
__device__ __forceinline__ void load_pieces_tile(const FieldPiecesIO& pio, int L, int64_t row_base, int64_t n, __half* tile, int tid) {
    const int own = L / pio.ranks;
    for (int idx = tid; idx < L * TILE_ROWS; idx += CTA_THREADS) {
        const int l = idx / TILE_ROWS, r = idx - l * TILE_ROWS;
        const int64_t row = row_base + r;
        const uint32_t v = row < n ? __ldg(pio.pieces + ((int64_t)(l % pio.ranks) * own + l / pio.ranks) * pio.cap + row) : 0u;
        *reinterpret_cast<uint32_t*>(&tile[r * TILE_STRIDE + 2 * l]) = v;
    }
}

template <class DS, class CS, bool WITH_LOSS, bool FROM_PIECES = false>
__global__ void __launch_bounds__(CTA_THREADS) field_forward_kernel(const __grid_constant__ GridParams gp, FieldIO io, __half* __restrict__ enc_save,
                                                                    float* __restrict__ sigma_out, float* __restrict__ logit_out,
                                                                    float* __restrict__ rgb_out, int rgb_stride, FieldLossIO lio,
                                                                    FieldPiecesIO pio) {
    static_assert(DS::OUT == 16 && CS::K0 == 32, "the colour network takes 16 density features and 16 SH coefficients");
    using FS = FieldSmem<DS, CS>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sWd = reinterpret_cast<__half*>(smem_raw);
    __half* sWc = sWd + DS::SW_TOTAL;
    float* sBd = reinterpret_cast<float*>(sWc + CS::SW_TOTAL);
    float* sBc = sBd + DS::B_TOTAL;
    __half* tile = reinterpret_cast<__half*>(sBc + CS::B_TOTAL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    const int64_t row_base = (int64_t)blockIdx.x * TILE_ROWS;
    if (io.count != nullptr) {
        // the launch covers an upper bound of the samples; tiles behind the count a kernel before this one left leave at once
        const int64_t counted = (int64_t)__ldg(io.count);
        if (counted < io.n) io.n = counted;
        if (row_base >= io.n) return;
    }
    load_weights_to_smem<DS>(io.Wd, io.bd, sWd, sBd, tid);
    load_weights_to_smem<CS>(io.Wc, io.bc, sWc, sBc, tid);
    cp_async_commit();
    if constexpr (FROM_PIECES) load_pieces_tile<FS::ENC_STRIDE>(pio, gp.L, row_base, io.n, tile, tid);
    else encode_tile<FS::ENC_STRIDE>(gp, io.pos4, io.table2, row_base, io.n, tile, tid);
    cp_async_wait_all();
    __syncthreads();
    if (enc_save != nullptr) store_enc_tile<FS::ENC_STRIDE>(tile, enc_save, gp.L, row_base, io.n, tid);

    const int64_t row0 = row_base + warp * 16;
    if constexpr (!WITH_LOSS) {
        if (row0 >= io.n) return;
    }
    float sq = 0.f;   // WITH_LOSS: this thread's share of the squared differences
    if (!WITH_LOSS || row0 < io.n) {
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
        if constexpr (!WITH_LOSS) {
            forward_layers<CS, 0, 1, false>(ca, cx);
        } else {
            float fin[1][4];
            forward_layers<CS, 0, 1, true>(ca, cx, fin);
            const int col = 2 * t;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int64_t r = row0 + g + 8 * h;
                if (r >= io.n) continue;
                const float px = fin[0][2 * h], py = fin[0][2 * h + 1];
                if (col < cx.out_valid) *reinterpret_cast<float2*>(&rgb_out[r * rgb_stride + col]) = make_float2(px, py);
                const float2 tg = __half22float2(*reinterpret_cast<const __half2*>(&lio.target[r * 8 + col]));
                const float dxv = (col < 3) ? (px - tg.x) : 0.0f;
                const float dyv = (col + 1 < 3) ? (py - tg.y) : 0.0f;
                sq += (dxv * dxv) + (dyv * dyv);
                float gx = dxv * lio.grad_scale, gy = dyv * lio.grad_scale;
                gx *= px * (1.0f - px);
                gy *= py * (1.0f - py);
                *reinterpret_cast<__half2*>(&lio.grad[r * 8 + col]) = __floats2half2_rn(gx, gy);
            }
        }
    }
    if constexpr (WITH_LOSS) {
        // one addition per CTA to the total; the tile is free by now, its first words carry the warps' sums
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_down_sync(0xffffffffu, sq, o);
        __syncthreads();
        float* warp_sums = reinterpret_cast<float*>(tile);
        if (lane == 0) warp_sums[warp] = sq;
        __syncthreads();
        if (tid == 0 && lio.total != nullptr) {
            float total = 0.f;
            for (int k = 0; k < CTA_THREADS / 32; k++) total += warp_sums[k];
            atomicAdd(lio.total, total);
        }
    }
}



// ---------------------------------------------------------------------------------------------
// forward with the coarse levels staged in shared memory
// ---------------------------------------------------------------------------------------------
// Same arithmetic and outputs as field_forward_kernel.  Differences: CTAs are persistent and walk over groups of
// FWD_GROUP_TILES consecutive tiles; per group the levels whose corner boxes fit are copied into shared memory once and
// gathered from there; the weights are staged once per CTA; rows may be visited through a permutation (perm[row] =
// sample), in which case the saved encoding is in ROW order (the backward visits the same rows) and every per-sample
// output lands at its sample's place.
constexpr int FWD_GROUP_TILES = 4;
constexpr int FWD_STAGE_CAP = 6144;   // entries of 4 bytes
constexpr int FWD_STAGE_LEVELS = 8;   // never look further than this many levels

template <class DS, class CS>
struct FieldStagedSmem {
    static constexpr int ENC_STRIDE = DS::K0 + 8;
    static constexpr size_t bytes() {
        return FieldSmem<DS, CS>::fwd_bytes() + (size_t)FWD_STAGE_CAP * 4 + sizeof(StagePlan) + 32;
    }
};

template <class DS, class CS>
__global__ void __launch_bounds__(CTA_THREADS) field_forward_staged_kernel(const __grid_constant__ GridParams gp, FieldIO io,
                                                                           const uint32_t* __restrict__ perm, __half* __restrict__ enc_save,
                                                                           float* __restrict__ sigma_out, float* __restrict__ logit_out,
                                                                           float* __restrict__ rgb_out, int rgb_stride, int stage_levels) {
    static_assert(DS::OUT == 16 && CS::K0 == 32 && CS::OUT == 8, "the colour network takes 16 density features and 16 SH coefficients");
    using FS = FieldSmem<DS, CS>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sWd = reinterpret_cast<__half*>(smem_raw);
    __half* sWc = sWd + DS::SW_TOTAL;
    float* sBd = reinterpret_cast<float*>(sWc + CS::SW_TOTAL);
    float* sBc = sBd + DS::B_TOTAL;
    __half* tile = reinterpret_cast<__half*>(sBc + CS::B_TOTAL);
    uint32_t* s_tab = reinterpret_cast<uint32_t*>(tile + TILE_ROWS * FS::ENC_STRIDE);
    StagePlan& plan = *reinterpret_cast<StagePlan*>(s_tab + FWD_STAGE_CAP);
    float* s_box = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(&plan) + sizeof(StagePlan));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    if (io.count != nullptr) {
        const int64_t counted = (int64_t)__ldg(io.count);
        if (counted < io.n) io.n = counted;
    }
    const int64_t group_rows = (int64_t)FWD_GROUP_TILES * TILE_ROWS;
    const int64_t groups = (io.n + group_rows - 1) / group_rows;
    if ((int64_t)blockIdx.x >= groups) return;
    load_weights_to_smem<DS>(io.Wd, io.bd, sWd, sBd, tid);
    load_weights_to_smem<CS>(io.Wc, io.bc, sWc, sBc, tid);
    cp_async_commit();
    cp_async_wait_all();

    for (int64_t grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        const int64_t group_base = grp * group_rows;
        // ---- which levels come from shared memory for this group, and their boxes ---------------------------------
        int staged = 0;
        if (stage_levels > 0) {
            plan_stage<false, CTA_THREADS>(gp, io.pos4, perm, group_base, (int)group_rows, io.n, FWD_STAGE_CAP, stage_levels, s_box, plan, tid,
                                           [] { __syncthreads(); });
            staged = plan.count;
        }
        for (int l = 0; l < staged; l++) {
            const uint32_t* tl = io.table2 + (size_t)l * gp.ls;
            const int N_l = __float2int_rd(gp.scales[l]);
            const bool dense = l < gp.dls;
            const int w = plan.w[l], wh = plan.wh[l], cnt = plan.whd[l], base = plan.base[l];
            const int ox = plan.ox[l], oy = plan.oy[l], oz = plan.oz[l];
            for (int e = tid; e < cnt; e += CTA_THREADS) {
                const int lz = e / wh, rem = e - lz * wh, ly = rem / w, lx = rem - ly * w;
                s_tab[base + e] = __ldg(tl + level_index(ox + lx, oy + ly, oz + lz, N_l, dense, gp.T));
            }
        }
        __syncthreads();

        for (int tl_i = 0; tl_i < FWD_GROUP_TILES; tl_i++) {
            const int64_t row_base = group_base + (int64_t)tl_i * TILE_ROWS;
            if (row_base >= io.n) break;
            // ---- encode: thread = (row, every other level), so staged and gathered levels split evenly over the halves ---
            {
                const int r = tid & (TILE_ROWS - 1), hsel = tid >> 7;
                const int64_t row = row_base + r;
                if (row < io.n) {
                    const int64_t smp = perm ? (int64_t)perm[row] : row;
                    const float4 p = ld_nc_f4(io.pos4 + smp * 4);
                    for (int li = hsel; li < gp.L; li += 4) {
                        // two levels at a time keeps 16 gathers in flight
                        const int la = li, lb = li + 2;
                        const bool has_b = lb < gp.L;
                        CornerBox ba, bb;
                        corner_box<false>(p.x, p.y, p.z, gp.scales[la], ba);
                        corner_box<false>(p.x, p.y, p.z, gp.scales[has_b ? lb : la], bb);
                        uint32_t fa[8], fb[8];
                        int loc[8];
                        if (la < staged && staged_corners(plan, la, ba, loc)) {
#pragma unroll
                            for (int k = 0; k < 8; k++) fa[k] = s_tab[loc[k]];
                        } else {
                            Corners c;
                            corners_from_box(ba, la < gp.dls, gp.T, c);
                            gather_corners(io.table2 + (size_t)la * gp.ls, c, gp.pair_ops != 0, fa);
                        }
                        if (has_b) {
                            if (lb < staged && staged_corners(plan, lb, bb, loc)) {
#pragma unroll
                                for (int k = 0; k < 8; k++) fb[k] = s_tab[loc[k]];
                            } else {
                                Corners c;
                                corners_from_box(bb, lb < gp.dls, gp.T, c);
                                gather_corners(io.table2 + (size_t)lb * gp.ls, c, gp.pair_ops != 0, fb);
                            }
                        }
                        Corners wa, wb;
                        wa.wx1 = ba.wx1; wa.wy1 = ba.wy1; wa.wz1 = ba.wz1;
                        wb.wx1 = bb.wx1; wb.wy1 = bb.wy1; wb.wz1 = bb.wz1;
                        float ka[8], kb[8];
                        corner_weights(wa, ka);
                        corner_weights(wb, kb);
                        *reinterpret_cast<uint32_t*>(&tile[r * FS::ENC_STRIDE + 2 * la]) = blend(fa, ka);
                        if (has_b) *reinterpret_cast<uint32_t*>(&tile[r * FS::ENC_STRIDE + 2 * lb]) = blend(fb, kb);
                    }
                } else {
                    for (int l = hsel; l < gp.L; l += 2) *reinterpret_cast<uint32_t*>(&tile[r * FS::ENC_STRIDE + 2 * l]) = 0u;
                }
            }
            __syncthreads();
            if (enc_save != nullptr) store_enc_tile<FS::ENC_STRIDE>(tile, enc_save, gp.L, row_base, io.n, tid);

            const int64_t row0 = row_base + warp * 16;
            if (row0 < io.n) {
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
                uint32_t ca[2][4];
                float raw0, raw1;
                build_color_input(dout, io, row0, lane, ca, raw0, raw1, perm);
                const int64_t r0 = row0 + g, r1 = r0 + 8;
                const int64_t s0 = (r0 < io.n) ? (perm ? (int64_t)perm[r0] : r0) : -1;
                const int64_t s1 = (r1 < io.n) ? (perm ? (int64_t)perm[r1] : r1) : -1;
                if (t == 0) {
                    if (s0 >= 0) {
                        if (logit_out) logit_out[s0] = raw0;
                        if (sigma_out) sigma_out[s0] = expf(fminf(sanitize_logit_f(raw0) - io.density_bias, 8.0f));
                    }
                    if (s1 >= 0) {
                        if (logit_out) logit_out[s1] = raw1;
                        if (sigma_out) sigma_out[s1] = expf(fminf(sanitize_logit_f(raw1) - io.density_bias, 8.0f));
                    }
                }
                FwdCtx cx{};
                cx.sW = sWc; cx.sBias = sBc; cx.row0 = row0; cx.n = io.n; cx.lane = lane;
                float fin[1][4];
                forward_layers<CS, 0, 1, true>(ca, cx, fin);
                // lane t holds columns 2t, 2t + 1 of rows g and g + 8: rgb and the padding column(s)
                const int col = 2 * t;
                if (col < (rgb_stride < 8 ? 4 : 8)) {
                    if (s0 >= 0) *reinterpret_cast<float2*>(&rgb_out[s0 * rgb_stride + col]) = make_float2(fin[0][0], fin[0][1]);
                    if (s1 >= 0) *reinterpret_cast<float2*>(&rgb_out[s1 * rgb_stride + col]) = make_float2(fin[0][2], fin[0][3]);
                }
            }
            __syncthreads();   // the next tile's encode overwrites the tile
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
// Block-level pieces; every tile involved has 128 rows.  "dZ" is the gradient tile (stride DZS halves), "A" the
// input-activation tile of the layer (stride AS halves).

__host__ __device__ constexpr int dw_tiles(int K, int NP) { return (NP / 16) * (K / 8); }
__host__ __device__ constexpr int dw_tpw(int K, int NP) { return (dw_tiles(K, NP) + 7) / 8; }

// dW (NP x K) += dZ^T x A in 16 x 8 register tiles.  Warp w owns the tpw consecutive tiles w*tpw .. w*tpw+tpw-1 of
// the row-major (mi, ni) tile grid; tpw divides the tiles of a row, so all of them share mi and one dZ^T fragment
// per 16-row step serves the whole group, and neighbouring ni pairs share one 4-matrix load of A.
template <int K, int NP, int DZS, int AS>
__device__ __forceinline__ void accumulate_dw(float (*acc)[4], const __half* sDZ, const __half* sA, int warp, int lane) {
    const int lq = lane >> 3, lr = lane & 7;
    constexpr int N8 = K / 8, TPW = dw_tpw(K, NP);
    static_assert(dw_tiles(K, NP) == 8 * TPW && N8 % TPW == 0 && (TPW == 1 || TPW % 2 == 0), "tile grid must split evenly over 8 warps");
    const int id0 = warp * TPW;
    const int mi = id0 / N8, ni0 = id0 % N8;
#pragma unroll
    for (int ks = 0; ks < TILE_ROWS / 16; ks++) {
        uint32_t a[4];
        // A operand = dZ^T: element (m, k) = sDZ[16ks + k][16mi + m]
        ldmatrix_x4_trans(a, &sDZ[(16 * ks + (lq >> 1) * 8 + lr) * DZS + 16 * mi + (lq & 1) * 8]);
        if constexpr (TPW == 1) {
            uint32_t b0, b1;
            // B operand = the layer input: element (k, nn) = sA[16ks + k][8ni + nn]
            ldmatrix_x2_trans(b0, b1, &sA[(16 * ks + (lq & 1) * 8 + lr) * AS + 8 * ni0]);
            mma_16816(acc[0], a, b0, b1);
        } else {
#pragma unroll
            for (int s = 0; s < TPW; s += 2) {
                uint32_t b[4];  // matrices: (k 0-7, ni), (k 8-15, ni), (k 0-7, ni+1), (k 8-15, ni+1)
                ldmatrix_x4_trans(b, &sA[(16 * ks + (lq & 1) * 8 + lr) * AS + 8 * (ni0 + s) + (lq >> 1) * 8]);
                mma_16816(acc[s], a, b[0], b[1]);
                mma_16816(acc[s + 1], a, b[2], b[3]);
            }
        }
    }
}

template <int K, int N, int NP>
__device__ __forceinline__ void flush_dw(const float (*acc)[4], float* __restrict__ dW, int warp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    constexpr int N8 = K / 8, TPW = dw_tpw(K, NP);
    const int id0 = warp * TPW;
    const int mi = id0 / N8, ni0 = id0 % N8;
#pragma unroll
    for (int s = 0; s < TPW; s++) {
        int m0 = 16 * mi + g, m1 = m0 + 8, nn = 8 * (ni0 + s) + 2 * t;
        if (m0 < N) red_add_v2(&dW[m0 * K + nn], acc[s][0], acc[s][1]);
        if (m1 < N) red_add_v2(&dW[m1 * K + nn], acc[s][2], acc[s][3]);
    }
}

template <int N, int DZS>
__device__ __forceinline__ void accumulate_db(float& db, const __half* sDZ, int tid) {
    constexpr int PARTS = CTA_THREADS / N;
    int col = tid % N, part = tid / N;
    float s = 0.f;
    for (int r = part; r < TILE_ROWS; r += PARTS) s += __half2float(sDZ[r * DZS + col]);
    db += s;
}

// dA[:, 0 .. KOUT) = dZ x W_l for the warp's 16 rows, rounded to fp16; MASK zeroes entries whose activation in
// sMask (the layer's input, this warp's rows) is not positive.
template <int K, int KOUT, int NP, int DZS, int AS, bool MASK>
__device__ __forceinline__ void compute_da(const __half* sWl, const __half* sDZ, const __half* sMask, int warp, int lane,
                                           uint32_t (&packed)[KOUT / 8][2]) {
    const int lq = lane >> 3, lr = lane & 7, g = lane >> 2, t = lane & 3;
    uint32_t a[NP / 16][4];
#pragma unroll
    for (int kc = 0; kc < NP / 16; kc++)
        ldmatrix_x4(a[kc], &sDZ[(16 * warp + lr + (lq & 1) * 8) * DZS + 16 * kc + (lq >> 1) * 8]);
#pragma unroll
    for (int j = 0; j < KOUT / 8; j++) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kc = 0; kc < NP / 16; kc++) {
            uint32_t b0, b1;
            ldmatrix_x2_trans(b0, b1, &sWl[(16 * kc + (lq & 1) * 8 + lr) * (K + 8) + 8 * j]);
            mma_16816(c, a[kc], b0, b1);
        }
        __half2 v0 = __floats2half2_rn(c[0], c[1]);  // row g
        __half2 v1 = __floats2half2_rn(c[2], c[3]);  // row g + 8
        if constexpr (MASK) {
            __half2 a0 = *reinterpret_cast<const __half2*>(&sMask[(16 * warp + g) * AS + 8 * j + 2 * t]);
            __half2 a1 = *reinterpret_cast<const __half2*>(&sMask[(16 * warp + g + 8) * AS + 8 * j + 2 * t]);
            const __half z = __float2half(0.f);
            if (!(__low2float(a0) > 0.f)) v0 = __halves2half2(z, __high2half(v0));
            if (!(__high2float(a0) > 0.f)) v0 = __halves2half2(__low2half(v0), z);
            if (!(__low2float(a1) > 0.f)) v1 = __halves2half2(z, __high2half(v1));
            if (!(__high2float(a1) > 0.f)) v1 = __halves2half2(__low2half(v1), z);
        }
        packed[j][0] = *reinterpret_cast<uint32_t*>(&v0);
        packed[j][1] = *reinterpret_cast<uint32_t*>(&v1);
    }
}

template <int KOUT, int DZS>
__device__ __forceinline__ void store_da(const uint32_t (&packed)[KOUT / 8][2], __half* sDZ, int warp, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int j = 0; j < KOUT / 8; j++) {
        *reinterpret_cast<uint32_t*>(&sDZ[(16 * warp + g) * DZS + 8 * j + 2 * t]) = packed[j][0];
        *reinterpret_cast<uint32_t*>(&sDZ[(16 * warp + g + 8) * DZS + 8 * j + 2 * t]) = packed[j][1];
    }
}

// fp16 pair + optional fp32 addend on the low half, clamped to the fp16 range, NaN -> 0 (compute_density_grad,
// modules/NeRF/otherKernels.cu:497-562)
__device__ __forceinline__ uint32_t sanitize_grad_pair(uint32_t v, float add_lo) {
    float2 f = unpack_half2(v);
    f.x += add_lo;
    f.x = fmaxf(-65504.0f, fminf(65504.0f, f.x));
    if (f.x != f.x) f.x = 0.0f;
    f.y = fmaxf(-65504.0f, fminf(65504.0f, f.y));
    if (f.y != f.y) f.y = 0.0f;
    return pack_half2(f.x, f.y);
}

struct FieldGradIO {
    const __half* enc;        // [n][K0] saved by the forward
    const __half* dcolor;     // [n][8] dL/d(colour pre-activation), channels 3..7 zero
    const float* dsigma;      // [n] dL/d(logit 0) through sigma, nullable
    float* dWd; float* dbd;   // density network gradients (accumulated)
    float* dWc; float* dbc;   // colour network gradients (accumulated)
    __half* denc;             // dL/d(encoding): the first denc_cols columns of every row, rows denc_cols halves apart
    int denc_cols;            // 32 = the full matrix; 4 * k = only the k levels the stand-alone scatter handles; 0 = nothing
    // gradient scatter done by this kernel for levels [scatter_begin, 16) when table_grads is set
    const float* pos4;
    float* table_grads;
    int scatter_begin;
    // level-partitioned step (level_partition.cu): dL/d(encoding) goes straight into the pieces for the levels' owners,
    // level l of sample i at pieces[((l % piece_ranks) * (L / piece_ranks) + l / piece_ranks) * piece_cap + i]
    uint32_t* pieces;
    int piece_ranks;
    int64_t piece_cap;
};

template <class DS, class CS>
struct FieldBwd {
    static_assert(DS::NL == 2 && CS::NL == 3 && DS::H == CS::H && DS::K0 == 32 && CS::K0 == 32 && DS::OUT == 16 && CS::OUT == 8,
                  "fused backward is written for the 32-H-16 density and 32-H-H-8 colour networks");
    static constexpr int H = DS::H;
    static constexpr int IS = 32 + 8;  // stride of the 32-wide tiles (encoding, colour input)
    static constexpr int HS = H + 8;   // stride of the H-wide tiles
    // register slots of the dW accumulators
    static constexpr int S_C2 = 0;
    static constexpr int S_C1 = S_C2 + dw_tpw(H, 16);
    static constexpr int S_C0 = S_C1 + dw_tpw(H, H);
    static constexpr int S_D1 = S_C0 + dw_tpw(32, H);
    static constexpr int S_D0 = S_D1 + dw_tpw(H, 16);
    static constexpr int SLOTS = S_D0 + dw_tpw(32, H);
    static constexpr size_t smem_bytes() {
        return (size_t)(DS::SW_TOTAL + CS::SW_TOTAL) * 2 + (size_t)(DS::B_TOTAL + CS::B_TOTAL) * 4 +
               (size_t)TILE_ROWS * (2 * IS + 3 * HS) * 2;
    }
};

template <class DS, class CS, bool GRAD_HALF>
__global__ void __launch_bounds__(CTA_THREADS, 2) field_backward_kernel(const __grid_constant__ GridParams gp, FieldIO io, FieldGradIO gio) {
    using FB = FieldBwd<DS, CS>;
    constexpr int H = FB::H, IS = FB::IS, HS = FB::HS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sWd = reinterpret_cast<__half*>(smem_raw);
    __half* sWc = sWd + DS::SW_TOTAL;
    float* sBd = reinterpret_cast<float*>(sWc + CS::SW_TOTAL);
    float* sBc = sBd + DS::B_TOTAL;
    __half* sE = reinterpret_cast<__half*>(sBc + CS::B_TOTAL);  // encoding            [128][IS]
    __half* sCI = sE + TILE_ROWS * IS;                          // colour input        [128][IS]
    __half* sC1 = sCI + TILE_ROWS * IS;                         // colour hidden 1, later density hidden [128][HS]
    __half* sC2 = sC1 + TILE_ROWS * HS;                         // colour hidden 2     [128][HS]
    __half* sDZ = sC2 + TILE_ROWS * HS;                         // gradient tile       [128][HS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    load_weights_to_smem<DS>(io.Wd, io.bd, sWd, sBd, tid);
    load_weights_to_smem<CS>(io.Wc, io.bc, sWc, sBc, tid);
    cp_async_commit();

    float acc[FB::SLOTS][4];
#pragma unroll
    for (int s = 0; s < FB::SLOTS; s++) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;
    float db_c2 = 0.f, db_c1 = 0.f, db_c0 = 0.f, db_d1 = 0.f, db_d0 = 0.f;

    const int64_t ntiles = (io.n + TILE_ROWS - 1) / TILE_ROWS;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t row_base = tile * TILE_ROWS;
        const int64_t row0 = row_base + 16 * warp;
        // ---- stage the encoding and the colour gradient (zero rows past n; columns 8..15 of dZ zero) -----------
        for (int c = tid; c < TILE_ROWS * 4; c += CTA_THREADS) {
            int r = c >> 2, c8 = c & 3;
            bool valid = row_base + r < io.n;
            cp_async16(&sE[r * IS + c8 * 8], valid ? &gio.enc[(row_base + r) * 32 + c8 * 8] : gio.enc, valid);
        }
        {
            int r = tid >> 1, c8 = tid & 1;
            bool valid = (row_base + r < io.n) && c8 == 0;
            cp_async16(&sDZ[r * HS + c8 * 8], valid ? &gio.dcolor[(row_base + r) * 8] : gio.dcolor, valid);
        }
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();

        // ---- re-derive the activations of the warp's 16 rows ------------------------------------------------------
        {
            uint32_t a0[2][4];
            load_frag_rows<32>(a0, sE + 16 * warp * IS, IS, lane);
            float c1[H / 8][4];
            layer_accumulate<32, H>(a0, sWd + DS::sw_off(0), sBd + DS::b_off(0), lane, c1);
            uint32_t d1[H / 16][4];
            relu_pack<H>(c1, d1);
            float dout[2][4];
            layer_accumulate<H, 16>(d1, sWd + DS::sw_off(1), sBd + DS::b_off(1), lane, dout);
            uint32_t ci[2][4];
            float raw0, raw1;
            build_color_input(dout, io, row0, lane, ci, raw0, raw1);
            store_frag_rows<32>(ci, sCI + 16 * warp * IS, IS, lane);
            float c2[H / 8][4];
            layer_accumulate<32, H>(ci, sWc + CS::sw_off(0), sBc + CS::b_off(0), lane, c2);
            uint32_t h1[H / 16][4];
            relu_pack<H>(c2, h1);
            store_frag_rows<H>(h1, sC1 + 16 * warp * HS, HS, lane);
            layer_accumulate<H, H>(h1, sWc + CS::sw_off(1), sBc + CS::b_off(1), lane, c2);
            relu_pack<H>(c2, h1);
            store_frag_rows<H>(h1, sC2 + 16 * warp * HS, HS, lane);
        }
        __syncthreads();

        // ---- colour layer 2: dZ = dcolor (8 valid of 16 columns), input C2 ---------------------------------------
        {
            accumulate_dw<H, 16, HS, HS>(&acc[FB::S_C2], sDZ, sC2, warp, lane);
            accumulate_db<8, HS>(db_c2, sDZ, tid);
            uint32_t pk[H / 8][2];
            compute_da<H, H, 16, HS, HS, true>(sWc + CS::sw_off(2), sDZ, sC2, warp, lane, pk);
            __syncthreads();
            store_da<H, HS>(pk, sDZ, warp, lane);
            __syncthreads();
        }
        // ---- colour layer 1: input C1 ------------------------------------------------------------------------------
        {
            accumulate_dw<H, H, HS, HS>(&acc[FB::S_C1], sDZ, sC1, warp, lane);
            accumulate_db<H, HS>(db_c1, sDZ, tid);
            uint32_t pk[H / 8][2];
            compute_da<H, H, H, HS, HS, true>(sWc + CS::sw_off(1), sDZ, sC1, warp, lane, pk);
            __syncthreads();
            store_da<H, HS>(pk, sDZ, warp, lane);
            __syncthreads();
        }
        // ---- colour layer 0: input CI; only the 16 density features carry a gradient further ----------------------
        {
            accumulate_dw<32, H, HS, IS>(&acc[FB::S_C0], sDZ, sCI, warp, lane);
            accumulate_db<H, HS>(db_c0, sDZ, tid);
            uint32_t pk[2][2];
            compute_da<32, 16, H, HS, IS, false>(sWc + CS::sw_off(0), sDZ, nullptr, warp, lane, pk);
            float ds0 = 0.f, ds1 = 0.f;
            if (t == 0 && gio.dsigma != nullptr) {
                if (row0 + g < io.n) ds0 = gio.dsigma[row0 + g];
                if (row0 + g + 8 < io.n) ds1 = gio.dsigma[row0 + g + 8];
            }
            pk[0][0] = sanitize_grad_pair(pk[0][0], ds0);
            pk[0][1] = sanitize_grad_pair(pk[0][1], ds1);
            pk[1][0] = sanitize_grad_pair(pk[1][0], 0.f);
            pk[1][1] = sanitize_grad_pair(pk[1][1], 0.f);
            // the density network's hidden activation, derived again into the tile colour hidden 1 no longer needs
            uint32_t a0[2][4];
            load_frag_rows<32>(a0, sE + 16 * warp * IS, IS, lane);
            float c1[H / 8][4];
            layer_accumulate<32, H>(a0, sWd + DS::sw_off(0), sBd + DS::b_off(0), lane, c1);
            uint32_t d1[H / 16][4];
            relu_pack<H>(c1, d1);
            __syncthreads();
            store_da<16, HS>(pk, sDZ, warp, lane);
            store_frag_rows<H>(d1, sC1 + 16 * warp * HS, HS, lane);
            __syncthreads();
        }
        // ---- density layer 1: dZ 16 wide, input D1 (in the C1 tile) -----------------------------------------------
        {
            accumulate_dw<H, 16, HS, HS>(&acc[FB::S_D1], sDZ, sC1, warp, lane);
            accumulate_db<16, HS>(db_d1, sDZ, tid);
            uint32_t pk[H / 8][2];
            compute_da<H, H, 16, HS, HS, true>(sWd + DS::sw_off(1), sDZ, sC1, warp, lane, pk);
            __syncthreads();
            store_da<H, HS>(pk, sDZ, warp, lane);
            __syncthreads();
        }
        // ---- density layer 0: input E; dA is the gradient of the encoding -----------------------------------------
        {
            accumulate_dw<32, H, HS, IS>(&acc[FB::S_D0], sDZ, sE, warp, lane);
            accumulate_db<H, HS>(db_d0, sDZ, tid);
            uint32_t pk[4][2];
            compute_da<32, 32, H, HS, IS, false>(sWd + DS::sw_off(0), sDZ, nullptr, warp, lane, pk);
            __syncthreads();
            store_da<32, HS>(pk, sDZ, warp, lane);
            __syncwarp();
            if (gio.denc_cols > 0) {
                // leading columns of the warp's 16 rows, 8-byte chunks
                const int cpr = gio.denc_cols >> 2;
                for (int ch = lane; ch < 16 * cpr; ch += 32) {
                    int r = ch / cpr, c4 = ch % cpr;
                    int64_t gr = row0 + r;
                    if (gr < io.n) {
                        uint2 v = *reinterpret_cast<const uint2*>(&sDZ[(16 * warp + r) * HS + c4 * 4]);
                        *reinterpret_cast<uint2*>(&gio.denc[gr * gio.denc_cols + c4 * 4]) = v;
                    }
                }
            }
            if (gio.pieces != nullptr) {
                // the warp's 16 rows, level by level: 64 contiguous bytes per level in the owner's piece
                const int own = (DS::K0 / 2) / gio.piece_ranks;
                for (int ch = lane; ch < 16 * (DS::K0 / 2); ch += 32) {
                    const int l = ch >> 4, r = ch & 15;
                    const int64_t gr = row0 + r;
                    if (gr < io.n)
                        gio.pieces[((int64_t)(l % gio.piece_ranks) * own + l / gio.piece_ranks) * gio.piece_cap + gr] =
                            *reinterpret_cast<const uint32_t*>(&sDZ[(16 * warp + r) * HS + 2 * l]);
                }
            }
            if (gio.table_grads != nullptr) {
                // Gradient scatter of this tile, fire-and-forget reductions that drain through L2 while the tensor
                // work of the next tile (and of the other CTA on this SM) goes on: thread = (row, every other level).
                __syncthreads();
                const int r = tid & (TILE_ROWS - 1), hsel = tid >> 7;  // a warp = 32 consecutive samples at one level
                const int64_t row = row_base + r;
                const bool has = row < io.n;
                float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
                if (has) p = ld_nc_f4(gio.pos4 + row * 4);
                for (int level = gio.scatter_begin + hsel; level < gp.L; level += 2) {
                    const float2 gq = __half22float2(*reinterpret_cast<const __half2*>(&sDZ[r * HS + 2 * level]));
                    scatter_level_warp<GRAD_HALF>(gp, level, p.x, p.y, p.z, gq, has, gio.table_grads, lane);
                }
            }
            __syncthreads();
        }
    }
    cp_async_wait_all();
    flush_dw<H, 8, 16>(&acc[FB::S_C2], gio.dWc + CS::w_off(2), warp, lane);
    flush_dw<H, H, H>(&acc[FB::S_C1], gio.dWc + CS::w_off(1), warp, lane);
    flush_dw<32, H, H>(&acc[FB::S_C0], gio.dWc + CS::w_off(0), warp, lane);
    flush_dw<H, 16, 16>(&acc[FB::S_D1], gio.dWd + DS::w_off(1), warp, lane);
    flush_dw<32, H, H>(&acc[FB::S_D0], gio.dWd + DS::w_off(0), warp, lane);
    red_add(&gio.dbc[CS::b_off(2) + tid % 8], db_c2);
    red_add(&gio.dbc[CS::b_off(1) + tid % H], db_c1);
    red_add(&gio.dbc[CS::b_off(0) + tid % H], db_c0);
    red_add(&gio.dbd[DS::b_off(1) + tid % 16], db_d1);
    red_add(&gio.dbd[DS::b_off(0) + tid % H], db_d0);
}

}  // namespace nb

namespace {

using DensityNet = nb::MlpShape<32, 64, 16, 2>;
using ColorNet = nb::MlpShape<32, 64, 8, 3>;

bool is_shape(const nb_mlp_desc* d, int k0, int h, int out, int nl) {
    return d->input_dim == k0 && d->hidden_dim == h && d->output_dim == out && d->num_layers == nl;
}
bool misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

}  // namespace

extern "C" int nb_field_supported(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color) {
    if (!grid || !density || !color) return 0;
    if (grid->num_levels != 16) return 0;
    return is_shape(density, 32, 64, 16, 2) && is_shape(color, 32, 64, 8, 3) && density->output_activation == 0 &&
           color->output_activation == 1;
}

namespace nb {
std::atomic<int> g_forward_staged{2};   // nb_set_tuning("forward_staged", ...): 0 never, 1 always, 2 when the call brings a sample order
std::atomic<int> g_forward_stage_levels{FWD_STAGE_LEVELS};   // "forward_stage_levels": leading levels the ordered forward may stage (0: none)
std::atomic<int> g_forward_persistent{1};                     // "forward_persistent": 0 = one CTA per tile group
}

static int field_forward_impl(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                                const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                                const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                                int64_t n, float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb,
                                int rgb_stride, const uint32_t* d_count, void* stream, const uint32_t* d_perm = nullptr,
                                const nb::FieldLossIO* loss = nullptr) {
    if (!grid || !density || !color || !d_pos4 || !d_table_h || !d_dirs3 || !d_density_w_h || !d_density_b || !d_color_w_h || !d_color_b ||
        !d_rgb || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_field_forward: null pointer or negative count");
    if (!nb_field_supported(grid, density, color))
        return nb_set_error(NB_ERR_UNSUPPORTED, "nb_field_forward: built for 16 levels, density 32-64-16 and colour 32-64-64-8 (sigmoid)");
    if (rgb_stride != 4 && rgb_stride != 8) return nb_set_error(NB_ERR_INVALID, "nb_field_forward: rgb_stride must be 4 or 8");
    if (misaligned(d_pos4, 16) || misaligned(d_table_h, 4) || misaligned(d_density_w_h, 16) || misaligned(d_color_w_h, 16) ||
        misaligned(d_enc_save_h, 16) || misaligned(d_rgb, 8) || misaligned(d_density_b, 8) || misaligned(d_color_b, 8))
        return nb_set_error(NB_ERR_INVALID, "nb_field_forward: misaligned device pointer");
    if (n == 0) return NB_OK;
    nb::FieldIO io{};
    io.pos4 = d_pos4; io.table2 = (const uint32_t*)d_table_h; io.dirs3 = d_dirs3; io.ray_idx = d_ray_indices;
    io.ray_idx_offset = ray_index_offset;
    io.Wd = (const __half*)d_density_w_h; io.bd = d_density_b; io.Wc = (const __half*)d_color_w_h; io.bc = d_color_b;
    io.n = n; io.density_bias = density_bias; io.count = d_count;
    nb::GridParams gp = nb::make_params(grid);
    if (misaligned(d_table_h, 8)) gp.pair_ops = 0;
    const int staged_mode = nb::g_forward_staged.load();
    if (loss != nullptr) {
        auto kern = nb::field_forward_kernel<DensityNet, ColorNet, true>;
        size_t smem = nb::FieldSmem<DensityNet, ColorNet>::fwd_bytes();
        NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int64_t grid_dim = (n + nb::TILE_ROWS - 1) / nb::TILE_ROWS;
        kern<<<(unsigned)grid_dim, nb::CTA_THREADS, smem, (cudaStream_t)stream>>>(gp, io, (__half*)d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride,
                                                                                  *loss, nb::FieldPiecesIO{});
        NB_CHECK_LAUNCH();
        nb::g_launch_count++;
        return NB_OK;
    }
    if (d_perm != nullptr || staged_mode == 1) {
        if (staged_mode == 0) return nb_set_error(NB_ERR_INVALID, "nb_field_forward_ordered: the staged forward is switched off (forward_staged = 0)");
        auto kern = nb::field_forward_staged_kernel<DensityNet, ColorNet>;
        const size_t smem = nb::FieldStagedSmem<DensityNet, ColorNet>::bytes();
        NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        int per_sm = 0;
        NB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, nb::CTA_THREADS, smem));
        if (per_sm < 1) per_sm = 1;
        const int64_t group_rows = (int64_t)nb::FWD_GROUP_TILES * nb::TILE_ROWS;
        const int64_t groups = (n + group_rows - 1) / group_rows;
        int64_t grid_dim = (int64_t)nb_num_sms() * per_sm;
        if (grid_dim > groups || nb::g_forward_persistent.load() == 0) grid_dim = groups;
        const int stage_levels = std::max(0, std::min(nb::g_forward_stage_levels.load(), (int)nb::FWD_STAGE_LEVELS));
        kern<<<(unsigned)grid_dim, nb::CTA_THREADS, smem, (cudaStream_t)stream>>>(gp, io, d_perm, (__half*)d_enc_save_h, d_sigma, d_logit0, d_rgb,
                                                                                  rgb_stride, stage_levels);
        NB_CHECK_LAUNCH();
        nb::g_launch_count++;
        return NB_OK;
    }
    auto kern = nb::field_forward_kernel<DensityNet, ColorNet, false>;
    size_t smem = nb::FieldSmem<DensityNet, ColorNet>::fwd_bytes();
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid_dim = (n + nb::TILE_ROWS - 1) / nb::TILE_ROWS;
    kern<<<(unsigned)grid_dim, nb::CTA_THREADS, smem, (cudaStream_t)stream>>>(gp, io, (__half*)d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride,
                                                                              nb::FieldLossIO{}, nb::FieldPiecesIO{});
    NB_CHECK_LAUNCH();
    nb::g_launch_count++;
    return NB_OK;
}

extern "C" int nb_field_forward(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                                const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                                const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                                int64_t n, float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb,
                                int rgb_stride, void* stream) {
    return field_forward_impl(grid, density, color, d_pos4, d_table_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b,
                              d_color_w_h, d_color_b, n, density_bias, d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride, nullptr, stream);
}

extern "C" int nb_field_forward_mse(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                                    const void* d_table_h, const float* d_dirs3, const void* d_density_w_h, const float* d_density_b,
                                    const void* d_color_w_h, const float* d_color_b, int64_t n, float density_bias, void* d_enc_save_h,
                                    float* d_sigma, float* d_logit0, float* d_rgb, int rgb_stride, const void* d_target_h, void* d_dcolor_h,
                                    float* d_total_loss, float loss_scale, void* stream) {
    if (!d_target_h || !d_dcolor_h) return nb_set_error(NB_ERR_INVALID, "nb_field_forward_mse: null target or gradient");
    if (misaligned(d_target_h, 4) || misaligned(d_dcolor_h, 4)) return nb_set_error(NB_ERR_INVALID, "nb_field_forward_mse: misaligned target or gradient");
    nb::FieldLossIO lio{};
    lio.target = (const __half*)d_target_h; lio.grad = (__half*)d_dcolor_h; lio.total = d_total_loss;
    lio.grad_scale = n > 0 ? (2.0f / (float)(n * 3)) * loss_scale : 0.0f;   // as nb_mse_loss_grad with valid_dim 3
    return field_forward_impl(grid, density, color, d_pos4, d_table_h, d_dirs3, nullptr, 0, d_density_w_h, d_density_b, d_color_w_h, d_color_b, n,
                              density_bias, d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride, nullptr, stream, nullptr, &lio);
}

extern "C" int nb_part_field_forward(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, int ranks, int64_t capacity,
                                     const void* d_pieces_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                                     const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                                     int64_t n, float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb,
                                     int rgb_stride, void* stream) {
    if (!grid || !density || !color || !d_pieces_h || !d_dirs3 || !d_density_w_h || !d_density_b || !d_color_w_h || !d_color_b || !d_rgb || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_part_field_forward: null pointer or negative count");
    if (!nb_field_supported(grid, density, color))
        return nb_set_error(NB_ERR_UNSUPPORTED, "nb_part_field_forward: built for 16 levels, density 32-64-16 and colour 32-64-64-8 (sigmoid)");
    if (ranks < 1 || grid->num_levels % ranks != 0 || capacity < n) return nb_set_error(NB_ERR_INVALID, "nb_part_field_forward: ranks must divide the levels, capacity >= n");
    if (rgb_stride != 4 && rgb_stride != 8) return nb_set_error(NB_ERR_INVALID, "nb_part_field_forward: rgb_stride must be 4 or 8");
    if (misaligned(d_pieces_h, 4) || misaligned(d_density_w_h, 16) || misaligned(d_color_w_h, 16) || misaligned(d_enc_save_h, 16) || misaligned(d_rgb, 8) ||
        misaligned(d_density_b, 8) || misaligned(d_color_b, 8))
        return nb_set_error(NB_ERR_INVALID, "nb_part_field_forward: misaligned device pointer");
    if (n == 0) return NB_OK;
    nb::FieldIO io{};
    io.dirs3 = d_dirs3; io.ray_idx = d_ray_indices; io.ray_idx_offset = ray_index_offset;
    io.Wd = (const __half*)d_density_w_h; io.bd = d_density_b; io.Wc = (const __half*)d_color_w_h; io.bc = d_color_b;
    io.n = n; io.density_bias = density_bias;
    nb::GridParams gp = nb::make_params(grid);
    nb::FieldPiecesIO pio{reinterpret_cast<const uint32_t*>(d_pieces_h), ranks, capacity};
    auto kern = nb::field_forward_kernel<DensityNet, ColorNet, false, true>;
    size_t smem = nb::FieldSmem<DensityNet, ColorNet>::fwd_bytes();
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid_dim = (n + nb::TILE_ROWS - 1) / nb::TILE_ROWS;
    kern<<<(unsigned)grid_dim, nb::CTA_THREADS, smem, (cudaStream_t)stream>>>(gp, io, (__half*)d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride,
                                                                              nb::FieldLossIO{}, pio);
    NB_CHECK_LAUNCH();
    nb::g_launch_count++;
    return NB_OK;
}

extern "C" int nb_field_forward_ordered(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                                        const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                                        const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                                        int64_t n, const uint32_t* d_order, float density_bias, void* d_enc_save_h, float* d_sigma,
                                        float* d_logit0, float* d_rgb, int rgb_stride, void* stream) {
    if (!d_order) return nb_set_error(NB_ERR_INVALID, "nb_field_forward_ordered: null sample order");
    return field_forward_impl(grid, density, color, d_pos4, d_table_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b,
                              d_color_w_h, d_color_b, n, density_bias, d_enc_save_h, d_sigma, d_logit0, d_rgb, rgb_stride, nullptr, stream, d_order);
}

extern "C" int nb_field_forward_counted(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                                        const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices,
                                        int64_t ray_index_offset, const void* d_density_w_h, const float* d_density_b,
                                        const void* d_color_w_h, const float* d_color_b, int64_t n_max, const uint32_t* d_count,
                                        float density_bias, float* d_sigma, float* d_rgb, int rgb_stride, void* stream) {
    if (!d_count) return nb_set_error(NB_ERR_INVALID, "nb_field_forward_counted: null count");
    return field_forward_impl(grid, density, color, d_pos4, d_table_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b,
                              d_color_w_h, d_color_b, n_max, density_bias, nullptr, d_sigma, nullptr, d_rgb, rgb_stride, d_count, stream);
}

static int field_backward_impl(const nb_mlp_desc* density, const nb_mlp_desc* color, const void* d_enc_h, const float* d_dirs3,
                               const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h,
                               const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n,
                               const void* d_dcolor_h, const float* d_dsigma, float* d_grad_density_w, float* d_grad_density_b,
                               float* d_grad_color_w, float* d_grad_color_b, void* d_denc_h, const nb_grid_desc* grid,
                               const float* d_pos4, float* d_table_grads, void* stream, const uint32_t* d_perm,
                               uint32_t* d_pieces = nullptr, int piece_ranks = 0, int64_t piece_cap = 0) {
    if (!density || !color || !d_enc_h || !d_dirs3 || !d_density_w_h || !d_density_b || !d_color_w_h || !d_color_b || !d_dcolor_h ||
        !d_grad_density_w || !d_grad_density_b || !d_grad_color_w || !d_grad_color_b || (!d_denc_h && !d_pieces) || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_field_backward: null pointer or negative count");
    if (!is_shape(density, 32, 64, 16, 2) || !is_shape(color, 32, 64, 8, 3))
        return nb_set_error(NB_ERR_UNSUPPORTED, "nb_field_backward: built for density 32-64-16 and colour 32-64-64-8");
    if (misaligned(d_enc_h, 16) || misaligned(d_dcolor_h, 16) || misaligned(d_denc_h, 16) || misaligned(d_density_w_h, 16) ||
        misaligned(d_color_w_h, 16) || misaligned(d_grad_density_w, 8) || misaligned(d_grad_color_w, 8) || misaligned(d_density_b, 8) ||
        misaligned(d_color_b, 8))
        return nb_set_error(NB_ERR_INVALID, "nb_field_backward: misaligned device pointer");
    if (nb::field_backward_tc_failed())
        return nb_set_error(NB_ERR_CUDA, "nb_field_backward: a bounded wait of an earlier tensor-memory launch ran out (its gradients are "
                                         "incomplete); nb_field_backward_tc_status() clears the condition");
    if (n == 0) return NB_OK;
    nb::FieldIO io{};
    io.dirs3 = d_dirs3; io.ray_idx = d_ray_indices; io.ray_idx_offset = ray_index_offset;
    io.Wd = (const __half*)d_density_w_h; io.bd = d_density_b; io.Wc = (const __half*)d_color_w_h; io.bc = d_color_b;
    io.n = n;
    nb::FieldGradIO gio{};
    gio.enc = (const __half*)d_enc_h; gio.dcolor = (const __half*)d_dcolor_h; gio.dsigma = d_dsigma;
    gio.dWd = d_grad_density_w; gio.dbd = d_grad_density_b; gio.dWc = d_grad_color_w; gio.dbc = d_grad_color_b;
    gio.denc = (__half*)d_denc_h; gio.denc_cols = 32;
    if (d_pieces != nullptr) { gio.denc = nullptr; gio.denc_cols = 0; gio.pieces = d_pieces; gio.piece_ranks = piece_ranks; gio.piece_cap = piece_cap; }
    nb::GridParams gp{};
    int shared_levels = 0;
    const bool scatter = d_table_grads != nullptr;
    if (scatter) {
        if (!grid || !d_pos4) return nb_set_error(NB_ERR_INVALID, "nb_field_backward: the fused scatter needs the grid descriptor and positions");
        if (grid->num_levels != 16) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_field_backward: built for 16 levels");
        if (misaligned(d_pos4, 16) || misaligned(d_table_grads, 8))
            return nb_set_error(NB_ERR_INVALID, "nb_field_backward: misaligned positions or table gradient");
        gp = nb::make_params(grid);
        if (misaligned(d_table_grads, 16) && !gp.grad_half) gp.pair_ops = 0;   // the fp32 pair is a 16-byte reduction, the fp16 pair 8 bytes
        shared_levels = nb::scatter_shared_levels(gp, n);
        gio.pos4 = d_pos4; gio.table_grads = d_table_grads; gio.scatter_begin = shared_levels;
        gio.denc_cols = 4 * shared_levels;   // only what the shared-memory scatter kernel below reads
    }
    // pieces are written by the register kernel only (it is also the faster one on the ray-ordered samples of the engine)
    const int tc_mode = d_pieces != nullptr ? 0 : (d_perm != nullptr ? 1 : nb::g_backward_tc.load());
    // The tensor-memory kernel adds its weight gradients with 16-byte reductions; the register kernel needs 8 bytes only.
    const bool grads_16 = !misaligned(d_grad_density_w, 16) && !misaligned(d_grad_color_w, 16);
    if (tc_mode == 1 && !grads_16)
        return nb_set_error(NB_ERR_INVALID, "nb_field_backward: the tensor-memory kernel needs 16-byte aligned weight gradients");
    if (d_perm != nullptr && scatter && misaligned(d_pos4, 16)) return nb_set_error(NB_ERR_INVALID, "nb_field_backward_ordered: misaligned positions");
    if (tc_mode == 1 || (tc_mode == 2 && d_ray_indices == nullptr && grads_16)) {
        // tensor-memory formulation (field_backward_tc.cu): same inputs, outputs and rounding points
        nb::tc::BackwardArgs ta{};
        ta.enc = gio.enc; ta.dcolor = gio.dcolor; ta.dsigma = gio.dsigma; ta.dirs3 = io.dirs3; ta.ray_idx = io.ray_idx;
        ta.ray_idx_offset = io.ray_idx_offset; ta.Wd = io.Wd; ta.Wc = io.Wc; ta.bd = io.bd; ta.bc = io.bc; ta.n = n;
        ta.dWd = gio.dWd; ta.dbd = gio.dbd; ta.dWc = gio.dWc; ta.dbc = gio.dbc; ta.denc = gio.denc; ta.denc_cols = gio.denc_cols;
        ta.pos4 = gio.pos4; ta.table_grads = gio.table_grads; ta.scatter_begin = gio.scatter_begin;
        ta.perm = d_perm;
        int rc = nb::launch_field_backward_tc(gp, ta, (cudaStream_t)stream);
        if (rc != NB_OK) return rc;
        if (scatter && shared_levels > 0)
            return nb::scatter_launch(gp, d_pos4, (const __half*)d_denc_h, 4 * shared_levels, n, d_table_grads, 0, shared_levels, (cudaStream_t)stream);
        return NB_OK;
    }
    auto kern = (scatter && gp.grad_half) ? nb::field_backward_kernel<DensityNet, ColorNet, true> : nb::field_backward_kernel<DensityNet, ColorNet, false>;
    size_t smem = nb::FieldBwd<DensityNet, ColorNet>::smem_bytes();
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    NB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, nb::CTA_THREADS, smem));
    if (per_sm < 1) per_sm = 1;
    int64_t ntiles = (n + nb::TILE_ROWS - 1) / nb::TILE_ROWS;
    int64_t grid_dim = (int64_t)nb_num_sms() * per_sm;
    if (grid_dim > ntiles) grid_dim = ntiles;
    kern<<<(unsigned)grid_dim, nb::CTA_THREADS, smem, (cudaStream_t)stream>>>(gp, io, gio);
    NB_CHECK_LAUNCH();
    nb::g_launch_count++;
    if (scatter && shared_levels > 0)
        return nb::scatter_launch(gp, d_pos4, (const __half*)d_denc_h, 4 * shared_levels, n, d_table_grads, 0, shared_levels, (cudaStream_t)stream);
    return NB_OK;
}

extern "C" int nb_field_backward(const nb_mlp_desc* density, const nb_mlp_desc* color, const void* d_enc_h, const float* d_dirs3,
                                 const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h,
                                 const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n,
                                 const void* d_dcolor_h, const float* d_dsigma, float* d_grad_density_w, float* d_grad_density_b,
                                 float* d_grad_color_w, float* d_grad_color_b, void* d_denc_h, const nb_grid_desc* grid,
                                 const float* d_pos4, float* d_table_grads, void* stream) {
    return field_backward_impl(density, color, d_enc_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b, d_color_w_h, d_color_b, n,
                               d_dcolor_h, d_dsigma, d_grad_density_w, d_grad_density_b, d_grad_color_w, d_grad_color_b, d_denc_h, grid, d_pos4,
                               d_table_grads, stream, nullptr);
}

extern "C" int nb_part_field_backward(const nb_mlp_desc* density, const nb_mlp_desc* color, int ranks, int64_t capacity, const void* d_enc_h,
                                      const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h,
                                      const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n, const void* d_dcolor_h,
                                      const float* d_dsigma, float* d_grad_density_w, float* d_grad_density_b, float* d_grad_color_w,
                                      float* d_grad_color_b, void* d_pieces_h, void* stream) {
    if (!d_pieces_h || ranks < 1 || 16 % ranks != 0 || capacity < n || misaligned(d_pieces_h, 4))
        return nb_set_error(NB_ERR_INVALID, "nb_part_field_backward: pieces required, ranks must divide the 16 levels, capacity >= n");
    return field_backward_impl(density, color, d_enc_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b, d_color_w_h, d_color_b, n,
                               d_dcolor_h, d_dsigma, d_grad_density_w, d_grad_density_b, d_grad_color_w, d_grad_color_b, nullptr, nullptr, nullptr,
                               nullptr, stream, nullptr, reinterpret_cast<uint32_t*>(d_pieces_h), ranks, capacity);
}

extern "C" int nb_field_backward_ordered(const nb_mlp_desc* density, const nb_mlp_desc* color, const void* d_enc_h, const float* d_dirs3,
                                         const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h,
                                         const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n,
                                         const uint32_t* d_order, const void* d_dcolor_h, const float* d_dsigma, float* d_grad_density_w,
                                         float* d_grad_density_b, float* d_grad_color_w, float* d_grad_color_b, void* d_denc_h,
                                         const nb_grid_desc* grid, const float* d_pos4, float* d_table_grads, void* stream) {
    if (!d_order) return nb_set_error(NB_ERR_INVALID, "nb_field_backward_ordered: null sample order");
    return field_backward_impl(density, color, d_enc_h, d_dirs3, d_ray_indices, ray_index_offset, d_density_w_h, d_density_b, d_color_w_h, d_color_b, n,
                               d_dcolor_h, d_dsigma, d_grad_density_w, d_grad_density_b, d_grad_color_w, d_grad_color_b, d_denc_h, grid, d_pos4,
                               d_table_grads, stream, d_order);
}
