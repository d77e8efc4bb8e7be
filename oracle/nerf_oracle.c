/*
 * CPU oracle for the NeRF training / rendering hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the arithmetic of the
 * reference's CUDA kernels (Ajitesh-07/3DMaker, modules/TinyMLP and modules/NeRF).  It is the
 * checker the parity tests compare the CUDA path against, and the timed CPU baseline of the
 * benchmark.  Nothing in the product library links, loads or calls it.
 *
 * Every function names the reference file:line it follows.  fp16 storage is passed as raw
 * uint16_t bit patterns; conversions use _Float16 (round-to-nearest-even, like __float2half).
 * Build with -ffp-contract=off: fused multiply-adds appear only where the reference spells
 * __fmaf_rn, everything else is separate IEEE fp32 operations as in the kernels.
 *
 * Parity pin: the functions of this file that have a CPU twin inside the reference's own test
 * executables (hash index + trilinear weights, gradient scatter, MLP forward, MLP backward,
 * Adam, MSE loss/grad, exclusive scan) are checked against those twins, compiled from the
 * reference sources where they lie (oracle/build_ref.sh -> oracle/_ref/), and against the
 * committed fixtures those twins produced (tests/golden/).  The reference holds no golden
 * vectors on disk and no CPU code for ray marching, compositing, loss gradients, SH and the
 * occupancy grid: for those functions parity is pinned only by running the reference's CUDA
 * kernels on a GPU next to ours (tests marked gpu, when oracle/_ref holds the reference build).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 orc_half;

static inline float h2f(uint16_t h) { orc_half x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t f2h(float f) { orc_half x = (orc_half)f; uint16_t h; memcpy(&h, &x, 2); return h; }

void orc_half_to_float(const uint16_t* in, float* out, long n) { for (long i = 0; i < n; i++) out[i] = h2f(in[i]); }
void orc_float_to_half(const float* in, uint16_t* out, long n) { for (long i = 0; i < n; i++) out[i] = f2h(in[i]); }

/* ------------------------------------------------------------------------------------------
 * Hash grid geometry
 * ------------------------------------------------------------------------------------------ */

/* First hashed (non dense) level.  modules/TinyMLP/networkFusionHashtable.cu:367-377 */
int orc_dense_level_start(int tableSize, int lowestSize, float b, int numLevels) {
    float inner_term = (cbrtf((float)tableSize) - 1.0f) / (float)lowestSize;
    float continuous_level = log2f(inner_term) / log2f(b);
    int s = (int)floorf(continuous_level) + 1;
    if (s > numLevels) s = numLevels;
    if (s < 0) s = 0;
    return s;
}

/* Per-level resolution as the forward kernel builds it: restarted with a power every four levels,
 * multiplied by b in between.  modules/TinyMLP/networkFusionHashtable.cu:124-128,218.
 * The kernel evaluates the power with the device's approximate __powf; this is the libm value.
 * Bit-exact index parity feeds the device-computed table into the functions below instead. */
void orc_level_scales(int lowestSize, float b, int numLevels, float* scales) {
    for (int l = 0; l < numLevels; l++) {
        int start = (l / 4) * 4;
        float v = (float)lowestSize * powf(b, (float)start);
        for (int i = start; i < l; i++) v *= b;
        scales[l] = v;
    }
}

/* modules/TinyMLP/networkFusionHashtable.cu:62-66 */
static inline uint32_t hash_coords(int cx, int cy, int cz, int T) {
    return (((uint32_t)cx * 1u) ^ ((uint32_t)cy * 2654435761u) ^ ((uint32_t)cz * 805459861u)) & (uint32_t)(T - 1);
}
/* modules/TinyMLP/networkFusionHashtable.cu:68-70 */
static inline uint32_t dense_index(int cx, int cy, int cz, int N_l) {
    return (uint32_t)(cx + cy * (N_l + 1) + cz * (N_l + 1) * (N_l + 1));
}

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

typedef struct {
    uint32_t idx[8];   /* element offset of feature 0 of each corner inside the whole table */
    float w[8];        /* trilinear weights, corner order 000,100,010,110,001,101,011,111 */
} orc_corners;

/* Corner indices + weights of one (point, level).
 * clamp_hi_minus: 0 = forward clamp of the low corner to [0, N_l]
 *                     (networkFusionHashtable.cu:134-148),
 *                 1 = backward clamp to [0, N_l-1]
 *                     (networkFusionBackwardHashtable.cu:812-826). */
static inline void corners_of(const float* p, float scale, int level, int T, int dls, int clamp_hi_minus,
                              orc_corners* c) {
    int N_l = (int)floorf(scale);
    float x_l = p[0] * scale, y_l = p[1] * scale, z_l = p[2] * scale;
    int x0 = (int)floorf(x_l), y0 = (int)floorf(y_l), z0 = (int)floorf(z_l);
    int hi = clamp_hi_minus ? N_l - 1 : N_l;
    x0 = imax(0, imin(x0, hi)); y0 = imax(0, imin(y0, hi)); z0 = imax(0, imin(z0, hi));
    int x1 = imin(x0 + 1, N_l), y1 = imin(y0 + 1, N_l), z1 = imin(z0 + 1, N_l);
    float wx1 = 1.0f - x_l + floorf(x_l);
    float wy1 = 1.0f - y_l + floorf(y_l);
    float wz1 = 1.0f - z_l + floorf(z_l);
    int dense = level < dls;
    int xs[2] = {x0, x1}, ys[2] = {y0, y1}, zs[2] = {z0, z1};
    float wx[2] = {wx1, 1.0f - wx1}, wy[2] = {wy1, 1.0f - wy1}, wz[2] = {wz1, 1.0f - wz1};
    for (int k = 0; k < 8; k++) {
        int ix = k & 1, iy = (k >> 1) & 1, iz = (k >> 2) & 1;
        uint32_t ti = dense ? dense_index(xs[ix], ys[iy], zs[iz], N_l) : hash_coords(xs[ix], ys[iy], zs[iz], T);
        c->idx[k] = (uint32_t)level * (uint32_t)T * 2u + ti * 2u;
        c->w[k] = wx[ix] * wy[iy] * wz[iz];   /* (wx*wy)*wz, networkFusionHashtable.cu:158-161 */
    }
}

/* Table element offsets of the 8 corners of every (point, level): idx_out[n][L][8]. */
void orc_hash_indices(const float* pos4, long n, const float* scales, int L, int T, int dls, int clamp_hi_minus,
                      uint32_t* idx_out, float* w_out) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        for (int l = 0; l < L; l++) {
            orc_corners c;
            corners_of(pos4 + 4 * i, scales[l], l, T, dls, clamp_hi_minus, &c);
            for (int k = 0; k < 8; k++) {
                idx_out[(i * L + l) * 8 + k] = c.idx[k];
                if (w_out) w_out[(i * L + l) * 8 + k] = c.w[k];
            }
        }
    }
}

/* Encode forward: fp16 feature pairs, fp32 trilinear blend in the kernel's fixed fma order,
 * rounded to fp16 once.  modules/TinyMLP/networkFusionHashtable.cu:111-222. */
void orc_encode_forward(const float* pos4, long n, const uint16_t* table, const float* scales, int L, int T, int dls,
                        uint16_t* enc_out) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        for (int l = 0; l < L; l++) {
            orc_corners c;
            corners_of(pos4 + 4 * i, scales[l], l, T, dls, 0, &c);
            for (int f = 0; f < 2; f++) {
                float r = h2f(table[c.idx[7] + f]) * c.w[7];
                for (int k = 6; k >= 0; k--) r = fmaf(h2f(table[c.idx[k] + f]), c.w[k], r);
                enc_out[i * 2 * L + 2 * l + f] = f2h(r);
            }
        }
    }
}

/* Gradient scatter: grad[l][idx][f] += dEnc[n][2l+f] * w_corner.
 * modules/TinyMLP/networkFusionBackwardHashtable.cu:783-910.  The kernel adds with fp32 atomics in
 * no fixed order; the oracle sums per level in double (as the reference's scatterCPU does,
 * tests_kernels/testScatterAB.cu:124-149) and rounds once. */
void orc_scatter_backward(const float* pos4, long n, const uint16_t* dEnc, const float* scales, int L, int T, int dls,
                          float* grads) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int l = 0; l < L; l++) {
        double* acc = (double*)calloc((size_t)T * 2, sizeof(double));
        uint32_t base = (uint32_t)l * (uint32_t)T * 2u;
        for (long i = 0; i < n; i++) {
            orc_corners c;
            corners_of(pos4 + 4 * i, scales[l], l, T, dls, 1, &c);
            float gx = h2f(dEnc[i * 2 * L + 2 * l]), gy = h2f(dEnc[i * 2 * L + 2 * l + 1]);
            for (int k = 0; k < 8; k++) {
                acc[c.idx[k] - base] += (double)(gx * c.w[k]);
                acc[c.idx[k] - base + 1] += (double)(gy * c.w[k]);
            }
        }
        for (long j = 0; j < (long)T * 2; j++) grads[base + j] = (float)((double)grads[base + j] + acc[j]);
        free(acc);
    }
}

/* ------------------------------------------------------------------------------------------
 * Fused MLP
 * ------------------------------------------------------------------------------------------ */

static inline int layer_in(int l, int in, int hid) { return l == 0 ? in : hid; }
static inline int layer_out(int l, int nl, int hid, int out) { return l == nl - 1 ? out : hid; }

long orc_mlp_weight_count(int in, int hid, int out, int nl) {
    long c = 0;
    for (int l = 0; l < nl; l++) c += (long)layer_in(l, in, hid) * layer_out(l, nl, hid, out);
    return c;
}
long orc_mlp_bias_count(int hid, int out, int nl) {
    long c = 0;
    for (int l = 0; l < nl; l++) c += layer_out(l, nl, hid, out);
    return c;
}

/* Forward: per layer relu(A W^T + b), W [out][in] row-major fp16, fp32 accumulate, hidden
 * activations rounded to fp16, last layer linear or sigmoid 1/(1+expf(-v)) in fp32.
 * modules/TinyMLP/networkFusion.cu:102-194 (plain) and networkFusionHashtable.cu:225-315 (grid net).
 * acts (nullable) receives the fp16 hidden activations, layer 1..nl-1, each [n][hid], back to back. */
void orc_mlp_forward(const uint16_t* in_h, long n, int in, int hid, int out, int nl, const uint16_t* W,
                     const float* bias, int out_act, float* out_f, uint16_t* acts) {
    long woff[16], boff[16];
    long wo = 0, bo = 0;
    for (int l = 0; l < nl; l++) {
        woff[l] = wo; boff[l] = bo;
        wo += (long)layer_in(l, in, hid) * layer_out(l, nl, hid, out);
        bo += layer_out(l, nl, hid, out);
    }
    int maxd = in > hid ? in : hid;
#pragma omp parallel
    {
        float* cur = (float*)malloc(sizeof(float) * maxd);
        float* nxt = (float*)malloc(sizeof(float) * maxd);
#pragma omp for schedule(static)
        for (long r = 0; r < n; r++) {
            for (int k = 0; k < in; k++) cur[k] = h2f(in_h[r * in + k]);
            for (int l = 0; l < nl; l++) {
                int K = layer_in(l, in, hid), N = layer_out(l, nl, hid, out);
                const uint16_t* Wl = W + woff[l];
                for (int o = 0; o < N; o++) {
                    float acc = 0.0f;
                    for (int k = 0; k < K; k++) acc += cur[k] * h2f(Wl[(long)o * K + k]);
                    float v = acc + bias[boff[l] + o];
                    if (l < nl - 1) {
                        v = fmaxf(v, 0.0f);
                        uint16_t hv = f2h(v);
                        if (acts) acts[(long)(l) * n * hid + r * hid + o] = hv;
                        nxt[o] = h2f(hv);
                    } else {
                        if (out_act == 1) v = 1.0f / (1.0f + expf(-v));
                        out_f[r * out + o] = v;
                    }
                }
                float* t = cur; cur = nxt; nxt = t;
            }
        }
        free(cur); free(nxt);
    }
}

/* Backward: per layer dW[o][i] += sum_n dZ[n][o] A[n][i], db[o] += sum_n dZ[n][o],
 * dA = dZ W rounded to fp16, then zeroed where the saved activation is <= 0.
 * modules/TinyMLP/networkFusionBackward.cu:92-644 (fp16 roundings at :253,:439,:626) and the CPU twin
 * tests_kernels/testFusionBackward.cu:38-85.  Sums run in double and round once (the kernel's fp32
 * atomic order is not fixed).  act0 = layer-0 input [n][in]; acts = hidden activations as orc_mlp_forward
 * stores them.  dX (nullable) = fp16 [n][in] gradient w.r.t. the input, not masked. */
void orc_mlp_backward(long n, int in, int hid, int out, int nl, const uint16_t* dL, const uint16_t* W,
                      const uint16_t* act0, const uint16_t* acts, float* dW, float* db, uint16_t* dX) {
    long woff[16], boff[16];
    long wo = 0, bo = 0;
    for (int l = 0; l < nl; l++) {
        woff[l] = wo; boff[l] = bo;
        wo += (long)layer_in(l, in, hid) * layer_out(l, nl, hid, out);
        bo += layer_out(l, nl, hid, out);
    }
    int maxd = in > hid ? in : hid;
    if (out > maxd) maxd = out;
    uint16_t* dz = (uint16_t*)malloc(sizeof(uint16_t) * n * maxd);
    uint16_t* dz_next = (uint16_t*)malloc(sizeof(uint16_t) * n * maxd);
    memcpy(dz, dL, sizeof(uint16_t) * n * out);
    for (int l = nl - 1; l >= 0; l--) {
        int K = layer_in(l, in, hid), N = layer_out(l, nl, hid, out);
        const uint16_t* A = (l == 0) ? act0 : acts + (long)(l - 1) * n * hid;
        const uint16_t* Wl = W + woff[l];
#pragma omp parallel for schedule(static)
        for (int o = 0; o < N; o++) {
            double sb = 0.0;
            double* sw = (double*)calloc(K, sizeof(double));
            for (long r = 0; r < n; r++) {
                float g = h2f(dz[r * N + o]);
                sb += (double)g;
                for (int k = 0; k < K; k++) sw[k] += (double)(g * h2f(A[r * K + k]));
            }
            db[boff[l] + o] = (float)((double)db[boff[l] + o] + sb);
            for (int k = 0; k < K; k++) dW[woff[l] + (long)o * K + k] = (float)((double)dW[woff[l] + (long)o * K + k] + sw[k]);
            free(sw);
        }
        if (l > 0 || dX) {
#pragma omp parallel for schedule(static)
            for (long r = 0; r < n; r++) {
                for (int k = 0; k < K; k++) {
                    float s = 0.0f;
                    for (int o = 0; o < N; o++) s += h2f(dz[r * N + o]) * h2f(Wl[(long)o * K + k]);
                    uint16_t hv = f2h(s);
                    if (l > 0) {
                        if (!(h2f(A[r * K + k]) > 0.0f)) hv = 0;
                        dz_next[r * K + k] = hv;
                    } else {
                        dX[r * K + k] = hv;
                    }
                }
            }
            uint16_t* t = dz; dz = dz_next; dz_next = t;
        }
    }
    free(dz); free(dz_next);
}

/* ------------------------------------------------------------------------------------------
 * Loss and optimizer
 * ------------------------------------------------------------------------------------------ */

/* MSE loss + gradient, optional sigmoid derivative folded in.
 * modules/TinyMLP/optimizerKernel.cu:169-224,369-401; CPU twin tests_kernels/testOptimizer.cu:27-52.
 * pred [n][padded] fp32, target [n][padded] fp16, grad [n][padded] fp16; returns the summed squared error. */
double orc_mse_loss_grad(const float* pred, const uint16_t* target, uint16_t* grad, long n, int padded, int valid,
                         float loss_scale, int out_act) {
    float grad_scale = (2.0f / (float)(n * valid)) * loss_scale;
    double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (long i = 0; i < n * padded; i++) {
        int col = (int)(i % padded);
        float p = pred[i];
        float diff = (col < valid) ? (p - h2f(target[i])) : 0.0f;
        total += (double)(diff * diff);
        float g = diff * grad_scale;
        if (out_act == 1) g *= p * (1.0f - p);
        grad[i] = f2h(g);
    }
    return total;
}

static inline float finite_or_zero(float x) { return isfinite(x) ? x : 0.0f; }

/* Dense Adam for MLP weights / biases with the non-finite self-heal.
 * modules/TinyMLP/optimizerKernel.cu:16-113; CPU twins tests_kernels/testOptimizer.cu:54-131.
 * w_half may be NULL (biases keep no fp16 copy). */
void orc_adam_dense(float* w, uint16_t* w_half, const float* g_in, float* m, float* v, long count, float lr,
                    float beta1, float beta2, float eps, float bc1, float bc2, float inv_loss_scale) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < count; i++) {
        float g = finite_or_zero(g_in[i] * inv_loss_scale);
        float mv = finite_or_zero(m[i]);
        float vv = finite_or_zero(v[i]);
        float wv = w[i];
        if (!isfinite(wv)) wv = 0.0f;
        mv = beta1 * mv + (1.0f - beta1) * g;
        vv = beta2 * vv + (1.0f - beta2) * g * g;
        float m_hat = mv / bc1;
        float v_hat = vv / bc2;
        wv = wv - (lr * m_hat / (sqrtf(v_hat) + eps));
        if (!isfinite(wv)) wv = 0.0f;
        m[i] = mv; v[i] = vv; w[i] = wv;
        if (w_half) w_half[i] = f2h(wv);
    }
}

/* Sparse Adam for the hash table: an entry whose gradient is exactly 0 is left untouched
 * (moments do not decay), the gradient is zeroed after it is read.
 * modules/TinyMLP/optimizerKernel.cu:116-167. */
void orc_adam_hash(float* w, uint16_t* w_half, float* g_io, float* m, float* v, long count, float lr, float beta1,
                   float beta2, float eps, float bc1, float bc2, float inv_loss_scale) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < count; i++) {
        float g_raw = g_io[i];
        if (g_raw == 0.0f) continue;
        g_io[i] = 0.0f;
        float g = finite_or_zero(g_raw * inv_loss_scale);
        float mv = beta1 * finite_or_zero(m[i]) + (1.0f - beta1) * g;
        float vv = beta2 * finite_or_zero(v[i]) + (1.0f - beta2) * g * g;
        float m_hat = mv / bc1;
        float v_hat = vv / bc2;
        float wv = w[i];
        if (!isfinite(wv)) wv = 0.0f;
        wv = wv - lr * m_hat / (sqrtf(v_hat) + eps);
        if (!isfinite(wv)) wv = 0.0f;
        m[i] = mv; v[i] = vv; w[i] = wv;
        w_half[i] = f2h(wv);
    }
}

/* Host-side bias corrections of step(): the step counter saturates at 50000.
 * modules/TinyMLP/TinyMLPHashGrid.cu:379-384, TinyMLP.cu:392-400. */
void orc_adam_bias_corrections(int step, float beta1, float beta2, float* bc1, float* bc2) {
    if (step > 50000) step = 50000;
    *bc1 = 1.0f - powf(beta1, (float)step);
    *bc2 = 1.0f - powf(beta2, (float)step);
}

/* ------------------------------------------------------------------------------------------
 * NeRF glue between the two networks
 * ------------------------------------------------------------------------------------------ */

static inline float sanitize_logit(float v) {
    v = fmaxf(-64.0f, fminf(64.0f, v));
    return (v != v) ? 0.0f : v;
}

/* Real spherical harmonics, bands l = 0..3 (16 coefficients), constants and signs of
 * modules/NeRF/otherKernels.cu:182-200. */
static inline void sh16(float x, float y, float z, float* sh) {
    float x2 = x * x, y2 = y * y, z2 = z * z;
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
}

/* Colour-network input: 16 clamped density logits ++ 16 SH of the ray direction, fp16; and
 * sigma = expf(min(logit0 - bias, 8)).  modules/NeRF/otherKernels.cu:156-273.
 * d_density_out is only read. */
void orc_sh_gather(const float* dirs3, const uint32_t* ray_indices, long offset, long n, float density_bias,
                   const float* density_out16, uint16_t* color_in32, float* sigma) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        const float* d = dirs3 + 3 * (long)ray_indices[i + offset];
        float sh[16];
        sh16(d[0], d[1], d[2], sh);
        float lg[16];
        for (int k = 0; k < 16; k++) lg[k] = sanitize_logit(density_out16[i * 16 + k]);
        sigma[i] = expf(fminf(lg[0] - density_bias, 8.0f));
        for (int k = 0; k < 16; k++) color_in32[i * 32 + k] = f2h(lg[k]);
        for (int k = 0; k < 16; k++) color_in32[i * 32 + 16 + k] = f2h(sh[k]);
    }
}

static inline float sanitize_65504(float v) {
    v = fmaxf(-65504.0f, fminf(65504.0f, v));
    return (v != v) ? 0.0f : v;
}

/* Density-network output gradient: the first 16 channels of the colour network's input gradient,
 * plus dL/dsigma*sigma on channel 0, clamped to the fp16 range, NaN -> 0.
 * modules/NeRF/otherKernels.cu:497-562. */
void orc_density_grad(long n, const float* tmp_dsigma, const uint16_t* color_dx32, uint16_t* density_grad16) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        for (int k = 0; k < 16; k++) {
            float f = h2f(color_dx32[i * 32 + k]);
            if (k == 0) f += tmp_dsigma[i];
            density_grad16[i * 16 + k] = f2h(sanitize_65504(f));
        }
    }
}
