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
 * Parity pin: the reference holds no golden vectors on disk and no CPU implementation of this path (the CPU
 * functions inside its test executables are not library code).  The pin is the reference's own CUDA code, compiled
 * for sm_100a from its sources where they lie (oracle/build_ref.py -> oracle/_ref/libref3dmaker.so, never copied into
 * this repository) and run on a GPU:
 *   - tests/golden/reference_vectors.npz holds its outputs on small seeded inputs (field forward/backward for both
 *     growth factors, ray/box test, occupancy march and compaction with 1 and 2 cascades and 2 samples per voxel,
 *     training and inference compositing, loss gradients, Philox sample jitter); tests/golden/make_golden.py is the
 *     script that produced it, and tests/test_golden_cpu.py checks every function of this file on that path against
 *     it without a GPU;
 *   - the tests marked gpu run the reference's kernels next to the product's on identical device buffers
 *     (tests/test_gpu_vs_reference.py).
 * Adam and the MSE loss have no reference vector of their own; they are pinned through the 30-step training
 * comparison against the reference's optimizer in tests/test_gpu_vs_reference.py.
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

/* ------------------------------------------------------------------------------------------
 * Rays, occupancy march, compaction
 *
 * The kernels these follow are compiled with --use_fast_math: divisions, log2f, exp2f and expf are
 * hardware approximations there.  The restatement uses IEEE / libm, so floats agree to a few ulp and
 * integer results (sample counts) can differ for a ray that grazes a voxel boundary within that
 * error.  Parity tests therefore compare counts exactly per ray but allow a small fraction of rays to
 * differ, and compare the GPU path with the reference's own kernels (same approximations) bit for bit.
 * Where the kernels write a * b + c in one expression nvcc contracts it into a fused multiply-add (its
 * default, -fmad=true, which the reference's build keeps); those spots use fmaf here.
 * ------------------------------------------------------------------------------------------ */

#define ORC_MAX_HITS 1024  /* modules/NeRF/InstantNerf.h:24 */

/* modules/NeRF/otherKernels.cu:91-154 */
void orc_ray_aabb(long num_rays, const float* rays_o, const float* rays_d, const float* aabb_min, const float* aabb_max,
                  int num_cascades, float* rays_d_inv, float* nears, float* fars) {
    float scale = exp2f((float)(num_cascades - 1));
#pragma omp parallel for schedule(static)
    for (long i = 0; i < num_rays; i++) {
        float o[3], d[3], tlo[3], thi[3];
        for (int a = 0; a < 3; a++) {
            o[a] = rays_o[3 * i + a];
            d[a] = rays_d[3 * i + a];
            if (fabsf(d[a]) < 1e-8f) d[a] = 1e-8f;
            float inv = 1.0f / d[a];
            rays_d_inv[3 * i + a] = inv;
            float t1 = (aabb_min[a] * scale - o[a]) * inv;
            float t2 = (aabb_max[a] * scale - o[a]) * inv;
            if (t1 > t2) { float tmp = t1; t1 = t2; t2 = tmp; }
            tlo[a] = t1; thi[a] = t2;
        }
        float t_enter = fmaxf(fmaxf(tlo[0], tlo[1]), tlo[2]);
        float t_exit = fminf(fminf(thi[0], thi[1]), thi[2]);
        if (t_enter > t_exit || t_exit < 0.0f) { nears[i] = 0.0f; fars[i] = 0.0f; }
        else { nears[i] = fmaxf(t_enter, 0.0f); fars[i] = t_exit; }
    }
}

/* modules/NeRF/processRays.cu:11-19 */
static inline int get_cascade(const float* pos, const float* aabb_min, const float* aabb_max, int num_cascades) {
    float rx = fmaxf(pos[0] / aabb_max[0], pos[0] / aabb_min[0]);
    float ry = fmaxf(pos[1] / aabb_max[1], pos[1] / aabb_min[1]);
    float rz = fmaxf(pos[2] / aabb_max[2], pos[2] / aabb_min[2]);
    float max_scale = fmaxf(rx, fmaxf(ry, rz));
    if (max_scale <= 1.0f) return 0;
    int cascade = (int)ceilf(log2f(max_scale));
    return imax(0, imin(cascade, num_cascades - 1));
}

/* modules/NeRF/processRays.cu:21-46 */
static inline void contract_pos(const float* pos, const float* aabb_min, const float* aabb_max, float* out) {
    for (int a = 0; a < 3; a++) {
        float extent = aabb_max[a] - aabb_min[a];
        float rel = (pos[a] - aabb_min[a]) / extent;
        float n = fmaf(rel, 2.0f, -1.0f);
        float c = fabsf(n) <= 1.0f ? n : (2.0f - 1.0f / fabsf(n)) * copysignf(1.0f, n);
        out[a] = fmaxf(0.0f, fminf((c + 2.0f) * 0.25f, 1.0f));
    }
}

void orc_contract_pos(long n, const float* pos3, const float* aabb_min, const float* aabb_max, float* out3) {
    for (long i = 0; i < n; i++) contract_pos(pos3 + 3 * i, aabb_min, aabb_max, out3 + 3 * i);
}

/* modules/NeRF/processRays.cu:83-93 */
static inline uint32_t mipmap_offset(const uint32_t* base_res, int target_level) {
    uint32_t offset = 0, rx = base_res[0], ry = base_res[1], rz = base_res[2];
    for (int l = 0; l < target_level; ++l) {
        offset += rx * ry * rz;
        rx >>= 1; ry >>= 1; rz >>= 1;
    }
    return offset;
}

uint32_t orc_pyramid_cells(const uint32_t* grid_res, int levels) { return mipmap_offset(grid_res, levels); }

/* One ray through the hierarchical DDA of march_rays_dda_calc_hits / march_rays_dda_offset
 * (modules/NeRF/processRays.cu:626-737, 801-929).  With t_out == NULL it only counts. */
static uint32_t march_one(const float* o, const float* d, const float* d_inv, float t_min, float t_max_ray,
                          const uint8_t* grid, const uint32_t* res, const float* aabb_min, const float* aabb_max,
                          int num_cascades, int levels, int spv, uint32_t ray_id, float* t_out, uint32_t* ray_out,
                          float* pos4_out) {
    float extent[3] = {aabb_max[0] - aabb_min[0], aabb_max[1] - aabb_min[1], aabb_max[2] - aabb_min[2]};
    int step[3] = {d[0] >= 0.0f ? 1 : -1, d[1] >= 0.0f ? 1 : -1, d[2] >= 0.0f ? 1 : -1};
    uint32_t hit_count = 0;
    float current_t = t_min;
    int level = levels - 1;
    uint32_t total_mip = mipmap_offset(res, levels);
    /* advances of the ray; bounded like the product's walk (see below) */
    uint32_t advances = 0;
    while (current_t < t_max_ray && hit_count < ORC_MAX_HITS && advances < (1u << 16)) {
        float pos[3] = {fmaf(current_t, d[0], o[0]), fmaf(current_t, d[1], o[1]), fmaf(current_t, d[2], o[2])};
        int cascade = get_cascade(pos, aabb_min, aabb_max, num_cascades);
        float cs = exp2f((float)cascade);
        float cmin[3], cext[3], vsize[3];
        uint32_t rl[3];
        int vi[3];
        for (int a = 0; a < 3; a++) {
            cmin[a] = aabb_min[a] * cs;
            cext[a] = extent[a] * cs;
            rl[a] = res[a] >> level;
            vsize[a] = cext[a] / (float)rl[a];
            float rel = (pos[a] - cmin[a]) / cext[a];
            vi[a] = imax(0, imin((int)floorf(rel * (float)rl[a]), (int)rl[a] - 1));
        }
        uint32_t flat = (uint32_t)cascade * total_mip + mipmap_offset(res, level) + (uint32_t)vi[2] * (rl[0] * rl[1]) +
                        (uint32_t)vi[1] * rl[0] + (uint32_t)vi[0];
        int occupied = (grid[flat >> 3] >> (flat & 7)) & 1;
        float tmax[3];
        for (int a = 0; a < 3; a++) {
            float nb = fmaf((float)vi[a] + (step[a] > 0 ? 1.0f : 0.0f), vsize[a], cmin[a]);
            tmax[a] = (nb - o[a]) * d_inv[a];
        }
        float next_t = fminf(fminf(tmax[0], tmax[1]), tmax[2]);
        if (occupied) {
            if (level > 0) { level--; continue; }
            if (t_out == NULL) {
                int n = spv, remaining = ORC_MAX_HITS - (int)hit_count;
                if (n > remaining) n = remaining;
                hit_count += (uint32_t)n;
            } else {
                float span = next_t - current_t;
                for (int k = 0; k < spv; ++k) {
                    if (hit_count >= ORC_MAX_HITS) break;
                    float t_k = fmaf(((float)k + 0.5f) / (float)spv, span, current_t);
                    t_out[hit_count] = t_k;
                    ray_out[hit_count] = ray_id;
                    float p[3] = {fmaf(t_k, d[0], o[0]), fmaf(t_k, d[1], o[1]), fmaf(t_k, d[2], o[2])};
                    contract_pos(p, aabb_min, aabb_max, pos4_out + 4 * hit_count);
                    pos4_out[4 * hit_count + 3] = 0.0f;
                    hit_count++;
                }
            }
        }
        /* The reference's advance (processRays.cu:733,925).  From t = 256 on, 1e-5 is rounded away and a voxel face a
         * rounding error behind t leaves t unchanged: the reference would loop forever.  Where the expression makes
         * progress it is kept bit for bit; otherwise t moves to the next float, and the advances are bounded. */
        {
            float nt = fmaxf(current_t + 1e-5f, next_t + 1e-6f);
            current_t = nt > current_t ? nt : nextafterf(current_t, INFINITY);
        }
        advances++;
        level = levels - 1;
    }
    return hit_count;
}

/* Pass 1: samples per ray.  modules/NeRF/processRays.cu:626-737 */
void orc_march_count(long num_rays, const float* rays_o, const float* rays_d, const float* rays_d_inv, const float* nears,
                     const float* fars, const uint8_t* grid, const uint32_t* res, const float* aabb_min,
                     const float* aabb_max, int num_cascades, int levels, int spv, uint32_t* num_steps) {
#pragma omp parallel for schedule(dynamic, 64)
    for (long i = 0; i < num_rays; i++)
        num_steps[i] = march_one(rays_o + 3 * i, rays_d + 3 * i, rays_d_inv + 3 * i, nears[i], fars[i], grid, res, aabb_min,
                                 aabb_max, num_cascades, levels, spv, (uint32_t)i, NULL, NULL, NULL);
}

/* Pass 2: t, ray id and contracted position of every sample, at ray_offsets[i] - base.
 * modules/NeRF/processRays.cu:801-929 */
void orc_march_emit(long num_rays, const float* rays_o, const float* rays_d, const float* rays_d_inv, const float* nears,
                    const float* fars, const uint8_t* grid, const uint32_t* res, const float* aabb_min,
                    const float* aabb_max, int num_cascades, int levels, int spv, const uint32_t* ray_offsets,
                    uint32_t base, float* t_out, uint32_t* ray_out, float* pos4_out) {
#pragma omp parallel for schedule(dynamic, 64)
    for (long i = 0; i < num_rays; i++) {
        uint32_t ob = ray_offsets[i] - base;
        march_one(rays_o + 3 * i, rays_d + 3 * i, rays_d_inv + 3 * i, nears[i], fars[i], grid, res, aabb_min, aabb_max,
                  num_cascades, levels, spv, (uint32_t)i, t_out + ob, ray_out + ob, pos4_out + 4 * (long)ob);
    }
}

/* Exclusive prefix sum (custom_exclusive_sum, modules/NeRF/processRays.cu:486-549; CPU twin
 * test_kernels/testProcessRays.cu cpu_exclusive_sum). */
void orc_exclusive_sum(long n, const uint32_t* in, uint32_t* out) {
    uint32_t acc = 0;
    for (long i = 0; i < n; i++) { out[i] = acc; acc += in[i]; }
}

/* Largest ray prefix that fits the sample budget, starting at rays_done.
 * find_cutoff_ray_kernel / find_cutoff_ray_from_kernel, modules/NeRF/processRays.cu:739-799.
 * Returns the absolute index one past the last ray that fits (rays_done if none fits). */
uint32_t orc_find_cutoff(long num_rays, const uint32_t* ray_offsets, const uint32_t* num_steps, uint32_t batch_size,
                         uint32_t rays_done) {
    uint32_t result = rays_done;
    if ((long)rays_done >= num_rays) return result;
    uint32_t base = ray_offsets[rays_done];
    for (long i = rays_done; i < num_rays; i++) {
        uint32_t incl = ray_offsets[i] + num_steps[i] - base;
        if (incl <= batch_size) {
            int boundary = 1;
            if (i < num_rays - 1 && ray_offsets[i + 1] + num_steps[i + 1] - base <= batch_size) boundary = 0;
            if (boundary) result = (uint32_t)(i + 1);
        }
    }
    return result;
}

/* ------------------------------------------------------------------------------------------
 * Compositing, distortion loss, loss gradients
 * ------------------------------------------------------------------------------------------ */

/* Inference compositing with early termination at T < 1e-4.  modules/NeRF/compositing.cu:5-78.
 * num_steps is indexed by r, ray_offsets by r + rays_done, samples start at ray_offsets[] - base. */
void orc_render_rays(long num_rays, uint32_t base, uint32_t rays_done, const uint32_t* ray_offsets, const uint32_t* num_steps,
                     const float* t_sorted, const float* sigma, const float* rgb, const float* rgb_true, float* final_rgb,
                     float* final_depth, float* phi_out, const float* bg) {
#pragma omp parallel for schedule(dynamic, 64)
    for (long r = 0; r < num_rays; r++) {
        uint32_t offset = ray_offsets[r + rays_done] - base;
        uint32_t count = num_steps[r];
        float T = 1.0f, rc = 0.0f, gc = 0.0f, bc = 0.0f, depth = 0.0f;
        for (uint32_t i = 0; i < count; ++i) {
            uint32_t idx = offset + i;
            float t = t_sorted[idx];
            float delta_t = (i < count - 1) ? t_sorted[idx + 1] - t : 1e-3f;
            if (delta_t < 0.0f) delta_t = 0.0f;
            float alpha = 1.0f - expf(-sigma[idx] * delta_t);
            float weight = alpha * T;
            rc += weight * rgb[idx * 3 + 0];
            gc += weight * rgb[idx * 3 + 1];
            bc += weight * rgb[idx * 3 + 2];
            depth += weight * t;
            T *= (1.0f - alpha);
            if (T < 1e-4f) break;
        }
        rc += T * bg[0]; gc += T * bg[1]; bc += T * bg[2];
        final_rgb[r * 3 + 0] = rc; final_rgb[r * 3 + 1] = gc; final_rgb[r * 3 + 2] = bc;
        final_depth[r] = depth;
        if (rgb_true && phi_out) {
            phi_out[r * 3 + 0] = 2.0f * (rc - rgb_true[r * 3 + 0]);
            phi_out[r * 3 + 1] = 2.0f * (gc - rgb_true[r * 3 + 1]);
            phi_out[r * 3 + 2] = 2.0f * (bc - rgb_true[r * 3 + 2]);
        }
    }
}

/* modules/NeRF/compositing.cu:80-82 */
static inline float disparity_warp(float t, float t_near, float inv_g_range) {
    return (1.0f - t_near / fmaxf(t, 1e-4f)) * inv_g_range;
}

/* Training compositing: colour, depth, phi = 2(C - C*), and per-sample dL/dw of the distortion loss
 * (+ depth prior term when depth_chunk != NULL), plus weight_sum[r] = sum_i w_i dL/dw_i.
 * modules/NeRF/compositing.cu:84-213. */
void orc_render_rays_distortion(long num_rays, const uint32_t* ray_offsets, const uint32_t* num_steps, const float* t_sorted,
                                const float* sigma_in, const float* depth_chunk, const float* sigma_chunk, const float* rgb,
                                const float* rgb_true, float* final_rgb, float* final_depth, float* phi_out, float* dw_out,
                                float* weight_sum, float lambda_dist, float lambda_depth, const float* bg) {
#pragma omp parallel for schedule(dynamic, 64)
    for (long r = 0; r < num_rays; r++) {
        uint32_t offset = ray_offsets[r];
        uint32_t count = num_steps[r];
        float d_prior = depth_chunk ? depth_chunk[r] : -1.0f;
        float sigma_prior = sigma_chunk ? sigma_chunk[r] : -1.0f;
        float depth_weight_loss = (d_prior >= 0) ? lambda_depth : 0.0f;
        float t_near = (count > 0) ? fmaxf(t_sorted[offset], 1e-4f) : 1.0f;
        float t_far_ray = (count > 0) ? t_sorted[offset + count - 1] : 1.0f;
        float g_far = 1.0f - t_near / fmaxf(t_far_ray, t_near + 1e-4f);
        float inv_g_range = (g_far > 1e-6f) ? (1.0f / g_far) : 0.0f;
        float T = 1.0f, rc = 0.0f, gc = 0.0f, bc = 0.0f, depth = 0.0f;
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
            float alpha = 1.0f - expf(-sigma_in[idx] * delta_t);
            float weight = alpha * T;
            rc += weight * rgb[idx * 3 + 0];
            gc += weight * rgb[idx * 3 + 1];
            bc += weight * rgb[idx * 3 + 2];
            depth += weight * t;
            T *= (1.0f - alpha);
            dw_global_sum += weight;
            dwm_global_sum += weight * m;
            float tx = (t - d_prior) / sigma_prior;
            depth_loss_sum += expf(-0.5f * tx * tx) * delta_t;
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
            float w = dw_out[idx];
            float tx = (t - d_prior) / sigma_prior;
            float depthWeight = expf(-0.5f * tx * tx) * delta_t * depth_loss_sum;
            float depthLoss = -depthWeight * (1.0f / fmaxf(w, 1e-6f));
            float dl_bilinear = m * (2 * dw_sum - dw_global_sum) + (dwm_global_sum - 2 * dwm_sum);
            float g = lambda_dist * (2 * (dl_bilinear) + c * w * delta_s) + depth_weight_loss * depthLoss;
            dw_out[idx] = g;
            weight_g_sum += w * g;
            dw_sum += w;
            dwm_sum += w * m;
        }
        weight_sum[r] = weight_g_sum;
        rc += T * bg[0]; gc += T * bg[1]; bc += T * bg[2];
        final_rgb[r * 3 + 0] = rc; final_rgb[r * 3 + 1] = gc; final_rgb[r * 3 + 2] = bc;
        final_depth[r] = depth;
        if (rgb_true && phi_out) {
            phi_out[r * 3 + 0] = 2.0f * (rc - rgb_true[r * 3 + 0]);
            phi_out[r * 3 + 1] = 2.0f * (gc - rgb_true[r * 3 + 1]);
            phi_out[r * 3 + 2] = 2.0f * (bc - rgb_true[r * 3 + 2]);
        }
    }
}

/* Per-ray walk producing dL/d(colour pre-sigmoid) (fp16) and dL/dsigma * sigma per sample.
 * modules/NeRF/otherKernels.cu:303-409 with initialOffset = 0 (the only value the training loop uses).
 * density_out is [n][16] (channel 0 is the density logit), color_out is [n][color_stride] (3 valid). */
void orc_color_grad(long num_rays, const uint32_t* num_steps, const uint32_t* ray_offsets, const float* t_sorted,
                    const float* density_out16, const float* color_out, int color_stride, const float* phi,
                    const float* final_rgb, const float* dw_out, const float* weight_sum, uint16_t* color_grad,
                    int grad_stride, float* tmp_dsigma, float loss_scale, float density_bias, uint32_t total_rays_batch) {
#pragma omp parallel for schedule(dynamic, 64)
    for (long r = 0; r < num_rays; r++) {
        float currentT = 1.0f, cur[3] = {0, 0, 0}, currentWeightG = 0.0f;
        uint32_t start = ray_offsets[r];
        float wsum = weight_sum[r];
        uint32_t maxDepth = num_steps[r];
        float ph[3] = {phi[r * 3], phi[r * 3 + 1], phi[r * 3 + 2]};
        float fin[3] = {final_rgb[r * 3], final_rgb[r * 3 + 1], final_rgb[r * 3 + 2]};
        float batch_scale = 1.0f / (float)total_rays_batch;
        for (uint32_t k = 0; k < maxDepth; k++) {
            uint32_t i = start + k;
            float t_current = t_sorted[i];
            float delta_t = (k == maxDepth - 1) ? 1e-3f : fmaxf(t_sorted[i + 1] - t_current, 0.0f);
            float sigma = expf(fminf(density_out16[(long)i * 16] - density_bias, 8.0f));
            float alpha = 1.0f - expf(-sigma * delta_t);
            float weight = currentT * alpha;
            float cg[3], col[3];
            int bad = 0;
            for (int ch = 0; ch < 3; ch++) {
                col[ch] = color_out[(long)i * color_stride + ch];
                cur[ch] += weight * col[ch];
                cg[ch] = ph[ch] * weight * col[ch] * (1.0f - col[ch]) * loss_scale * batch_scale;
                cg[ch] = fmaxf(-65504.0f, fminf(65504.0f, cg[ch]));
                if (cg[ch] != cg[ch]) bad = 1;
            }
            if (bad) cg[0] = cg[1] = cg[2] = 0.0f;
            for (int ch = 0; ch < 3; ch++) color_grad[(long)i * grad_stride + ch] = f2h(cg[ch]);
            float acc = 0.0f;
            {
                float ds_r = currentT * col[0] * (1.0f - alpha) - (fin[0] - cur[0]);
                float ds_g = currentT * col[1] * (1.0f - alpha) - (fin[1] - cur[1]);
                float ds_b = currentT * col[2] * (1.0f - alpha) - (fin[2] - cur[2]);
                acc = ds_r * ph[0] + ds_g * ph[1] + ds_b * ph[2];
            }
            float g_i = dw_out[i];
            currentWeightG += weight * g_i;
            float suffix_weight = wsum - currentWeightG;
            float d_sigma_i = delta_t * acc;
            d_sigma_i += delta_t * (g_i * currentT * (1.0f - alpha) - suffix_weight);
            float ds = d_sigma_i * sigma * loss_scale * batch_scale;
            ds = fmaxf(-65504.0f, fminf(65504.0f, ds));
            if (ds != ds) ds = 0.0f;
            tmp_dsigma[i] = ds;
            currentT = currentT * (1.0f - alpha);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Occupancy grid maintenance
 * ------------------------------------------------------------------------------------------ */

/* Philox4x32-10 counter-based generator (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy
 * as 1, 2, 3", SC'11), as the CUDA toolkit's cuRAND device API (12.9, curand_kernel.h) uses it for
 * curandStatePhilox4_32_10_t: curand_init(seed, subsequence, 0) sets key = (seed lo, seed hi) and counter =
 * (0, 0, subsequence lo, subsequence hi); the first curand_uniform4 returns the four outputs of that counter
 * mapped to (0, 1] by x * 2^-32 + 2^-33.  The reference draws its occupancy samples this way
 * (modules/NeRF/otherKernels.cu:604-607, 852-855). */
static inline void philox_round(uint32_t* c, const uint32_t* k) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0];
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1];
    uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void orc_philox_uniform4(uint64_t seed, uint64_t subsequence, float* out4) {
    uint32_t c[4] = {0u, 0u, (uint32_t)subsequence, (uint32_t)(subsequence >> 32)};
    uint32_t k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    for (int r = 0; r < 10; r++) {
        philox_round(c, k);
        if (r < 9) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    }
    for (int i = 0; i < 4; i++) out4[i] = fmaf((float)c[i], 2.3283064e-10f, 2.3283064e-10f / 2.0f);
}

static inline void cell_sample(int cell_idx, const float* rnd, const float* aabb_min, const float* aabb_max,
                               const uint32_t* res, float* out4) {
    int cells = (int)(res[0] * res[1] * res[2]);
    int cascade = cell_idx / cells, local = cell_idx % cells;
    int g[3] = {local % (int)res[0], (local / (int)res[0]) % (int)res[1], local / (int)(res[0] * res[1])};
    float cs = exp2f((float)cascade);
    float pos[3];
    for (int a = 0; a < 3; a++) {
        float lo = aabb_min[a] * cs, hi = aabb_max[a] * cs;
        float cell = (hi - lo) / (float)res[a];
        pos[a] = fmaf((float)g[a] + rnd[a], cell, lo);
    }
    contract_pos(pos, aabb_min, aabb_max, out4);
    memcpy(out4 + 3, &cell_idx, 4);
}

/* One jittered sample per thread, cell id carried in .w.  modules/NeRF/otherKernels.cu:591-648 */
void orc_sample_aabb(float* samples4, const float* aabb_min, const float* aabb_max, const uint32_t* res, int N,
                     int total_cells, int cell_offset, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < N; idx++) {
        float rnd[4];
        orc_philox_uniform4(seed, (uint64_t)idx, rnd);
        int cell_idx = (N == total_cells) ? cell_offset + idx
                                          : cell_offset + imin((int)(rnd[3] * (float)total_cells), total_cells - 1);
        cell_sample(cell_idx, rnd, aabb_min, aabb_max, res, samples4 + 4 * (long)idx);
    }
}

/* Samples inside cells drawn from the active list.  modules/NeRF/otherKernels.cu:836-888 */
void orc_sample_occupied(float* samples4, const int* active, int total_active, const float* aabb_min,
                         const float* aabb_max, const uint32_t* res, int N, uint64_t seed) {
    if (total_active == 0) return;
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < N; idx++) {
        float rnd[4];
        orc_philox_uniform4(seed, (uint64_t)idx, rnd);
        int li = imin((int)(rnd[3] * (float)total_active), total_active - 1);
        cell_sample(active[li], rnd, aabb_min, aabb_max, res, samples4 + 4 * (long)idx);
    }
}

/* Per-cell maximum of sigma = expf(min(logit - bias, 8)).  modules/NeRF/otherKernels.cu:650-678
 * (an integer atomicMax on the float bits: correct for the non-negative values stored here). */
void orc_update_tmp_grid(const float* samples4, const float* density_out16, float* tmp_grid, float density_bias, int N) {
    for (int idx = 0; idx < N; idx++) {
        int cell;
        memcpy(&cell, samples4 + 4 * (long)idx + 3, 4);
        float sigma = expf(fminf(density_out16[(long)idx * 16] - density_bias, 8.0f));
        int32_t cur, val;
        memcpy(&cur, &tmp_grid[cell], 4);
        memcpy(&val, &sigma, 4);
        if (val > cur) tmp_grid[cell] = sigma;
    }
}

/* modules/NeRF/otherKernels.cu:680-694 */
void orc_update_master_grid(const float* tmp_grid, float* master, float decay, int N) {
    for (int i = 0; i < N; i++) {
        float prev = master[i];
        master[i] = (prev < 0.f) ? prev : fmaxf(prev * decay, tmp_grid[i]);
    }
}

/* Threshold min((bar / base_voxel) / 2^cascade, mean) -> level-0 bits of every cascade's pyramid.
 * modules/NeRF/otherKernels.cu:700-750.  `sum` is the sum of the master grid (the kernel takes it from
 * a CUB reduction; summation order there is not fixed). */
void orc_update_occupancy_bits(uint8_t* bitfield, const float* master, float sum, int total_cells, int cells_per_cascade,
                               int pyramid_cells, float min_optical_thickness, float base_voxel) {
    float mean = sum / (float)total_cells;
    for (int c = 0; c < total_cells; c++) {
        int cascade = c / cells_per_cascade, local = c % cells_per_cascade;
        float thr = fminf((min_optical_thickness / base_voxel) / exp2f((float)cascade), mean);
        uint32_t bit = (uint32_t)cascade * (uint32_t)pyramid_cells + (uint32_t)local;
        if (master[c] > thr) bitfield[bit >> 3] |= (uint8_t)(1u << (bit & 7));
        else bitfield[bit >> 3] &= (uint8_t)~(1u << (bit & 7));
    }
}

/* 2x2x2 OR-pooling of every level into the next, per cascade.
 * modules/NeRF/otherKernels.cu:752-807 + InstantNerf::buildMipmaps, InstantNerf.cu:1177-1204. */
void orc_build_mipmaps(uint8_t* bitfield, const uint32_t* res, int levels, int num_cascades) {
    uint32_t S = mipmap_offset(res, levels);
    for (int c = 0; c < num_cascades; c++) {
        uint8_t* cur = bitfield + (size_t)c * (S / 8);
        uint32_t r[3] = {res[0], res[1], res[2]};
        for (int l = 0; l < levels - 1; l++) {
            uint32_t o[3] = {r[0] / 2, r[1] / 2, r[2] / 2};
            uint8_t* nxt = cur + (r[0] * r[1] * r[2]) / 8;
            uint32_t total = o[0] * o[1] * o[2];
            for (uint32_t idx = 0; idx < total; idx++) {
                uint32_t ox = idx % o[0], oy = (idx / o[0]) % o[1], oz = idx / (o[0] * o[1]);
                int occ = 0;
                for (int dz = 0; dz < 2; dz++)
                    for (int dy = 0; dy < 2; dy++)
                        for (int dx = 0; dx < 2; dx++) {
                            uint32_t in = (2 * oz + dz) * (r[0] * r[1]) + (2 * oy + dy) * r[0] + (2 * ox + dx);
                            occ |= (cur[in >> 3] >> (in & 7)) & 1;
                        }
                if (occ) nxt[idx >> 3] |= (uint8_t)(1u << (idx & 7));
                else nxt[idx >> 3] &= (uint8_t)~(1u << (idx & 7));
            }
            cur = nxt;
            r[0] = o[0]; r[1] = o[1]; r[2] = o[2];
        }
    }
}

/* Dense ids of the set level-0 cells, in increasing order (the kernel appends with an atomic counter, so
 * its order is not fixed; the set is).  modules/NeRF/otherKernels.cu:809-834 */
int orc_extract_active_cells(const uint8_t* bitfield, int* active, int total_cells, int cells_per_cascade, int pyramid_cells) {
    int n = 0;
    for (int c = 0; c < total_cells; c++) {
        uint32_t bit = (uint32_t)(c / cells_per_cascade) * (uint32_t)pyramid_cells + (uint32_t)(c % cells_per_cascade);
        if ((bitfield[bit >> 3] >> (bit & 7)) & 1) active[n++] = c;
    }
    return n;
}

/* ------------------------------------------------------------------------------------------------
 * Ray batches from a posed image set: fetchRayChunkStreamingKernel, modules/NeRF/DataLoader.cu:542-662.
 * PCG hash (:542-546), hold-out aware image / pixel pick (:566-592), depth-prior slots (:606-626), pinhole ray
 * (:628-646), RGBA over background (:651-664).  Parity unpinned for this function: the reference's loader does not build
 * without its image-decoding dependencies, so there is no reference vector; the selection is integer arithmetic on a
 * published hash, the rest a handful of fp32 operations.
 * ------------------------------------------------------------------------------------------------ */
static uint32_t orc_pcg_hash(uint32_t input) {
    uint32_t state = input * 747796405u + 2891336453u;
    uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
    return (word >> 22u) ^ word;
}
uint32_t orc_pcg(uint32_t v) { return orc_pcg_hash(v); }

void orc_fetch_ray_chunk(int offset, int size, int total_rays, uint32_t seed, int randomize, int width, int height, float focal,
                         const float* transforms, const uint8_t* images, float* rays_o, float* rays_d, float* rgb, float* out_depth,
                         float* out_sigma, uint32_t* picked, const int* rec_frame, const float* rec_u, const float* rec_v, const float* rec_D,
                         const float* rec_sigma, uint32_t num_records, float dense_fraction, float uv_scale_x, float uv_scale_y,
                         const float* bg, int holdout_every) {
    const int pixels = width * height;
    for (int idx = 0; idx < size; idx++) {
        uint32_t global_idx;
        if (randomize) {
            uint32_t rand_val = orc_pcg_hash((uint32_t)(offset + idx) + seed);
            if (holdout_every >= 2) {
                int num_imgs = total_rays / pixels;
                int num_test = (num_imgs + holdout_every - 1) / holdout_every;
                int num_train = num_imgs - num_test;
                if (num_train < 1) {
                    global_idx = rand_val % (uint32_t)total_rays;
                } else {
                    int train_slot = (int)(rand_val % (uint32_t)num_train);
                    int block = train_slot / (holdout_every - 1);
                    int within = train_slot % (holdout_every - 1);
                    int img_idx = block * holdout_every + within + 1;
                    uint32_t r2 = orc_pcg_hash(rand_val);
                    global_idx = (uint32_t)img_idx * (uint32_t)pixels + r2 % (uint32_t)pixels;
                }
            } else {
                global_idx = rand_val % (uint32_t)total_rays;
            }
        } else {
            global_idx = (uint32_t)(offset + idx) % (uint32_t)total_rays;
        }
        int img_idx = (int)(global_idx / (uint32_t)pixels);
        int pixel_idx = (int)(global_idx % (uint32_t)pixels);
        float px = (float)(pixel_idx % width), py = (float)(pixel_idx / width);
        float oD = -1.0f, oS = -1.0f;
        if (randomize && dense_fraction > 0.0f && num_records > 0) {
            uint32_t hsel = orc_pcg_hash((uint32_t)(idx + 0x9E3779B9u) ^ (seed * 2654435761u));
            if ((float)hsel * (1.0f / 4294967296.0f) < dense_fraction) {
                uint32_t r = orc_pcg_hash(hsel) % num_records;
                int f = rec_frame[r];
                if (!(holdout_every >= 2 && (f % holdout_every == 0))) {
                    img_idx = f;
                    px = rec_u[r] * uv_scale_x;
                    py = rec_v[r] * uv_scale_y;
                    oD = rec_D[r];
                    oS = rec_sigma[r];
                    int px_i = (int)(px + 0.5f), py_i = (int)(py + 0.5f);
                    px_i = px_i < 0 ? 0 : (px_i > width - 1 ? width - 1 : px_i);
                    py_i = py_i < 0 ? 0 : (py_i > height - 1 ? height - 1 : py_i);
                    global_idx = (uint32_t)img_idx * (uint32_t)pixels + (uint32_t)(py_i * width + px_i);
                }
            }
        }
        float dx = (px - width * 0.5f) / focal, dy = -(py - height * 0.5f) / focal, dz = -1.0f;
        float inv = 1.0f / sqrtf(dx * dx + dy * dy + dz * dz);
        dx *= inv; dy *= inv; dz *= inv;
        const float* m = transforms + (size_t)img_idx * 16;
        rays_o[3 * idx + 0] = m[3]; rays_o[3 * idx + 1] = m[7]; rays_o[3 * idx + 2] = m[11];
        rays_d[3 * idx + 0] = m[0] * dx + m[1] * dy + m[2] * dz;
        rays_d[3 * idx + 1] = m[4] * dx + m[5] * dy + m[6] * dz;
        rays_d[3 * idx + 2] = m[8] * dx + m[9] * dy + m[10] * dz;
        const uint8_t* c = images + (size_t)global_idx * 4;
        float fa = c[3] / 255.0f;
        for (int k = 0; k < 3; k++) rgb[3 * idx + k] = (c[k] / 255.0f) * fa + bg[k] * (1.0f - fa);
        if (out_depth) out_depth[idx] = oD;
        if (out_sigma) out_sigma[idx] = oS;
        if (picked) picked[idx] = global_idx;
    }
}
