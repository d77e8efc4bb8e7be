// Warp-level fused MLP forward on mma.sync m16n8k16 (fp16 x fp16 -> fp32).
//
// One warp owns 16 consecutive rows of the batch through every layer.  Layer outputs never leave
// registers: the accumulator fragments of two adjacent 8-column tiles, rounded to fp16, are exactly the
// A fragment of the next layer's 16-wide k chunk.  Weights of all layers sit in shared memory for the
// lifetime of the CTA, row stride padded by 8 halves so ldmatrix is bank-conflict free.
//
// Arithmetic follows the reference's WMMA kernels (modules/TinyMLP/networkFusion.cu:102-194):
// fp32 accumulation over k, bias added in fp32 after the sum, ReLU, hidden activations rounded to fp16,
// last layer linear or sigmoid 1/(1+expf(-v)).
#pragma once

#include "common.cuh"

namespace nb {

constexpr int TILE_ROWS = 128;  // batch rows per CTA tile (8 warps x 16 rows)
constexpr int CTA_THREADS = 256;

// K0V: input columns that exist in global memory (weights of layer 0 are [out][K0V], the input rows K0V wide); the
// kernels work on K0 >= K0V columns, the extra ones zero.  Only the forward kernels accept K0V != K0.
template <int K0_, int H_, int OUT_, int NL_, int K0V_ = K0_>
struct MlpShape {
    static constexpr int K0 = K0_, H = H_, OUT = OUT_, NL = NL_, K0V = K0V_;
    static_assert(K0 % 16 == 0 && H % 16 == 0 && OUT % 8 == 0, "dims must fit m16n8k16 tiles");
    static_assert(K0V % 8 == 0 && K0V > 0 && K0V <= K0, "valid input columns come in 16-byte chunks");
    static_assert(NL >= 1 && NL <= NB_MAX_LAYERS, "layer count");
    __host__ __device__ static constexpr int in_dim(int l) { return l == 0 ? K0 : H; }
    __host__ __device__ static constexpr int in_dim_global(int l) { return l == 0 ? K0V : H; }
    __host__ __device__ static constexpr int out_dim(int l) { return l == NL - 1 ? OUT : H; }
    // rows of layer l in the shared copy: the last layer is padded to 16 rows of zeros when OUT == 8 so
    // a 16-deep k chunk over the output dimension (backward) never reads past the layer
    __host__ __device__ static constexpr int out_rows_padded(int l) { return out_dim(l) < 16 ? 16 : out_dim(l); }
    __host__ __device__ static constexpr int w_off(int l) {
        int o = 0;
        for (int i = 0; i < l; i++) o += in_dim_global(i) * out_dim(i);
        return o;
    }
    __host__ __device__ static constexpr int b_off(int l) {
        int o = 0;
        for (int i = 0; i < l; i++) o += out_dim(i);
        return o;
    }
    __host__ __device__ static constexpr int sw_off(int l) {
        int o = 0;
        for (int i = 0; i < l; i++) o += (in_dim(i) + 8) * out_rows_padded(i);
        return o;
    }
    static constexpr int W_TOTAL = w_off(NL);
    static constexpr int B_TOTAL = b_off(NL);
    static constexpr int SW_TOTAL = sw_off(NL);  // halves
    static constexpr int MAXW = (K0 > H ? K0 : H);
    static constexpr int TILE_STRIDE = MAXW + 8;  // halves; (MAXW+8)*2 bytes is a multiple of 16
};

template <class S, int L>
__device__ __forceinline__ void load_layer_weights(const __half* __restrict__ W, __half* sW, int tid) {
    if constexpr (L < S::NL) {
        constexpr int K = S::in_dim(L), KG = S::in_dim_global(L), N = S::out_dim(L), NP = S::out_rows_padded(L);
        constexpr int CPR = K / 8;  // 16-byte chunks per row
        for (int c = tid; c < NP * CPR; c += CTA_THREADS) {
            int r = c / CPR, c8 = c % CPR;
            const bool valid = r < N && c8 * 8 < KG;   // rows past the layer and columns past the real input are zero
            cp_async16(&sW[S::sw_off(L) + r * (K + 8) + c8 * 8], valid ? &W[S::w_off(L) + r * KG + c8 * 8] : W, valid);
        }
        load_layer_weights<S, L + 1>(W, sW, tid);
    }
}

// All layers' fp16 weights -> padded shared layout (cp.async, caller waits), fp32 biases behind them.
template <class S>
__device__ __forceinline__ void load_weights_to_smem(const __half* __restrict__ W, const float* __restrict__ bias,
                                                     __half* sW, float* sBias, int tid) {
    load_layer_weights<S, 0>(W, sW, tid);
    if (bias != nullptr && sBias != nullptr)
        for (int i = tid; i < S::B_TOTAL; i += CTA_THREADS) sBias[i] = bias[i];
}

struct FwdCtx {
    const __half* sW;
    const float* sBias;
    __half* tile_rows;  // this warp's 16 rows of the CTA tile (input on entry, staging afterwards)
    float* out;         // fp32 output rows, out_stride floats apart; only columns < out_valid are written
    int out_stride;
    int out_valid;      // even
    __half* acts;       // hidden activations in global memory, nullable
    __half* smem_act[NB_MAX_LAYERS];  // per hidden layer: this warp's 16 rows of a shared-memory tile to receive the
    int smem_act_stride;              // activation (nullable), rows smem_act_stride halves apart
    int64_t row0;       // global row of the warp's first row
    int64_t n;
    int lane;
};

// c[j][.] = (A x W_l^T)[:, 8j .. 8j+7] + bias for the warp's 16 rows; sWl has rows K + 8 halves apart.
template <int K, int N>
__device__ __forceinline__ void layer_accumulate(const uint32_t (&a)[K / 16][4], const __half* sWl, const float* sBl, int lane,
                                                 float (&c)[N / 8][4]) {
    const int t = lane & 3;
#pragma unroll
    for (int j = 0; j < N / 8; j++) {
        c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.0f;
#pragma unroll
        for (int kc = 0; kc < K / 16; kc++) {
            uint32_t b0, b1;
            ldmatrix_x2(b0, b1, &sWl[(8 * j + (lane & 7)) * (K + 8) + 16 * kc + ((lane >> 3) & 1) * 8]);
            mma_16816(c[j], a[kc], b0, b1);
        }
        float2 bb = *reinterpret_cast<const float2*>(&sBl[8 * j + 2 * t]);
        c[j][0] += bb.x; c[j][1] += bb.y; c[j][2] += bb.x; c[j][3] += bb.y;
    }
}

// ReLU + fp16 rounding of accumulator tiles = the A fragments of the next layer.
template <int N>
__device__ __forceinline__ void relu_pack(const float (&c)[N / 8][4], uint32_t (&an)[N / 16][4]) {
#pragma unroll
    for (int q = 0; q < N / 16; q++) {
        an[q][0] = pack_half2(fmaxf(c[2 * q][0], 0.f), fmaxf(c[2 * q][1], 0.f));
        an[q][1] = pack_half2(fmaxf(c[2 * q][2], 0.f), fmaxf(c[2 * q][3], 0.f));
        an[q][2] = pack_half2(fmaxf(c[2 * q + 1][0], 0.f), fmaxf(c[2 * q + 1][1], 0.f));
        an[q][3] = pack_half2(fmaxf(c[2 * q + 1][2], 0.f), fmaxf(c[2 * q + 1][3], 0.f));
    }
}

// A-fragment layout -> 16 rows of a shared tile (rows `stride` halves apart).
template <int N>
__device__ __forceinline__ void store_frag_rows(const uint32_t (&an)[N / 16][4], __half* st, int stride, int lane) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int q = 0; q < N / 16; q++) {
        *reinterpret_cast<uint32_t*>(&st[g * stride + 16 * q + 2 * t]) = an[q][0];
        *reinterpret_cast<uint32_t*>(&st[(g + 8) * stride + 16 * q + 2 * t]) = an[q][1];
        *reinterpret_cast<uint32_t*>(&st[g * stride + 16 * q + 8 + 2 * t]) = an[q][2];
        *reinterpret_cast<uint32_t*>(&st[(g + 8) * stride + 16 * q + 8 + 2 * t]) = an[q][3];
    }
}

// A fragments of the warp's 16 rows from a shared tile.
template <int K>
__device__ __forceinline__ void load_frag_rows(uint32_t (&a)[K / 16][4], const __half* rows, int stride, int lane) {
#pragma unroll
    for (int kc = 0; kc < K / 16; kc++) {
        int q = lane >> 3, r = lane & 7;
        ldmatrix_x4(a[kc], &rows[(r + (q & 1) * 8) * stride + 16 * kc + (q >> 1) * 8]);
    }
}

// TO_REGS: the last layer's accumulators (bias added, output activation applied) are handed back in fin[OUT/8][4]
// instead of being written to cx.out.
template <class S, int L, int OUT_ACT, bool TO_REGS = false>
__device__ __forceinline__ void forward_layers(const uint32_t (&a)[S::in_dim(L) / 16][4], const FwdCtx& cx, float (*fin)[4] = nullptr) {
    constexpr int K = S::in_dim(L), N = S::out_dim(L);
    const int lane = cx.lane, g = lane >> 2, t = lane & 3;
    float c[N / 8][4];
    layer_accumulate<K, N>(a, cx.sW + S::sw_off(L), cx.sBias + S::b_off(L), lane, c);
    if constexpr (L < S::NL - 1) {
        uint32_t an[N / 16][4];
        relu_pack<N>(c, an);
        if (cx.smem_act[L] != nullptr) store_frag_rows<N>(an, cx.smem_act[L], cx.smem_act_stride, lane);
        if (cx.acts != nullptr) {
            // stage the 16 x N fp16 block in the warp's own tile rows, then write 16-byte chunks coalesced
            __half* st = cx.tile_rows;
            store_frag_rows<N>(an, st, S::TILE_STRIDE, lane);
            __syncwarp();
            __half* dst = cx.acts + (int64_t)L * cx.n * N;
            constexpr int CPR = N / 8;
#pragma unroll
            for (int i = 0; i < (16 * CPR) / 32; i++) {
                int ch = lane + 32 * i;
                int r = ch / CPR, c8 = ch % CPR;
                if (cx.row0 + r < cx.n) {
                    uint4 v = *reinterpret_cast<const uint4*>(&st[r * S::TILE_STRIDE + c8 * 8]);
                    st_cs_v4(&dst[(cx.row0 + r) * N + c8 * 8], v);
                }
            }
            __syncwarp();
        }
        forward_layers<S, L + 1, OUT_ACT, TO_REGS>(an, cx, fin);
    } else {
#pragma unroll
        for (int j = 0; j < N / 8; j++) {
            if constexpr (OUT_ACT == 1) {
#pragma unroll
                for (int e = 0; e < 4; e++) c[j][e] = 1.0f / (1.0f + expf(-c[j][e]));
            }
            if constexpr (TO_REGS) {
#pragma unroll
                for (int e = 0; e < 4; e++) fin[j][e] = c[j][e];
                continue;
            }
            int64_t r0 = cx.row0 + g, r1 = r0 + 8;
            const int col = 8 * j + 2 * t;
            if (col < cx.out_valid) {
                if (r0 < cx.n) *reinterpret_cast<float2*>(&cx.out[r0 * cx.out_stride + col]) = make_float2(c[j][0], c[j][1]);
                if (r1 < cx.n) *reinterpret_cast<float2*>(&cx.out[r1 * cx.out_stride + col]) = make_float2(c[j][2], c[j][3]);
            }
        }
    }
}

// Runs every layer for the warp's 16 rows whose layer-0 input sits in cx.tile_rows.
template <class S, int OUT_ACT>
__device__ __forceinline__ void mlp_forward_warp(const FwdCtx& cx) {
    uint32_t a[S::K0 / 16][4];
    load_frag_rows<S::K0>(a, cx.tile_rows, S::TILE_STRIDE, cx.lane);
    __syncwarp();
    forward_layers<S, 0, OUT_ACT>(a, cx);
}

}  // namespace nb
