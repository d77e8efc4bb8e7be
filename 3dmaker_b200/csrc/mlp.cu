// Plain fused MLP: forward (inference and activation-saving) and backward (dW, db, optional dX).
//
// Forward replaces networkFusionMMA_2d / networkFusionMMAGrad_2d (modules/TinyMLP/networkFusion.cu:56-355),
// backward replaces networkFusionMMA_Backward (modules/TinyMLP/networkFusionBackward.cu:49-646).
//
// Backward design (differs from the reference on purpose):
//   * persistent CTAs, one or more per SM, each walking 128-row tiles of the batch;
//   * dW (a reduction over batch rows) is a block-level GEMM dZ^T x A per tile whose accumulator tiles stay
//     in registers across ALL tiles of the CTA and are added to global memory once, at the end, so the
//     number of fp32 atomics is (#CTAs x #weights) instead of (#tiles x #weights);
//   * dA = dZ x W is row-parallel, one warp per 16 rows, operands through ldmatrix from shared memory;
//   * dZ between layers is rounded to fp16 and ReLU-masked with the saved activation, as the reference does.
#include <atomic>

#include "mlp_core.cuh"

namespace nb {

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <class S, int OUT_ACT>
__global__ void __launch_bounds__(CTA_THREADS) mlp_forward_kernel(const __half* __restrict__ in, const __half* __restrict__ W,
                                                                  const float* __restrict__ bias, int64_t n,
                                                                  float* __restrict__ out, __half* __restrict__ acts) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sW = reinterpret_cast<__half*>(smem_raw);
    float* sBias = reinterpret_cast<float*>(sW + S::SW_TOTAL);
    __half* tile = reinterpret_cast<__half*>(sBias + S::B_TOTAL);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    load_weights_to_smem<S>(W, bias, sW, sBias, tid);

    const int64_t row_base = (int64_t)blockIdx.x * TILE_ROWS;
    constexpr int CPR = S::K0 / 8;
    for (int c = tid; c < TILE_ROWS * CPR; c += CTA_THREADS) {
        int r = c / CPR, c8 = c % CPR;
        bool valid = row_base + r < n;
        const __half* src = valid ? &in[(row_base + r) * S::K0 + c8 * 8] : in;
        cp_async16(&tile[r * S::TILE_STRIDE + c8 * 8], src, valid);
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();

    FwdCtx cx{};
    cx.sW = sW; cx.sBias = sBias;
    cx.tile_rows = tile + warp * 16 * S::TILE_STRIDE;
    cx.out = out; cx.out_stride = S::OUT; cx.out_valid = S::OUT; cx.acts = acts;
    cx.row0 = row_base + warp * 16; cx.n = n; cx.lane = lane;
    if (cx.row0 < n) mlp_forward_warp<S, OUT_ACT>(cx);
}

template <class S>
static size_t forward_smem_bytes() {
    return (size_t)S::SW_TOTAL * 2 + (size_t)S::B_TOTAL * 4 + (size_t)TILE_ROWS * S::TILE_STRIDE * 2;
}

extern std::atomic<uint64_t> g_launch_count;

template <class S>
static int launch_forward(const nb_mlp_desc* d, const void* in, const void* W, const float* bias, int64_t n, float* out,
                          void* acts, cudaStream_t st) {
    size_t smem = forward_smem_bytes<S>();
    int grid = (int)((n + TILE_ROWS - 1) / TILE_ROWS);
    if (d->output_activation == 1) {
        NB_CUDA(cudaFuncSetAttribute(mlp_forward_kernel<S, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        mlp_forward_kernel<S, 1><<<grid, CTA_THREADS, smem, st>>>((const __half*)in, (const __half*)W, bias, n, out, (__half*)acts);
    } else {
        NB_CUDA(cudaFuncSetAttribute(mlp_forward_kernel<S, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        mlp_forward_kernel<S, 0><<<grid, CTA_THREADS, smem, st>>>((const __half*)in, (const __half*)W, bias, n, out, (__half*)acts);
    }
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
template <class S>
struct BwdShape {
    static constexpr int OUT16 = S::OUT < 16 ? 16 : S::OUT;
    static constexpr int DZ_W = (S::H > OUT16 ? S::H : OUT16);
    static constexpr int DZ_STRIDE = DZ_W + 8;
    static constexpr int A_STRIDE = S::MAXW + 8;
    // dW tiles (16 output features x 8 input features) of layer l, spread over the 8 warps
    __host__ __device__ static constexpr int m16(int l) { return S::out_rows_padded(l) / 16; }
    __host__ __device__ static constexpr int n8(int l) { return S::in_dim(l) / 8; }
    __host__ __device__ static constexpr int tiles(int l) { return m16(l) * n8(l); }
    __host__ __device__ static constexpr int tpw(int l) { return (tiles(l) + 7) / 8; }
    __host__ __device__ static constexpr int slot_off(int l) {
        int o = 0;
        for (int i = 0; i < l; i++) o += tpw(i);
        return o;
    }
    static constexpr int SLOTS = slot_off(S::NL);
};

template <class S>
struct BwdState {
    float acc[BwdShape<S>::SLOTS][4];  // dW accumulator tiles, live for the whole kernel
    float db[S::NL];                   // per-thread partial bias gradient of each layer
};

template <class S, int L, bool WRITE_DX>
__device__ __forceinline__ void backward_layer(BwdState<S>& stt, const __half* sW, __half* sDZ, __half* sA,
                                               const __half* __restrict__ act0, const __half* __restrict__ acts,
                                               __half* __restrict__ dX, int64_t row_base, int64_t n, int tid) {
    using B = BwdShape<S>;
    constexpr int K = S::in_dim(L);      // input features of layer L  (columns of A, of dA)
    constexpr int N = S::out_dim(L);     // output features of layer L (columns of dZ)
    constexpr int NP = S::out_rows_padded(L);
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int lq = lane >> 3, lr = lane & 7;

    // ---- dW_L += dZ^T x A over the 128 rows of the tile ------------------------------------------
#pragma unroll
    for (int s = 0; s < B::tpw(L); s++) {
        int id = warp + 8 * s;
        if (id < B::tiles(L)) {
            int mi = id / B::n8(L), ni = id % B::n8(L);
            float(&c)[4] = stt.acc[B::slot_off(L) + s];
#pragma unroll
            for (int ks = 0; ks < TILE_ROWS / 16; ks++) {
                uint32_t a[4], b0, b1;
                // A = dZ^T: element (m, k) = sDZ[16ks + k][16mi + m]
                ldmatrix_x4_trans(a, &sDZ[(16 * ks + (lq >> 1) * 8 + lr) * B::DZ_STRIDE + 16 * mi + (lq & 1) * 8]);
                // B = A_L: element (k, nn) = sA[16ks + k][8ni + nn]
                ldmatrix_x2_trans(b0, b1, &sA[(16 * ks + (lq & 1) * 8 + lr) * B::A_STRIDE + 8 * ni]);
                mma_16816(c, a, b0, b1);
            }
        }
    }
    // ---- db_L += column sums of dZ ------------------------------------------------------------------
    {
        constexpr int PARTS = CTA_THREADS / N;
        int col = tid % N, part = tid / N;
        float s = 0.f;
        for (int r = part; r < TILE_ROWS; r += PARTS) s += __half2float(sDZ[r * B::DZ_STRIDE + col]);
        stt.db[L] += s;
    }
    // ---- dA = dZ x W_L for the warp's 16 rows --------------------------------------------------------
    constexpr bool NEED_DA = (L > 0) || WRITE_DX;
    uint32_t packed[K / 8][2];
    if constexpr (NEED_DA) {
        const __half* sWl = sW + S::sw_off(L);
        uint32_t a[NP / 16][4];
#pragma unroll
        for (int kc = 0; kc < NP / 16; kc++)
            ldmatrix_x4(a[kc], &sDZ[(16 * warp + lr + (lq & 1) * 8) * B::DZ_STRIDE + 16 * kc + (lq >> 1) * 8]);
#pragma unroll
        for (int j = 0; j < K / 8; j++) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kc = 0; kc < NP / 16; kc++) {
                uint32_t b0, b1;
                // B element (k = out feature, nn = in feature) = W_L[16kc + k][8j + nn]
                ldmatrix_x2_trans(b0, b1, &sWl[(16 * kc + (lq & 1) * 8 + lr) * (K + 8) + 8 * j]);
                mma_16816(c, a[kc], b0, b1);
            }
            __half2 v0 = __floats2half2_rn(c[0], c[1]);  // row g
            __half2 v1 = __floats2half2_rn(c[2], c[3]);  // row g + 8
            if constexpr (L > 0) {
                // ReLU mask with the saved input activation of layer L
                __half2 a0 = *reinterpret_cast<const __half2*>(&sA[(16 * warp + g) * B::A_STRIDE + 8 * j + 2 * t]);
                __half2 a1 = *reinterpret_cast<const __half2*>(&sA[(16 * warp + g + 8) * B::A_STRIDE + 8 * j + 2 * t]);
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
    __syncthreads();  // everyone is done reading sDZ and sA of layer L

    if constexpr (NEED_DA) {
#pragma unroll
        for (int j = 0; j < K / 8; j++) {
            *reinterpret_cast<uint32_t*>(&sDZ[(16 * warp + g) * B::DZ_STRIDE + 8 * j + 2 * t]) = packed[j][0];
            *reinterpret_cast<uint32_t*>(&sDZ[(16 * warp + g + 8) * B::DZ_STRIDE + 8 * j + 2 * t]) = packed[j][1];
        }
    }
    if constexpr (L > 0) {
        // stage the input activation of layer L-1
        constexpr int KP = S::in_dim(L - 1);
        constexpr int CPR = KP / 8;
        const __half* src_base = (L - 1 == 0) ? act0 : acts + (int64_t)(L - 2) * n * S::H;
        for (int c = tid; c < TILE_ROWS * CPR; c += CTA_THREADS) {
            int r = c / CPR, c8 = c % CPR;
            bool valid = row_base + r < n;
            const __half* src = valid ? &src_base[(row_base + r) * KP + c8 * 8] : src_base;
            cp_async16(&sA[r * B::A_STRIDE + c8 * 8], src, valid);
        }
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();
        backward_layer<S, L - 1, WRITE_DX>(stt, sW, sDZ, sA, act0, acts, dX, row_base, n, tid);
    } else {
        if constexpr (WRITE_DX) {
            __syncwarp();
            constexpr int CPR = K / 8;
#pragma unroll
            for (int i = 0; i < (16 * CPR + 31) / 32; i++) {
                int ch = lane + 32 * i;
                int r = ch / CPR, c8 = ch % CPR;
                int64_t gr = row_base + 16 * warp + r;
                if (ch < 16 * CPR && gr < n) {
                    uint4 v = *reinterpret_cast<const uint4*>(&sDZ[(16 * warp + r) * B::DZ_STRIDE + c8 * 8]);
                    *reinterpret_cast<uint4*>(&dX[gr * K + c8 * 8]) = v;
                }
            }
        }
        __syncthreads();  // sDZ / sA are refilled by the next tile
    }
}

template <class S, int L>
__device__ __forceinline__ void flush_layer(const BwdState<S>& stt, float* __restrict__ dW, float* __restrict__ db, int tid) {
    using B = BwdShape<S>;
    if constexpr (L < S::NL) {
        constexpr int K = S::in_dim(L), N = S::out_dim(L);
        const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int s = 0; s < B::tpw(L); s++) {
            int id = warp + 8 * s;
            if (id < B::tiles(L)) {
                int mi = id / B::n8(L), ni = id % B::n8(L);
                const float(&c)[4] = stt.acc[B::slot_off(L) + s];
                int m0 = 16 * mi + g, m1 = m0 + 8, nn = 8 * ni + 2 * t;
                if (m0 < N) red_add_v2(&dW[S::w_off(L) + m0 * K + nn], c[0], c[1]);
                if (m1 < N) red_add_v2(&dW[S::w_off(L) + m1 * K + nn], c[2], c[3]);
            }
        }
        red_add(&db[S::b_off(L) + tid % N], stt.db[L]);
        flush_layer<S, L + 1>(stt, dW, db, tid);
    }
}

template <class S, bool WRITE_DX>
__global__ void __launch_bounds__(CTA_THREADS) mlp_backward_kernel(const __half* __restrict__ dL, const __half* __restrict__ W,
                                                                   const __half* __restrict__ act0,
                                                                   const __half* __restrict__ acts, int64_t n,
                                                                   float* __restrict__ dW, float* __restrict__ db,
                                                                   __half* __restrict__ dX) {
    using B = BwdShape<S>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sW = reinterpret_cast<__half*>(smem_raw);
    __half* sDZ = sW + S::SW_TOTAL;
    __half* sA = sDZ + TILE_ROWS * B::DZ_STRIDE;
    const int tid = threadIdx.x;

    load_weights_to_smem<S>(W, nullptr, sW, nullptr, tid);
    cp_async_commit();

    BwdState<S> stt;
#pragma unroll
    for (int s = 0; s < B::SLOTS; s++) stt.acc[s][0] = stt.acc[s][1] = stt.acc[s][2] = stt.acc[s][3] = 0.f;
#pragma unroll
    for (int l = 0; l < S::NL; l++) stt.db[l] = 0.f;

    const int64_t ntiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int64_t row_base = tile * TILE_ROWS;
        // dZ of the last layer = the loss gradient; columns up to 16 zero-filled when OUT == 8
        {
            constexpr int CPR = B::OUT16 / 8;
            constexpr int CPR_VALID = S::OUT / 8;
            for (int c = tid; c < TILE_ROWS * CPR; c += CTA_THREADS) {
                int r = c / CPR, c8 = c % CPR;
                bool valid = (row_base + r < n) && (c8 < CPR_VALID);
                const __half* src = valid ? &dL[(row_base + r) * S::OUT + c8 * 8] : dL;
                cp_async16(&sDZ[r * B::DZ_STRIDE + c8 * 8], src, valid);
            }
        }
        {
            constexpr int KP = S::in_dim(S::NL - 1);
            constexpr int CPR = KP / 8;
            const __half* src_base = (S::NL - 1 == 0) ? act0 : acts + (int64_t)(S::NL - 2) * n * S::H;
            for (int c = tid; c < TILE_ROWS * CPR; c += CTA_THREADS) {
                int r = c / CPR, c8 = c % CPR;
                bool valid = row_base + r < n;
                const __half* src = valid ? &src_base[(row_base + r) * KP + c8 * 8] : src_base;
                cp_async16(&sA[r * B::A_STRIDE + c8 * 8], src, valid);
            }
        }
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();
        backward_layer<S, S::NL - 1, WRITE_DX>(stt, sW, sDZ, sA, act0, acts, dX, row_base, n, tid);
    }
    cp_async_wait_all();
    flush_layer<S, 0>(stt, dW, db, tid);
}

template <class S>
static size_t backward_smem_bytes() {
    using B = BwdShape<S>;
    return (size_t)S::SW_TOTAL * 2 + (size_t)TILE_ROWS * B::DZ_STRIDE * 2 + (size_t)TILE_ROWS * B::A_STRIDE * 2;
}

template <class S, bool WRITE_DX>
static int launch_backward_t(const void* dL, const void* W, const void* act0, const void* acts, int64_t n, float* dW, float* db,
                             void* dX, cudaStream_t st) {
    size_t smem = backward_smem_bytes<S>();
    auto kern = mlp_backward_kernel<S, WRITE_DX>;
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    NB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, CTA_THREADS, smem));
    if (per_sm < 1) per_sm = 1;
    int64_t ntiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    int64_t grid = (int64_t)nb_num_sms() * per_sm;
    if (grid > ntiles) grid = ntiles;
    kern<<<(int)grid, CTA_THREADS, smem, st>>>((const __half*)dL, (const __half*)W, (const __half*)act0, (const __half*)acts, n,
                                               dW, db, (__half*)dX);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

template <class S>
static int launch_backward(const void* dL, const void* W, const void* act0, const void* acts, int64_t n, float* dW, float* db,
                           void* dX, cudaStream_t st) {
    if (dX != nullptr) return launch_backward_t<S, true>(dL, W, act0, acts, n, dW, db, dX, st);
    return launch_backward_t<S, false>(dL, W, act0, acts, n, dW, db, dX, st);
}

// ---------------------------------------------------------------------------------------------
// shape dispatch
// ---------------------------------------------------------------------------------------------
#define NB_MLP_SHAPES(X) \
    X(32, 64, 16, 2)     \
    X(32, 64, 8, 3)      \
    X(32, 64, 8, 2)      \
    X(32, 32, 8, 3)      \
    X(32, 32, 16, 2)     \
    X(32, 64, 16, 3)     \
    X(64, 64, 64, 2)     \
    X(64, 64, 64, 4)     \
    X(32, 32, 32, 2)     \
    X(16, 16, 16, 2)     \
    X(16, 32, 16, 3)     \
    X(32, 64, 16, 1)

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int mlp_forward_dispatch(const nb_mlp_desc* d, const void* in, const void* W, const float* bias, int64_t n, float* out, void* acts,
                         cudaStream_t st) {
#define X(K0, H, OUT, NL)                                                                           \
    if (d->input_dim == K0 && (d->hidden_dim == H || NL == 1) && d->output_dim == OUT && d->num_layers == NL) \
        return launch_forward<MlpShape<K0, H, OUT, NL>>(d, in, W, bias, n, out, acts, st);
    NB_MLP_SHAPES(X)
#undef X
    return nb_set_error(NB_ERR_UNSUPPORTED, "nb_mlp_forward: no kernel built for this (input, hidden, output, layers) shape");
}

int mlp_backward_dispatch(const nb_mlp_desc* d, const void* dL, const void* W, const void* act0, const void* acts, int64_t n,
                          float* dW, float* db, void* dX, cudaStream_t st) {
#define X(K0, H, OUT, NL)                                                                           \
    if (d->input_dim == K0 && (d->hidden_dim == H || NL == 1) && d->output_dim == OUT && d->num_layers == NL) \
        return launch_backward<MlpShape<K0, H, OUT, NL>>(dL, W, act0, acts, n, dW, db, dX, st);
    NB_MLP_SHAPES(X)
#undef X
    return nb_set_error(NB_ERR_UNSUPPORTED, "nb_mlp_backward: no kernel built for this (input, hidden, output, layers) shape");
}

}  // namespace nb

extern "C" int nb_mlp_forward(const nb_mlp_desc* mlp, const void* d_in_h, const void* d_weights_h, const float* d_biases, int64_t n,
                              float* d_out, void* d_save_acts_h, void* stream) {
    if (!mlp || !d_in_h || !d_weights_h || !d_biases || !d_out || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_mlp_forward: null pointer or negative batch");
    if (!nb::aligned16(d_in_h) || !nb::aligned16(d_weights_h) || !nb::aligned16(d_out) || !nb::aligned16(d_save_acts_h))
        return nb_set_error(NB_ERR_INVALID, "nb_mlp_forward: device pointers must be 16-byte aligned");
    if (n == 0) return NB_OK;
    return nb::mlp_forward_dispatch(mlp, d_in_h, d_weights_h, d_biases, n, d_out, d_save_acts_h, (cudaStream_t)stream);
}

extern "C" int nb_mlp_backward(const nb_mlp_desc* mlp, const void* d_dloss_h, const void* d_weights_h, const void* d_act0_h,
                               const void* d_acts_h, int64_t n, float* d_grad_w, float* d_grad_b, void* d_dx_h, void* stream) {
    if (!mlp || !d_dloss_h || !d_weights_h || !d_act0_h || !d_grad_w || !d_grad_b || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_mlp_backward: null pointer or negative batch");
    if (mlp->num_layers > 1 && !d_acts_h) return nb_set_error(NB_ERR_INVALID, "nb_mlp_backward: hidden activations missing");
    if (!nb::aligned16(d_dloss_h) || !nb::aligned16(d_weights_h) || !nb::aligned16(d_act0_h) || !nb::aligned16(d_acts_h) ||
        !nb::aligned16(d_dx_h) || (reinterpret_cast<uintptr_t>(d_grad_w) & 7u))
        return nb_set_error(NB_ERR_INVALID, "nb_mlp_backward: device pointers must be 16-byte aligned");
    if (n == 0) return NB_OK;
    return nb::mlp_backward_dispatch(mlp, d_dloss_h, d_weights_h, d_act0_h, d_acts_h, n, d_grad_w, d_grad_b, d_dx_h,
                                     (cudaStream_t)stream);
}
