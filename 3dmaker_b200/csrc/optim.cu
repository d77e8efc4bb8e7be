// Loss gradient and the fused Adam update.
//
// nb_adam_step walks ONE flat parameter arena (hash table first, MLP weights and biases behind it) in a
// single launch.  It replaces fusedAdamHashGridOptim, fusedAdamWeightsOptim, fusedAdamBiasOptim and
// zeroGradientsKernel of modules/TinyMLP/optimizerKernel.cu (three launches per network there).
// The element rules are the reference's: the hash part skips entries whose gradient is exactly zero
// (their moments do not decay) and zeroes the gradient it consumed; the dense part always updates;
// non-finite gradients, moments and weights are replaced by zero.
#include <algorithm>
#include <atomic>
#include <cstring>

#include "common.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;
extern std::atomic<int> g_grad_table_half;        // hashgrid.cu: the hash part of a gradient arena is __half2 per entry
extern std::atomic<int> g_grad_table_scale_log2;

__device__ __forceinline__ float finite_or_zero(float x) { return isfinite(x) ? x : 0.0f; }

struct AdamHyper {
    float lr, beta1, beta2, eps, bc1, bc2, inv_loss_scale;
};

// Four consecutive gradients of the hash part.  fp32 table: element 4i of the arena.  Half-precision table: the hash
// part's gradients are packed as fp16 at the start of the arena (8 bytes per group of four), scaled by the factor the
// scatter applied; the caller folds that factor into inv_loss_scale.
template <bool GRAD_HALF>
__device__ __forceinline__ float4 load_hash_grad4(const void* g, int64_t i) {
    if constexpr (GRAD_HALF) {
        uint2 raw;
        asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];\n" : "=r"(raw.x), "=r"(raw.y) : "l"(reinterpret_cast<const uint2*>(g) + i));
        const float2 a = unpack_half2(raw.x), b = unpack_half2(raw.y);
        return make_float4(a.x, a.y, b.x, b.y);
    } else {
        float4 v;
        asm volatile("ld.global.cs.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(reinterpret_cast<const float4*>(g) + i));
        return v;
    }
}
template <bool GRAD_HALF>
__device__ __forceinline__ void clear_hash_grad4(void* g, int64_t i) {
    if constexpr (GRAD_HALF) reinterpret_cast<uint2*>(g)[i] = make_uint2(0u, 0u);
    else reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// optimizerKernel.cu:142-166
__device__ __forceinline__ bool adam_sparse(float g_raw, float& m, float& v, float& w, const AdamHyper& h) {
    if (g_raw == 0.0f) return false;
    float g = finite_or_zero(g_raw * h.inv_loss_scale);
    float m_val = h.beta1 * finite_or_zero(m) + (1.0f - h.beta1) * g;
    float v_val = h.beta2 * finite_or_zero(v) + (1.0f - h.beta2) * g * g;
    float m_hat = m_val / h.bc1;
    float v_hat = v_val / h.bc2;
    float w_val = w;
    if (!isfinite(w_val)) w_val = 0.0f;
    w_val = w_val - h.lr * m_hat / (sqrtf(v_hat) + h.eps);
    if (!isfinite(w_val)) w_val = 0.0f;
    m = m_val; v = v_val; w = w_val;
    return true;
}

// optimizerKernel.cu:41-63
__device__ __forceinline__ void adam_dense(float g_raw, float& m, float& v, float& w, const AdamHyper& h) {
    float g = finite_or_zero(g_raw * h.inv_loss_scale);
    float m_val = finite_or_zero(m);
    float v_val = finite_or_zero(v);
    float w_val = w;
    if (!isfinite(w_val)) w_val = 0.0f;
    m_val = h.beta1 * m_val + (1.0f - h.beta1) * g;
    v_val = h.beta2 * v_val + (1.0f - h.beta2) * g * g;
    float m_hat = m_val / h.bc1;
    float v_hat = v_val / h.bc2;
    w_val = w_val - (h.lr * m_hat / (sqrtf(v_hat) + h.eps));
    if (!isfinite(w_val)) w_val = 0.0f;
    m = m_val; v = v_val; w = w_val;
}

// Four consecutive parameters per thread (16-byte loads).  sparse4 / total4 are counts of such groups.
template <bool GRAD_HALF>
__global__ void __launch_bounds__(256) adam_arena_kernel(float4* __restrict__ w, uint2* __restrict__ w_h, float4* __restrict__ g,
                                                         float4* __restrict__ m, float4* __restrict__ v, int64_t sparse4,
                                                         int64_t total4, AdamHyper h, AdamHyper h_hash, int zero_dense) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
        if (i < sparse4) {
            float4 gv;
            if constexpr (GRAD_HALF) gv = load_hash_grad4<true>(g, i);
            else gv = g[i];
            if (gv.x == 0.f && gv.y == 0.f && gv.z == 0.f && gv.w == 0.f) continue;  // untouched group: 16 bytes read, nothing else
            float4 mv = m[i], vv = v[i], wv = w[i];
            uint2 hv = w_h[i];
            __half2 h01 = *reinterpret_cast<__half2*>(&hv.x), h23 = *reinterpret_cast<__half2*>(&hv.y);
            if (adam_sparse(gv.x, mv.x, vv.x, wv.x, h_hash)) h01 = __halves2half2(__float2half(wv.x), __high2half(h01));
            if (adam_sparse(gv.y, mv.y, vv.y, wv.y, h_hash)) h01 = __halves2half2(__low2half(h01), __float2half(wv.y));
            if (adam_sparse(gv.z, mv.z, vv.z, wv.z, h_hash)) h23 = __halves2half2(__float2half(wv.z), __high2half(h23));
            if (adam_sparse(gv.w, mv.w, vv.w, wv.w, h_hash)) h23 = __halves2half2(__low2half(h23), __float2half(wv.w));
            m[i] = mv; v[i] = vv; w[i] = wv;
            hv.x = *reinterpret_cast<uint32_t*>(&h01); hv.y = *reinterpret_cast<uint32_t*>(&h23);
            w_h[i] = hv;
            clear_hash_grad4<GRAD_HALF>(g, i);
        } else {
            const float4 gv = g[i];
            float4 mv = m[i], vv = v[i], wv = w[i];
            adam_dense(gv.x, mv.x, vv.x, wv.x, h);
            adam_dense(gv.y, mv.y, vv.y, wv.y, h);
            adam_dense(gv.z, mv.z, vv.z, wv.z, h);
            adam_dense(gv.w, mv.w, vv.w, wv.w, h);
            m[i] = mv; v[i] = vv; w[i] = wv;
            __half2 h01 = __floats2half2_rn(wv.x, wv.y), h23 = __floats2half2_rn(wv.z, wv.w);
            uint2 hv;
            hv.x = *reinterpret_cast<uint32_t*>(&h01); hv.y = *reinterpret_cast<uint32_t*>(&h23);
            w_h[i] = hv;
            if (zero_dense) g[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}

// ---- reduce-scatter + Adam + all-gather in one kernel, over peer memory ------------------------------------------------
// Data-parallel training ends every step with: sum the ranks' gradients, update, make every replica equal again.  With
// collectives that is a reduce-scatter (or all-reduce), an optimizer launch and an all-gather, each a pass over the
// table through its own buffers.  Here every rank runs ONE kernel over its slice of the hash table: it loads the slice
// of every rank's gradient straight from that rank's memory (NVLink peer loads, summed in rank order), applies the
// reference's sparse Adam rule to its own master copy and moments, and stores the updated fp16 parameters into every
// rank's forward copy (peer stores).  Untouched 16-byte groups cost their gradient reads and nothing else.  The small
// dense tail (network weights) is summed and updated by every rank for itself - same order, same bits.
// No rank waits for another inside the kernel: the caller puts a barrier across the ranks before the launch (all
// gradients complete) and after it (all parameters delivered, all gradient reads done), then clears its own gradient.
constexpr int MAX_PEERS = 8;
struct PeerArenas {
    const float4* g[MAX_PEERS];   // gradient arena of every rank (entry `rank` = this rank's own)
    uint2* w_h[MAX_PEERS];        // fp16 parameter arena of every rank, as groups of four
};

__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.cs.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

template <bool GRAD_HALF>
__global__ void __launch_bounds__(256) adam_peer_kernel(float4* __restrict__ w, float4* __restrict__ m, float4* __restrict__ v, PeerArenas peers,
                                                        int rank, int world, int64_t lo4, int64_t hi4, int64_t sparse4, int64_t total4,
                                                        AdamHyper h, AdamHyper h_hash) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // this rank's slice of the hash table
    for (int64_t i = lo4 + first; i < hi4; i += stride) {
        float4 gv = load_hash_grad4<GRAD_HALF>(peers.g[0], i);
        for (int r = 1; r < world; r++) {
            const float4 o = load_hash_grad4<GRAD_HALF>(peers.g[r], i);
            gv.x += o.x; gv.y += o.y; gv.z += o.z; gv.w += o.w;
        }
        if (gv.x == 0.f && gv.y == 0.f && gv.z == 0.f && gv.w == 0.f) continue;
        float4 mv = m[i], vv = v[i], wv = w[i];
        uint2 hv = peers.w_h[rank][i];
        __half2 h01 = *reinterpret_cast<__half2*>(&hv.x), h23 = *reinterpret_cast<__half2*>(&hv.y);
        if (adam_sparse(gv.x, mv.x, vv.x, wv.x, h_hash)) h01 = __halves2half2(__float2half(wv.x), __high2half(h01));
        if (adam_sparse(gv.y, mv.y, vv.y, wv.y, h_hash)) h01 = __halves2half2(__low2half(h01), __float2half(wv.y));
        if (adam_sparse(gv.z, mv.z, vv.z, wv.z, h_hash)) h23 = __halves2half2(__float2half(wv.z), __high2half(h23));
        if (adam_sparse(gv.w, mv.w, vv.w, wv.w, h_hash)) h23 = __halves2half2(__low2half(h23), __float2half(wv.w));
        m[i] = mv; v[i] = vv; w[i] = wv;
        hv.x = *reinterpret_cast<uint32_t*>(&h01); hv.y = *reinterpret_cast<uint32_t*>(&h23);
        for (int r = 0; r < world; r++) peers.w_h[r][i] = hv;
    }
    // the dense tail: every rank for itself
    for (int64_t i = sparse4 + first; i < total4; i += stride) {
        float4 gv = ld_stream_f4(peers.g[0] + i);
        for (int r = 1; r < world; r++) {
            const float4 o = ld_stream_f4(peers.g[r] + i);
            gv.x += o.x; gv.y += o.y; gv.z += o.z; gv.w += o.w;
        }
        float4 mv = m[i], vv = v[i], wv = w[i];
        adam_dense(gv.x, mv.x, vv.x, wv.x, h);
        adam_dense(gv.y, mv.y, vv.y, wv.y, h);
        adam_dense(gv.z, mv.z, vv.z, wv.z, h);
        adam_dense(gv.w, mv.w, vv.w, wv.w, h);
        m[i] = mv; v[i] = vv; w[i] = wv;
        __half2 h01 = __floats2half2_rn(wv.x, wv.y), h23 = __floats2half2_rn(wv.z, wv.w);
        uint2 hv;
        hv.x = *reinterpret_cast<uint32_t*>(&h01); hv.y = *reinterpret_cast<uint32_t*>(&h23);
        peers.w_h[rank][i] = hv;
    }
}

// MSE loss and its gradient, two elements per thread.  optimizerKernel.cu:169-224.
template <int OUT_ACT>
__global__ void __launch_bounds__(256) mse_loss_grad_kernel(const float* __restrict__ pred, const __half* __restrict__ target,
                                                            __half* __restrict__ grad, float* __restrict__ total_loss,
                                                            int64_t num_elements, int padded_dim, int valid_dim, float grad_scale) {
    float local = 0.f;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < num_elements; i += (int64_t)gridDim.x * blockDim.x * 2) {
        int c1 = (int)(i % padded_dim), c2 = c1 + 1;
        float2 p = *reinterpret_cast<const float2*>(&pred[i]);
        float2 t = __half22float2(*reinterpret_cast<const __half2*>(&target[i]));
        float dx = (c1 < valid_dim) ? (p.x - t.x) : 0.0f;
        float dy = (c2 < valid_dim) ? (p.y - t.y) : 0.0f;
        local += (dx * dx) + (dy * dy);
        float gx = dx * grad_scale, gy = dy * grad_scale;
        if (OUT_ACT == 1) {
            gx *= p.x * (1.0f - p.x);
            gy *= p.y * (1.0f - p.y);
        }
        *reinterpret_cast<__half2*>(&grad[i]) = __floats2half2_rn(gx, gy);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xffffffffu, local, o);
    __shared__ float warp_sums[8];
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0 && total_loss != nullptr) {
        float s = 0.f;
        for (int k = 0; k < 8; k++) s += warp_sums[k];
        atomicAdd(total_loss, s);
    }
}

}  // namespace nb

using namespace nb;

extern "C" int nb_adam_step(float* d_w, void* d_w_h, float* d_g, float* d_m, float* d_v, int64_t sparse_count, int64_t total_count,
                            float lr, float beta1, float beta2, float eps, float bias_correction1, float bias_correction2,
                            float inv_loss_scale, int zero_dense_grads, void* stream) {
    if (!d_w || !d_w_h || !d_g || !d_m || !d_v || sparse_count < 0 || total_count < sparse_count)
        return nb_set_error(NB_ERR_INVALID, "nb_adam_step: null pointer or bad counts");
    if ((sparse_count & 3) || (total_count & 3))
        return nb_set_error(NB_ERR_INVALID, "nb_adam_step: sparse_count and total_count must be multiples of 4");
    uintptr_t bits = reinterpret_cast<uintptr_t>(d_w) | reinterpret_cast<uintptr_t>(d_g) | reinterpret_cast<uintptr_t>(d_m) |
                     reinterpret_cast<uintptr_t>(d_v);
    if ((bits & 15u) || (reinterpret_cast<uintptr_t>(d_w_h) & 7u))
        return nb_set_error(NB_ERR_INVALID, "nb_adam_step: arrays must be 16-byte aligned (fp16 copy 8-byte)");
    if (total_count == 0) return NB_OK;
    AdamHyper h{lr, beta1, beta2, eps, bias_correction1, bias_correction2, inv_loss_scale};
    int64_t total4 = total_count / 4;
    int64_t blocks = (total4 + 255) / 256;
    int64_t cap = (int64_t)nb_num_sms() * 32;
    if (blocks > cap) blocks = cap;
    const bool grad_half = g_grad_table_half.load() != 0;
    AdamHyper h_hash = h;
    if (grad_half) h_hash.inv_loss_scale = inv_loss_scale / (float)(1u << g_grad_table_scale_log2.load());
    if (grad_half)
        adam_arena_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((float4*)d_w, (uint2*)d_w_h, (float4*)d_g, (float4*)d_m,
                                                                                    (float4*)d_v, sparse_count / 4, total4, h, h_hash, zero_dense_grads);
    else
        adam_arena_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((float4*)d_w, (uint2*)d_w_h, (float4*)d_g, (float4*)d_m,
                                                                                     (float4*)d_v, sparse_count / 4, total4, h, h_hash, zero_dense_grads);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_adam_step_peer(float* d_w, float* d_m, float* d_v, const float* const* peer_grads, void* const* peer_w_h, int rank, int world,
                                 int64_t sparse_count, int64_t total_count, float lr, float beta1, float beta2, float eps,
                                 float bias_correction1, float bias_correction2, float inv_loss_scale, void* stream) {
    if (!d_w || !d_m || !d_v || !peer_grads || !peer_w_h || sparse_count < 0 || total_count < sparse_count)
        return nb_set_error(NB_ERR_INVALID, "nb_adam_step_peer: null pointer or bad counts");
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) return nb_set_error(NB_ERR_LIMIT, "nb_adam_step_peer: 1 to 8 ranks, rank below that");
    if ((sparse_count % (4 * (int64_t)world)) || (total_count & 3))
        return nb_set_error(NB_ERR_INVALID, "nb_adam_step_peer: sparse_count must be a multiple of 4 x ranks, total_count of 4");
    PeerArenas peers{};
    uintptr_t bits = reinterpret_cast<uintptr_t>(d_w) | reinterpret_cast<uintptr_t>(d_m) | reinterpret_cast<uintptr_t>(d_v);
    for (int r = 0; r < world; r++) {
        if (!peer_grads[r] || !peer_w_h[r]) return nb_set_error(NB_ERR_INVALID, "nb_adam_step_peer: null peer pointer");
        bits |= reinterpret_cast<uintptr_t>(peer_grads[r]) | (reinterpret_cast<uintptr_t>(peer_w_h[r]) << 1);
        peers.g[r] = reinterpret_cast<const float4*>(peer_grads[r]);
        peers.w_h[r] = reinterpret_cast<uint2*>(peer_w_h[r]);
    }
    if (bits & 15u) return nb_set_error(NB_ERR_INVALID, "nb_adam_step_peer: arrays must be 16-byte aligned (fp16 copies 8-byte)");
    if (total_count == 0) return NB_OK;
    AdamHyper h{lr, beta1, beta2, eps, bias_correction1, bias_correction2, inv_loss_scale};
    const int64_t shard4 = sparse_count / world / 4;
    const int64_t lo4 = rank * shard4, hi4 = lo4 + shard4;
    const int64_t work = std::max<int64_t>(shard4, 1);
    int64_t blocks = (work + 255) / 256;
    const int64_t cap = (int64_t)nb_num_sms() * 8;   // enough loads in flight to cover the latency of the peer reads
    if (blocks > cap) blocks = cap;
    const bool grad_half = g_grad_table_half.load() != 0;
    AdamHyper h_hash = h;
    if (grad_half) h_hash.inv_loss_scale = inv_loss_scale / (float)(1u << g_grad_table_scale_log2.load());
    if (grad_half)
        adam_peer_kernel<true><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((float4*)d_w, (float4*)d_m, (float4*)d_v, peers, rank, world, lo4,
                                                                                   hi4, sparse_count / 4, total_count / 4, h, h_hash);
    else
        adam_peer_kernel<false><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((float4*)d_w, (float4*)d_m, (float4*)d_v, peers, rank, world, lo4,
                                                                                    hi4, sparse_count / 4, total_count / 4, h, h_hash);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

// Device memory another process of this machine can map (cudaIpc*): the hand-shake that gives every rank the peer
// pointers nb_adam_step_peer takes.  handle64: 64 bytes (cudaIpcMemHandle_t).
extern "C" int nb_ipc_export(void* d_base, void* handle64) {
    if (!d_base || !handle64) return nb_set_error(NB_ERR_INVALID, "nb_ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
    NB_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), d_base));
    return NB_OK;
}
extern "C" int nb_ipc_open(const void* handle64, void** d_ptr_out) {
    if (!handle64 || !d_ptr_out) return nb_set_error(NB_ERR_INVALID, "nb_ipc_open: null pointer");
    cudaIpcMemHandle_t hnd;
    memcpy(&hnd, handle64, sizeof(hnd));
    NB_CUDA(cudaIpcOpenMemHandle(d_ptr_out, hnd, cudaIpcMemLazyEnablePeerAccess));
    return NB_OK;
}
extern "C" int nb_ipc_close(void* d_ptr) {
    if (!d_ptr) return NB_OK;
    NB_CUDA(cudaIpcCloseMemHandle(d_ptr));
    return NB_OK;
}
// cudaMalloc / cudaFree for hosts that hold their arrays in another runtime's allocator: memory that can be exported.
extern "C" int nb_device_alloc(int64_t bytes, void** d_ptr_out) {
    if (bytes <= 0 || !d_ptr_out) return nb_set_error(NB_ERR_INVALID, "nb_device_alloc: bad size or null pointer");
    NB_CUDA(cudaMalloc(d_ptr_out, (size_t)bytes));
    NB_CUDA(cudaMemset(*d_ptr_out, 0, (size_t)bytes));
    return NB_OK;
}
extern "C" int nb_device_free(void* d_ptr) {
    if (d_ptr) NB_CUDA(cudaFree(d_ptr));
    return NB_OK;
}

extern "C" int nb_mse_loss_grad(const float* d_pred, const void* d_target_h, void* d_grad_h, float* d_total_loss, int64_t n,
                                int padded_dim, int valid_dim, float loss_scale, int output_activation, void* stream) {
    if (!d_pred || !d_target_h || !d_grad_h || n < 0 || padded_dim < 2 || (padded_dim & 1) || valid_dim < 1 || valid_dim > padded_dim)
        return nb_set_error(NB_ERR_INVALID, "nb_mse_loss_grad: null pointer or bad dims (padded_dim even, 1 <= valid_dim <= padded_dim)");
    if (n == 0) return NB_OK;
    int64_t num = n * padded_dim;
    // (2 / (batch * validDim)) * loss_scale, optimizerKernel.cu:388
    float grad_scale = (2.0f / (float)(n * valid_dim)) * loss_scale;
    int64_t blocks = ((num + 1) / 2 + 255) / 256;
    int64_t cap = (int64_t)nb_num_sms() * 16;
    if (blocks > cap) blocks = cap;
    if (output_activation == 1)
        mse_loss_grad_kernel<1><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_pred, (const __half*)d_target_h, (__half*)d_grad_h,
                                                                                    d_total_loss, num, padded_dim, valid_dim, grad_scale);
    else
        mse_loss_grad_kernel<0><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_pred, (const __half*)d_target_h, (__half*)d_grad_h,
                                                                                    d_total_loss, num, padded_dim, valid_dim, grad_scale);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}
