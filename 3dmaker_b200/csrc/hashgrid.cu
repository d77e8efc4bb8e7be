// Multiresolution hash grid: geometry set-up, index dump, encode forward (stand-alone and fused with the
// MLP), gradient scatter.
//
// Replaces the encode body and launchers of modules/TinyMLP/networkFusionHashtable.cu and the
// hashTableScatter_Backward kernel of modules/TinyMLP/networkFusionBackwardHashtable.cu:783-910.
//
// Thread mapping of the encode (differs from the reference, which gives each thread 4 levels of one
// point): a CTA owns 128 points; thread t works on point (t & 127) and on one half of the levels, so a
// warp always works on 32 consecutive points of ONE level at a time.  Coarse dense levels then hit a
// handful of cache lines per warp, and the 8 corner loads of two levels are issued back to back before
// either blend starts (16 independent 4-byte gathers in flight per thread).
#include <algorithm>
#include <atomic>
#include <string>

#include "hashgrid_core.cuh"
#include "field_backward_tc.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

// Resolution of every level.  out[l]: the forward kernel's expression sequence, a power at levels 0,4,8,12 and
// repeated multiplication by b in between (modules/TinyMLP/networkFusionHashtable.cu:124-128,218).
// out[NB_MAX_LEVELS + l]: the split scatter kernel's expression (networkFusionBackwardHashtable.cu:805).
__global__ void level_scales_kernel(int lowestSize, float b, float log2b, int L, float* out) {
    int l = threadIdx.x;
    if (l >= L) return;
    int levelStart = (l / 4) * 4;
    float N_l_float = lowestSize * __powf(b, levelStart);
    for (int i = levelStart; i < l; i++) N_l_float *= b;
    out[l] = N_l_float;
    int level = l;
    out[NB_MAX_LEVELS + l] = lowestSize * exp2f(level * log2b);
}

constexpr int ENC_STRIDE = 2 * NB_MAX_LEVELS + 8;

__global__ void __launch_bounds__(CTA_THREADS) encode_forward_kernel(const __grid_constant__ GridParams gp, const float* __restrict__ pos4,
                                                                     const uint32_t* __restrict__ table2, int64_t n,
                                                                     __half* __restrict__ enc_out) {
    __shared__ __align__(16) __half tile[TILE_ROWS * ENC_STRIDE];
    const int64_t row_base = (int64_t)blockIdx.x * TILE_ROWS;
    encode_tile<ENC_STRIDE>(gp, pos4, table2, row_base, n, tile, threadIdx.x);
    __syncthreads();
    store_enc_tile<ENC_STRIDE>(tile, enc_out, gp.L, row_base, n, threadIdx.x);
}

__global__ void hash_indices_kernel(const __grid_constant__ GridParams gp, const float* __restrict__ pos4, int64_t n, int clamp_mode,
                                    uint32_t* __restrict__ idx_out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * gp.L) return;
    int64_t p = i / gp.L;
    int l = (int)(i % gp.L);
    float4 pt = ld_nc_f4(pos4 + p * 4);
    Corners c;
    if (clamp_mode == 0) corners_of<false>(pt.x, pt.y, pt.z, gp.scales[l], l < gp.dls, gp.T, c);
    else corners_of<true>(pt.x, pt.y, pt.z, gp.sscales[l], l < gp.dls, gp.T, c);
#pragma unroll
    for (int k = 0; k < 8; k++) idx_out[i * 8 + k] = (uint32_t)l * (uint32_t)gp.T * 2u + c.idx[k] * 2u;
}

// Encode fused with the MLP: the encoded 128 x 2L tile is built in shared memory, optionally saved, then
// every warp runs all layers for its 16 rows out of registers.
template <class S, bool SAVE>
__global__ void __launch_bounds__(CTA_THREADS) grid_mlp_forward_kernel(const __grid_constant__ GridParams gp, const float* __restrict__ pos4,
                                                                       const uint32_t* __restrict__ table2,
                                                                       const __half* __restrict__ W, const float* __restrict__ bias,
                                                                       int64_t n, float* __restrict__ out,
                                                                       __half* __restrict__ save_enc, __half* __restrict__ save_acts) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sW = reinterpret_cast<__half*>(smem_raw);
    float* sBias = reinterpret_cast<float*>(sW + S::SW_TOTAL);
    __half* tile = reinterpret_cast<__half*>(sBias + S::B_TOTAL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    load_weights_to_smem<S>(W, bias, sW, sBias, tid);
    cp_async_commit();

    const int64_t row_base = (int64_t)blockIdx.x * TILE_ROWS;
    encode_tile<S::TILE_STRIDE>(gp, pos4, table2, row_base, n, tile, tid);
    if constexpr (S::K0V < S::K0) {
        // fewer levels than the 16-wide k chunk: the columns behind the encoding are zero
        for (int c = tid; c < TILE_ROWS * (S::K0 - S::K0V) / 2; c += CTA_THREADS) {
            const int r = c / ((S::K0 - S::K0V) / 2), c2 = c % ((S::K0 - S::K0V) / 2);
            *reinterpret_cast<uint32_t*>(&tile[r * S::TILE_STRIDE + S::K0V + 2 * c2]) = 0u;
        }
    }
    cp_async_wait_all();
    __syncthreads();
    if (SAVE && save_enc != nullptr) {
        store_enc_tile<S::TILE_STRIDE>(tile, save_enc, gp.L, row_base, n, tid);
        __syncthreads();
    }
    FwdCtx cx{};
    cx.sW = sW; cx.sBias = sBias;
    cx.tile_rows = tile + warp * 16 * S::TILE_STRIDE;
    cx.out = out; cx.out_stride = S::OUT; cx.out_valid = S::OUT; cx.acts = SAVE ? save_acts : nullptr;
    cx.row0 = row_base + warp * 16; cx.n = n; cx.lane = lane;
    if (cx.row0 < n) mlp_forward_warp<S, 0>(cx);
}

// Tunables of the scatter (nb_set_tuning): levels below `smem_levels` whose dense grid fits shared memory are
// accumulated per CTA in shared memory and flushed once; [level_begin, level_end) restricts the launch (profiling
// experiments).
struct ScatterTuning {
    int smem_levels = 2;
    int level_begin = 0;
    int level_end = NB_MAX_LEVELS;
};
static ScatterTuning g_scatter_tuning;
std::atomic<int> g_pair_ops{1};
std::atomic<int> g_run_merge{20};
// Half-precision gradient table (opt-in): the hash part of a gradient arena holds one __half2 per entry in its first
// half instead of two floats; scatter kernels multiply by 2^scale_log2 before rounding and the optimizer divides again.
std::atomic<int> g_grad_table_half{0};
std::atomic<int> g_grad_table_scale_log2{7};

// Where a scatter kernel finds sample i's position and the gradient of its encoding on a level.
// RowsDenc: the samples of one batch, gradients row-major ([n][denc_stride] halves, level l at columns 2l, 2l + 1).
struct RowsDenc {
    const float* pos4; const __half* denc; int stride; int64_t n;
    __device__ __forceinline__ int64_t rows() const { return n; }
    __device__ __forceinline__ bool fetch(int64_t i, int level, float4& p, float2& g) const {
        if (i >= n) return false;
        p = ld_nc_f4(pos4 + i * 4);
        g = __half22float2(*reinterpret_cast<const __half2*>(&denc[i * stride + 2 * level]));
        return true;
    }
};
// PiecesDenc: the samples of ALL ranks of a level-partitioned grid (level_partition.cu): rank q's slot of the gathered
// positions holds `cap` positions and its sample count in element `cap`; the gradients of the owner's level k for rank q's
// samples are the contiguous run pieces[(q * own + k) * cap ...].
struct PiecesDenc {
    const float* pos_all; const uint32_t* pieces; int ranks, own; int64_t cap;
    __device__ __forceinline__ int64_t rows() const { return (int64_t)ranks * cap; }
    __device__ __forceinline__ bool fetch(int64_t i, int level, float4& p, float2& g) const {
        const int q = (int)(i / cap);
        const int64_t j = i - (int64_t)q * cap;
        if (q >= ranks) return false;
        const float* slot = pos_all + (int64_t)q * (cap + 1) * 4;
        if (j >= (int64_t)__float_as_uint(__ldg(slot + cap * 4))) return false;
        p = ld_nc_f4(slot + j * 4);
        g = unpack_half2(__ldg(pieces + ((int64_t)q * own + level) * cap + j));
        return true;
    }
};

// Gradient scatter, one thread per (sample, level), level = level_base + blockIdx.y so that all CTAs resident at one
// time work on the same 2T-float slice of the gradient table.  A feature pair is one 8-byte vector reduction.
template <bool GRAD_HALF, class Fetch>
__global__ void __launch_bounds__(256) scatter_backward_kernel(const __grid_constant__ GridParams gp, const Fetch in, float* __restrict__ grads,
                                                               int level_base) {
    const int level = level_base + blockIdx.y;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
    float2 g = make_float2(0.f, 0.f);
    const bool has = in.fetch(i, level, p, g);
    scatter_level_warp<GRAD_HALF>(gp, level, p.x, p.y, p.z, g, has, grads, threadIdx.x & 31);
}

// Coarse dense levels whose whole grid fits shared memory: every CTA accumulates its share of the samples into a
// private copy of the level with shared-memory atomics and adds the non-zero entries to global memory once, so the
// heavily contended coarse entries see (#CTAs) global reductions instead of (#samples x 8).  Runs of consecutive
// samples in one cell are merged in the warp first (scatter_level_runs): on these levels a ray spends ten or more
// samples per cell, and same-address shared-memory atomics serialise.
template <class Fetch>
__global__ void __launch_bounds__(256) scatter_smem_kernel(const __grid_constant__ GridParams gp, const Fetch in, float* __restrict__ grads,
                                                           int level_base) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* acc = reinterpret_cast<float2*>(smem_raw);
    const int level = level_base + blockIdx.y;
    const float scale = gp.sscales[level];
    const int N_l = __float2int_rd(scale);
    const int cells = (N_l + 1) * (N_l + 1) * (N_l + 1);
    for (int c = threadIdx.x; c < cells; c += blockDim.x) acc[c] = make_float2(0.f, 0.f);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t n = in.rows();
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x; i0 < n; i0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = i0 + threadIdx.x;
        float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
        float2 g = make_float2(0.f, 0.f);
        const bool has = in.fetch(i, level, p, g);
        scatter_level_runs(gp, level, p.x, p.y, p.z, g, has, lane, [&](const Corners& c, const float (&v)[16]) {
#pragma unroll
            for (int k = 0; k < 8; k++) {
                atomicAdd(&acc[c.idx[k]].x, v[2 * k]);
                atomicAdd(&acc[c.idx[k]].y, v[2 * k + 1]);
            }
        });
    }
    __syncthreads();
    if (gp.grad_half) {
        uint32_t* base = reinterpret_cast<uint32_t*>(grads) + (size_t)level * gp.ls;
        for (int c = threadIdx.x; c < cells; c += blockDim.x) {
            float2 v = acc[c];
            if (v.x != 0.f || v.y != 0.f) red_add_h2(base + c, pack_half2(v.x * gp.grad_scale, v.y * gp.grad_scale));
        }
        return;
    }
    float* base = grads + (size_t)level * gp.ls * 2;
    for (int c = threadIdx.x; c < cells; c += blockDim.x) {
        float2 v = acc[c];
        if (v.x != 0.f || v.y != 0.f) red_add_v2(base + (size_t)c * 2, v.x, v.y);
    }
}

template <class S>
static int launch_grid_mlp(const GridParams& gp, const float* pos4, const void* table, const void* W, const float* bias, int64_t n,
                           float* out, void* save_enc, void* save_acts, cudaStream_t st) {
    size_t smem = (size_t)S::SW_TOTAL * 2 + (size_t)S::B_TOTAL * 4 + (size_t)TILE_ROWS * S::TILE_STRIDE * 2;
    int grid = (int)((n + TILE_ROWS - 1) / TILE_ROWS);
    if (save_enc != nullptr || save_acts != nullptr) {
        NB_CUDA(cudaFuncSetAttribute(grid_mlp_forward_kernel<S, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        grid_mlp_forward_kernel<S, true><<<grid, CTA_THREADS, smem, st>>>(gp, pos4, (const uint32_t*)table, (const __half*)W, bias, n,
                                                                          out, (__half*)save_enc, (__half*)save_acts);
    } else {
        NB_CUDA(cudaFuncSetAttribute(grid_mlp_forward_kernel<S, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        grid_mlp_forward_kernel<S, false><<<grid, CTA_THREADS, smem, st>>>(gp, pos4, (const uint32_t*)table, (const __half*)W, bias, n,
                                                                           out, nullptr, nullptr);
    }
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

static int check_desc(const nb_grid_desc* d, const char* who) {
    if (!d) return nb_set_error(NB_ERR_INVALID, who);
    if (d->num_levels < 2 || d->num_levels > NB_MAX_LEVELS || (d->num_levels & 1))
        return nb_set_error(NB_ERR_UNSUPPORTED, "hash grid: num_levels must be even and between 2 and 16");
    if (d->table_size < 2 || (d->table_size & (d->table_size - 1)))
        return nb_set_error(NB_ERR_UNSUPPORTED, "hash grid: table_size must be a power of two");
    if ((int64_t)d->num_levels * d->table_size * 2 > 0xffffffffLL)
        return nb_set_error(NB_ERR_LIMIT, "hash grid: table beyond 2^32 elements");
    return NB_OK;
}

// Leading dense levels whose (N+1)^3 float2 grid fits shared memory.
static constexpr size_t SCATTER_SMEM_CAP = 112 * 1024;

int scatter_shared_levels(const GridParams& gp, int64_t n) {
    const ScatterTuning tn = g_scatter_tuning;
    int k = 0;
    while (k < gp.L && k < gp.dls && k < tn.smem_levels && n >= 16384) {
        int N_l = (int)std::floor(gp.sscales[k]);
        if ((size_t)(N_l + 1) * (N_l + 1) * (N_l + 1) * sizeof(float2) > SCATTER_SMEM_CAP) break;
        k++;
    }
    return k;
}

// Launches the scatter of levels [level_begin, level_end) over in.rows() samples; n_hint = how many of them are real
// (decides whether the shared-memory kernel is worth its fixed cost).
template <class Fetch>
static int scatter_launch_from(const GridParams& gp, const Fetch& in, int64_t rows, int64_t n_hint, float* d_table_grads, int level_begin,
                               int level_end, cudaStream_t st) {
    const ScatterTuning tn = g_scatter_tuning;
    const int lb = std::max(level_begin, std::max(0, tn.level_begin)), le = std::min(level_end, std::min(gp.L, tn.level_end));
    if (le <= lb || rows <= 0) return NB_OK;
    const int smem_end = std::max(lb, std::min(le, scatter_shared_levels(gp, n_hint)));
    if (smem_end > lb) {
        size_t smem_bytes = 0;
        for (int l = lb; l < smem_end; l++) {
            int N_l = (int)std::floor(gp.sscales[l]);
            smem_bytes = std::max(smem_bytes, (size_t)(N_l + 1) * (N_l + 1) * (N_l + 1) * sizeof(float2));
        }
        // always the cap, not this launch's size: the attribute belongs to the function, and two host threads launching
        // levels of different size would otherwise lower it under each other's feet
        NB_CUDA(cudaFuncSetAttribute(scatter_smem_kernel<Fetch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCATTER_SMEM_CAP));
        int per_level = std::max(1, nb_num_sms() * 2 / (smem_end - lb));
        int64_t need = (rows + 255) / 256;
        dim3 grid((unsigned)std::min<int64_t>(per_level, need), smem_end - lb, 1);
        scatter_smem_kernel<Fetch><<<grid, 256, smem_bytes, st>>>(gp, in, d_table_grads, lb);
        NB_CHECK_LAUNCH();
        g_launch_count++;
    }
    if (le > smem_end) {
        dim3 grid((unsigned)((rows + 255) / 256), le - smem_end, 1);
        if (gp.grad_half) scatter_backward_kernel<true, Fetch><<<grid, 256, 0, st>>>(gp, in, d_table_grads, smem_end);
        else scatter_backward_kernel<false, Fetch><<<grid, 256, 0, st>>>(gp, in, d_table_grads, smem_end);
        NB_CHECK_LAUNCH();
        g_launch_count++;
    }
    return NB_OK;
}

int scatter_launch(const GridParams& gp, const float* d_pos4, const __half* d_denc, int denc_stride, int64_t n, float* d_table_grads,
                   int level_begin, int level_end, cudaStream_t st) {
    return scatter_launch_from(gp, RowsDenc{d_pos4, d_denc, denc_stride, n}, n, n, d_table_grads, level_begin, level_end, st);
}

int scatter_launch_pieces(const GridParams& view, const float* d_pos_all, const uint32_t* d_pieces, int ranks, int own, int64_t cap,
                          float* d_table_grads_view, cudaStream_t st) {
    return scatter_launch_from(view, PiecesDenc{d_pos_all, d_pieces, ranks, own, cap}, (int64_t)ranks * cap, (int64_t)ranks * cap, d_table_grads_view, 0,
                               view.L, st);
}

}  // namespace nb

using namespace nb;

extern "C" int nb_grid_setup(nb_grid_desc* desc, int num_levels, int table_size, int base_resolution, float growth, void* stream) {
    if (!desc) return nb_set_error(NB_ERR_INVALID, "nb_grid_setup: null descriptor");
    desc->num_levels = num_levels;
    desc->table_size = table_size;
    desc->base_resolution = base_resolution;
    desc->growth = growth;
    desc->dense_level_start = 0;
    for (int i = 0; i < NB_MAX_LEVELS; i++) desc->scales[i] = desc->scatter_scales[i] = 0.f;
    int rc = check_desc(desc, "nb_grid_setup");
    if (rc != NB_OK) return rc;
    if (base_resolution < 1 || !(growth > 1.0f)) return nb_set_error(NB_ERR_INVALID, "nb_grid_setup: base_resolution >= 1 and growth > 1 required");
    // first hashed level, host float math as in the reference's launchers (networkFusionHashtable.cu:367-377)
    float inner_term = (std::cbrt(static_cast<float>(table_size)) - 1.0f) / base_resolution;
    float continuous_level = std::log2(inner_term) / std::log2(growth);
    int dls = static_cast<int>(std::floor(continuous_level)) + 1;
    dls = std::max(0, std::min(dls, num_levels));
    desc->dense_level_start = dls;

    cudaStream_t st = (cudaStream_t)stream;
    float* d_scales = nullptr;
    NB_CUDA(cudaMalloc(&d_scales, 2 * NB_MAX_LEVELS * sizeof(float)));
    level_scales_kernel<<<1, 32, 0, st>>>(base_resolution, growth, std::log2(growth), num_levels, d_scales);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(desc->scales, d_scales, num_levels * sizeof(float), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(desc->scatter_scales, d_scales + NB_MAX_LEVELS, num_levels * sizeof(float), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_scales);
    if (e != cudaSuccess) return nb_set_cuda_error(e);
    g_launch_count++;
    return NB_OK;
}

// ---------------------------------------------------------------------------------------------------
// nb_grid_setup_noalloc: the same set-up without any allocation.
//
// Some host programs may not allocate device memory at the point where they configure a grid: a renderer
// plug-in that was handed a fixed memory budget by its host application, or a real-time loop that forbids
// cudaMalloc / cudaFree because they synchronise the whole device.  For them the 32-float scratch that
// nb_grid_setup allocates and frees lives in the library image instead: every GPU that loads the library holds
// these 128 bytes (at a 256-byte aligned address) until the process exits.
// Like nb_grid_setup the call reads the scales back to the host and waits for the stream before it returns.
// ---------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_static_level_scales[2 * NB_MAX_LEVELS];

// Device address of g_static_level_scales on each device, looked up on the first call made with that
// device current.  In host code the array's name is only a handle for cudaGetSymbolAddress, never a pointer
// a kernel could use.  Threads may race to fill an entry; they all store the same address.  The addresses
// belong to the device's context: after cudaDeviceReset they are stale and the library must be reloaded.
static std::atomic<float*> g_static_level_scales_addr[64];

extern "C" int nb_grid_setup_noalloc(nb_grid_desc* desc, int num_levels, int table_size, int base_resolution, float growth,
                                     void* stream) {
    if (!desc) return nb_set_error(NB_ERR_INVALID, "nb_grid_setup_noalloc: null descriptor");
    if (num_levels > NB_MAX_LEVELS)
        return nb_set_error(NB_ERR_LIMIT, "nb_grid_setup_noalloc: num_levels exceeds the 16 levels the static scratch holds");
    desc->num_levels = num_levels;
    desc->table_size = table_size;
    desc->base_resolution = base_resolution;
    desc->growth = growth;
    desc->dense_level_start = 0;
    for (int i = 0; i < NB_MAX_LEVELS; i++) desc->scales[i] = desc->scatter_scales[i] = 0.f;
    int rc = check_desc(desc, "nb_grid_setup_noalloc");
    if (rc != NB_OK) return rc;
    if (base_resolution < 1 || !(growth > 1.0f))
        return nb_set_error(NB_ERR_INVALID, "nb_grid_setup_noalloc: base_resolution >= 1 and growth > 1 required");
    float inner_term = (std::cbrt(static_cast<float>(table_size)) - 1.0f) / base_resolution;
    float continuous_level = std::log2(inner_term) / std::log2(growth);
    int dls = static_cast<int>(std::floor(continuous_level)) + 1;
    desc->dense_level_start = std::max(0, std::min(dls, num_levels));

    int dev = -1;
    NB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return nb_set_error(NB_ERR_LIMIT, "nb_grid_setup_noalloc: device ordinal beyond 63");
    float* d_scales = g_static_level_scales_addr[dev].load(std::memory_order_acquire);
    if (d_scales == nullptr) {
        NB_CUDA(cudaGetSymbolAddress((void**)&d_scales, g_static_level_scales));
        if (d_scales == nullptr) return nb_set_error(NB_ERR_CUDA, "nb_grid_setup_noalloc: cudaGetSymbolAddress returned a null address");
        g_static_level_scales_addr[dev].store(d_scales, std::memory_order_release);
    }
    cudaStream_t st = (cudaStream_t)stream;
    // the kernel writes entries [0, num_levels) and only those are read back, so nothing has to start at zero
    level_scales_kernel<<<1, 32, 0, st>>>(base_resolution, growth, std::log2(growth), num_levels, d_scales);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    NB_CUDA(cudaMemcpyAsync(desc->scales, d_scales, num_levels * sizeof(float), cudaMemcpyDeviceToHost, st));
    NB_CUDA(cudaMemcpyAsync(desc->scatter_scales, d_scales + NB_MAX_LEVELS, num_levels * sizeof(float), cudaMemcpyDeviceToHost, st));
    NB_CUDA(cudaStreamSynchronize(st));
    return NB_OK;
}

extern "C" int nb_hash_indices(const nb_grid_desc* desc, const float* d_pos4, int64_t n, int clamp_mode, uint32_t* d_idx_out,
                               void* stream) {
    int rc = check_desc(desc, "nb_hash_indices: null descriptor");
    if (rc != NB_OK) return rc;
    if (!d_pos4 || !d_idx_out || n < 0) return nb_set_error(NB_ERR_INVALID, "nb_hash_indices: null pointer or negative count");
    if (n == 0) return NB_OK;
    GridParams gp = make_params(desc);
    int64_t total = n * gp.L;
    hash_indices_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gp, d_pos4, n, clamp_mode, d_idx_out);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_hash_encode_forward(const nb_grid_desc* desc, const float* d_pos4, const void* d_table_h, int64_t n,
                                      void* d_enc_out_h, void* stream) {
    int rc = check_desc(desc, "nb_hash_encode_forward: null descriptor");
    if (rc != NB_OK) return rc;
    if (!d_pos4 || !d_table_h || !d_enc_out_h || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_hash_encode_forward: null pointer or negative count");
    if ((reinterpret_cast<uintptr_t>(d_pos4) & 15u) || (reinterpret_cast<uintptr_t>(d_enc_out_h) & 15u) ||
        (reinterpret_cast<uintptr_t>(d_table_h) & 3u) || (desc->num_levels % 4))
        return nb_set_error(NB_ERR_INVALID, "nb_hash_encode_forward: positions/output must be 16-byte aligned, levels a multiple of 4");
    if (n == 0) return NB_OK;
    GridParams gp = make_params(desc);
    if (reinterpret_cast<uintptr_t>(d_table_h) & 7u) gp.pair_ops = 0;
    encode_forward_kernel<<<(unsigned)((n + TILE_ROWS - 1) / TILE_ROWS), CTA_THREADS, 0, (cudaStream_t)stream>>>(
        gp, d_pos4, (const uint32_t*)d_table_h, n, (__half*)d_enc_out_h);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_grid_mlp_forward(const nb_grid_desc* desc, const nb_mlp_desc* mlp, const float* d_pos4, const void* d_table_h,
                                   const void* d_weights_h, const float* d_biases, int64_t n, float* d_out, void* d_save_enc_h,
                                   void* d_save_acts_h, void* stream) {
    int rc = check_desc(desc, "nb_grid_mlp_forward: null descriptor");
    if (rc != NB_OK) return rc;
    if (!mlp || !d_pos4 || !d_table_h || !d_weights_h || !d_biases || !d_out || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_grid_mlp_forward: null pointer or negative count");
    if (mlp->input_dim != 2 * desc->num_levels)
        return nb_set_error(NB_ERR_INVALID, "nb_grid_mlp_forward: mlp input_dim must equal 2 * num_levels");
    if (mlp->output_activation != 0) return nb_set_error(NB_ERR_UNSUPPORTED, "nb_grid_mlp_forward: the grid network has a linear output");
    uintptr_t bits = reinterpret_cast<uintptr_t>(d_pos4) | reinterpret_cast<uintptr_t>(d_weights_h) | reinterpret_cast<uintptr_t>(d_out) |
                     reinterpret_cast<uintptr_t>(d_save_enc_h) | reinterpret_cast<uintptr_t>(d_save_acts_h);
    if (bits & 15u) return nb_set_error(NB_ERR_INVALID, "nb_grid_mlp_forward: device pointers must be 16-byte aligned");
    if (n == 0) return NB_OK;
    GridParams gp = make_params(desc);
    if (reinterpret_cast<uintptr_t>(d_table_h) & 7u) gp.pair_ops = 0;
    cudaStream_t st = (cudaStream_t)stream;
#define X(K0, H, OUT, NL)                                                                                         \
    if (mlp->input_dim == K0 && (mlp->hidden_dim == H || NL == 1) && mlp->output_dim == OUT && mlp->num_layers == NL) \
        return launch_grid_mlp<MlpShape<K0, H, OUT, NL>>(gp, d_pos4, d_table_h, d_weights_h, d_biases, n, d_out, d_save_enc_h, d_save_acts_h, st);
    X(32, 64, 16, 2)
    X(32, 32, 16, 2)
    X(32, 64, 16, 3)
    X(32, 64, 16, 1)
    X(16, 16, 16, 2)
#undef X
    // four levels: 8 encoded features, run as a 16-wide input whose upper half is zero (forward only)
    if (mlp->input_dim == 8 && mlp->hidden_dim == 64 && mlp->output_dim == 16 && mlp->num_layers == 2)
        return launch_grid_mlp<MlpShape<16, 64, 16, 2, 8>>(gp, d_pos4, d_table_h, d_weights_h, d_biases, n, d_out, d_save_enc_h, d_save_acts_h, st);
    return nb_set_error(NB_ERR_UNSUPPORTED, "nb_grid_mlp_forward: no kernel built for this (levels, hidden, output, layers) shape");
}

extern "C" int nb_set_tuning(const char* key, int value) {
    if (!key) return nb_set_error(NB_ERR_INVALID, "nb_set_tuning: null key");
    std::string k(key);
    if (k == "scatter_run_merge") g_run_merge = value;
    else if (k == "backward_tc") g_backward_tc = value;
    else if (k == "backward_tc_wait_us") g_backward_tc_wait_us = value;
    else if (k == "forward_staged") g_forward_staged = value;
    else if (k == "forward_stage_levels") g_forward_stage_levels = value;
    else if (k == "forward_persistent") g_forward_persistent = value;
    else if (k == "scatter_smem_levels") g_scatter_tuning.smem_levels = value;
    else if (k == "pair_ops") g_pair_ops = value;
    else if (k == "grad_table_half") g_grad_table_half = value != 0;
    else if (k == "grad_table_scale_log2") {
        if (value < 0 || value > 24) return nb_set_error(NB_ERR_INVALID, "nb_set_tuning: grad_table_scale_log2 must be 0..24");
        g_grad_table_scale_log2 = value;
    }
    else if (k == "scatter_level_begin") g_scatter_tuning.level_begin = value;
    else if (k == "scatter_level_end") g_scatter_tuning.level_end = value;
    else return nb_set_error(NB_ERR_INVALID, "nb_set_tuning: unknown key");
    return NB_OK;
}

extern "C" int nb_get_tuning(const char* key, int* value) {
    if (!key || !value) return nb_set_error(NB_ERR_INVALID, "nb_get_tuning: null pointer");
    std::string k(key);
    if (k == "grad_table_half") *value = g_grad_table_half.load();
    else if (k == "grad_table_scale_log2") *value = g_grad_table_scale_log2.load();
    else if (k == "pair_ops") *value = g_pair_ops.load();
    else if (k == "scatter_run_merge") *value = g_run_merge.load();
    else if (k == "backward_tc") *value = g_backward_tc.load();
    else return nb_set_error(NB_ERR_INVALID, "nb_get_tuning: unknown key");
    return NB_OK;
}

extern "C" int nb_hash_scatter_backward(const nb_grid_desc* desc, const float* d_pos4, const void* d_denc_h, int64_t n,
                                        float* d_table_grads, void* stream) {
    int rc = check_desc(desc, "nb_hash_scatter_backward: null descriptor");
    if (rc != NB_OK) return rc;
    if (!d_pos4 || !d_denc_h || !d_table_grads || n < 0)
        return nb_set_error(NB_ERR_INVALID, "nb_hash_scatter_backward: null pointer or negative count");
    if ((reinterpret_cast<uintptr_t>(d_pos4) & 15u) || (reinterpret_cast<uintptr_t>(d_table_grads) & 7u))
        return nb_set_error(NB_ERR_INVALID, "nb_hash_scatter_backward: misaligned device pointer");
    if (n == 0) return NB_OK;
    GridParams gp = make_params(desc);
    if ((reinterpret_cast<uintptr_t>(d_table_grads) & 15u) && !gp.grad_half) gp.pair_ops = 0;
    return scatter_launch(gp, d_pos4, (const __half*)d_denc_h, 2 * gp.L, n, d_table_grads, 0, gp.L, (cudaStream_t)stream);
}
