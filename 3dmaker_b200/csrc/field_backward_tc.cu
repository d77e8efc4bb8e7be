// Backward pass of the whole field on the 5th-generation tensor cores: tcgen05.mma with accumulators in tensor memory.
//
// Same contract and same fp16 rounding points as field_backward_kernel (field_fused.cu).  What changes is where the
// GEMM operands and accumulators live.  The mma.sync formulation pulls every operand fragment through the load/store
// pipe (ldmatrix) and keeps the weight-gradient accumulators in 40 registers per thread; measured, that operand traffic
// is half of the kernel's L1TEX time - the pipe the gradient scatter's reductions also need.  Here
//   * every activation / gradient tile sits in shared memory in the tensor core's own core-matrix layout (8 rows x 16
//     bytes per core, no swizzle) and is read by the MMA unit directly, as a K-major operand in the layer GEMMs and, the
//     same bytes viewed MN-major, as an operand of the weight-gradient GEMMs (dW = dZ^T x A, a reduction over the rows);
//   * the weight-gradient accumulators of all five layers, and the bias gradients of the three wide layers (a GEMM with a
//     tile of ones), stay in tensor memory for the lifetime of the persistent CTA and are added to global memory once;
//   * a thread owns one sample row: it reads its row of a layer's result from tensor memory, applies bias / ReLU / mask,
//     rounds to fp16 and writes the row of the next operand tile; after the last layer it holds the 32 encoding gradients
//     of its sample in registers and scatters them into the hash-table gradient without a round trip through memory.
// One elected thread issues the MMAs of a stage and commits them to an mbarrier.
//
// The CTA is two warpgroups.  Warps 0-3 (thread = row) run the chain of layer GEMMs and epilogues above; that chain is a
// sequence of dependent stages, each waiting on the tensor core, so its warps are mostly asleep.  Warps 4-7 do nothing but
// the gradient scatter: they receive a tile's encoding gradients through a double-buffered shared-memory hand-over and
// issue its reductions while warps 0-3 are already on the next tile.  The scatter's index arithmetic and its L1TEX
// traffic thus run underneath the tensor-core chain instead of after it.  (SCATTER_GROUPS = 2 adds a second
// scatter warpgroup, registers split by setmaxnreg; measured at 2^20 unordered samples it is slower, 0.654 against
// 0.630 ms - the reductions' own rate binds by then - and on ray-ordered samples faster, 0.234 against 0.282 ms, where
// the register kernel's 0.214 ms is what gets used anyway.)
// Every wait - MMA barrier, hand-over full / empty - is bounded in TIME (the global timer, one second); a CTA whose wait
// runs out drops its accumulated weight gradients, raises an error flag in mapped host memory that the next
// nb_field_backward call (and nb_field_backward_tc_status) reports, waits for its MMAs in flight and leaves.
#include <atomic>
#include <type_traits>

#include "hashgrid_core.cuh"
#include "field_backward_tc.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

namespace tc {

constexpr int ROWS = 128;      // rows of a tile = TMEM lanes = threads of the CTA
constexpr int SCATTER_GROUPS = 1;  // warpgroups that only scatter; a row's levels are dealt round-robin to them
constexpr int THREADS = 128 * (1 + SCATTER_GROUPS);  // warps 0-3: GEMM chain (thread = row); the rest: gradient scatter
constexpr int CHAIN_THREADS = 128;
constexpr uint64_t WAIT_LIMIT_NS = 1000000000ull;   // one second: the longest any wait inside the kernel lasts

// ---- shared-memory map (bytes); every tile is [rows][cols] fp16 in core-matrix order --------------------------
__host__ __device__ constexpr uint32_t tile_bytes(int rows, int cols) { return (uint32_t)rows * cols * 2; }
// byte offset of element (row, col) in a tile with `cols` columns: cores of one 8-row block are contiguous
__host__ __device__ constexpr uint32_t core_off(int row, int col, int cols) {
    return (uint32_t)(row >> 3) * (cols >> 3) * 128 + (uint32_t)(col >> 3) * 128 + (uint32_t)(row & 7) * 16 + (uint32_t)(col & 7) * 2;
}

constexpr uint32_t OFF_WD0 = 0;                                   // [64][32]
constexpr uint32_t OFF_WD1 = OFF_WD0 + tile_bytes(64, 32);        // [16][64]
constexpr uint32_t OFF_WC0 = OFF_WD1 + tile_bytes(16, 64);        // [64][32]
constexpr uint32_t OFF_WC1 = OFF_WC0 + tile_bytes(64, 32);        // [64][64]
constexpr uint32_t OFF_WC2 = OFF_WC1 + tile_bytes(64, 64);        // [16][64], rows 8..15 zero
constexpr uint32_t OFF_ONES = OFF_WC2 + tile_bytes(16, 64);       // [128][8] of 1.0
constexpr uint32_t OFF_E = OFF_ONES + tile_bytes(ROWS, 8);        // encoding            [128][32]
constexpr uint32_t OFF_CI = OFF_E + tile_bytes(ROWS, 32);         // colour input        [128][32]
constexpr uint32_t OFF_A = OFF_CI + tile_bytes(ROWS, 32);         // density hidden, later its gradient  [128][64]
constexpr uint32_t OFF_B = OFF_A + tile_bytes(ROWS, 64);          // colour hidden 1, later its gradient [128][64]
constexpr uint32_t OFF_C = OFF_B + tile_bytes(ROWS, 64);          // colour hidden 2, later its gradient [128][64]
constexpr uint32_t OFF_Z = OFF_C + tile_bytes(ROWS, 64);          // 16-wide gradients: colour output, then density output [128][16]
constexpr uint32_t OFF_BIAS = OFF_Z + tile_bytes(ROWS, 16);       // fp32 biases: density 64 + 16, colour 64 + 64 + 8
constexpr uint32_t OFF_X = OFF_BIAS + (64 + 16 + 64 + 64 + 8) * 4;   // hand-over: 2 buffers x [16 levels][128 rows] fp16 pairs
constexpr int GROUP_TILES = 1;        // consecutive tiles a CTA takes at a time
constexpr uint32_t SMEM_BYTES = OFF_X + 2 * 16 * ROWS * 4;   // 107 KB: two CTAs per SM (measured: at 111 KB only one is resident)

// ---- tensor-memory map (32-bit columns) ----------------------------------------------------------------------
constexpr uint32_t COL_WORK = 0;      // result of the current layer GEMM, up to 64 columns, 128 lanes
constexpr uint32_t COL_DWC1 = 64;     // dW colour 1   [64 out][64 in]   (64-row accumulators use lanes 0-15 of each warp's 32)
constexpr uint32_t COL_DWC0 = 128;    // dW colour 0   [64 out][32 in]
constexpr uint32_t COL_DWD0 = 160;    // dW density 0  [64 out][32 in]
constexpr uint32_t COL_DWC2T = 192;   // dW colour 2, transposed  [64 in][16 out]
constexpr uint32_t COL_DWD1T = 208;   // dW density 1, transposed [64 in][16 out]
constexpr uint32_t COL_DBC1 = 224;    // db colour 1 in column 0 of [64 out][8]
constexpr uint32_t COL_DBC0 = 232;
constexpr uint32_t COL_DBD0 = 240;
constexpr uint32_t TMEM_COLS = 256;   // two CTAs per SM share the 512 columns

// ---- PTX wrappers -----------------------------------------------------------------------------------------------
// shared-memory matrix descriptor: no swizzle; lbo = byte step between cores along K, sbo = along M/N (K-major), or
// lbo = along K, sbo = along M/N for MN-major as well - what differs between the two views is which storage step is K
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | ((uint64_t)1 << 46);
}
// instruction descriptor: fp16 operands, fp32 accumulate
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int a_mn_major, int b_mn_major) {
    return (1u << 4) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar_addr, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(bar_addr), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity, for at most limit_ns nanoseconds of the global timer (false when the time
// ran out, or when *give_up - a flag another warp of the CTA raises - became non-zero).  limit_ns == 0 does not wait at
// all: one non-blocking test decides.  That setting exists for the test of the give-up path.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns, volatile int* give_up = nullptr) {
    const uint32_t a = smem_u32(bar);
    if (mbar_test(a, parity)) return true;
    if (limit_ns == 0) return false;
    // the timer is looked at once in 256 failed polls (a poll itself waits a while in hardware): the common case, a
    // barrier that completes within a few polls, never reads it
    uint64_t t0 = 0;
    for (uint32_t polls = 1;; polls++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (give_up != nullptr && *give_up != 0) return false;
        if ((polls & 255u) == 0u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}

// 32 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// ---- GEMM issue helpers (one thread) ------------------------------------------------------------------------------
// D[128][N] (+)= X[128][K] x W[N][K]^T : both operands K-major tiles with K columns
__device__ __forceinline__ void gemm_layer(uint32_t tmem_d, uint32_t x_addr, uint32_t w_addr, int K, int N) {
    const uint32_t idesc = instr_desc(ROWS, N, 0, 0);
    const uint32_t sbo = (uint32_t)(K >> 3) * 128;
    for (int k = 0; k < K; k += 16)
        umma_f16(tmem_d, smem_desc(x_addr + (k >> 3) * 128, 128, sbo), smem_desc(w_addr + (k >> 3) * 128, 128, sbo), idesc, k > 0);
}
// D[128][N] = dZ[128][KO] x W[KO][wcols] restricted to the first N input columns: dZ K-major, W viewed MN-major
__device__ __forceinline__ void gemm_dinput(uint32_t tmem_d, uint32_t dz_addr, int KO, uint32_t w_addr, int wcols, int N) {
    const uint32_t idesc = instr_desc(ROWS, N, 0, 1);
    const uint32_t dz_sbo = (uint32_t)(KO >> 3) * 128, w_lbo = (uint32_t)(wcols >> 3) * 128;
    for (int k = 0; k < KO; k += 16)
        umma_f16(tmem_d, smem_desc(dz_addr + (k >> 3) * 128, 128, dz_sbo), smem_desc(w_addr + (k >> 3) * w_lbo, w_lbo, 128), idesc, k > 0);
}
// D[64][N] += P[128][pcols(first 64)]^T x Q[128][qcols(first N)] : a reduction over the 128 rows, both operands MN-major
__device__ __forceinline__ void gemm_outer(uint32_t tmem_d, uint32_t p_addr, int pcols, uint32_t q_addr, int qcols, int N, bool accumulate) {
    const uint32_t idesc = instr_desc(64, N, 1, 1);
    const uint32_t p_lbo = (uint32_t)(pcols >> 3) * 128, q_lbo = (uint32_t)(qcols >> 3) * 128;
    for (int r = 0; r < ROWS; r += 16)
        umma_f16(tmem_d, smem_desc(p_addr + (r >> 3) * p_lbo, p_lbo, 128), smem_desc(q_addr + (r >> 3) * q_lbo, q_lbo, 128), idesc, accumulate || r > 0);
}

// ---- row helpers (thread = row) -------------------------------------------------------------------------------------
// 8 fp32 -> 8 fp16 -> the 16-byte chunk (row, c8) of a tile with `cols` columns
__device__ __forceinline__ void store_chunk(unsigned char* tile, int row, int c8, int cols, const float* v) {
    uint4 q = make_uint4(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]), pack_half2(v[4], v[5]), pack_half2(v[6], v[7]));
    *reinterpret_cast<uint4*>(tile + core_off(row, c8 * 8, cols)) = q;
}
__device__ __forceinline__ uint4 load_chunk(const unsigned char* tile, int row, int c8, int cols) {
    return *reinterpret_cast<const uint4*>(tile + core_off(row, c8 * 8, cols));
}
// gradient chunk rounded to fp16, entries whose activation (same chunk of the layer's input tile) is not positive zeroed
__device__ __forceinline__ uint4 masked_chunk(const float* g, uint4 act) {
    const uint32_t a[4] = {act.x, act.y, act.z, act.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 av = unpack_half2(a[i]);
        o[i] = pack_half2(av.x > 0.f ? g[2 * i] : 0.f, av.y > 0.f ? g[2 * i + 1] : 0.f);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}


// The 16 SH coefficients of a direction (bands 0..3, constants of modules/NeRF/otherKernels.cu:182-200).
__device__ __forceinline__ void sh16(float x, float y, float z, float (&sh)[16]) {
    const float x2 = x * x, y2 = y * y, z2 = z * z;
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

__device__ __forceinline__ float clamp_logit(float v) {
    v = fmaxf(-64.0f, fminf(64.0f, v));
    return (v != v) ? 0.0f : v;
}
__device__ __forceinline__ float clamp_half_range(float v) {
    v = fmaxf(-65504.0f, fminf(65504.0f, v));
    return (v != v) ? 0.0f : v;
}

// All threads: make this thread's shared-memory writes visible to the tensor core, order its tensor-memory reads, meet.
__device__ __forceinline__ void chain_barrier() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }
__device__ __forceinline__ void stage_sync() {
    proxy_fence();
    tc_fence_before();
    chain_barrier();
    tc_fence_after();
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

template <bool GRAD_HALF>
__global__ void __launch_bounds__(THREADS, 2) field_backward_tc_kernel(const __grid_constant__ GridParams gp, const BackwardArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) uint64_t mbar;         // MMAs of the current stage done
    __shared__ __align__(8) uint64_t x_full[2];    // hand-over buffer written by the 128 chain threads
    __shared__ __align__(8) uint64_t x_empty[2];   // ... read by the 128 scatter threads
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag_s;
    volatile int* abort_flag = &abort_flag_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = smem_u32(smem);
    float* sBias = reinterpret_cast<float*>(smem + OFF_BIAS);
    const float* bD0 = sBias, *bD1 = sBias + 64, *bC0 = sBias + 80, *bC1 = sBias + 144;

    // ---- one-time set-up (all 256 threads): weights and the ones tile in core-matrix order, biases, tensor memory, barriers
    auto stage_weights = [&](uint32_t off, const __half* W, int rows_valid, int rows, int cols) {
        const int cpr = cols >> 3;
        for (int c = tid; c < rows * cpr; c += THREADS) {
            const int r = c / cpr, c8 = c % cpr;
            cp_async16(smem + off + core_off(r, c8 * 8, cols), r < rows_valid ? (const void*)(W + r * cols + c8 * 8) : (const void*)W, r < rows_valid);
        }
    };
    stage_weights(OFF_WD0, a.Wd, 64, 64, 32);
    stage_weights(OFF_WD1, a.Wd + 64 * 32, 16, 16, 64);
    stage_weights(OFF_WC0, a.Wc, 64, 64, 32);
    stage_weights(OFF_WC1, a.Wc + 64 * 32, 64, 64, 64);
    stage_weights(OFF_WC2, a.Wc + 64 * 32 + 64 * 64, 8, 16, 64);
    cp_async_commit();
    for (int i = tid; i < 80; i += THREADS) sBias[i] = a.bd[i];
    for (int i = tid; i < 136; i += THREADS) sBias[80 + i] = a.bc[i];
    if (tid < ROWS) {
        const uint32_t one2 = pack_half2(1.0f, 1.0f);
        *reinterpret_cast<uint4*>(smem + OFF_ONES + core_off(tid, 0, 8)) = make_uint4(one2, one2, one2, one2);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&mbar)), "r"(1u) : "memory");
#pragma unroll
        for (int b = 0; b < 2; b++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&x_full[b])), "r"((uint32_t)CHAIN_THREADS) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&x_empty[b])), "r"((uint32_t)(THREADS - CHAIN_THREADS)) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        abort_flag_s = 0;
    }
    cp_async_wait_all();
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    const int64_t ntiles = (a.n + ROWS - 1) / ROWS;
    const int64_t ngroups = (ntiles + GROUP_TILES - 1) / GROUP_TILES;   // a CTA takes whole groups of consecutive tiles
    bool ok = true;
    uint32_t phase_out = 0;   // chain warps: commits awaited or given up on so far

    if (warp >= 4) {
        // ================= scatter warpgroup: thread = row of the tile handed over =====================================
        if constexpr (SCATTER_GROUPS > 1) asm volatile("setmaxnreg.dec.sync.aligned.u32 64;\n");
        if (a.table_grads != nullptr) {
            const int r = (tid - CHAIN_THREADS) & (ROWS - 1), group = (tid - CHAIN_THREADS) >> 7;
            int it = 0;
            for (int64_t grp = blockIdx.x; grp < ngroups && ok; grp += gridDim.x) {
                for (int tl = 0; tl < GROUP_TILES; tl++) {
                    const int64_t tile = grp * GROUP_TILES + tl;
                    if (tile >= ntiles) break;
                    const int buf = it & 1, use = it >> 1;
                    const bool got = __all_sync(0xffffffffu, mbar_wait(&x_full[buf], use & 1, WAIT_LIMIT_NS, abort_flag));
                    if (!got) { ok = false; break; }   // the chain gave up (or never came): leave, every wait here is bounded
                    const uint32_t* x = reinterpret_cast<const uint32_t*>(smem + OFF_X) + buf * 16 * ROWS;
                    uint32_t pk[16];
#pragma unroll
                    for (int l = 0; l < 16; l++) pk[l] = x[l * ROWS + r];
                    mbar_arrive(&x_empty[buf]);
                    it++;
                    const int64_t row = tile * ROWS + r;
                    const bool has = row < a.n;
                    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (has) p = ld_nc_f4(a.pos4 + (a.perm ? (int64_t)a.perm[row] : row) * 4);
                    // a warp is 32 consecutive rows working on one level at a time
#pragma unroll
                    for (int l = 0; l < 16; l++)
                        if (l >= a.scatter_begin && (l % SCATTER_GROUPS) == group)
                            scatter_level_warp<GRAD_HALF>(gp, l, p.x, p.y, p.z, unpack_half2(pk[l]), has, a.table_grads, lane);
                }
            }
        }
    } else {
        if constexpr (SCATTER_GROUPS > 1) asm volatile("setmaxnreg.inc.sync.aligned.u32 112;\n");
        // ================= chain warpgroup: thread = row = tensor-memory lane ============================================
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);  // this warp's 32 lanes
        uint32_t phase = 0;
        bool first_tile = true;
        int it = 0;
        float db_c2 = 0.f, db_d1 = 0.f;  // lane j of every warp: partial bias gradient of output j (colour 8, density 16)

        // wait for the MMAs committed last; uniform verdict over the warpgroup
        auto await = [&]() -> bool {
            if (!mbar_wait(&mbar, phase & 1, a.wait_ns)) *abort_flag = 1;
            phase++;
            chain_barrier();
            tc_fence_after();
            return *abort_flag == 0;
        };

        for (int64_t tile_seq = (int64_t)blockIdx.x * GROUP_TILES; tile_seq < ntiles && ok; it++,
                     tile_seq = ((tile_seq % GROUP_TILES) == GROUP_TILES - 1) ? tile_seq - (GROUP_TILES - 1) + (int64_t)gridDim.x * GROUP_TILES : tile_seq + 1) {
            const int64_t tile = tile_seq;
            const int64_t row_base = tile * ROWS;
            const int64_t row = row_base + tid;
            const bool has = row < a.n;
            const int64_t smp = has ? (a.perm ? (int64_t)a.perm[row] : row) : 0;   // the sample in this row
            // ---- stage 0: encoding tile and colour gradient (zero rows past n; gradient columns 8..15 zero) -------------
            for (int c = tid; c < ROWS * 4; c += CHAIN_THREADS) {
                const int r = c >> 2, c8 = c & 3;
                const bool v = row_base + r < a.n;
                cp_async16(smem + OFF_E + core_off(r, c8 * 8, 32), v ? (const void*)(a.enc + (row_base + r) * 32 + c8 * 8) : (const void*)a.enc, v);
            }
            cp_async16(smem + OFF_Z + core_off(tid, 0, 16), has ? (const void*)(a.dcolor + smp * 8) : (const void*)a.dcolor, has);
            *reinterpret_cast<uint4*>(smem + OFF_Z + core_off(tid, 8, 16)) = make_uint4(0u, 0u, 0u, 0u);
            cp_async_commit();
            // direction of this row's ray, for the SH half of the colour input
            float sh[16];
            {
                int64_t r = has ? smp : (a.perm ? (int64_t)a.perm[a.n - 1] : a.n - 1);
                int64_t ray = a.ray_idx ? (int64_t)a.ray_idx[r + a.ray_idx_offset] : r;
                const float* dp = a.dirs3 + 3 * ray;
                sh16(dp[0], dp[1], dp[2], sh);
            }
            cp_async_wait_all();
            stage_sync();

            // ---- stage 1: density hidden = relu(E Wd0^T + b) -> tile A ----------------------------------------------------
            if (tid == 0) { gemm_layer(tmem + COL_WORK, sbase + OFF_E, sbase + OFF_WD0, 32, 64); umma_commit(&mbar); }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = fmaxf(v[i] + bD0[32 * h + i], 0.f);
#pragma unroll
                for (int c = 0; c < 4; c++) store_chunk(smem + OFF_A, tid, 4 * h + c, 64, v + 8 * c);
            }
            stage_sync();

            // ---- stage 2: 16 logits = A Wd1^T + b; clamp; with the SH -> colour input tile ---------------------------------
            if (tid == 0) { gemm_layer(tmem + COL_WORK, sbase + OFF_A, sbase + OFF_WD1, 64, 16); umma_commit(&mbar); }
            if (!(ok = await())) break;
            {
                float v[16];
                tmem_ld16(lane_base + COL_WORK, v);
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = clamp_logit(v[i] + bD1[i]);
                store_chunk(smem + OFF_CI, tid, 0, 32, v);
                store_chunk(smem + OFF_CI, tid, 1, 32, v + 8);
                store_chunk(smem + OFF_CI, tid, 2, 32, sh);
                store_chunk(smem + OFF_CI, tid, 3, 32, sh + 8);
            }
            stage_sync();

            // ---- stage 3: colour hidden 1 = relu(CI Wc0^T + b) -> tile B -----------------------------------------------------
            if (tid == 0) { gemm_layer(tmem + COL_WORK, sbase + OFF_CI, sbase + OFF_WC0, 32, 64); umma_commit(&mbar); }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = fmaxf(v[i] + bC0[32 * h + i], 0.f);
#pragma unroll
                for (int c = 0; c < 4; c++) store_chunk(smem + OFF_B, tid, 4 * h + c, 64, v + 8 * c);
            }
            stage_sync();

            // ---- stage 4: colour hidden 2 = relu(B Wc1^T + b) -> tile C ------------------------------------------------------
            if (tid == 0) { gemm_layer(tmem + COL_WORK, sbase + OFF_B, sbase + OFF_WC1, 64, 64); umma_commit(&mbar); }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int i = 0; i < 32; i++) v[i] = fmaxf(v[i] + bC1[32 * h + i], 0.f);
#pragma unroll
                for (int c = 0; c < 4; c++) store_chunk(smem + OFF_C, tid, 4 * h + c, 64, v + 8 * c);
            }
            // bias gradient of the colour output layer: column sums of this tile's colour gradient (8 valid columns)
            {
                const uint4 q = load_chunk(smem + OFF_Z, tid, 0, 16);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                float g8[8];
#pragma unroll
                for (int i = 0; i < 4; i++) { const float2 f = unpack_half2(w[i]); g8[2 * i] = f.x; g8[2 * i + 1] = f.y; }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float s = g8[j];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (lane == j) db_c2 += s;
                }
            }
            stage_sync();

            // ---- stage 5: colour layer 2 backward: dW2^T += C^T Z ; dA = Z Wc2, masked by C > 0 -> tile C (in place) --------
            if (tid == 0) {
                gemm_outer(tmem + COL_DWC2T, sbase + OFF_C, 64, sbase + OFF_Z, 16, 16, !first_tile);
                gemm_dinput(tmem + COL_WORK, sbase + OFF_Z, 16, sbase + OFF_WC2, 64, 64);
                umma_commit(&mbar);
            }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    unsigned char* p = smem + OFF_C + core_off(tid, (4 * h + c) * 8, 64);
                    *reinterpret_cast<uint4*>(p) = masked_chunk(v + 8 * c, *reinterpret_cast<const uint4*>(p));
                }
            }
            stage_sync();

            // ---- stage 6: colour layer 1 backward: dW1 += C^T B ; db1 += C^T 1 ; dA = C Wc1, masked by B > 0 -> tile B --------
            if (tid == 0) {
                gemm_outer(tmem + COL_DWC1, sbase + OFF_C, 64, sbase + OFF_B, 64, 64, !first_tile);
                gemm_outer(tmem + COL_DBC1, sbase + OFF_C, 64, sbase + OFF_ONES, 8, 8, !first_tile);
                gemm_dinput(tmem + COL_WORK, sbase + OFF_C, 64, sbase + OFF_WC1, 64, 64);
                umma_commit(&mbar);
            }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    unsigned char* p = smem + OFF_B + core_off(tid, (4 * h + c) * 8, 64);
                    *reinterpret_cast<uint4*>(p) = masked_chunk(v + 8 * c, *reinterpret_cast<const uint4*>(p));
                }
            }
            stage_sync();

            // ---- stage 7: colour layer 0 backward: dW0 += B^T CI ; db0 += B^T 1 ; gradient of the 16 density outputs ---------
            if (tid == 0) {
                gemm_outer(tmem + COL_DWC0, sbase + OFF_B, 64, sbase + OFF_CI, 32, 32, !first_tile);
                gemm_outer(tmem + COL_DBC0, sbase + OFF_B, 64, sbase + OFF_ONES, 8, 8, !first_tile);
                gemm_dinput(tmem + COL_WORK, sbase + OFF_B, 64, sbase + OFF_WC0, 32, 16);
                umma_commit(&mbar);
            }
            if (!(ok = await())) break;
            {
                float v[16];
                tmem_ld16(lane_base + COL_WORK, v);
                // compute_density_grad (modules/NeRF/otherKernels.cu:497-562): fp16 gradient, + dL/dsigma on logit 0, clamp, NaN -> 0
                const float ds = (has && a.dsigma != nullptr) ? a.dsigma[smp] : 0.f;
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = clamp_half_range(__half2float(__float2half_rn(v[i])) + (i == 0 ? ds : 0.f));
                store_chunk(smem + OFF_Z, tid, 0, 16, v);
                store_chunk(smem + OFF_Z, tid, 1, 16, v + 8);
                // bias gradient of the density output layer: column sums of the fp16 values just written
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    float s = __half2float(__float2half_rn(v[j]));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                    if (lane == j) db_d1 += s;
                }
            }
            stage_sync();

            // ---- stage 8: density layer 1 backward: dW1^T += A^T Z ; dA = Z Wd1, masked by A > 0 -> tile A ---------------------
            if (tid == 0) {
                gemm_outer(tmem + COL_DWD1T, sbase + OFF_A, 64, sbase + OFF_Z, 16, 16, !first_tile);
                gemm_dinput(tmem + COL_WORK, sbase + OFF_Z, 16, sbase + OFF_WD1, 64, 64);
                umma_commit(&mbar);
            }
            if (!(ok = await())) break;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v[32];
                tmem_ld32(lane_base + COL_WORK + 32 * h, v);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    unsigned char* p = smem + OFF_A + core_off(tid, (4 * h + c) * 8, 64);
                    *reinterpret_cast<uint4*>(p) = masked_chunk(v + 8 * c, *reinterpret_cast<const uint4*>(p));
                }
            }
            stage_sync();

            // ---- stage 9: density layer 0 backward: dW0 += A^T E ; db0 += A^T 1 ; dL/d(encoding) = A Wd0 -------------------------
            if (tid == 0) {
                gemm_outer(tmem + COL_DWD0, sbase + OFF_A, 64, sbase + OFF_E, 32, 32, !first_tile);
                gemm_outer(tmem + COL_DBD0, sbase + OFF_A, 64, sbase + OFF_ONES, 8, 8, !first_tile);
                gemm_dinput(tmem + COL_WORK, sbase + OFF_A, 64, sbase + OFF_WD0, 32, 32);
                umma_commit(&mbar);
            }
            if (!(ok = await())) break;
            {
                float v[32];
                tmem_ld32(lane_base + COL_WORK, v);
                uint32_t pk[16];  // the sample's 16 feature-pair gradients, fp16 as the reference rounds them
#pragma unroll
                for (int l = 0; l < 16; l++) pk[l] = pack_half2(v[2 * l], v[2 * l + 1]);
                if (has && a.denc_cols > 0) {
                    uint2* dst = reinterpret_cast<uint2*>(a.denc + smp * a.denc_cols);
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if (4 * q < a.denc_cols) dst[q] = make_uint2(pk[2 * q], pk[2 * q + 1]);
                }
                if (a.table_grads != nullptr) {
                    // hand the tile's gradients to the scatter warps: buffer `it & 1`, free again once they have read it
                    const int buf = it & 1, use = it >> 1;
                    bool free_now = true;
                    if (use > 0) free_now = mbar_wait(&x_empty[buf], (use - 1) & 1, a.wait_ns);
                    if (free_now) {
                        uint32_t* x = reinterpret_cast<uint32_t*>(smem + OFF_X) + buf * 16 * ROWS;
#pragma unroll
                        for (int l = 0; l < 16; l++) x[l * ROWS + tid] = pk[l];
                        mbar_arrive(&x_full[buf]);
                    } else {
                        *abort_flag = 1;
                    }
                }
            }
            first_tile = false;
            // the next tile's stage 0 overwrites E and Z: every MMA that read them has completed (awaited above), and all
            // threads have finished reading tensor memory before the next MMA is issued
            tc_fence_before();
            chain_barrier();
            tc_fence_after();
            if (*abort_flag != 0) ok = false;
        }

        // ---- flush: accumulators of this CTA -> global (fp32 reductions), once ---------------------------------------------
        if (ok && !first_tile) {
            // a 64-row accumulator keeps row m in lane (m % 16) of warp (m / 16): lanes 0..15 of every warp hold rows
            const int m = 16 * warp + lane;
            const bool holds = lane < 16;
            float v[32];
#pragma unroll
            for (int h = 0; h < 2; h++) {  // colour layer 1: [64 out][64 in]
                tmem_ld32(lane_base + COL_DWC1 + 32 * h, v);
                if (holds)
#pragma unroll
                    for (int q = 0; q < 8; q++) red_add_v4(a.dWc + 64 * 32 + m * 64 + 32 * h + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
            tmem_ld32(lane_base + COL_DWC0, v);  // colour layer 0: [64 out][32 in]
            if (holds)
#pragma unroll
                for (int q = 0; q < 8; q++) red_add_v4(a.dWc + m * 32 + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            tmem_ld32(lane_base + COL_DWD0, v);  // density layer 0: [64 out][32 in]
            if (holds)
#pragma unroll
                for (int q = 0; q < 8; q++) red_add_v4(a.dWd + m * 32 + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            tmem_ld32(lane_base + COL_DWC2T, v);  // columns 0-15: colour layer 2 transposed [64 in][16 out], 16-31: density layer 1 transposed
            if (holds) {
#pragma unroll
                for (int o = 0; o < 8; o++) red_add(a.dWc + 64 * 32 + 64 * 64 + o * 64 + m, v[o]);
#pragma unroll
                for (int o = 0; o < 16; o++) red_add(a.dWd + 64 * 32 + o * 64 + m, v[16 + o]);
            }
            tmem_ld32(lane_base + COL_DBC1, v);  // columns 0, 8, 16: bias gradients of colour 1, colour 0, density 0
            if (holds) {
                red_add(a.dbc + 64 + m, v[0]);
                red_add(a.dbc + m, v[8]);
                red_add(a.dbd + m, v[16]);
            }
            if (lane < 8) red_add(a.dbc + 128 + lane, db_c2);
            if (lane < 16) red_add(a.dbd + 64 + lane, db_d1);
        }
        phase_out = phase;
    }
    if (!ok && lane == 0 && a.error_flag != nullptr) atomicExch_system(a.error_flag, 1);
    if (!ok && warp < 4 && phase_out > 0) {
        // A chain that gave up may still have MMAs in flight that write tensor memory: before the columns are handed
        // back, wait (bounded, the full limit whatever the tuning says) for the last commit.
        mbar_wait(&mbar, (phase_out - 1) & 1, WAIT_LIMIT_NS);
        tc_fence_after();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

}  // namespace tc
}  // namespace nb

namespace nb {

std::atomic<int> g_backward_tc{2};        // nb_set_tuning("backward_tc", ...)
std::atomic<int> g_backward_tc_wait_us{1000000};   // nb_set_tuning("backward_tc_wait_us", ...): the chain's wait limit

// The error flag lives in mapped, portable host memory: the kernel raises it with a system-scope atomic, the host
// reads it without a CUDA call.  One flag per process, allocated on the first launch.
static std::atomic<int*> g_tc_error_flag{nullptr};

static int* tc_error_flag() {
    int* p = g_tc_error_flag.load(std::memory_order_acquire);
    if (p != nullptr) return p;
    int* fresh = nullptr;
    if (cudaHostAlloc((void**)&fresh, 64, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess || fresh == nullptr) return nullptr;
    *fresh = 0;
    int* expected = nullptr;
    if (!g_tc_error_flag.compare_exchange_strong(expected, fresh)) { cudaFreeHost(fresh); return expected; }
    return fresh;
}

// Non-zero when a wait of the tensor-memory backward kernel has run out since the flag was last cleared.
int field_backward_tc_failed() {
    int* p = g_tc_error_flag.load(std::memory_order_acquire);
    return p != nullptr && *reinterpret_cast<volatile int*>(p) != 0;
}

// Host side: launched by nb_field_backward when the tensor-memory path is selected.
int launch_field_backward_tc(const GridParams& gp, const tc::BackwardArgs& args_in, cudaStream_t st) {
    tc::BackwardArgs args = args_in;
    args.error_flag = tc_error_flag();
    if (args.error_flag == nullptr) return nb_set_error(NB_ERR_CUDA, "field backward: no mapped host memory for the error flag");
    const int wait_us = g_backward_tc_wait_us.load();
    args.wait_ns = wait_us <= 0 ? 0ull : (uint64_t)wait_us * 1000ull;
    auto kern = gp.grad_half ? tc::field_backward_tc_kernel<true> : tc::field_backward_tc_kernel<false>;
    NB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc::SMEM_BYTES));
    const int64_t ntiles = (args.n + tc::ROWS - 1) / tc::ROWS;
    // Two CTAs per SM: 107 KB of shared memory, 128 registers x 256 threads and 256 tensor-memory columns each.  The grid is
    // sized by that count, not by cudaOccupancyMaxActiveBlocksPerMultiprocessor, which answers 1 for this kernel although
    // two CTAs are resident (measured: 0.60 ms with 296 CTAs, 0.91 ms with the 148 the query suggests).
    int64_t grid = (int64_t)nb_num_sms() * 2;
    const int64_t ngroups = (ntiles + tc::GROUP_TILES - 1) / tc::GROUP_TILES;
    if (grid > ngroups) grid = ngroups;
    kern<<<(unsigned)grid, tc::THREADS, tc::SMEM_BYTES, st>>>(gp, args);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

}  // namespace nb

// NB_OK when no wait of the tensor-memory backward kernel has run out since the last call; otherwise NB_ERR_CUDA, and
// the flag is cleared.  Synchronises the device first, so that it speaks for every launch enqueued so far.
extern "C" int nb_field_backward_tc_status(void) {
    NB_CUDA(cudaDeviceSynchronize());
    if (nb::field_backward_tc_failed()) {
        *reinterpret_cast<volatile int*>(nb::g_tc_error_flag.load()) = 0;
        return nb_set_error(NB_ERR_CUDA, "field backward (tensor memory): a bounded wait inside the kernel ran out; the gradients of that launch are incomplete");
    }
    return NB_OK;
}
