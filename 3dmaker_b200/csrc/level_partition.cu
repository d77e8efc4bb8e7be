// Level-partitioned hash grid: data-parallel training in which every rank OWNS some levels of the table instead of
// holding a replica of all of them.  The reference is single-GPU (modules/NeRF/InstantNerf.cu:300-566 is one device's
// loop); this is the layout for tables whose parameters outweigh a step's samples (T = 2^22: 268 MB of fp16 parameters
// and 537 MB of fp32 gradient per step against 2^21 samples x 128 B of encodings and their gradients).
//
// Rank r of R owns levels r, r + R, r + 2R, ... (interleaved, so that every rank gets coarse and fine levels).  A step:
//   1. every rank's sample positions are gathered on every rank (one all-gather of fixed-size slots; the slot's last
//      element carries the rank's sample count: nb_part_stamp_count);
//   2. nb_part_encode: the owner encodes ITS levels for ALL ranks' samples into pieces, one contiguous piece per
//      destination rank;
//   3. all-to-all of the pieces: every rank now holds all 16 levels' features of its own samples;
//   4. nb_part_field_forward: the networks, exactly as nb_field_forward, reading the encoding from the pieces;
//      compositing, loss, the networks' backward (no table gradient here);
//   5. dL/d(encoding) by owner (nb_part_field_backward writes the pieces itself; nb_part_pack_denc makes them from a
//      row-major matrix) + all-to-all back: the owner receives the gradient of its levels for all ranks' samples;
//   6. nb_part_scatter: the owner adds them to ITS levels of the table gradient (the scatter kernels of hashgrid.cu on the
//      level view); the optimizer then updates owned levels only - no gradient or parameter exchange for the table at all.
// The collectives are the caller's (NCCL through the host); the kernels here only define the buffer layouts:
//   positions  [R][cap + 1] float4      slot q = rank q's samples, element cap = (count as uint bits, 0, 0, 0)
//   pieces     [R][own][cap] half2      piece q, owned level k, sample j of rank q (send side of the forward exchange and
//                                       receive side of the backward one); on the other side piece q = the levels OWNED BY
//                                       rank q of this rank's own samples
#include <atomic>

#include "hashgrid_core.cuh"

namespace nb {

extern std::atomic<uint64_t> g_launch_count;

__global__ void stamp_count_kernel(float* __restrict__ slot_tail, uint32_t n) {
    reinterpret_cast<uint4*>(slot_tail)[0] = make_uint4(n, 0u, 0u, 0u);
}

// One thread per (sample of some rank, owned level): blockIdx.y = rank whose samples, blockIdx.z = owned level.
__global__ void __launch_bounds__(256) part_encode_kernel(const __grid_constant__ GridParams view, const float* __restrict__ pos_all,
                                                          const uint32_t* __restrict__ table_view, int own, int64_t cap,
                                                          uint32_t* __restrict__ pieces) {
    const int q = blockIdx.y, k = blockIdx.z;
    const float* slot = pos_all + (int64_t)q * (cap + 1) * 4;
    const int64_t count = (int64_t)__float_as_uint(__ldg(slot + cap * 4));
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= count || j >= cap) return;
    const float4 p = ld_nc_f4(slot + j * 4);
    Corners c;
    corners_of<false>(p.x, p.y, p.z, view.scales[k], k < view.dls, view.T, c);
    uint32_t f[8];
    gather_corners(table_view + (size_t)k * view.ls, c, view.pair_ops != 0, f);
    float w[8];
    corner_weights(c, w);
    pieces[((int64_t)q * own + k) * cap + j] = blend(f, w);
}

// dL/d(encoding) of this rank's n samples, row-major [n][2L] halves, into pieces: level l goes to piece l % ranks, owned
// level l / ranks.  A CTA moves 128 rows through shared memory so that both sides are coalesced.
__global__ void __launch_bounds__(256) part_pack_kernel(const uint32_t* __restrict__ denc, int64_t n, int L, int ranks, int own, int64_t cap,
                                                        uint32_t* __restrict__ pieces) {
    __shared__ uint32_t tile[128 * (NB_MAX_LEVELS + 1)];
    const int64_t row_base = (int64_t)blockIdx.x * 128;
    for (int idx = threadIdx.x; idx < 128 * L; idx += blockDim.x) {
        const int r = idx / L, l = idx - r * L;
        tile[r * (NB_MAX_LEVELS + 1) + l] = (row_base + r < n) ? __ldg(denc + (row_base + r) * L + l) : 0u;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 128 * L; idx += blockDim.x) {
        const int l = idx >> 7, r = idx & 127;
        if (row_base + r < n) pieces[((int64_t)(l % ranks) * own + l / ranks) * cap + row_base + r] = tile[r * (NB_MAX_LEVELS + 1) + l];
    }
}

}  // namespace nb

using namespace nb;

static int check_part(const nb_grid_desc* grid, int ranks, int rank, int64_t cap, const char* who) {
    if (!grid) return nb_set_error(NB_ERR_INVALID, who);
    if (ranks < 1 || rank < 0 || rank >= ranks || cap < 1 || cap > 0x7fffffffLL) return nb_set_error(NB_ERR_INVALID, who);
    if (grid->num_levels % ranks != 0) return nb_set_error(NB_ERR_UNSUPPORTED, "level partition: the number of ranks must divide the number of levels");
    return NB_OK;
}

extern "C" int nb_part_stamp_count(float* d_pos_slot, int64_t capacity, int64_t n, void* stream) {
    if (!d_pos_slot || capacity < 1 || n < 0 || n > capacity) return nb_set_error(NB_ERR_INVALID, "nb_part_stamp_count: null slot or count outside [0, capacity]");
    if (reinterpret_cast<uintptr_t>(d_pos_slot) & 15u) return nb_set_error(NB_ERR_INVALID, "nb_part_stamp_count: the slot must be 16-byte aligned");
    stamp_count_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(d_pos_slot + capacity * 4, (uint32_t)n);
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_part_encode(const nb_grid_desc* grid, int ranks, int rank, int64_t capacity, const float* d_pos_all, const void* d_table_h,
                              void* d_pieces_h, void* stream) {
    int rc = check_part(grid, ranks, rank, capacity, "nb_part_encode: bad descriptor, rank or capacity");
    if (rc != NB_OK) return rc;
    if (!d_pos_all || !d_table_h || !d_pieces_h) return nb_set_error(NB_ERR_INVALID, "nb_part_encode: null pointer");
    if ((reinterpret_cast<uintptr_t>(d_pos_all) & 15u) || (reinterpret_cast<uintptr_t>(d_table_h) & 3u) || (reinterpret_cast<uintptr_t>(d_pieces_h) & 3u))
        return nb_set_error(NB_ERR_INVALID, "nb_part_encode: misaligned device pointer");
    const GridParams whole = make_params(grid);
    GridParams view = level_view(whole, rank, ranks);
    const uint32_t* table_view = reinterpret_cast<const uint32_t*>(d_table_h) + (size_t)rank * whole.T;
    if (reinterpret_cast<uintptr_t>(table_view) & 7u) view.pair_ops = 0;
    dim3 g((unsigned)((capacity + 255) / 256), (unsigned)ranks, (unsigned)view.L);
    part_encode_kernel<<<g, 256, 0, (cudaStream_t)stream>>>(view, d_pos_all, table_view, view.L, capacity, reinterpret_cast<uint32_t*>(d_pieces_h));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_part_pack_denc(const nb_grid_desc* grid, int ranks, int64_t capacity, const void* d_denc_h, int64_t n, void* d_pieces_h, void* stream) {
    int rc = check_part(grid, ranks, 0, capacity, "nb_part_pack_denc: bad descriptor, ranks or capacity");
    if (rc != NB_OK) return rc;
    if (!d_denc_h || !d_pieces_h || n < 0 || n > capacity) return nb_set_error(NB_ERR_INVALID, "nb_part_pack_denc: null pointer or count outside [0, capacity]");
    if ((reinterpret_cast<uintptr_t>(d_denc_h) & 3u) || (reinterpret_cast<uintptr_t>(d_pieces_h) & 3u))
        return nb_set_error(NB_ERR_INVALID, "nb_part_pack_denc: misaligned device pointer");
    if (n == 0) return NB_OK;
    part_pack_kernel<<<(unsigned)((n + 127) / 128), 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint32_t*>(d_denc_h), n, grid->num_levels, ranks,
                                                                                    grid->num_levels / ranks, capacity,
                                                                                    reinterpret_cast<uint32_t*>(d_pieces_h));
    NB_CHECK_LAUNCH();
    g_launch_count++;
    return NB_OK;
}

extern "C" int nb_part_scatter(const nb_grid_desc* grid, int ranks, int rank, int64_t capacity, const float* d_pos_all, const void* d_pieces_h,
                               float* d_table_grads, void* stream) {
    int rc = check_part(grid, ranks, rank, capacity, "nb_part_scatter: bad descriptor, rank or capacity");
    if (rc != NB_OK) return rc;
    if (!d_pos_all || !d_pieces_h || !d_table_grads) return nb_set_error(NB_ERR_INVALID, "nb_part_scatter: null pointer");
    if ((reinterpret_cast<uintptr_t>(d_pos_all) & 15u) || (reinterpret_cast<uintptr_t>(d_table_grads) & 7u) || (reinterpret_cast<uintptr_t>(d_pieces_h) & 3u))
        return nb_set_error(NB_ERR_INVALID, "nb_part_scatter: misaligned device pointer");
    const GridParams whole = make_params(grid);
    GridParams view = level_view(whole, rank, ranks);
    // the owner's first level inside the gradient array: two floats per entry, or one __half2 with the half-precision table
    float* grads_view = view.grad_half ? reinterpret_cast<float*>(reinterpret_cast<uint32_t*>(d_table_grads) + (size_t)rank * whole.T)
                                       : d_table_grads + (size_t)rank * whole.T * 2;
    if ((reinterpret_cast<uintptr_t>(grads_view) & 15u) && !view.grad_half) view.pair_ops = 0;
    return scatter_launch_pieces(view, d_pos_all, reinterpret_cast<const uint32_t*>(d_pieces_h), ranks, view.L, capacity, grads_view, (cudaStream_t)stream);
}
