// Argument block and launcher of the tensor-memory (tcgen05) backward kernel of the field, shared between
// field_backward_tc.cu (the kernel) and field_fused.cu (the nb_field_backward entry point that selects it).
#pragma once

#include <atomic>

#include "hashgrid_core.cuh"

namespace nb {
namespace tc {

struct BackwardArgs {
    // inputs
    const __half* enc;        // [n][32]
    const __half* dcolor;     // [n][8]
    const float* dsigma;      // [n], nullable
    const float* dirs3;
    const uint32_t* ray_idx;  // nullable
    int64_t ray_idx_offset;
    const __half *Wd, *Wc;    // density [64][32] [16][64]; colour [64][32] [64][64] [8][64]
    const float *bd, *bc;
    int64_t n;
    // outputs
    float *dWd, *dbd, *dWc, *dbc;
    __half* denc;             // leading denc_cols columns, rows denc_cols halves apart
    int denc_cols;
    const float* pos4;        // scatter
    float* table_grads;
    int scatter_begin;
    const uint32_t* perm;     // nullable: row r of the tile order is sample perm[r] (enc is in row order, everything else by sample)
    int* error_flag;          // mapped host memory; set when a wait ran out
    uint64_t wait_ns;         // limit of the chain's waits (0: give up at once when a barrier is not ready - test only)
};

}  // namespace tc

extern std::atomic<int> g_backward_tc;
extern std::atomic<int> g_backward_tc_wait_us;
extern std::atomic<int> g_forward_staged;
extern std::atomic<int> g_forward_stage_levels;
extern std::atomic<int> g_forward_persistent;
int field_backward_tc_failed();
int launch_field_backward_tc(const GridParams& gp, const tc::BackwardArgs& args, cudaStream_t st);

}  // namespace nb
