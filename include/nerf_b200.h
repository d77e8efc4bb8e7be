/*
 * C ABI of the B200 (sm_100a) NeRF hot-path library, libnerf_b200.so.
 *
 * Plain pointers and sizes only.  Every pointer named d_* is a device pointer owned by the caller;
 * `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Every entry point
 * enqueues on that stream and returns an int status (NB_OK = 0); nothing aborts and nothing is a
 * silent no-op: an unsupported shape returns NB_ERR_UNSUPPORTED and nb_last_error() says why.
 *
 * Each declaration cites the interface of the reference (Ajitesh-07/3DMaker) that it replaces.
 * Parameter layout differs from the reference's launchers in one way: per-layer weights, biases,
 * activations and gradients are flat, layer after layer, instead of device arrays of device
 * pointers, so that one allreduce and one optimizer launch cover everything.
 *
 *   weights  fp16  layer l is [out_l][in_l] row-major, layers back to back
 *   biases   fp32  layer l is [out_l], layers back to back
 *   in_0 = input_dim, in_l = hidden_dim; out_l = hidden_dim, out_last = output_dim
 *   hidden activations fp16: layer 1 .. num_layers-1 inputs, each [n][hidden_dim], back to back
 */
#ifndef NERF_B200_H
#define NERF_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB_OK 0
#define NB_ERR_INVALID 1      /* bad argument (null pointer, negative size, misaligned) */
#define NB_ERR_UNSUPPORTED 2  /* shape outside what the kernels are built for */
#define NB_ERR_CUDA 3         /* a CUDA runtime call or launch failed */
#define NB_ERR_LIMIT 4        /* size beyond a fixed capacity */

#define NB_MAX_LEVELS 16
#define NB_MAX_LAYERS 8

/* Multiresolution hash grid geometry.  Mirrors the grid fields of MLPGridOptions
 * (modules/TinyMLP/TinyMLPHashGrid.h:11-23); features per level is fixed to 2 as the reference's
 * constructor requires (TinyMLPHashGrid.cu:39). */
typedef struct nb_grid_desc {
    int32_t num_levels;        /* numLevels, even, <= NB_MAX_LEVELS */
    int32_t table_size;        /* tableSize: entries per level, power of two */
    int32_t base_resolution;   /* lowestSize */
    int32_t dense_level_start; /* first hashed level (levels below use dense indexing) */
    float growth;              /* b */
    float scales[NB_MAX_LEVELS]; /* per-level resolution N_l as the forward kernel computes it */
    float scatter_scales[NB_MAX_LEVELS]; /* N_l as the reference's gradient scatter computes it:
                                            lowestSize * exp2f(level * log2(b)), a few ulp away from scales[] */
} nb_grid_desc;

/* Mirrors MLPOption (modules/TinyMLP/TinyMLP.h:26-33) with dims already padded the way the
 * reference pads them (powers of two, minimum 8). */
typedef struct nb_mlp_desc {
    int32_t input_dim;
    int32_t hidden_dim;
    int32_t output_dim;
    int32_t num_layers;
    int32_t output_activation; /* 0 none, 1 sigmoid (OUT_ACT_SIGMOID) */
} nb_mlp_desc;

/* Text of the last error on this thread ("" if none). */
const char* nb_last_error(void);
/* Library version and the SM architecture the kernels were built for (100 = sm_100a). */
int nb_version(void);
int nb_built_arch(void);
/* Number of kernel launches this library has issued since load (bench accounting). */
uint64_t nb_launch_count(void);

/* Measurement aid (no counterpart in the reference): `blocks` x 256 threads x per_thread scattered accesses to seeded
 * random entries of d_table and nothing else - kind 0: 4-byte gathers from 2^entries_log2 4-byte entries; kind 1: 8-byte
 * fp32-pair reductions into 2^entries_log2 8-byte entries (the gradient scatter's operation; it adds to the table).  The
 * rates it reaches are the ceilings bench.py reports the hash-grid gathers and the gradient scatter against. */
int nb_probe_random_access(int kind, int entries_log2, int blocks, int per_thread, void* d_table, void* stream);
/* cudaMemsetAsync(d_ptr, 0, bytes) on the caller's stream (the reference's classes call
 * cudaMemsetAsync directly, e.g. TinyMLPHashGrid.cu:312). */
int nb_zero_async(void* d_ptr, int64_t bytes, void* stream);

/* ---- hash grid --------------------------------------------------------------------------- */

/* Fills dense_level_start (host float math of networkFusionHashtable.cu:367-377), scales[]
 * (computed on the device with the forward kernel's own expression sequence, restarted every four
 * levels, networkFusionHashtable.cu:124-128,218) and scatter_scales[] (the expression of the split
 * scatter kernel, networkFusionBackwardHashtable.cu:805, with log2(b) taken on the host as its launcher
 * does, :994).  The reference encodes with the first and scatters with the second; so do we.
 * Synchronises the stream once. */
int nb_grid_setup(nb_grid_desc* desc, int num_levels, int table_size, int base_resolution, float growth, void* stream);

/* nb_grid_setup for callers that must not allocate device memory (no counterpart in the reference,
 * whose launchers recompute the geometry inside every kernel).  Think of a plug-in running inside a
 * host application's fixed memory budget, or a loop that cannot afford the device-wide synchronisation
 * of cudaMalloc/cudaFree.  Same inputs, same results as nb_grid_setup; the 32-float scratch the set-up
 * kernel writes is a static device array inside the library (128 bytes per GPU at a 256-byte aligned
 * address, held until the process exits) instead of a cudaMalloc'd buffer, and no cudaMalloc, cudaFree
 * or other allocating call is made.  Like nb_grid_setup it copies the scales back to the host and waits
 * for the stream (cudaStreamSynchronize) before returning.
 * Limits and rules:
 *   - num_levels > 16 (NB_MAX_LEVELS) is rejected with NB_ERR_LIMIT;
 *   - the first call on each device (with that device current) looks up the array's device address;
 *     make that first call before any stream capture begins.  The address belongs to the device's
 *     context and does not survive cudaDeviceReset;
 *   - all calls on one GPU share the array, which keeps the previous call's values (each call overwrites
 *     exactly the entries it reads back, so nothing needs clearing); two calls that overlap on the GPU
 *     (different streams or threads) race on it - serialise them. */
int nb_grid_setup_noalloc(nb_grid_desc* desc, int num_levels, int table_size, int base_resolution, float growth, void* stream);

/* Element offsets (feature 0) of the 8 corners of every (point, level): d_idx_out[n][L][8].
 * clamp_mode 0 = forward clamp, 1 = backward clamp (networkFusionHashtable.cu:134-156,
 * networkFusionBackwardHashtable.cu:812-834).  For bit-exact index parity tests. */
int nb_hash_indices(const nb_grid_desc* desc, const float* d_pos4, int64_t n, int clamp_mode, uint32_t* d_idx_out,
                    void* stream);

/* Encode only: d_enc_out[n][2L] fp16.  The encode body of networkFusionHashTableMMA_2d_vector3
 * (networkFusionHashtable.cu:111-222).  d_pos4 is float4 per point, w ignored. */
int nb_hash_encode_forward(const nb_grid_desc* desc, const float* d_pos4, const void* d_table_h, int64_t n,
                           void* d_enc_out_h, void* stream);

/* Encode fused with the MLP.  Replaces launchNetworkFusionHashTableKernel (d_save_* NULL) and
 * launchNetworkFusionHashTableGradKernel (TinyMLPHashGrid.h:172-194).  d_out is fp32 [n][output_dim].
 * d_save_enc_h [n][2L] and d_save_acts_h (hidden activations) may be NULL. */
int nb_grid_mlp_forward(const nb_grid_desc* desc, const nb_mlp_desc* mlp, const float* d_pos4, const void* d_table_h,
                        const void* d_weights_h, const float* d_biases, int64_t n, float* d_out, void* d_save_enc_h,
                        void* d_save_acts_h, void* stream);

/* Gradient scatter into the fp32 table gradient.  Replaces the hashTableScatter_Backward half of
 * launchNetworkFusionScatterBackwardKernel (TinyMLPHashGrid.h:213-226).  d_denc_h is [n][2L] fp16. */
int nb_hash_scatter_backward(const nb_grid_desc* desc, const float* d_pos4, const void* d_denc_h, int64_t n,
                             float* d_table_grads, void* stream);

/* A/B switches for benchmarking, in the spirit of the reference's TinyMLPHashGrid::setSplitScatter
 * (TinyMLPHashGrid.h:60-63).  Keys: "scatter_run_merge" (consecutive samples in one grid cell are summed inside the
 * warp before the reduction, in warps with at most this many runs; default 20, 0 = never), "scatter_smem_levels" (dense levels below it that fit shared memory are
 * accumulated per CTA; default 2), "scatter_level_begin" / "scatter_level_end" (restrict the scatter to a level range),
 * "pair_ops" (x-neighbour corners that share an aligned slot pair are gathered with one 8-byte load and scattered with
 * one 16-byte reduction; default 1).  Results do not depend on these beyond fp32 summation order of the scatter.
 * Further keys, described where they act: "backward_tc", "backward_tc_wait_us" (nb_field_backward), "forward_staged",
 * "forward_stage_levels", "forward_persistent" (nb_field_forward_ordered).
 *
 * "grad_table_half" (default 0) switches the TABLE GRADIENT to half precision, process-wide; the reference keeps fp32
 * only (TinyMLPHashGrid.h:119).  With it on, the hash part of every gradient array handed to this library -
 * d_table_grads of nb_hash_scatter_backward / nb_field_backward, the first sparse_count elements of d_g of nb_adam_step
 * and of the peer arrays of nb_adam_step_peer - is ONE __half2 PER ENTRY (4 bytes, entry e of level l at element
 * l * T + e) packed at the start of the array, instead of two floats; the array keeps its fp32 size and everything
 * behind the hash part (network weights and biases) keeps its fp32 place and type.  The scatter multiplies every
 * contribution by 2^"grad_table_scale_log2" (default 7, 0..24) before rounding it to fp16 (on top of the loss scale the
 * activations' gradients already carry) and adds it with red.global.add.noftz.f16x2 (x-neighbour corners in one 8-byte
 * vector reduction); levels accumulated in shared memory are rounded once per CTA.  The optimizer divides by the same
 * factor.  An entry whose fp16 sum overflows reads as non-finite and is treated like any non-finite gradient: it
 * counts as zero (optimizerKernel.cu:145-150 does the same for its fp32 gradients).  Set both keys before the first
 * backward and leave them alone between a backward and the optimizer step that consumes it.  Not available with
 * gradient exchanges that treat the arena as one fp32 array (all-reduce, reduce-scatter): nb_adam_step_peer reads the
 * half-precision slices of every rank itself. */
int nb_set_tuning(const char* key, int value);
/* Current value of a switch ("grad_table_half", "grad_table_scale_log2", "pair_ops", "scatter_run_merge",
 * "backward_tc"); NB_ERR_INVALID for any other key. */
int nb_get_tuning(const char* key, int* value);

/* ---- level-partitioned grid (no counterpart in the reference, which trains on one GPU) --------------------------
 *
 * Data-parallel training in which rank r of R OWNS levels r, r + R, r + 2R, ... of the table instead of holding a
 * replica of all levels: the ranks exchange positions, encodings and encoding gradients (128 bytes per sample and step)
 * and nothing of the table.  R must divide the number of levels.  The collectives are the caller's; these entry points
 * define the layouts they move:
 *   position slots  float4 [R][capacity + 1]: slot q = rank q's sample positions, element `capacity` = its sample
 *                   count (uint32 bits in .x; nb_part_stamp_count writes it).  One all-gather of a rank's slot fills it.
 *   pieces          half2 [R][levels / R][capacity]: piece q, owned level k, sample j.  After nb_part_encode piece q
 *                   holds THIS rank's levels for rank q's samples; one all-to-all of whole pieces later piece q holds the
 *                   levels OWNED BY rank q for this rank's samples, which is what nb_part_field_forward reads.  The
 *                   backward exchange runs the other way: nb_part_pack_denc, all-to-all, nb_part_scatter.
 * Results equal those of the replicated path sample by sample (the encoding bit for bit; gradients up to summation order). */
int nb_part_stamp_count(float* d_pos_slot, int64_t capacity, int64_t n, void* stream);
int nb_part_encode(const nb_grid_desc* grid, int ranks, int rank, int64_t capacity, const float* d_pos_all, const void* d_table_h,
                   void* d_pieces_h, void* stream);
/* nb_field_forward with the encoding taken from the received pieces (d_enc_save_h row-major [n][32] as before). */
int nb_part_field_forward(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, int ranks, int64_t capacity,
                          const void* d_pieces_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                          const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                          int64_t n, float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb,
                          int rgb_stride, void* stream);
/* d_denc_h fp16 [n][2 levels] as nb_field_backward (without a table gradient) writes it -> pieces for the owners. */
int nb_part_pack_denc(const nb_grid_desc* grid, int ranks, int64_t capacity, const void* d_denc_h, int64_t n, void* d_pieces_h, void* stream);
/* nb_field_backward without a table gradient whose dL/d(encoding) goes straight into the pieces (no row-major copy, no
 * nb_part_pack_denc); always the register formulation of the kernel. */
int nb_part_field_backward(const nb_mlp_desc* density, const nb_mlp_desc* color, int ranks, int64_t capacity, const void* d_enc_h,
                           const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h,
                           const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n, const void* d_dcolor_h,
                           const float* d_dsigma, float* d_grad_density_w, float* d_grad_density_b, float* d_grad_color_w,
                           float* d_grad_color_b, void* d_pieces_h, void* stream);
/* The owner's levels of d_table_grads (the WHOLE gradient array, standard layout) receive the gradients of all ranks'
 * samples: hashTableScatter_Backward (networkFusionBackwardHashtable.cu:783-910) restricted to the owned levels. */
int nb_part_scatter(const nb_grid_desc* grid, int ranks, int rank, int64_t capacity, const float* d_pos_all, const void* d_pieces_h,
                    float* d_table_grads, void* stream);

/* ---- fused MLP ---------------------------------------------------------------------------- */

/* Replaces launchNetworkFusionKernel / launchNetworkFusionGradKernel (TinyMLP.h:172-206). */
int nb_mlp_forward(const nb_mlp_desc* mlp, const void* d_in_h, const void* d_weights_h, const float* d_biases, int64_t n,
                   float* d_out, void* d_save_acts_h, void* stream);

/* Replaces launchNetworkFusionBackwardKernel (TinyMLP.h:183-194) and the MLP half of
 * launchNetworkFusionScatterBackwardKernel.  d_dloss_h [n][output_dim] fp16; d_act0_h the layer-0
 * input [n][input_dim]; gradients are ADDED into d_grad_w / d_grad_b; d_dx_h [n][input_dim] may be NULL. */
int nb_mlp_backward(const nb_mlp_desc* mlp, const void* d_dloss_h, const void* d_weights_h, const void* d_act0_h,
                    const void* d_acts_h, int64_t n, float* d_grad_w, float* d_grad_b, void* d_dx_h, void* stream);

/* ---- loss and optimizer ------------------------------------------------------------------- */

/* Replaces launchMSELossGrad (TinyMLP.h:244-255).  d_total_loss: one float, the summed squared
 * error is ADDED to it. */
int nb_mse_loss_grad(const float* d_pred, const void* d_target_h, void* d_grad_h, float* d_total_loss, int64_t n,
                     int padded_dim, int valid_dim, float loss_scale, int output_activation, void* stream);

/* One Adam launch over a flat parameter arena.  Elements [0, sparse_count) follow the hash-table
 * rule of fusedAdamHashGridOptim (optimizerKernel.cu:116-167: skip when the gradient is exactly 0,
 * zero the gradient after reading); elements [sparse_count, total_count) follow the dense rule of
 * fusedAdamWeightsOptim / fusedAdamBiasOptim (optimizerKernel.cu:16-113).  Replaces
 * launchAdamHashGridOptim + launchAdamWeightsOptim + launchAdamBiasOptim (+ launchZeroGradients when
 * zero_dense_grads != 0).  d_w_h receives the fp16 copy of every element. */
int nb_adam_step(float* d_w, void* d_w_h, float* d_g, float* d_m, float* d_v, int64_t sparse_count, int64_t total_count,
                 float lr, float beta1, float beta2, float eps, float bias_correction1, float bias_correction2,
                 float inv_loss_scale, int zero_dense_grads, void* stream);

/* Data-parallel tail of a step as ONE kernel over peer memory (no counterpart in the reference, which is single-GPU):
 * this rank's slice [rank, rank + 1) * sparse_count / world of the hash table gets the SUM of all ranks' gradients -
 * loaded straight from the ranks' gradient arenas, peer_grads[r] (HOST array of `world` device pointers, entry `rank`
 * this rank's own) -, the sparse Adam rule of nb_adam_step on this rank's d_w / d_m / d_v, and the updated fp16 groups are
 * stored into EVERY rank's forward copy, peer_w_h[r].  The dense tail [sparse_count, total_count) is summed and updated
 * by every rank for itself.  Replaces reduce-scatter + optimizer + all-gather.  The caller provides what the kernel
 * does not: a barrier across the ranks before the launch (gradients complete) and after it (parameters delivered,
 * gradients read), after which each rank clears its own gradient arena; peer pointers come from nb_ipc_open or
 * cudaDeviceEnablePeerAccess.  At most 8 ranks; sparse_count a multiple of 4 x world.  The fp32 master copy and the
 * moments of a slice are current on its owner only. */
int nb_adam_step_peer(float* d_w, float* d_m, float* d_v, const float* const* peer_grads, void* const* peer_w_h, int rank, int world,
                      int64_t sparse_count, int64_t total_count, float lr, float beta1, float beta2, float eps, float bias_correction1,
                      float bias_correction2, float inv_loss_scale, void* stream);
/* cudaIpcGetMemHandle / cudaIpcOpenMemHandle (lazy peer access) / cudaIpcCloseMemHandle: handle64 is the 64-byte
 * cudaIpcMemHandle_t; d_base must be the start of a cudaMalloc allocation (nb_device_alloc's, or the arenas of
 * nb_nerf_get_arena).  nb_device_alloc returns zeroed memory. */
int nb_ipc_export(void* d_base, void* handle64);
int nb_ipc_open(const void* handle64, void** d_ptr_out);
int nb_ipc_close(void* d_ptr);
int nb_device_alloc(int64_t bytes, void** d_ptr_out);
int nb_device_free(void* d_ptr);

/* ---- NeRF glue between the two networks ------------------------------------------------------ */

/* Replaces compute_SH_gather (modules/NeRF/otherKernels.cu:156-273).  d_dirs3: float3 per ray;
 * d_ray_indices[offset + i] = ray of sample i; d_density_out fp32 [n][16] (read only);
 * d_color_in_h fp16 [n][32] = 16 clamped logits ++ 16 SH; d_sigma[n] = expf(min(logit0 - bias, 8)). */
int nb_sh_gather(const float* d_dirs3, const uint32_t* d_ray_indices, int64_t offset, int64_t n, float density_bias,
                 const float* d_density_out, void* d_color_in_h, float* d_sigma, void* stream);

/* Replaces compute_density_grad (modules/NeRF/otherKernels.cu:497-562).  d_color_dx_h fp16 [n][32]
 * (only the first 16 channels are read), d_tmp_dsigma[n] added to channel 0 (NULL = zeros),
 * d_density_grad_h fp16 [n][16], clamped to +-65504, NaN -> 0. */
int nb_density_grad(int64_t n, const float* d_tmp_dsigma, const void* d_color_dx_h, void* d_density_grad_h, void* stream);

/* Samples in their compact host layout - position float3, target colour three halves: 18 bytes where the kernels' own
 * layouts take 32 - into position float4 (w = 0) and target eight halves (channels 3..7 zero), the job of the
 * reference's hg_pad kernels and fusedPadAndCastKernel (TinyMLPHashGrid.cu:11-34, TinyMLP.cu:23-45).  Either pair may
 * be NULL.  Lets a training loop that feeds samples from the host move 30 instead of 44 bytes per sample over PCIe. */
int nb_unpack_samples(const float* d_pos3, const void* d_target3_h, int64_t n, float* d_pos4, void* d_target8_h, void* stream);
/* Replaces generate_custom_rays_kernel (modules/NeRF/NerfTrainer.cu:25-47): pinhole rays of pixels
 * [first_pixel, first_pixel + count) of a width x height frame; c2w_3x4 is a HOST pointer to the row-major 3x4
 * camera-to-world matrix.  The pixel range is what pixel-sharded rendering splits across ranks. */
int nb_generate_rays(int width, int height, float focal, const float* c2w_3x4, int64_t first_pixel, int64_t count, float* d_rays_o,
                     float* d_rays_d, void* stream);
/* The same rays for the tiles first_tile, first_tile + tile_stride, ... of `tile` consecutive pixels each, written one tile
 * after the other: ray i is pixel (first_tile + (i / tile) * tile_stride) * tile + i % tile.  One launch generates all the
 * tiles a rank of a pixel-sharded frame renders (distributed.pixel_tiles); only the last tile may be cut short by count. */
int nb_generate_rays_tiled(int width, int height, float focal, const float* c2w_3x4, int64_t tile, int64_t first_tile, int64_t tile_stride,
                           int64_t count, float* d_rays_o, float* d_rays_d, void* stream);
/* Inverse of that deal, for the rank that assembles a pixel-sharded frame (no counterpart in the reference, which renders
 * on one GPU): d_blocks holds `ranks` blocks of rows_per_rank pixels (3 floats each), block r = the tiles r, r + ranks,
 * r + 2 ranks, ... of the frame one after the other as rank r rendered them; d_frame receives the num_pixels x 3 frame. */
int nb_undeal_tiles(const float* d_blocks, int ranks, int64_t rows_per_rank, int64_t tile, int64_t num_pixels, float* d_frame,
                    void* stream);
/* Replaces mse_kernel (modules/NeRF/NerfTrainer.cu:15-23): ADDS sum over rays of mean((pred - target)^2) to *d_loss_sum. */
int nb_mse_rays(const float* d_pred3, const float* d_target3, float* d_loss_sum, int64_t n, void* stream);

/* ---- the whole field in one launch each way ------------------------------------------------------ */

/* 1 when nb_field_forward / nb_field_backward are built for this (grid, density, colour) combination: 16 levels,
 * density 32-64-16 (linear), colour 32-64-64-8 (sigmoid) - the shapes of NerfOptions' defaults
 * (modules/NeRF/InstantNerf.h:20-33).  Other shapes run the separate kernels above. */
int nb_field_supported(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color);

/* Positions -> (sigma, logit 0, rgb) of n samples.  Replaces, in one launch, the sequence
 * TinyMLPHashGrid::forward / inference -> compute_SH_gather -> TinyMLP::forward / inference that InstantNerf runs per
 * chunk (modules/NeRF/InstantNerf.cu:436-459 training, 930-960 rendering).  Ray of sample i =
 * d_ray_indices[ray_index_offset + i] (NULL: ray i).  d_enc_save_h fp16 [n][32] is all the backward needs
 * (NULL when rendering); d_sigma[n] = expf(min(clamp(logit0) - density_bias, 8)); d_logit0[n] the raw first output
 * of the density network; d_rgb rows are rgb_stride (4 or 8) floats apart, sigmoid applied, columns >= 3 padding. */
int nb_field_forward(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                     const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                     const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n,
                     float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb, int rgb_stride,
                     void* stream);
/* nb_field_forward for explicit samples (direction i belongs to sample i) followed by nb_mse_loss_grad on its colour
 * output (valid_dim 3, padded_dim 8, sigmoid derivative folded in), in one launch: the loss is taken in the forward's
 * epilogue from the colour it still has in registers.  Replaces TinyMLP::forward -> launchMSELossGrad
 * (modules/TinyMLP/optimizerKernel.cu:169-224, 380-400) for the field.  d_target_h fp16 [n][8], d_dcolor_h fp16 [n][8]
 * (what nb_field_backward takes), *d_total_loss (nullable) is ADDED the sum of squared differences. */
int nb_field_forward_mse(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                         const void* d_table_h, const float* d_dirs3, const void* d_density_w_h, const float* d_density_b,
                         const void* d_color_w_h, const float* d_color_b, int64_t n, float density_bias, void* d_enc_save_h,
                         float* d_sigma, float* d_logit0, float* d_rgb, int rgb_stride, const void* d_target_h, void* d_dcolor_h,
                         float* d_total_loss, float loss_scale, void* stream);


/* nb_field_forward for rendering when the sample count is known only on the device: the launch covers n_max samples
 * and tiles at or behind *d_count (read when the kernel runs; at most n_max) leave at once. */
int nb_field_forward_counted(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                             const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                             const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b,
                             int64_t n_max, const uint32_t* d_count, float density_bias, float* d_sigma, float* d_rgb, int rgb_stride,
                             void* stream);

/* ---- samples in spatial order ---------------------------------------------------------------------------------
 * The reference keeps a Morton ordering of the samples in its legacy march (morton keys from the sample position and a
 * radix sort, modules/NeRF/processRays.cu:70-81,412-448); its field kernels take samples in whatever order they come.
 * Here the order is an input of the field kernels: neighbouring samples share their corners on the coarser levels, and a
 * CTA that works on neighbours keeps those corners' boxes in shared memory instead of going to L2 for each of them.
 *
 * nb_sample_order: d_order[k] = the k-th sample when the samples are listed brick by brick, the 16^3 bricks of the unit
 * cube in Morton order (a counting sort over 12-bit keys; samples of one brick in no particular order).  d_scratch:
 * nb_sample_order_scratch_bytes() bytes, 16-byte aligned.  Positions outside [0, 1] count for the nearest brick. */
int64_t nb_sample_order_scratch_bytes(void);
int nb_sample_order(const float* d_pos4, int64_t n, uint32_t* d_order, void* d_scratch, void* stream);

/* nb_field_forward visiting the samples in the order d_order (any permutation of 0 .. n-1; nb_sample_order's makes it
 * fast): persistent CTAs take groups of four consecutive 128-row tiles, copy the boxes of the leading levels that the
 * group's positions span into shared memory (as many levels as fit 24 KB) and gather those levels from there.  Results
 * are identical to nb_field_forward's, sample by sample: d_sigma, d_logit0 and d_rgb are indexed by SAMPLE; only
 * d_enc_save_h is in ROW order (row k = sample d_order[k]), which is what nb_field_backward_ordered expects.
 * nb_set_tuning("forward_staged", 1) makes nb_field_forward itself use this kernel (rows = samples); 0 switches it off. */
int nb_field_forward_ordered(const nb_grid_desc* grid, const nb_mlp_desc* density, const nb_mlp_desc* color, const float* d_pos4,
                             const void* d_table_h, const float* d_dirs3, const uint32_t* d_ray_indices, int64_t ray_index_offset,
                             const void* d_density_w_h, const float* d_density_b, const void* d_color_w_h, const float* d_color_b, int64_t n,
                             const uint32_t* d_order, float density_bias, void* d_enc_save_h, float* d_sigma, float* d_logit0, float* d_rgb,
                             int rgb_stride, void* stream);

/* nb_field_backward for the same order: d_enc_h in ROW order as nb_field_forward_ordered saved it, d_dcolor_h, d_dsigma,
 * d_pos4 and d_denc_h by SAMPLE.  Always the tensor-memory kernel; its scatter warps visit the rows in the given order, so
 * that the reductions of neighbouring samples on the coarser levels meet in the same L2 sectors.  Gradients agree with
 * nb_field_backward's to fp32 summation order. */
int nb_field_backward_ordered(const nb_mlp_desc* density, const nb_mlp_desc* color, const void* d_enc_h, const float* d_dirs3,
                              const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h, const float* d_density_b,
                              const void* d_color_w_h, const float* d_color_b, int64_t n, const uint32_t* d_order, const void* d_dcolor_h,
                              const float* d_dsigma, float* d_grad_density_w, float* d_grad_density_b, float* d_grad_color_w,
                              float* d_grad_color_b, void* d_denc_h, const nb_grid_desc* grid, const float* d_pos4, float* d_table_grads,
                              void* stream);

/* Gradients of both networks, of the encoding and (optionally) of the hash table from the colour gradient.  Replaces
 * TinyMLP::backward (colour) -> compute_density_grad -> TinyMLPHashGrid::backward (modules/NeRF/InstantNerf.cu:506-561).
 * Hidden activations are derived again from d_enc_h inside the kernel.  d_dcolor_h fp16 [n][8] = dL/d(colour
 * pre-activation) as nb_color_grad / nb_mse_loss_grad write it; d_dsigma[n] (NULL = zeros) is added to the gradient
 * of logit 0.  d_grad_* are ACCUMULATED (fp32).
 *   d_table_grads == NULL: d_denc_h receives fp16 [n][32] for nb_hash_scatter_backward (grid, d_pos4 unused).
 *   d_table_grads != NULL: the kernel also scatters into the table gradient as nb_hash_scatter_backward would (its
 *     reductions drain through L2 underneath the tensor work); d_denc_h is then scratch of at least n * 8 bytes whose
 *     content is unspecified, grid and d_pos4 (float4 per sample) are required. */
/* The backward kernel exists in two formulations with the same inputs, outputs and fp16 rounding points:
 * nb_set_tuning("backward_tc", 1) selects tcgen05.mma with accumulators in tensor memory, 0 mma.sync with register
 * accumulators, 2 (default) picks by the sample order the call implies: d_ray_indices == NULL means explicit,
 * unordered samples, where the scatter's reductions are the long pole and the tensor-memory kernel (its scatter on
 * warps of their own) is faster (0.63 against 0.74 ms at 2^20 samples); ray-ordered samples from the marcher come with
 * ray indices, merge into few reductions, and the register kernel is the faster one there (0.21 against 0.23 ms at 2^18).
 * The tensor-memory kernel adds its weight gradients with 16-byte reductions: with weight-gradient pointers that are only
 * 8-byte aligned mode 2 uses the register kernel and mode 1 returns NB_ERR_INVALID.
 * Every wait inside the tensor-memory kernel is bounded by the GPU's global timer (one second;
 * nb_set_tuning("backward_tc_wait_us", v) changes the limit of the MMA and hand-over waits, v = 0 makes a wait give up
 * as soon as its barrier is not ready, which is how the give-up path is tested).  A CTA whose wait runs out drops its
 * weight gradients and raises a flag in mapped host memory; from then on nb_field_backward returns NB_ERR_CUDA until
 * nb_field_backward_tc_status() - which synchronises the device, reports the condition (NB_ERR_CUDA) and clears it - has
 * been called. */
int nb_field_backward_tc_status(void);
int nb_field_backward(const nb_mlp_desc* density, const nb_mlp_desc* color, const void* d_enc_h, const float* d_dirs3,
                      const uint32_t* d_ray_indices, int64_t ray_index_offset, const void* d_density_w_h, const float* d_density_b,
                      const void* d_color_w_h, const float* d_color_b, int64_t n, const void* d_dcolor_h, const float* d_dsigma,
                      float* d_grad_density_w, float* d_grad_density_b, float* d_grad_color_w, float* d_grad_color_b, void* d_denc_h,
                      const nb_grid_desc* grid, const float* d_pos4, float* d_table_grads, void* stream);

/* ---- ray batches from an image set ------------------------------------------------------------------ */

/* A posed image set in device memory: what the reference's DataLoader holds after loading (DataLoader.h), with the
 * images in HBM instead of mapped host memory.  Depth-prior records are optional (num_records 0). */
typedef struct nb_image_set {
    const uint8_t* d_images_rgba;  /* [num_images][height][width][4] */
    const float* d_transforms;     /* [num_images][16] row-major camera-to-world */
    int32_t num_images, width, height;
    float focal;                   /* pixels */
    const int32_t* d_rec_frame;    /* depth priors: image index, pixel position (in a prior_width x prior_height frame), depth, sigma */
    const float *d_rec_u, *d_rec_v, *d_rec_depth, *d_rec_sigma;
    uint32_t num_records;
    float dense_fraction;          /* share of the random slots redirected to a prior's keypoint */
    int32_t prior_width, prior_height;
} nb_image_set;

/* Replaces DataLoader::fetchRayChunk / fetchRayChunkStreamingKernel (modules/NeRF/DataLoader.cu:542-690): `size` rays
 * and blended target colours for slots [offset, offset + size).  randomize != 0: PCG-hashed image and pixel per slot
 * (seed = the epoch seed), images 0, N, 2N, ... never drawn when holdout_every = N >= 2; randomize == 0: pixels in
 * order (validation, INerfTrainer::validate).  d_prior_depth / d_prior_sigma (nullable) receive -1 for plain colour
 * rays.  float3 rays, float3 colours. */
int nb_fetch_ray_chunk(const nb_image_set* set, int offset, int size, uint32_t seed, int randomize, const float* bg_color3,
                       int holdout_every, float* d_rays_o, float* d_rays_d, float* d_rgb, float* d_prior_depth, float* d_prior_sigma,
                       void* stream);

/* ---- rays, occupancy march, compaction ------------------------------------------------------- */

/* Scene geometry of the marcher: the fields of NerfOptions it reads (modules/NeRF/InstantNerf.h:35-42). */
typedef struct nb_scene_desc {
    uint32_t grid_res[3];      /* gridResolution (level 0 of each cascade) */
    float aabb_min[3];         /* aabbMin; must be negative, aabb_max positive (get_cascade divides by both) */
    float aabb_max[3];
    int32_t num_cascades;
    int32_t mip_levels;        /* levelsMipmap */
    int32_t samples_per_voxel; /* samplesPerVoxel */
} nb_scene_desc;

/* Replaces compute_ray_aabb_inv_kernel (modules/NeRF/otherKernels.cu:91-154). float3 per ray in and out. */
int nb_ray_aabb(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, int64_t num_rays, float* d_rays_d_inv,
                float* d_nears, float* d_fars, void* stream);

/* Pass 1 of the march, samples per ray (cap 1024).  Replaces march_rays_dda_calc_hits
 * (modules/NeRF/processRays.cu:626-737). */
int nb_march_count(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv,
                   const float* d_nears, const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays, uint32_t* d_num_steps,
                   void* stream);

/* Exclusive scan of the counts + sample-budget cutoff from ray 0.  Replaces custom_exclusive_sum and
 * find_cutoff_ray_kernel (processRays.cu:486-549,739-769) and the three host read-backs of
 * processRaysHitLinear (:979-1013).  d_block_sums: scratch of ceil(num_rays/1024) uint32.  d_plan[4]:
 * [0] rays that fit, [1] their sample total, [2] first sample of the batch (0), [3] samples of all rays. */
int nb_march_scan(const uint32_t* d_num_steps, uint32_t* d_ray_offsets, uint32_t* d_block_sums, int64_t num_rays, uint32_t batch_size,
                  uint32_t* d_plan, void* stream);

/* Cutoff for the next batch of an already scanned chunk, starting at rays_done.  Replaces
 * find_cutoff_ray_from_kernel (processRays.cu:771-799).  d_plan as above, [0] absolute end ray. */
int nb_march_cutoff(const uint32_t* d_num_steps, const uint32_t* d_ray_offsets, int64_t num_rays, uint32_t rays_done, uint32_t batch_size,
                    uint32_t* d_plan, void* stream);

/* Pass 2: t, ray id (relative to rays_done) and contracted float4 position of every sample of rays
 * [rays_done, d_plan[0]), written at ray_offsets[i] - d_plan[2].  Replaces march_rays_dda_offset
 * (processRays.cu:801-929).  The plan is read on the device; max_rays_in_batch bounds the launch. */
int nb_march_emit(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv,
                  const float* d_nears, const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays, uint32_t rays_done,
                  int64_t max_rays_in_batch, const uint32_t* d_ray_offsets, const uint32_t* d_plan, float* d_t_out,
                  uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream);

/* The single walk: as nb_march_count, but the sample distances of ray i are also stored in row i of d_t_rows
 * (nb_march_row_stride() = 1024 floats per ray), and the counts are scanned into d_ray_offsets[num_rays + 1] (exclusive
 * offsets, last entry = sample total).  d_block_sums: scratch of 1028 uint32.  At most 1048576 rays per call.  A host
 * that reads d_ray_offsets back can cut any number of sample batches out of the rows with nb_march_compact without
 * walking a ray again.  No counterpart in the reference, which walks every ray twice per batch. */
int nb_march_row_stride(void);
int nb_march_fill(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, const float* d_rays_d_inv, const float* d_nears,
                  const float* d_fars, const uint8_t* d_bitfield, int64_t num_rays, uint32_t* d_num_steps, float* d_t_rows,
                  uint32_t* d_ray_offsets, uint32_t* d_block_sums, void* stream);
/* Samples of rays [ray_begin, ray_begin + ray_count) from the rows into the compact arrays the field kernels read:
 * sample k of ray i lands at d_ray_offsets[i] - sample_base + k with its t, its ray id relative to ray_begin and its
 * contracted float4 position - the output of march_rays_dda_offset (processRays.cu:801-929). */
int nb_march_compact(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, uint32_t ray_begin, uint32_t ray_count,
                     const uint32_t* d_num_steps, const uint32_t* d_ray_offsets, uint32_t sample_base, const float* d_t_rows,
                     float* d_t_out, uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream);
/* Rendering in rounds (no counterpart in the reference, whose renderImageHit, InstantNerf.cu:880-990, evaluates every
 * sample of every ray and lets render_rays_kernel skip the ones behind an opaque surface): round [round_begin,
 * round_begin + round_width) of the rows of rays [ray_begin, ray_begin + ray_count) - all arrays are indexed by the ray's
 * place in the walked chunk.  A ray takes part when it has more than round_begin samples and (round_begin > 0) its
 * d_transmittance is still at least 1e-4.  Its samples land contiguously at d_round_offsets[ray] of the compact arrays
 * (ray id = place in the chunk, contracted float4 position); *d_counter (zero before the call) is advanced by the
 * round's sample total, which stays on the device: nb_field_forward_counted reads it there.  capacity = size of the
 * compact arrays in samples; the caller bounds the round (rays x round_width) so that it fits.  d_emitted_total
 * (nullable) is a running 64-bit sum of the samples emitted, for statistics. */
int nb_march_round_emit(const nb_scene_desc* scene, const float* d_rays_o, const float* d_rays_d, uint32_t ray_begin, uint32_t ray_count,
                        const uint32_t* d_num_steps, const float* d_transmittance, uint32_t round_begin, uint32_t round_width,
                        const float* d_t_rows, uint32_t capacity, uint32_t* d_counter, uint64_t* d_emitted_total,
                        uint32_t* d_round_offsets, uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream);

/* ---- compositing and loss gradients ---------------------------------------------------------- */

/* The three compositing entry points give every ray a warp; ray r of the call has num_steps[r] samples starting at
 * d_ray_offsets[r] - sample_base of the sample arrays. */

/* Replaces render_rays_kernel via launchVolumeRendering with d_dw_out == NULL (modules/NeRF/compositing.cu:5-78,
 * InstantNerf.h launchVolumeRendering).  Ray r reads d_ray_offsets[rays_done + r] - base and d_num_steps[r].
 * d_rgb rows are rgb_stride floats apart (3 valid). */
int nb_composite_infer(int64_t num_rays, uint32_t base, uint32_t rays_done, const uint32_t* d_ray_offsets, const uint32_t* d_num_steps,
                       const float* d_t_sorted, const float* d_sigma, const float* d_rgb, int rgb_stride, const float* d_rgb_true,
                       float* d_final_rgb, float* d_final_depth, float* d_phi, const float* bg_color3, void* stream);

/* One round of nb_composite_infer's sum for the rays nb_march_round_emit planned (same arguments, same predicate):
 * continues from d_transmittance / d_composited4 (r, g, b, depth per ray; not read when round_begin == 0), stops a ray
 * for good once its transmittance is below 1e-4 exactly where render_rays_kernel (compositing.cu:5-78) leaves its loop,
 * and writes colour (+ transmittance x background) and depth so far into d_final_rgb / d_final_depth (nullable) at the
 * ray's place in the chunk.  Round 0 writes every ray of the range (background for rays without samples).
 * next_width > 0: the same launch also does nb_march_round_emit's work for the round that follows
 * ([round_begin + round_width, ... + next_width)) for the rays that are still visible, into d_ray_idx_out / d_pos4_out
 * (free by then: this round's field kernel has read them), *d_next_counter (zero before the call) and d_round_offsets;
 * then scene, rays, capacity and the arrays are needed, otherwise they may be NULL / 0.  All ray ranges of one round share
 * the sample arrays, so with next_width > 0 a chunk is processed range by range (all rounds of a range, then the next). */
int nb_composite_round(uint32_t ray_begin, uint32_t ray_count, const uint32_t* d_num_steps, uint32_t* d_round_offsets,
                       const float* d_t_rows, uint32_t round_begin, uint32_t round_width, const float* d_sigma, const float* d_rgb,
                       int rgb_stride, float* d_transmittance, float* d_composited4, float* d_final_rgb, float* d_final_depth,
                       const float* bg_color3, uint32_t next_width, const nb_scene_desc* scene, const float* d_rays_o,
                       const float* d_rays_d, uint32_t capacity, uint32_t* d_next_counter, uint64_t* d_emitted_total,
                       uint32_t* d_ray_idx_out, float* d_pos4_out, void* stream);

/* Replaces render_rays_distortion_kernel via launchVolumeRendering with d_dw_out != NULL
 * (modules/NeRF/compositing.cu:84-213).  d_depth_prior / d_sigma_prior may be NULL (depth supervision off). */
int nb_composite_train(int64_t num_rays, uint32_t sample_base, const uint32_t* d_ray_offsets, const uint32_t* d_num_steps,
                       const float* d_t_sorted, const float* d_sigma, const float* d_depth_prior, const float* d_sigma_prior,
                       const float* d_rgb, int rgb_stride, const float* d_rgb_true, float* d_final_rgb, float* d_final_depth, float* d_phi,
                       float* d_dw_out, float* d_weight_sum, float lambda_dist, float lambda_depth, const float* bg_color3, void* stream);

/* Replaces compute_color_grad (modules/NeRF/otherKernels.cu:303-409).  d_logit0 holds the raw first density output of
 * sample i at d_logit0[i * logit_stride] (16 for a full density-output matrix, 1 for the compact array of
 * nb_field_forward); d_color_out rows are color_stride floats apart; gradient rows are grad_stride (3 or 8) halves,
 * channels 3..7 written as zero. */
int nb_color_grad(int64_t num_rays, uint32_t sample_base, const uint32_t* d_num_steps, const uint32_t* d_ray_offsets,
                  const float* d_t_sorted, const float* d_logit0, int logit_stride, const float* d_color_out, int color_stride,
                  const float* d_phi, const float* d_final_rgb, const float* d_dw_out, const float* d_weight_sum, void* d_color_grad_h,
                  int grad_stride, float* d_tmp_dsigma, float loss_scale, float density_bias, uint32_t total_rays_batch, void* stream);

/* ---- occupancy grid ------------------------------------------------------------------------------ */

/* Replaces sampleAABB (modules/NeRF/otherKernels.cu:591-648): one Philox-jittered, contracted sample per thread,
 * cell id in .w; n == total_cells covers every cell of [cell_offset, cell_offset + n). */
int nb_occ_sample_cells(const nb_scene_desc* scene, float* d_samples4, int n, int total_cells, int cell_offset, uint64_t seed,
                        void* stream);
/* Replaces sampleOccupiedAABB (otherKernels.cu:836-888). */
int nb_occ_sample_occupied(const nb_scene_desc* scene, float* d_samples4, const int* d_active_cells, const int* d_num_active, int n,
                           uint64_t seed, void* stream);
/* Replaces updateTmpGrid (otherKernels.cu:657-678). */
int nb_occ_update_tmp_grid(const float* d_samples4, const float* d_density_out16, float* d_tmp_grid, float density_bias, int n,
                           void* stream);
/* Bytes of scratch nb_occ_update_master_grid needs for total_cells cells. */
int64_t nb_occ_scratch_bytes(int total_cells);
/* Replaces updateMasterGrid + the CUB sum of the master grid (otherKernels.cu:680-698): d_sum[0] = sum of the
 * updated grid. */
int nb_occ_update_master_grid(const float* d_tmp_grid, float* d_master_grid, float decay, int total_cells, void* d_scratch,
                              float* d_sum, void* stream);
/* Replaces updateOccupancyGrid + buildMipmaps / bitfield_max_pool (otherKernels.cu:700-807, InstantNerf.cu:1177-1204). */
int nb_occ_update_bitfield(const nb_scene_desc* scene, uint8_t* d_bitfield, const float* d_master_grid, const float* d_sum,
                           float min_optical_thickness, void* stream);
/* Replaces extractActiveCells (otherKernels.cu:809-834); zeroes *d_num_active first. */
int nb_occ_extract_active(const nb_scene_desc* scene, const uint8_t* d_bitfield, int* d_active_cells, int* d_num_active, void* stream);

/* ---- scene engine (C handle over the InstantNerf host class) ------------------------------------- */

/* Byte-for-byte mirror of NerfOptions (modules/NeRF/InstantNerf.h:35-76); the raw struct is also what the
 * .inerf file stores after its magic. */
typedef struct nb_nerf_options {
    uint32_t grid_resolution[3];
    float aabb_min[3];
    float aabb_max[3];
    int32_t levels_mipmap, num_cascades, samples_per_voxel;
    int32_t density_hidden_dim, density_num_layers;
    int32_t color_hidden_dim, color_num_layers;
    int32_t hash_table_size, num_levels;
    float growth_factor;
    int32_t base_resolution, features_per_level;
    int32_t render_batch_size, batch_size, ray_chunk_size;
    float lambda_depth, lambda_dist, learning_rate, beta1, beta2, epsilon, loss_scale;
    float bg_color[3];
    float min_density_threshold, decay_value, density_bias;
    uint8_t legacy_render_flag, is_profiling;
} nb_nerf_options;

typedef struct nb_nerf nb_nerf;
typedef void (*nb_grad_sync_fn)(void* user, float* d_grads, int64_t count, void* stream);

typedef struct nb_nerf_arena_view {
    float* w; void* w_h; float* g; float* m; float* v;
    int64_t total, sparse_count;
    int64_t density_weight_offset, density_bias_offset, color_weight_offset, color_bias_offset;
    int64_t density_weight_count, density_bias_count, color_weight_count, color_bias_count;
} nb_nerf_arena_view;

typedef struct nb_nerf_step_view {
    const uint32_t *num_steps, *ray_offsets, *ray_indices;
    const float *t_sorted, *positions, *density_out, *sigma, *color_out, *render_rgb, *phi, *dw, *weight_sum, *tmp_dsigma;
    const void *color_in, *color_grad, *density_grad;
    uint32_t last_total_hits;
    int32_t train_steps;
    int32_t logit_stride; /* density_out[i * logit_stride] = raw logit 0 of sample i: 16 (full rows) or 1 (fused field) */
    int32_t color_stride; /* floats between rows of color_out: 8 or 4 (fused field) */
    uint32_t rays_consumed; /* rays of the last nb_nerf_train_rays call that were trained on */
    uint32_t sample_base;   /* num_steps / ray_offsets point at the last step's first ray; ray_offsets[r] - sample_base = its first sample */
} nb_nerf_step_view;

/* NerfOptions defaults (InstantNerf.h:35-76). */
int nb_nerf_default_options(nb_nerf_options* out);
/* InstantNerf::init (InstantNerf.cu:282-339); memory_mode 0 = TRAINING, 1 = INFERENCE.  NULL on failure. */
nb_nerf* nb_nerf_create(const nb_nerf_options* options, int memory_mode);
void nb_nerf_destroy(nb_nerf* h);
/* InstantNerf::trainWithRaysHit (InstantNerf.cu:359-583): float3 rays, optional depth priors, float3 targets. */
int nb_nerf_train_rays(nb_nerf* h, const float* d_rays_o, const float* d_rays_d, const float* d_rays_depth, const float* d_rays_sigma,
                       const float* d_rgb_true, uint32_t num_rays, int* step_count, uint32_t* hit_counts, float* d_rgb_out, void* stream);
/* InstantNerf::renderImageHit (InstantNerf.cu:713-864). */
int nb_nerf_render(nb_nerf* h, const float* d_rays_o, const float* d_rays_d, uint32_t num_rays, float* d_rgb_out, void* stream);
/* setLearningRate / setBgColor / setProfiling / setMemoryMode (InstantNerf.h:289-293). */
int nb_nerf_set_learning_rate(nb_nerf* h, float lr);
int nb_nerf_set_bg_color(nb_nerf* h, float r, float g, float b);
int nb_nerf_set_profiling(nb_nerf* h, int on);
int nb_nerf_set_memory_mode(nb_nerf* h, int memory_mode);
/* Data parallelism (no counterpart in the reference, which is single-GPU): loss gradients are normalised by
 * num_rays * scale, and fn runs on the gradient arena between backward and the optimizer of every step. */
int nb_nerf_set_global_ray_scale(nb_nerf* h, uint32_t scale);
int nb_nerf_set_grad_sync(nb_nerf* h, nb_grad_sync_fn fn, void* user);
/* Sharded optimizer for data parallelism (no counterpart in the reference): this rank applies Adam to slice
 * [rank, rank + 1) * sparse_count / world of the hash table only - nb_grad_sync_fn is expected to leave the summed
 * gradient of that slice in place (reduce-scatter) and the summed gradient of the dense tail (network weights) - clears
 * the rest of the table gradient and then calls fn on the fp16 parameter copy, where the caller all-gathers the slices.
 * Adam's launch and the bytes on the wire shrink; the fp32 master copy and the moments of a slice are current on its
 * owner only.  world <= 1 switches back.  sparse_count must be a multiple of 4 x world. */
typedef void (*nb_param_sync_fn)(void* user, void* d_params_h, int64_t sparse_count, void* stream);
int nb_nerf_set_optimizer_shard(nb_nerf* h, uint32_t rank, uint32_t world, nb_param_sync_fn fn, void* user);
/* Data parallelism through nb_adam_step_peer (no counterpart in the reference): peer_grads[r] / peer_w_h[r] = rank r's
 * gradient arena and fp16 parameter arena (nb_nerf_get_arena's g and w_h) as this process addresses them - its own for
 * r == rank, nb_ipc_open'ed for the others; fn must meet all ranks on the stream it is given (e.g. a one-element
 * all-reduce).  Every optimizer step then runs: fn, the kernel, fn, clearing of this rank's gradient.  nb_grad_sync_fn is
 * not called in this mode.  world <= 1 switches back. */
typedef void (*nb_barrier_fn)(void* user, void* stream);
int nb_nerf_set_peer_exchange(nb_nerf* h, uint32_t rank, uint32_t world, const float* const* peer_grads, void* const* peer_w_h,
                              nb_barrier_fn fn, void* user);
/* Data parallelism with the table partitioned by level instead of replicated (see "level-partitioned grid" above): rank
 * `rank` of `world` owns levels rank, rank + world, ...  Per optimizer step the engine calls
 *   gather(user, send, recv, bytes, stream)    once: recv = every rank's `bytes`-sized block, rank order (an all-gather;
 *                                               send may be the rank's own block inside recv: the in-place form);
 *   exchange(user, send, recv, bytes, stream)  twice: block q of send to rank q, block r of recv from rank r (all-to-all);
 *   reduce(user, d_grads, count, stream)       once: SUM over the ranks of the networks' gradients (a few thousand floats);
 * and `gather` again, per block of `world` levels, before every occupancy update and in nb_nerf_sync_levels, which
 * brings the levels a rank does not own up to date in its copy of the table (fp16 forward copy; master != 0: the fp32
 * copy as well) - call it before rendering, saving or comparing replicas.  world must divide the number of levels; the
 * fused field kernels are required; not together with nb_nerf_set_optimizer_shard / nb_nerf_set_peer_exchange /
 * nb_nerf_set_grad_sync.  world <= 1 switches back. */
/* Data parallelism: rank `rank` evaluates only its share of the density queries of every occupancy update
 * (InstantNerf.cu:1009-1204 evaluates all of them on its one GPU) and reduce_max - an all-reduce with MAX over the ranks,
 * on `count` floats - merges the per-cell maxima before they are folded into the grid; the resulting bits are those of a
 * single GPU.  world <= 1 switches back. */
int nb_nerf_set_occupancy_shard(nb_nerf* h, uint32_t rank, uint32_t world, nb_grad_sync_fn reduce_max, void* user);
typedef void (*nb_block_fn)(void* user, const void* d_send, void* d_recv, int64_t bytes, void* stream);
int nb_nerf_set_level_partition(nb_nerf* h, uint32_t rank, uint32_t world, nb_block_fn gather, nb_block_fn exchange, nb_grad_sync_fn reduce,
                                void* user);
int nb_nerf_sync_levels(nb_nerf* h, int master, void* stream);
/* on != 0: nb_nerf_train_rays runs exactly one optimizer step (one fn call) per call; rays that do not fit the sample
 * batch are left untrained (nb_nerf_step_view.rays_consumed says how many were used) instead of starting a second
 * step, so that every rank of a data-parallel job issues the same number of gradient exchanges. */
int nb_nerf_set_single_step(nb_nerf* h, int on);
/* The general form: exactly `steps` optimizer steps per nb_nerf_train_rays call (0 = as many as the rays need, the
 * reference's loop).  A rank whose rays are used up before the last step takes the remaining steps with no samples
 * of its own: it still calls fn and applies the update. */
int nb_nerf_set_steps_per_call(nb_nerf* h, int steps);
/* Size of the hit_counts array passed to nb_nerf_train_rays (one entry per optimizer step of the call; the reference's
 * trainWithRaysHit writes it unbounded, InstantNerf.cu:429): steps at or beyond `capacity` are not recorded.  0 = unbounded. */
int nb_nerf_set_hit_counts_capacity(nb_nerf* h, uint32_t capacity);
/* Switches between nb_field_forward / nb_field_backward (default when nb_field_supported) and the reference's
 * kernel-by-kernel sequence; returns 1 when the fused kernels are in effect afterwards, 0 otherwise.  Results agree
 * to the fp32 summation order of the weight gradients.  No counterpart in the reference. */
int nb_nerf_set_fused_field(nb_nerf* h, int on);
/* Rendering in rounds of samples per ray (nb_march_round_emit / nb_field_forward_counted / nb_composite_round), so that
 * nothing is evaluated behind the point where a ray turned opaque.  Off by default (every sample of every ray, as the
 * reference's renderImageHit does): it pays when surfaces hide much of what the occupancy grid keeps and costs a few
 * launches per ray chunk when they do not.  Needs the fused field kernels; returns 1 when rounds are in effect afterwards.
 * Frames agree to fp32 rounding (the skipped samples have weight zero in both).  No counterpart in the reference. */
int nb_nerf_set_render_rounds(nb_nerf* h, int on);
/* Samples the field was evaluated on during the last nb_nerf_render call (waits for the device). */
int nb_nerf_last_render_samples(nb_nerf* h, uint64_t* samples);
/* The gradient arena moves into caller-owned device memory of at least `count` >= arena total floats (16-byte aligned;
 * zeroed by the call; the caller keeps it alive until nb_nerf_destroy or a call with NULL, which returns to an own
 * allocation).  For data-parallel training: a buffer allocated by the collective library's allocator and registered
 * with the communicator is all-reduced in place through NVSwitch without staging copies.  Call between steps. */
int nb_nerf_set_grad_buffer(nb_nerf* h, float* d_grads, int64_t count);
/* Device pointers of the parameter arena [hash | density W,b | colour W,b] and the slice offsets. */
int nb_nerf_get_arena(nb_nerf* h, nb_nerf_arena_view* out);
/* loadHashgrid / loadWeights of both networks from host fp32 arrays (any may be NULL);
 * TinyMLPHashGrid.cu:457-497, TinyMLP.cu:483-512. */
int nb_nerf_load_params(nb_nerf* h, const float* hash, const float* density_w, const float* density_b, const float* color_w,
                        const float* color_b);
/* occupancyGrid() / occupancyBytes() (InstantNerf.h:327-328) and the fp32 master grid. */
int nb_nerf_occupancy(nb_nerf* h, uint8_t** d_bitfield, int64_t* bitfield_bytes, float** d_master_grid);
/* earlyOccupancyGridUpdate (InstantNerf.cu:1108-1171) on demand, e.g. after nb_nerf_load_params. */
int nb_nerf_rebuild_occupancy(nb_nerf* h, void* stream);
/* Buffers of the last step (parity tests). */
int nb_nerf_get_step_view(nb_nerf* h, nb_nerf_step_view* out);
/* Summed per-phase device milliseconds when profiling is on: march, occupancy, density fwd, SH, colour fwd,
 * compositing, loss grad, colour bwd, density grad, density bwd, scatter, optimizer (GPUStats, InstantNerf.h:128-277). */
int nb_nerf_phase_times(nb_nerf* h, double* out_ms12, int64_t* steps);
/* InstantNerf::save / load, the .inerf format (InstantNerf.cu:1206-1352). */
int nb_nerf_save(nb_nerf* h, const char* path);
int nb_nerf_load(nb_nerf* h, const char* path);

#ifdef __cplusplus
}
#endif
#endif /* NERF_B200_H */
