"""B200-native NeRF hot path: loader for libnerf_b200.so and thin ctypes bindings.

The package name starts with a digit, so import it with
``importlib.import_module("3dmaker_b200")``.

The product is the shared library (hand-written sm_100a CUDA behind a C ABI, ``include/nerf_b200.h``)
and the C++ host classes built into it.  This module only loads the library, declares the argument
types of its entry points and offers helpers that take torch CUDA tensors (torch is used for device
memory and streams, nothing else).  There is no CPU fallback: if the library is missing, or a call
returns a non-zero status, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnerf_b200.so")

NB_MAX_LEVELS = 16

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_float = ctypes.c_float


class GridDesc(ctypes.Structure):
    """nb_grid_desc of include/nerf_b200.h."""
    _fields_ = [
        ("num_levels", ctypes.c_int32),
        ("table_size", ctypes.c_int32),
        ("base_resolution", ctypes.c_int32),
        ("dense_level_start", ctypes.c_int32),
        ("growth", ctypes.c_float),
        ("scales", ctypes.c_float * NB_MAX_LEVELS),
        ("scatter_scales", ctypes.c_float * NB_MAX_LEVELS),
    ]


class MlpDesc(ctypes.Structure):
    """nb_mlp_desc of include/nerf_b200.h."""
    _fields_ = [
        ("input_dim", ctypes.c_int32),
        ("hidden_dim", ctypes.c_int32),
        ("output_dim", ctypes.c_int32),
        ("num_layers", ctypes.c_int32),
        ("output_activation", ctypes.c_int32),
    ]

    def layer_dims(self):
        dims = []
        for l in range(self.num_layers):
            i = self.input_dim if l == 0 else self.hidden_dim
            o = self.output_dim if l == self.num_layers - 1 else self.hidden_dim
            dims.append((i, o))
        return dims

    @property
    def weight_count(self):
        return sum(i * o for i, o in self.layer_dims())

    @property
    def bias_count(self):
        return sum(o for _, o in self.layer_dims())


class SceneDesc(ctypes.Structure):
    """nb_scene_desc of include/nerf_b200.h."""
    _fields_ = [
        ("grid_res", ctypes.c_uint32 * 3),
        ("aabb_min", ctypes.c_float * 3),
        ("aabb_max", ctypes.c_float * 3),
        ("num_cascades", ctypes.c_int32),
        ("mip_levels", ctypes.c_int32),
        ("samples_per_voxel", ctypes.c_int32),
    ]

    @property
    def cells_per_cascade(self):
        return int(self.grid_res[0]) * int(self.grid_res[1]) * int(self.grid_res[2])

    @property
    def pyramid_cells(self):
        x, y, z, s = int(self.grid_res[0]), int(self.grid_res[1]), int(self.grid_res[2]), 0
        for _ in range(self.mip_levels):
            s += x * y * z
            x, y, z = x >> 1, y >> 1, z >> 1
        return s


def scene_desc(grid_res, aabb_min, aabb_max, num_cascades=1, mip_levels=4, samples_per_voxel=1):
    d = SceneDesc()
    for a in range(3):
        d.grid_res[a] = int(grid_res[a]); d.aabb_min[a] = float(aabb_min[a]); d.aabb_max[a] = float(aabb_max[a])
    d.num_cascades, d.mip_levels, d.samples_per_voxel = num_cascades, mip_levels, samples_per_voxel
    return d


class NerfOptions(ctypes.Structure):
    """nb_nerf_options of include/nerf_b200.h (mirror of the reference's NerfOptions)."""
    _fields_ = [
        ("grid_resolution", ctypes.c_uint32 * 3), ("aabb_min", ctypes.c_float * 3), ("aabb_max", ctypes.c_float * 3),
        ("levels_mipmap", ctypes.c_int32), ("num_cascades", ctypes.c_int32), ("samples_per_voxel", ctypes.c_int32),
        ("density_hidden_dim", ctypes.c_int32), ("density_num_layers", ctypes.c_int32),
        ("color_hidden_dim", ctypes.c_int32), ("color_num_layers", ctypes.c_int32),
        ("hash_table_size", ctypes.c_int32), ("num_levels", ctypes.c_int32), ("growth_factor", ctypes.c_float),
        ("base_resolution", ctypes.c_int32), ("features_per_level", ctypes.c_int32),
        ("render_batch_size", ctypes.c_int32), ("batch_size", ctypes.c_int32), ("ray_chunk_size", ctypes.c_int32),
        ("lambda_depth", ctypes.c_float), ("lambda_dist", ctypes.c_float), ("learning_rate", ctypes.c_float),
        ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("epsilon", ctypes.c_float), ("loss_scale", ctypes.c_float),
        ("bg_color", ctypes.c_float * 3),
        ("min_density_threshold", ctypes.c_float), ("decay_value", ctypes.c_float), ("density_bias", ctypes.c_float),
        ("legacy_render_flag", ctypes.c_uint8), ("is_profiling", ctypes.c_uint8),
    ]


class ImageSet(ctypes.Structure):
    _fields_ = [("d_images_rgba", c_void_p), ("d_transforms", c_void_p), ("num_images", ctypes.c_int32), ("width", ctypes.c_int32),
                ("height", ctypes.c_int32), ("focal", c_float), ("d_rec_frame", c_void_p), ("d_rec_u", c_void_p), ("d_rec_v", c_void_p),
                ("d_rec_depth", c_void_p), ("d_rec_sigma", c_void_p), ("num_records", ctypes.c_uint32), ("dense_fraction", c_float),
                ("prior_width", ctypes.c_int32), ("prior_height", ctypes.c_int32)]


class ArenaView(ctypes.Structure):
    _fields_ = [("w", c_void_p), ("w_h", c_void_p), ("g", c_void_p), ("m", c_void_p), ("v", c_void_p),
                ("total", c_int64), ("sparse_count", c_int64),
                ("density_weight_offset", c_int64), ("density_bias_offset", c_int64), ("color_weight_offset", c_int64),
                ("color_bias_offset", c_int64), ("density_weight_count", c_int64), ("density_bias_count", c_int64),
                ("color_weight_count", c_int64), ("color_bias_count", c_int64)]


class StepView(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("num_steps", "ray_offsets", "ray_indices", "t_sorted", "positions", "density_out", "sigma",
                                        "color_out", "render_rgb", "phi", "dw", "weight_sum", "tmp_dsigma", "color_in", "color_grad",
                                        "density_grad")] + [("last_total_hits", ctypes.c_uint32), ("train_steps", ctypes.c_int32),
                                                            ("logit_stride", ctypes.c_int32), ("color_stride", ctypes.c_int32),
                                                            ("rays_consumed", ctypes.c_uint32), ("sample_base", ctypes.c_uint32)]


GRAD_SYNC_FN = ctypes.CFUNCTYPE(None, c_void_p, c_void_p, c_int64, c_void_p)
PARAM_SYNC_FN = ctypes.CFUNCTYPE(None, c_void_p, c_void_p, c_int64, c_void_p)
BARRIER_FN = ctypes.CFUNCTYPE(None, c_void_p, c_void_p)
BLOCK_FN = ctypes.CFUNCTYPE(None, c_void_p, c_void_p, c_void_p, c_int64, c_void_p)


class NerfB200Error(RuntimeError):
    pass


_SIGNATURES = {
    "nb_last_error": (ctypes.c_char_p, []),
    "nb_version": (c_int, []),
    "nb_built_arch": (c_int, []),
    "nb_launch_count": (ctypes.c_uint64, []),
    "nb_zero_async": (c_int, [c_void_p, c_int64, c_void_p]),
    "nb_grid_setup": (c_int, [ctypes.POINTER(GridDesc), c_int, c_int, c_int, c_float, c_void_p]),
    "nb_grid_setup_noalloc": (c_int, [ctypes.POINTER(GridDesc), c_int, c_int, c_int, c_float, c_void_p]),
    "nb_hash_indices": (c_int, [ctypes.POINTER(GridDesc), c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "nb_hash_encode_forward": (c_int, [ctypes.POINTER(GridDesc), c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "nb_grid_mlp_forward": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_hash_scatter_backward": (c_int, [ctypes.POINTER(GridDesc), c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "nb_set_tuning": (c_int, [ctypes.c_char_p, c_int]),
    "nb_get_tuning": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_int)]),
    "nb_field_backward_tc_status": (c_int, []),
    "nb_field_supported": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc)]),
    "nb_field_forward": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_void_p]),
    "nb_field_forward_counted": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_float,
                                         c_void_p, c_void_p, c_int, c_void_p]),
    "nb_sample_order_scratch_bytes": (c_int64, []),
    "nb_sample_order": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "nb_part_stamp_count": (c_int, [c_void_p, c_int64, c_int64, c_void_p]),
    "nb_part_encode": (c_int, [ctypes.POINTER(GridDesc), c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_part_field_forward": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_int, c_int64, c_void_p, c_void_p,
                              c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_void_p]),
    "nb_part_field_backward": (c_int, [ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_part_pack_denc": (c_int, [ctypes.POINTER(GridDesc), c_int, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "nb_part_scatter": (c_int, [ctypes.POINTER(GridDesc), c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_field_forward_mse": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "nb_field_forward_ordered": (c_int, [ctypes.POINTER(GridDesc), ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_float, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_void_p]),
    "nb_field_backward_ordered": (c_int, [ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, ctypes.POINTER(GridDesc), c_void_p, c_void_p, c_void_p]),
    "nb_field_backward": (c_int, [ctypes.POINTER(MlpDesc), ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, ctypes.POINTER(GridDesc), c_void_p, c_void_p, c_void_p]),
    "nb_mlp_forward": (c_int, [ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "nb_mlp_backward": (c_int, [ctypes.POINTER(MlpDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                c_void_p, c_void_p, c_void_p]),
    "nb_adam_step_peer": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int, c_int64, c_int64,
                                  c_float, c_float, c_float, c_float, c_float, c_float, c_float, c_void_p]),
    "nb_ipc_export": (c_int, [c_void_p, c_void_p]),
    "nb_ipc_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "nb_ipc_close": (c_int, [c_void_p]),
    "nb_device_alloc": (c_int, [c_int64, ctypes.POINTER(c_void_p)]),
    "nb_device_free": (c_int, [c_void_p]),
    "nb_mse_loss_grad": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "nb_adam_step": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_float,
                             c_float, c_float, c_float, c_float, c_float, c_int, c_void_p]),
    "nb_sh_gather": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_density_grad": (c_int, [c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_fetch_ray_chunk": (c_int, [ctypes.POINTER(ImageSet), c_int, c_int, ctypes.c_uint32, c_int, ctypes.POINTER(c_float), c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_generate_rays": (c_int, [c_int, c_int, c_float, ctypes.POINTER(c_float), c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "nb_generate_rays_tiled": (c_int, [c_int, c_int, c_float, ctypes.POINTER(c_float), c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                       c_void_p]),
    "nb_mse_rays": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "nb_ray_aabb": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_march_count": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                               c_void_p]),
    "nb_march_scan": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, ctypes.c_uint32, c_void_p, c_void_p]),
    "nb_march_cutoff": (c_int, [c_void_p, c_void_p, c_int64, ctypes.c_uint32, ctypes.c_uint32, c_void_p, c_void_p]),
    "nb_march_row_stride": (c_int, []),
    "nb_march_fill": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_march_compact": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, ctypes.c_uint32, ctypes.c_uint32, c_void_p, c_void_p,
                                 ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_march_round_emit": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, ctypes.c_uint32, ctypes.c_uint32, c_void_p, c_void_p,
                                    ctypes.c_uint32, ctypes.c_uint32, c_void_p, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p]),
    "nb_march_emit": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                              ctypes.c_uint32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_composite_infer": (c_int, [c_int64, ctypes.c_uint32, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_float), c_void_p]),
    "nb_composite_round": (c_int, [ctypes.c_uint32, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, ctypes.c_uint32, ctypes.c_uint32, c_void_p,
                                   c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_float), ctypes.c_uint32,
                                   ctypes.POINTER(SceneDesc), c_void_p, c_void_p, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p]),
    "nb_composite_train": (c_int, [c_int64, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, ctypes.POINTER(c_float), c_void_p]),
    "nb_color_grad": (c_int, [c_int64, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_int, c_void_p, c_float, c_float, ctypes.c_uint32, c_void_p]),
    "nb_occ_sample_cells": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_int, c_int, c_int, ctypes.c_uint64, c_void_p]),
    "nb_occ_sample_occupied": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_int, ctypes.c_uint64, c_void_p]),
    "nb_occ_update_tmp_grid": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p]),
    "nb_occ_scratch_bytes": (c_int64, [c_int]),
    "nb_occ_update_master_grid": (c_int, [c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "nb_occ_update_bitfield": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "nb_occ_extract_active": (c_int, [ctypes.POINTER(SceneDesc), c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_probe_random_access": (c_int, [c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "nb_unpack_samples": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "nb_undeal_tiles": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "nb_nerf_default_options": (c_int, [ctypes.POINTER(NerfOptions)]),
    "nb_nerf_create": (c_void_p, [ctypes.POINTER(NerfOptions), c_int]),
    "nb_nerf_destroy": (None, [c_void_p]),
    "nb_nerf_train_rays": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_uint32, ctypes.POINTER(c_int),
                                   c_void_p, c_void_p, c_void_p]),
    "nb_nerf_render": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.c_uint32, c_void_p, c_void_p]),
    "nb_nerf_set_learning_rate": (c_int, [c_void_p, c_float]),
    "nb_nerf_set_bg_color": (c_int, [c_void_p, c_float, c_float, c_float]),
    "nb_nerf_set_profiling": (c_int, [c_void_p, c_int]),
    "nb_nerf_set_memory_mode": (c_int, [c_void_p, c_int]),
    "nb_nerf_set_global_ray_scale": (c_int, [c_void_p, ctypes.c_uint32]),
    "nb_nerf_set_fused_field": (c_int, [c_void_p, c_int]),
    "nb_nerf_set_render_rounds": (c_int, [c_void_p, c_int]),
    "nb_nerf_last_render_samples": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint64)]),
    "nb_nerf_set_single_step": (c_int, [c_void_p, c_int]),
    "nb_nerf_set_steps_per_call": (c_int, [c_void_p, c_int]),
    "nb_nerf_set_optimizer_shard": (c_int, [c_void_p, ctypes.c_uint32, ctypes.c_uint32, PARAM_SYNC_FN, c_void_p]),
    "nb_nerf_set_peer_exchange": (c_int, [c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), BARRIER_FN,
                                          c_void_p]),
    "nb_nerf_set_hit_counts_capacity": (c_int, [c_void_p, ctypes.c_uint32]),
    "nb_nerf_set_grad_sync": (c_int, [c_void_p, GRAD_SYNC_FN, c_void_p]),
    "nb_nerf_set_level_partition": (c_int, [c_void_p, ctypes.c_uint32, ctypes.c_uint32, BLOCK_FN, BLOCK_FN, GRAD_SYNC_FN, c_void_p]),
    "nb_nerf_set_occupancy_shard": (c_int, [c_void_p, ctypes.c_uint32, ctypes.c_uint32, GRAD_SYNC_FN, c_void_p]),
    "nb_nerf_sync_levels": (c_int, [c_void_p, c_int, c_void_p]),
    "nb_nerf_set_grad_buffer": (c_int, [c_void_p, c_void_p, c_int64]),
    "nb_nerf_get_arena": (c_int, [c_void_p, ctypes.POINTER(ArenaView)]),
    "nb_nerf_load_params": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "nb_nerf_occupancy": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), ctypes.POINTER(c_void_p)]),
    "nb_nerf_rebuild_occupancy": (c_int, [c_void_p, c_void_p]),
    "nb_nerf_get_step_view": (c_int, [c_void_p, ctypes.POINTER(StepView)]),
    "nb_nerf_phase_times": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(c_int64)]),
    "nb_nerf_save": (c_int, [c_void_p, ctypes.c_char_p]),
    "nb_nerf_load": (c_int, [c_void_p, ctypes.c_char_p]),
}

_lib = None


def declared_symbols():
    """Names of every entry point this module binds (a subset check against include/*.h lives in tests)."""
    return sorted(_SIGNATURES)


def load():
    """Loads libnerf_b200.so (once).  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NerfB200Error(
            "libnerf_b200.so is missing (%s): build it with `python 3dmaker_b200/build.py`; "
            "there is no CPU or PyTorch fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status, what=""):
    if status != 0:
        msg = load().nb_last_error().decode("utf-8", "replace")
        raise NerfB200Error("%s failed with status %d: %s" % (what or "libnerf_b200 call", status, msg))


def get_tuning(key):
    v = c_int(0)
    check(load().nb_get_tuning(key.encode(), ctypes.byref(v)), "nb_get_tuning(%s)" % key)
    return v.value


def set_grad_table_half(on, scale_log2=None):
    """Process-wide: the hash part of every gradient arena becomes one __half2 per entry (see nb_set_tuning in
    include/nerf_b200.h).  Call it before the first backward, never between a backward and its optimizer step."""
    if scale_log2 is not None:
        check(load().nb_set_tuning(b"grad_table_scale_log2", int(scale_log2)), "nb_set_tuning(grad_table_scale_log2)")
    check(load().nb_set_tuning(b"grad_table_half", 1 if on else 0), "nb_set_tuning(grad_table_half)")


def grad_table_half():
    return get_tuning("grad_table_half") != 0


def grad_table_scale():
    return float(1 << get_tuning("grad_table_scale_log2")) if grad_table_half() else 1.0


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise NerfB200Error("expected a CUDA tensor")
    if not t.is_contiguous():
        raise NerfB200Error("expected a contiguous tensor")
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def grid_setup(num_levels, table_size, base_resolution, growth, stream=None):
    d = GridDesc()
    check(load().nb_grid_setup(ctypes.byref(d), num_levels, table_size, base_resolution, growth, stream_ptr(stream)),
          "nb_grid_setup")
    return d


def mlp_desc(input_dim, hidden_dim, output_dim, num_layers, output_activation=0):
    return MlpDesc(input_dim, hidden_dim, output_dim, num_layers, output_activation)
