"""ctypes front end of oracle/_ref/libref3dmaker.so: the reference's own CUDA classes and kernels, compiled for
sm_100a by oracle/build_ref.py.  TEST INFRASTRUCTURE ONLY (tests marked gpu, and bench.py --impl reference).
Device pointers are passed as integers / c_void_p; torch supplies the memory."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref3dmaker.so")

V, I, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_uint

_SIG = {
    "ref_field_create": (V, [I, I, I, F, I, I, I, I, I]),
    "ref_field_destroy": (None, [V]),
    "ref_field_load": (None, [V, V, V, V, V, V]),
    "ref_field_save": (None, [V, V, V, V, V, V]),
    "ref_field_density_out": (V, [V]),
    "ref_field_color_out": (V, [V]),
    "ref_field_color_in": (V, [V]),
    "ref_field_hash_grads": (V, [V]),
    "ref_field_layer_grads": (V, [V, I, I, I]),
    "ref_field_forward": (None, [V, V, V, I, F, V]),
    "ref_field_forward_backward": (None, [V, V, V, V, I, F, F, V]),
    "ref_field_train_step": (None, [V, V, V, V, I, F, F, F, F, F, F, V]),
    "ref_field_grid_activation": (V, [V, I]),
    "ref_field_step": (None, [V, F, F, F, F, F, V]),
    "ref_nerf_set_learning_rate": (None, [V, F]),
    "ref_nerf_save": (I, [V, ctypes.c_char_p]),
    "ref_nerf_load": (I, [V, ctypes.c_char_p]),
    "ref_volume_rendering_priors": (None, [U, V, V, V, V, V, V, V, V, V, V, V, V, V, F, F, V, V]),
    "ref_nerf_create": (V, [V, I]),
    "ref_nerf_options_size": (I, []),
    "ref_nerf_destroy": (None, [V]),
    "ref_nerf_load_params": (None, [V, V, V, V, V, V]),
    "ref_nerf_save_params": (None, [V, V, V, V, V, V]),
    "ref_nerf_rebuild_occupancy": (None, [V]),
    "ref_nerf_set_train_steps": (None, [V, I]),
    "ref_nerf_bitfield": (V, [V, ctypes.POINTER(ctypes.c_long)]),
    "ref_nerf_master_grid": (V, [V]),
    "ref_nerf_train": (I, [V, V, V, V, V, V, U, V, V, V]),
    "ref_nerf_render": (None, [V, V, V, U, V, V]),
    "ref_nerf_set_memory_mode": (None, [V, I]),
    "ref_nerf_buffer": (V, [V, I]),
    "ref_ray_aabb": (None, [U, V, V, V, V, I, V, V, V, V]),
    "ref_process_rays_hit_linear": (I, [U, V, V, V, V, V, V, V, V, V, I, I, I, I, V, V, V, V, V, V, V, V, V]),
    "ref_volume_rendering": (None, [U, V, V, V, V, V, V, V, V, V, V, V, F, F, V, U, U, V]),
    "ref_color_grad": (None, [U, V, V, V, V, V, V, V, V, V, V, V, F, F, U, V]),
    "ref_sample_aabb": (None, [V, V, V, V, I, I, I, ctypes.c_ulonglong, V]),
}

BUFFERS = {"num_steps": 0, "ray_offsets": 1, "ray_indices": 2, "t_sorted": 3, "positions": 4, "density_out": 5, "sigma": 6, "color_out": 7,
           "render_rgb": 8, "phi": 9, "dw": 10, "weight_sum": 11, "tmp_dsigma": 12, "color_grad": 13, "density_grad": 14, "nears": 15, "fars": 16,
           "rays_d_inv": 17}

_lib = None


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIG.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def hptr(a):
    """Host pointer of a contiguous numpy array (None -> NULL)."""
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)
