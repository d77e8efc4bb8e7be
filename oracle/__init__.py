"""ctypes front end of the CPU oracle (oracle/nerf_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the cpu_baseline /
reference legs of bench.py, never by the product package.  All arrays are numpy; fp16 data travels as
uint16 bit patterns (``arr.view(np.uint16)``).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
SRC = os.path.join(_HERE, "nerf_oracle.c")

# x86-64-v3 (AVX2, FMA, F16C) instead of -march=native so the prebuilt library also runs on the GPU
# box's host CPU.  -ffp-contract=off: fused multiply-adds only where the source says fmaf.
CFLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-std=gnu11", "-Wall"]


def build(force=False):
    if (not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= os.path.getmtime(SRC)):
        return LIB_PATH
    cmd = ["gcc"] + CFLAGS + [SRC, "-o", LIB_PATH, "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + r.stderr)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.orc_mse_loss_grad.restype = ctypes.c_double
        _lib.orc_dense_level_start.restype = ctypes.c_int
        _lib.orc_mlp_weight_count.restype = ctypes.c_long
        _lib.orc_mlp_bias_count.restype = ctypes.c_long
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f(x):
    return ctypes.c_float(float(x))


def _c(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def dense_level_start(table_size, base, growth, num_levels):
    return int(lib().orc_dense_level_start(int(table_size), int(base), _f(growth), int(num_levels)))


def level_scales(base, growth, num_levels):
    out = np.zeros(num_levels, np.float32)
    lib().orc_level_scales(int(base), _f(growth), int(num_levels), _p(out))
    return out


def hash_indices(pos4, scales, table_size, dls, clamp_mode=0, want_weights=False):
    pos4 = _c(pos4, np.float32)
    scales = _c(scales, np.float32)
    n, L = pos4.shape[0], scales.shape[0]
    idx = np.zeros((n, L, 8), np.uint32)
    w = np.zeros((n, L, 8), np.float32) if want_weights else None
    lib().orc_hash_indices(_p(pos4), ctypes.c_long(n), _p(scales), L, int(table_size), int(dls), int(clamp_mode), _p(idx), _p(w))
    return (idx, w) if want_weights else idx


def encode_forward(pos4, table_h, scales, table_size, dls):
    """table_h: uint16 view of the fp16 table [L][T][2]; returns uint16 [n][2L]."""
    pos4 = _c(pos4, np.float32)
    table_h = _c(table_h, np.uint16)
    scales = _c(scales, np.float32)
    n, L = pos4.shape[0], scales.shape[0]
    out = np.zeros((n, 2 * L), np.uint16)
    lib().orc_encode_forward(_p(pos4), ctypes.c_long(n), _p(table_h), _p(scales), L, int(table_size), int(dls), _p(out))
    return out


def scatter_backward(pos4, denc_h, scales, table_size, dls, grads=None):
    pos4 = _c(pos4, np.float32)
    denc_h = _c(denc_h, np.uint16)
    scales = _c(scales, np.float32)
    n, L = pos4.shape[0], scales.shape[0]
    if grads is None:
        grads = np.zeros(L * table_size * 2, np.float32)
    lib().orc_scatter_backward(_p(pos4), ctypes.c_long(n), _p(denc_h), _p(scales), L, int(table_size), int(dls), _p(grads))
    return grads


def mlp_forward(in_h, dims, W_h, bias, out_act=0, save_acts=False):
    """dims = (input, hidden, output, layers).  Returns (out fp32 [n][out], acts uint16 or None)."""
    i, h, o, nl = dims
    in_h = _c(in_h, np.uint16)
    W_h = _c(W_h, np.uint16)
    bias = _c(bias, np.float32)
    n = in_h.shape[0]
    out = np.zeros((n, o), np.float32)
    acts = np.zeros((max(nl - 1, 0), n, h), np.uint16) if save_acts else None
    lib().orc_mlp_forward(_p(in_h), ctypes.c_long(n), i, h, o, nl, _p(W_h), _p(bias), int(out_act), _p(out), _p(acts))
    return out, acts


def mlp_backward(dL_h, dims, W_h, act0_h, acts_h, want_dx=False):
    i, h, o, nl = dims
    dL_h = _c(dL_h, np.uint16)
    W_h = _c(W_h, np.uint16)
    act0_h = _c(act0_h, np.uint16)
    acts_h = _c(acts_h, np.uint16) if acts_h is not None else np.zeros(1, np.uint16)
    n = dL_h.shape[0]
    dW = np.zeros(int(lib().orc_mlp_weight_count(i, h, o, nl)), np.float32)
    db = np.zeros(int(lib().orc_mlp_bias_count(h, o, nl)), np.float32)
    dX = np.zeros((n, i), np.uint16) if want_dx else None
    lib().orc_mlp_backward(ctypes.c_long(n), i, h, o, nl, _p(dL_h), _p(W_h), _p(act0_h), _p(acts_h), _p(dW), _p(db), _p(dX))
    return dW, db, dX


def mse_loss_grad(pred, target_h, valid, loss_scale, out_act=0):
    pred = _c(pred, np.float32)
    target_h = _c(target_h, np.uint16)
    n, padded = pred.shape
    grad = np.zeros((n, padded), np.uint16)
    total = lib().orc_mse_loss_grad(_p(pred), _p(target_h), _p(grad), ctypes.c_long(n), int(padded), int(valid),
                                    _f(loss_scale), int(out_act))
    return float(total), grad


def adam_dense(w, g, m, v, lr, b1, b2, eps, bc1, bc2, ils, want_half=True):
    """In place on w, m, v; returns the fp16 copy (uint16) or None."""
    wh = np.zeros(w.shape, np.uint16) if want_half else None
    lib().orc_adam_dense(_p(w), _p(wh), _p(_c(g, np.float32)), _p(m), _p(v), ctypes.c_long(w.size), _f(lr), _f(b1), _f(b2),
                         _f(eps), _f(bc1), _f(bc2), _f(ils))
    return wh


def adam_hash(w, wh, g, m, v, lr, b1, b2, eps, bc1, bc2, ils):
    """In place on w, wh, g (zeroed where consumed), m, v."""
    lib().orc_adam_hash(_p(w), _p(wh), _p(g), _p(m), _p(v), ctypes.c_long(w.size), _f(lr), _f(b1), _f(b2), _f(eps), _f(bc1),
                        _f(bc2), _f(ils))


def adam_bias_corrections(step, b1, b2):
    a, b = ctypes.c_float(), ctypes.c_float()
    lib().orc_adam_bias_corrections(int(step), _f(b1), _f(b2), ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


def half_bits(x):
    """float32 array -> uint16 bit patterns of its fp16 rounding (round to nearest even)."""
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def half_values(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def sh_gather(dirs3, ray_indices, density_out16, density_bias, offset=0):
    dirs3 = _c(dirs3, np.float32)
    ray_indices = _c(ray_indices, np.uint32)
    density_out16 = _c(density_out16, np.float32)
    n = density_out16.shape[0]
    color_in = np.zeros((n, 32), np.uint16)
    sigma = np.zeros(n, np.float32)
    lib().orc_sh_gather(_p(dirs3), _p(ray_indices), ctypes.c_long(offset), ctypes.c_long(n), _f(density_bias), _p(density_out16),
                        _p(color_in), _p(sigma))
    return color_in, sigma


def density_grad(tmp_dsigma, color_dx32_h):
    tmp_dsigma = _c(tmp_dsigma, np.float32)
    color_dx32_h = _c(color_dx32_h, np.uint16)
    n = tmp_dsigma.shape[0]
    out = np.zeros((n, 16), np.uint16)
    lib().orc_density_grad(ctypes.c_long(n), _p(tmp_dsigma), _p(color_dx32_h), _p(out))
    return out


# ---- rays, march, compositing, occupancy ------------------------------------------------------------------

def _u32x3(res):
    return np.ascontiguousarray(res, np.uint32)


def _f3(v):
    return np.ascontiguousarray(v, np.float32)


def ray_aabb(rays_o, rays_d, aabb_min, aabb_max, num_cascades):
    rays_o, rays_d = _c(rays_o, np.float32), _c(rays_d, np.float32)
    n = rays_o.shape[0]
    d_inv = np.zeros((n, 3), np.float32); nears = np.zeros(n, np.float32); fars = np.zeros(n, np.float32)
    lib().orc_ray_aabb(ctypes.c_long(n), _p(rays_o), _p(rays_d), _p(_f3(aabb_min)), _p(_f3(aabb_max)), int(num_cascades), _p(d_inv),
                       _p(nears), _p(fars))
    return d_inv, nears, fars


def contract_pos(pos3, aabb_min, aabb_max):
    pos3 = _c(pos3, np.float32)
    out = np.zeros_like(pos3)
    lib().orc_contract_pos(ctypes.c_long(pos3.shape[0]), _p(pos3), _p(_f3(aabb_min)), _p(_f3(aabb_max)), _p(out))
    return out


def pyramid_cells(res, levels):
    lib().orc_pyramid_cells.restype = ctypes.c_uint32
    return int(lib().orc_pyramid_cells(_p(_u32x3(res)), int(levels)))


def march_count(rays_o, rays_d, d_inv, nears, fars, grid, res, aabb_min, aabb_max, num_cascades, levels, spv):
    n = rays_o.shape[0]
    out = np.zeros(n, np.uint32)
    lib().orc_march_count(ctypes.c_long(n), _p(_c(rays_o, np.float32)), _p(_c(rays_d, np.float32)), _p(_c(d_inv, np.float32)),
                          _p(_c(nears, np.float32)), _p(_c(fars, np.float32)), _p(_c(grid, np.uint8)), _p(_u32x3(res)), _p(_f3(aabb_min)),
                          _p(_f3(aabb_max)), int(num_cascades), int(levels), int(spv), _p(out))
    return out


def march_emit(rays_o, rays_d, d_inv, nears, fars, grid, res, aabb_min, aabb_max, num_cascades, levels, spv, ray_offsets, base, total):
    n = rays_o.shape[0]
    t = np.zeros(total, np.float32); ray = np.zeros(total, np.uint32); pos = np.zeros((total, 4), np.float32)
    lib().orc_march_emit(ctypes.c_long(n), _p(_c(rays_o, np.float32)), _p(_c(rays_d, np.float32)), _p(_c(d_inv, np.float32)),
                         _p(_c(nears, np.float32)), _p(_c(fars, np.float32)), _p(_c(grid, np.uint8)), _p(_u32x3(res)), _p(_f3(aabb_min)),
                         _p(_f3(aabb_max)), int(num_cascades), int(levels), int(spv), _p(_c(ray_offsets, np.uint32)), ctypes.c_uint32(base),
                         _p(t), _p(ray), _p(pos))
    return t, ray, pos


def exclusive_sum(counts):
    counts = _c(counts, np.uint32)
    out = np.zeros_like(counts)
    lib().orc_exclusive_sum(ctypes.c_long(counts.size), _p(counts), _p(out))
    return out


def find_cutoff(ray_offsets, num_steps, batch_size, rays_done=0):
    lib().orc_find_cutoff.restype = ctypes.c_uint32
    return int(lib().orc_find_cutoff(ctypes.c_long(len(num_steps)), _p(_c(ray_offsets, np.uint32)), _p(_c(num_steps, np.uint32)),
                                     ctypes.c_uint32(batch_size), ctypes.c_uint32(rays_done)))


def render_rays(num_rays, base, rays_done, ray_offsets, num_steps, t_sorted, sigma, rgb3, rgb_true, bg):
    rgb = np.zeros((num_rays, 3), np.float32); depth = np.zeros(num_rays, np.float32)
    phi = np.zeros((num_rays, 3), np.float32) if rgb_true is not None else None
    lib().orc_render_rays(ctypes.c_long(num_rays), ctypes.c_uint32(base), ctypes.c_uint32(rays_done), _p(_c(ray_offsets, np.uint32)),
                          _p(_c(num_steps, np.uint32)), _p(_c(t_sorted, np.float32)), _p(_c(sigma, np.float32)), _p(_c(rgb3, np.float32)),
                          _p(_c(rgb_true, np.float32)) if rgb_true is not None else None, _p(rgb), _p(depth), _p(phi), _p(_f3(bg)))
    return rgb, depth, phi


def render_rays_distortion(num_rays, ray_offsets, num_steps, t_sorted, sigma, rgb3, rgb_true, lambda_dist, lambda_depth, bg,
                           depth_prior=None, sigma_prior=None):
    n = len(t_sorted)
    rgb = np.zeros((num_rays, 3), np.float32); depth = np.zeros(num_rays, np.float32); phi = np.zeros((num_rays, 3), np.float32)
    dw = np.zeros(n, np.float32); wsum = np.zeros(num_rays, np.float32)
    lib().orc_render_rays_distortion(ctypes.c_long(num_rays), _p(_c(ray_offsets, np.uint32)), _p(_c(num_steps, np.uint32)),
                                     _p(_c(t_sorted, np.float32)), _p(_c(sigma, np.float32)),
                                     _p(_c(depth_prior, np.float32)) if depth_prior is not None else None,
                                     _p(_c(sigma_prior, np.float32)) if sigma_prior is not None else None, _p(_c(rgb3, np.float32)),
                                     _p(_c(rgb_true, np.float32)), _p(rgb), _p(depth), _p(phi), _p(dw), _p(wsum), _f(lambda_dist),
                                     _f(lambda_depth), _p(_f3(bg)))
    return rgb, depth, phi, dw, wsum


def color_grad(num_rays, num_steps, ray_offsets, t_sorted, density_out16, color_out, phi, final_rgb, dw, wsum, loss_scale, density_bias,
               total_rays, grad_stride=8):
    color_out = _c(color_out, np.float32)
    n = len(t_sorted)
    grad = np.zeros((n, grad_stride), np.uint16); dsig = np.zeros(n, np.float32)
    lib().orc_color_grad(ctypes.c_long(num_rays), _p(_c(num_steps, np.uint32)), _p(_c(ray_offsets, np.uint32)), _p(_c(t_sorted, np.float32)),
                         _p(_c(density_out16, np.float32)), _p(color_out), int(color_out.shape[1]), _p(_c(phi, np.float32)),
                         _p(_c(final_rgb, np.float32)), _p(_c(dw, np.float32)), _p(_c(wsum, np.float32)), _p(grad), int(grad_stride), _p(dsig),
                         _f(loss_scale), _f(density_bias), ctypes.c_uint32(total_rays))
    return grad, dsig


def philox_uniform4(seed, subsequence):
    out = np.zeros(4, np.float32)
    lib().orc_philox_uniform4(ctypes.c_uint64(seed), ctypes.c_uint64(subsequence), _p(out))
    return out


def sample_aabb(aabb_min, aabb_max, res, n, total_cells, cell_offset, seed):
    out = np.zeros((n, 4), np.float32)
    lib().orc_sample_aabb(_p(out), _p(_f3(aabb_min)), _p(_f3(aabb_max)), _p(_u32x3(res)), int(n), int(total_cells), int(cell_offset),
                          ctypes.c_uint64(seed))
    return out


def sample_occupied(active, aabb_min, aabb_max, res, n, seed):
    active = _c(active, np.int32)
    out = np.zeros((n, 4), np.float32)
    lib().orc_sample_occupied(_p(out), _p(active), int(active.size), _p(_f3(aabb_min)), _p(_f3(aabb_max)), _p(_u32x3(res)), int(n),
                              ctypes.c_uint64(seed))
    return out


def update_tmp_grid(samples4, density_out16, tmp_grid, density_bias):
    samples4 = _c(samples4, np.float32)
    lib().orc_update_tmp_grid(_p(samples4), _p(_c(density_out16, np.float32)), _p(tmp_grid), _f(density_bias), int(samples4.shape[0]))


def update_master_grid(tmp_grid, master, decay):
    lib().orc_update_master_grid(_p(_c(tmp_grid, np.float32)), _p(master), _f(decay), int(master.size))


def update_occupancy_bits(bitfield, master, total_sum, cells_per_cascade, pyramid, min_optical_thickness, base_voxel):
    lib().orc_update_occupancy_bits(_p(bitfield), _p(_c(master, np.float32)), _f(total_sum), int(master.size), int(cells_per_cascade),
                                    int(pyramid), _f(min_optical_thickness), _f(base_voxel))


def build_mipmaps(bitfield, res, levels, num_cascades):
    lib().orc_build_mipmaps(_p(bitfield), _p(_u32x3(res)), int(levels), int(num_cascades))


def extract_active_cells(bitfield, total_cells, cells_per_cascade, pyramid):
    out = np.zeros(total_cells, np.int32)
    n = lib().orc_extract_active_cells(_p(_c(bitfield, np.uint8)), _p(out), int(total_cells), int(cells_per_cascade), int(pyramid))
    return out[:n].copy()


def pcg_hash(v):
    lib().orc_pcg.restype = ctypes.c_uint32
    return int(lib().orc_pcg(ctypes.c_uint32(int(v) & 0xffffffff)))


def fetch_ray_chunk(offset, size, seed, randomize, width, height, focal, transforms, images_rgba, bg, holdout_every=0, records=None,
                    dense_fraction=0.0, prior_wh=(0, 0)):
    """fetchRayChunkStreamingKernel on the CPU.  images_rgba uint8 [n][h][w][4], transforms float32 [n][16].
    records = (frame int32, u, v, depth, sigma float32 arrays) or None.  Returns rays_o, rays_d, rgb, depth, sigma, picked."""
    images_rgba = _c(images_rgba, np.uint8)
    n = images_rgba.shape[0]
    total = n * width * height
    ro, rd, rgb = np.zeros((size, 3), np.float32), np.zeros((size, 3), np.float32), np.zeros((size, 3), np.float32)
    dep, sig, pick = np.zeros(size, np.float32), np.zeros(size, np.float32), np.zeros(size, np.uint32)
    if records is None:
        rf = ru = rv = rD = rs = None
        nrec = 0
    else:
        rf, ru, rv, rD, rs = (_c(records[0], np.int32), _c(records[1], np.float32), _c(records[2], np.float32), _c(records[3], np.float32),
                              _c(records[4], np.float32))
        nrec = len(rf)
    sx = float(width) / prior_wh[0] if prior_wh[0] > 0 else 1.0
    sy = float(height) / prior_wh[1] if prior_wh[1] > 0 else 1.0
    P = lambda a: None if a is None else _p(a)
    lib().orc_fetch_ray_chunk(int(offset), int(size), int(total), ctypes.c_uint32(int(seed)), int(randomize), int(width), int(height), _f(focal),
                              _p(_c(transforms, np.float32)), _p(images_rgba), _p(ro), _p(rd), _p(rgb), _p(dep), _p(sig), _p(pick), P(rf), P(ru), P(rv),
                              P(rD), P(rs), ctypes.c_uint32(nrec), _f(dense_fraction), _f(sx), _f(sy), _p(_c(np.asarray(bg, np.float32), np.float32)),
                              int(holdout_every))
    return ro, rd, rgb, dep, sig, pick
