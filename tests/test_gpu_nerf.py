"""GPU parity of the NeRF-level kernels (ray slab test, DDA march, scan + cutoff, compositing, loss
gradients, occupancy grid) against the CPU oracle, through the C ABI.

The march kernels use the device's approximate division / log2 / exp2 (the reference is built with
--use_fast_math); the oracle uses IEEE and libm.  Floats therefore agree to a few ulp, and a ray that grazes a
voxel face within that error may gain or lose a sample: counts are compared per ray with a small allowance
(MARCH_MISMATCH), everything downstream is compared on the rays whose counts agree."""
import ctypes
import importlib

import numpy as np
import pytest

from helpers import ABS_RGB, REL_MLP, Uploader, dev_half_bits, half_vals, rel_err
from test_oracle_nerf_cpu import camera_rays, speckled_bitfield, sphere_bitfield

pytestmark = pytest.mark.gpu

MARCH_MISMATCH = 5e-3   # fraction of rays whose sample count may differ from the IEEE restatement


def _scene(nb, res, cascades, levels, spv, aabb=0.5):
    return nb.scene_desc(res, [-aabb] * 3, [aabb] * 3, cascades, levels, spv)


def _march_gpu(torch, nb, up, sc, o, d, bits, batch):
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    n = o.shape[0]
    f32, u32 = torch.float32, torch.int32
    d_o, d_d = up.f(o), up.f(d)
    d_inv = torch.zeros((n, 3), dtype=f32, device="cuda"); nears = torch.zeros(n, dtype=f32, device="cuda"); fars = torch.zeros_like(nears)
    nb.check(lib.nb_ray_aabb(ctypes.byref(sc), d_o, d_d, n, P(d_inv), P(nears), P(fars), st), "nb_ray_aabb")
    d_bits = torch.from_numpy(bits).cuda()
    steps = torch.zeros(n, dtype=u32, device="cuda"); offs = torch.zeros_like(steps)
    nb.check(lib.nb_march_count(ctypes.byref(sc), d_o, d_d, P(d_inv), P(nears), P(fars), P(d_bits), n, P(steps), st), "nb_march_count")
    bsums = torch.zeros((n + 1023) // 1024 + 1, dtype=u32, device="cuda"); plan = torch.zeros(4, dtype=u32, device="cuda")
    nb.check(lib.nb_march_scan(P(steps), P(offs), P(bsums), n, batch, P(plan), st), "nb_march_scan")
    torch.cuda.synchronize()
    return dict(d_o=d_o, d_d=d_d, d_inv=d_inv, nears=nears, fars=fars, bits=d_bits, steps=steps, offs=offs, plan=plan)


@pytest.mark.parametrize("cascades,spv,res", [(1, 1, 128), (3, 1, 128), (1, 2, 64)])
def test_march_count_scan_emit(cuda, nb, orc, cascades, spv, res):
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    levels, R = 4, 20000
    r3 = (res, res, res)
    sc = _scene(nb, r3, cascades, levels, spv)
    bits = sphere_bitfield(orc, r3, levels, cascades)
    o, d = camera_rays(R, seed=2)
    batch = 1 << 18
    g = _march_gpu(torch, nb, up, sc, o, d, bits, batch)
    amin, amax = [-.5] * 3, [.5] * 3
    # slab test: same formulas, device reciprocal is approximate
    d_inv_ref, n_ref, f_ref = orc.ray_aabb(o, d, amin, amax, cascades)
    d_inv, nears, fars = (g[k].cpu().numpy() for k in ("d_inv", "nears", "fars"))
    assert np.allclose(d_inv, d_inv_ref, rtol=2e-6) and np.allclose(nears, n_ref, rtol=1e-5, atol=1e-6) and np.allclose(fars, f_ref, rtol=1e-5)
    # counts: the oracle walks with the GPU's own d_inv / near / far
    cnt = g["steps"].cpu().numpy().view(np.uint32)
    cnt_ref = orc.march_count(o, d, d_inv, nears, fars, bits, r3, amin, amax, cascades, levels, spv)
    mism = np.mean(cnt != cnt_ref)
    assert mism <= MARCH_MISMATCH, "sample counts differ on %.3f%% of rays" % (100 * mism)
    assert np.max(np.abs(cnt.astype(np.int64) - cnt_ref.astype(np.int64))) <= 2 * spv
    assert cnt.sum() > 100000
    # scan and cutoff are integer work on the GPU's own counts: bit-exact
    offs = g["offs"].cpu().numpy().view(np.uint32)
    assert np.array_equal(offs, orc.exclusive_sum(cnt))
    plan = g["plan"].cpu().numpy().view(np.uint32)
    active = orc.find_cutoff(offs, cnt, batch)
    assert plan[0] == active and plan[1] == (offs[active - 1] + cnt[active - 1] if active else 0) and plan[2] == 0 and plan[3] == cnt.sum()
    assert 0 < active < R                               # the budget cuts the chunk: the cutoff path is exercised
    # emit
    total = int(plan[1])
    t = torch.zeros(batch, dtype=torch.float32, device="cuda"); ray = torch.zeros(batch, dtype=torch.int32, device="cuda")
    pos = torch.zeros((batch, 4), dtype=torch.float32, device="cuda")
    nb.check(lib.nb_march_emit(ctypes.byref(sc), g["d_o"], g["d_d"], P(g["d_inv"]), P(g["nears"]), P(g["fars"]), P(g["bits"]), R, 0, R,
                               P(g["offs"]), P(g["plan"]), P(t), P(ray), P(pos), st), "nb_march_emit")
    torch.cuda.synchronize()
    t, ray, pos = t.cpu().numpy()[:total], ray.cpu().numpy().view(np.uint32)[:total], pos.cpu().numpy()[:total]
    assert np.array_equal(ray, np.repeat(np.arange(active, dtype=np.uint32), cnt[:active]))      # ray-ordered, ids exact
    good = np.nonzero(cnt[:active] == cnt_ref[:active])[0]
    offs_ref = orc.exclusive_sum(cnt_ref)
    t_ref, _, pos_ref = orc.march_emit(o, d, d_inv, nears, fars, bits, r3, amin, amax, cascades, levels, spv, offs_ref, 0, int(cnt_ref.sum()))
    idx = np.concatenate([np.arange(offs[r], offs[r] + cnt[r]) for r in good])
    idx_ref = np.concatenate([np.arange(offs_ref[r], offs_ref[r] + cnt_ref[r]) for r in good])
    assert np.allclose(t[idx], t_ref[idx_ref], rtol=2e-5, atol=2e-6)
    assert np.allclose(pos[idx], pos_ref[idx_ref], atol=2e-6)
    # second batch of the same chunk: cutoff from rays_done, emit relative to it
    nb.check(lib.nb_march_cutoff(P(g["steps"]), P(g["offs"]), R, active, batch, P(g["plan"]), st), "nb_march_cutoff")
    torch.cuda.synchronize()
    plan2 = g["plan"].cpu().numpy().view(np.uint32)
    nxt = orc.find_cutoff(offs, cnt, batch, rays_done=active)
    assert plan2[0] == nxt and plan2[2] == offs[active] and plan2[1] == offs[nxt - 1] + cnt[nxt - 1] - offs[active]
    ray2 = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
    nb.check(lib.nb_march_emit(ctypes.byref(sc), g["d_o"], g["d_d"], P(g["d_inv"]), P(g["nears"]), P(g["fars"]), P(g["bits"]), R, active, R,
                               P(g["offs"]), P(g["plan"]), P(t := torch.zeros(batch, dtype=torch.float32, device="cuda")), P(ray2),
                               P(pos := torch.zeros((batch, 4), dtype=torch.float32, device="cuda")), st), "nb_march_emit")
    torch.cuda.synchronize()
    r2 = ray2.cpu().numpy()[:int(plan2[1])]
    assert np.array_equal(r2, np.repeat(np.arange(nxt - active), cnt[active:nxt]))


@pytest.mark.parametrize("cascades,spv,res,levels", [(1, 1, 128, 4), (3, 1, 128, 4), (1, 2, 64, 3)])
def test_single_walk_and_compaction_equal_the_two_pass_march(cuda, nb, orc, cascades, spv, res, levels):
    """nb_march_fill + nb_march_compact against nb_march_count / scan / cutoff / emit on the same rays: counts,
    offsets, ray ids, distances and positions are the same bits, batch after batch."""
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    R, batch = 30000, 1 << 17
    r3 = (res, res, res)
    sc = _scene(nb, r3, cascades, levels, spv)
    bits = speckled_bitfield(orc, r3, levels, cascades)
    o, d = camera_rays(R, seed=4)
    g = _march_gpu(torch, nb, up, sc, o, d, bits, batch)
    i32, f32 = torch.int32, torch.float32
    steps2 = torch.zeros(R, dtype=i32, device="cuda"); offs2 = torch.zeros(R + 1, dtype=i32, device="cuda")
    rows = torch.zeros((R, lib.nb_march_row_stride()), dtype=f32, device="cuda"); scratch = torch.zeros(1028, dtype=i32, device="cuda")
    nb.check(lib.nb_march_fill(ctypes.byref(sc), g["d_o"], g["d_d"], P(g["d_inv"]), P(g["nears"]), P(g["fars"]), P(g["bits"]), R, P(steps2), P(rows),
                               P(offs2), P(scratch), st), "nb_march_fill")
    torch.cuda.synchronize()
    cnt = g["steps"].cpu().numpy().view(np.uint32)
    assert np.array_equal(steps2.cpu().numpy().view(np.uint32), cnt)
    offs = offs2.cpu().numpy().view(np.uint32)
    assert np.array_equal(offs[:R], g["offs"].cpu().numpy().view(np.uint32)) and offs[R] == cnt.sum()
    assert cnt.sum() > 2 * batch                                                # several batches
    done, batches = 0, 0
    while done < R:
        nb.check(lib.nb_march_cutoff(P(g["steps"]), P(g["offs"]), R, done, batch, P(g["plan"]), st), "nb_march_cutoff")
        torch.cuda.synchronize()
        plan = g["plan"].cpu().numpy().view(np.uint32)
        # the host's cut from the offsets: the last ray whose samples still fit
        end = int(np.searchsorted(offs[done + 1:], offs[done] + batch, side="right")) + done
        assert end == plan[0] and offs[end] - offs[done] == plan[1] and end > done
        total = int(plan[1])
        a = [torch.zeros(batch, dtype=f32, device="cuda"), torch.full((batch,), -1, dtype=i32, device="cuda"), torch.zeros((batch, 4), dtype=f32, device="cuda")]
        b = [torch.zeros(batch, dtype=f32, device="cuda"), torch.full((batch,), -1, dtype=i32, device="cuda"), torch.zeros((batch, 4), dtype=f32, device="cuda")]
        nb.check(lib.nb_march_emit(ctypes.byref(sc), g["d_o"], g["d_d"], P(g["d_inv"]), P(g["nears"]), P(g["fars"]), P(g["bits"]), R, done, R,
                                   P(g["offs"]), P(g["plan"]), P(a[0]), P(a[1]), P(a[2]), st), "nb_march_emit")
        nb.check(lib.nb_march_compact(ctypes.byref(sc), g["d_o"], g["d_d"], done, end - done, P(steps2), P(offs2), int(offs[done]), P(rows),
                                      P(b[0]), P(b[1]), P(b[2]), st), "nb_march_compact")
        torch.cuda.synchronize()
        for x, y in zip(a, b):
            assert torch.equal(x[:total].view(i32), y[:total].view(i32))
        done, batches = end, batches + 1
    assert batches >= 3


def test_march_edge_cases(cuda, nb, orc):
    torch = cuda
    up = Uploader(torch, nb)
    sc = _scene(nb, (32, 32, 32), 1, 3, 1)
    bits = sphere_bitfield(orc, (32, 32, 32), 3, 1)
    o = np.array([[0, 0, -1.5], [3, 3, 3], [0, 0, 0]], np.float32); d = np.array([[0, 0, 1], [0, 1, 0], [0, 0, 1]], np.float32)
    g = _march_gpu(torch, nb, up, sc, o, d, bits, 10)              # budget smaller than the first ray: nothing fits
    cnt = g["steps"].cpu().numpy()
    assert cnt[0] >= 18 and cnt[1] == 0 and cnt[2] > 0
    assert g["plan"].cpu().numpy()[0] == 0
    g = _march_gpu(torch, nb, up, sc, o, d, np.zeros_like(bits), 10)   # empty grid: all rays fit with zero samples
    p = g["plan"].cpu().numpy()
    assert p[0] == 3 and p[1] == 0 and p[3] == 0


def _random_ray_samples(R, seed, max_count=60):
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, max_count, R).astype(np.uint32)
    counts[:3] = [0, 1, max_count]
    if R > 100:
        counts[3:8] = [31, 32, 33, 300, 1024]          # around the 32-sample window of the warp-per-ray kernels, and the cap
    n = int(counts.sum())
    off = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    t = np.concatenate([np.sort(rng.uniform(0.5, 3.0, c)) for c in counts]).astype(np.float32)
    dens = rng.normal(1.5, 1.5, (n, 16)).astype(np.float32)
    col = np.zeros((n, 8), np.float32); col[:, :3] = rng.random((n, 3), dtype=np.float32)
    target = rng.random((R, 3), dtype=np.float32)
    return counts, off, t, dens, col, target


@pytest.mark.parametrize("R", [1, 5000])
def test_compositing_and_color_grad(cuda, nb, orc, R):
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    counts, off, t, dens, col, target = _random_ray_samples(max(R, 3), 5)
    R = len(counts)
    n = len(t)
    bias, lam, scale = 1.0, 0.1, 128.0
    sigma = np.exp(np.minimum(dens[:, 0] - np.float32(bias), 8)).astype(np.float32)
    bg = (ctypes.c_float * 3)(1.0, 0.5, 0.25)
    bg_np = np.array([1.0, 0.5, 0.25], np.float32)
    f32 = torch.float32
    rgb = torch.zeros((R, 3), dtype=f32, device="cuda"); depth = torch.zeros(R, dtype=f32, device="cuda"); phi = torch.zeros((R, 3), dtype=f32, device="cuda")
    dw = torch.zeros(n, dtype=f32, device="cuda"); wsum = torch.zeros(R, dtype=f32, device="cuda")
    d_off, d_cnt, d_t, d_sig, d_col, d_tgt = up.f(off.view(np.int32)), up.f(counts.view(np.int32)), up.f(t), up.f(sigma), up.f(col), up.f(target)
    nb.check(lib.nb_composite_train(R, 0, d_off, d_cnt, d_t, d_sig, None, None, d_col, 8, d_tgt, P(rgb), P(depth), P(phi), P(dw), P(wsum), lam, 0.0,
                                    bg, st), "nb_composite_train")
    torch.cuda.synchronize()
    r_rgb, r_depth, r_phi, r_dw, r_wsum = orc.render_rays_distortion(R, off, counts, t, sigma, col[:, :3].copy(), target, lam, 0.0, bg_np)
    assert np.max(np.abs(rgb.cpu().numpy() - r_rgb)) <= ABS_RGB
    assert np.allclose(depth.cpu().numpy(), r_depth, rtol=1e-4, atol=1e-4) and np.max(np.abs(phi.cpu().numpy() - r_phi)) <= 2 * ABS_RGB
    assert rel_err(dw.cpu().numpy(), r_dw) <= REL_MLP and rel_err(wsum.cpu().numpy(), r_wsum) <= REL_MLP
    # inference variant (early termination) agrees on colour within the termination threshold
    rgb2 = torch.zeros_like(rgb)
    nb.check(lib.nb_composite_infer(R, 0, 0, d_off, d_cnt, d_t, d_sig, d_col, 8, None, P(rgb2), None, None, bg, st), "nb_composite_infer")
    torch.cuda.synchronize()
    i_rgb, _, _ = orc.render_rays(R, 0, 0, off, counts, t, sigma, col[:, :3].copy(), None, bg_np)
    assert np.max(np.abs(rgb2.cpu().numpy() - i_rgb)) <= ABS_RGB
    # loss gradients from the GPU's own forward results
    grad = torch.full((n, 8), 9.0, dtype=torch.float16, device="cuda"); dsig = torch.zeros(n, dtype=f32, device="cuda")
    nb.check(lib.nb_color_grad(R, 0, d_cnt, d_off, d_t, up.f(dens), 16, d_col, 8, P(phi), P(rgb), P(dw), P(wsum), P(grad), 8, P(dsig), scale, bias, R,
                               st), "nb_color_grad")
    torch.cuda.synchronize()
    g_ref, ds_ref = orc.color_grad(R, counts, off, t, dens, col, phi.cpu().numpy(), rgb.cpu().numpy(), dw.cpu().numpy(), wsum.cpu().numpy(),
                                   scale, bias, R, 8)
    got = half_vals(dev_half_bits(grad))
    assert np.all(got[:, 3:] == 0)
    assert rel_err(got, half_vals(g_ref)) <= REL_MLP and rel_err(dsig.cpu().numpy(), ds_ref) <= REL_MLP
    if R < 100:
        return
    # the same rays as the second half of a longer sample list: offsets carry a base, results do not change
    k = R // 2
    base = int(off[k])
    sh = lambda a: up.f(np.ascontiguousarray(a[base:]))
    rgb_b = torch.zeros((R - k, 3), dtype=f32, device="cuda"); phi_b = torch.zeros_like(rgb_b); dw_b = torch.zeros(n - base, dtype=f32, device="cuda")
    ws_b = torch.zeros(R - k, dtype=f32, device="cuda"); grad_b = torch.zeros((n - base, 8), dtype=torch.float16, device="cuda")
    dsig_b = torch.zeros(n - base, dtype=f32, device="cuda")
    o_b, c_b = up.f(off[k:].view(np.int32).copy()), up.f(counts[k:].view(np.int32).copy())
    t_b, s_b, col_b, dens_b, tgt_b = sh(t), sh(sigma), sh(col), sh(dens), up.f(target[k:].copy())
    nb.check(lib.nb_composite_train(R - k, base, o_b, c_b, t_b, s_b, None, None, col_b, 8, tgt_b, P(rgb_b), None, P(phi_b), P(dw_b), P(ws_b), lam, 0.0,
                                    bg, st), "nb_composite_train")
    nb.check(lib.nb_color_grad(R - k, base, c_b, o_b, t_b, dens_b, 16, col_b, 8, P(phi_b), P(rgb_b), P(dw_b), P(ws_b), P(grad_b), 8, P(dsig_b), scale,
                               bias, R, st), "nb_color_grad")
    rgb_i = torch.zeros_like(rgb_b)
    nb.check(lib.nb_composite_infer(R - k, base, k, d_off, c_b, t_b, s_b, col_b, 8, None, P(rgb_i), None, None, bg, st), "nb_composite_infer")
    torch.cuda.synchronize()
    assert torch.equal(rgb_b, rgb[k:]) and torch.equal(dw_b, dw[base:]) and torch.equal(ws_b, wsum[k:])
    assert torch.equal(grad_b, grad[base:]) and torch.equal(dsig_b, dsig[base:]) and torch.equal(rgb_i, rgb2[k:])


@pytest.mark.parametrize("capacity_rays,fused", [(None, False), (700, False), (None, True), (700, True)])
def test_rendering_in_rounds_equals_the_single_pass(cuda, nb, orc, capacity_rays, fused):
    """nb_march_round_emit + nb_composite_round over the rounds 16, 16, 32, ... against nb_composite_infer on the same
    rays: same colour and depth to fp32 rounding, and rays that turned opaque are not emitted again.  fused: the
    compositing launch of a round copies the next round out itself (range by range instead of round by round)."""
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    counts, off, t, dens, col, _ = _random_ray_samples(5000, 11, max_count=200)
    R, n = len(counts), len(t)
    sigma = np.exp(np.minimum(dens[:, 0] - np.float32(1.0), 8)).astype(np.float32)
    bg = (ctypes.c_float * 3)(1.0, 0.5, 0.25)
    f32, i32 = torch.float32, torch.int32
    d_off, d_cnt, d_t, d_sig, d_col = up.f(off.view(np.int32)), up.f(counts.view(np.int32)), up.f(t), up.f(sigma), up.f(col)
    want = torch.zeros((R, 3), dtype=f32, device="cuda"); want_depth = torch.zeros(R, dtype=f32, device="cuda")
    nb.check(lib.nb_composite_infer(R, 0, 0, d_off, d_cnt, d_t, d_sig, d_col, 8, None, P(want), P(want_depth), None, bg, st), "nb_composite_infer")
    # rows as the walk leaves them
    stride = lib.nb_march_row_stride()
    rows_np = np.zeros((R, stride), np.float32)
    for r in range(R):
        rows_np[r, :counts[r]] = t[off[r]:off[r] + counts[r]]
    rows = torch.from_numpy(rows_np).cuda()
    sc = _scene(nb, (32, 32, 32), 1, 3, 1)
    rng = np.random.default_rng(3)
    o = torch.from_numpy(rng.normal(0, 0.1, (R, 3)).astype(np.float32)).cuda()
    dirs = rng.normal(0, 1, (R, 3)).astype(np.float32); dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    d = torch.from_numpy(dirs).cuda()
    cap = 1 << 20
    pos = torch.zeros((cap, 4), dtype=f32, device="cuda"); ridx = torch.zeros(cap, dtype=i32, device="cuda")
    roff = torch.zeros(R, dtype=i32, device="cuda"); T = torch.full((R,), 7.0, dtype=f32, device="cuda")
    acc = torch.full((R, 4), 7.0, dtype=f32, device="cuda")
    got = torch.full((R, 3), -1.0, dtype=f32, device="cuda"); got_depth = torch.full((R,), -1.0, dtype=f32, device="cuda")
    sig_all, col_all, off_all = torch.from_numpy(sigma).cuda(), torch.from_numpy(col).cuda(), torch.from_numpy(off.astype(np.int64)).cuda()
    total = torch.zeros(1, dtype=torch.int64, device="cuda")
    widths = (16, 16, 32, 64, 128, 256, 512)
    begins = (0, 16, 32, 64, 128, 256, 512)
    step = R if capacity_rays is None else capacity_rays
    stats = {"emitted": 0, "reached": 0}

    def field(r0, rc, begin, width, m):
        """sigma and colour of the m samples in the arrays, looked up by (ray, sample index in the ray); checks the copy-out"""
        reach = np.clip(counts[r0:r0 + rc].astype(np.int64) - begin, 0, width)
        assert m <= reach.sum()
        stats["emitted"] += m; stats["reached"] += int(reach.sum())
        ray = ridx[:m].long()
        assert m == 0 or (int(ray.min()) >= r0 and int(ray.max()) < r0 + rc)
        k = begin + torch.arange(m, device="cuda") - roff.long()[ray]
        assert m == 0 or (int(k.min()) >= begin and int(k.max()) < begin + width)
        src = off_all[ray] + k
        if m:
            tt = rows[ray, k]
            p_want = orc.contract_pos((o[ray] + tt[:, None] * d[ray]).cpu().numpy(), (-0.5,) * 3, (0.5,) * 3)
            assert np.allclose(pos[:m, :3].cpu().numpy(), p_want, atol=2e-6)
            return sig_all[src].contiguous(), col_all[src].contiguous()
        return torch.zeros(1, device="cuda"), torch.zeros((1, 8), device="cuda")

    def emit(r0, rc, begin, width, counter):
        nb.check(lib.nb_march_round_emit(ctypes.byref(sc), P(o), P(d), r0, rc, d_cnt, P(T), begin, width, P(rows), cap, P(counter), P(total), P(roff),
                                         P(ridx), P(pos), st), "nb_march_round_emit")
        torch.cuda.synchronize()

    def composite(r0, rc, begin, width, s_round, c_round, next_width=0, next_counter=None):
        nb.check(lib.nb_composite_round(r0, rc, d_cnt, P(roff), P(rows), begin, width, P(s_round), P(c_round), 8, P(T), P(acc), P(got), P(got_depth),
                                        bg, next_width, ctypes.byref(sc) if next_width else None, P(o) if next_width else None,
                                        P(d) if next_width else None, cap if next_width else 0, P(next_counter) if next_width else None,
                                        P(total) if next_width else None, P(ridx) if next_width else None, P(pos) if next_width else None, st),
                 "nb_composite_round")
        torch.cuda.synchronize()

    if not fused:
        for begin, width in zip(begins, widths):
            for r0 in range(0, R, step):
                rc = min(step, R - r0)
                counter = torch.zeros(1, dtype=i32, device="cuda")
                emit(r0, rc, begin, width, counter)
                s_round, c_round = field(r0, rc, begin, width, int(counter.item()))
                composite(r0, rc, begin, width, s_round, c_round)
    else:
        for r0 in range(0, R, step):
            rc = min(step, R - r0)
            counters = torch.zeros(len(widths) + 1, dtype=i32, device="cuda")
            emit(r0, rc, 0, widths[0], counters[0:1])
            for j, (begin, width) in enumerate(zip(begins, widths)):
                s_round, c_round = field(r0, rc, begin, width, int(counters[j].item()))
                nxt = widths[j + 1] if j + 1 < len(widths) else 0
                composite(r0, rc, begin, width, s_round, c_round, nxt, counters[j + 1:j + 2] if nxt else None)
    assert float((got - want).abs().max()) <= 1e-5
    assert torch.allclose(got_depth, want_depth, rtol=1e-5, atol=1e-5)
    assert int(total.item()) == stats["emitted"]
    assert stats["emitted"] < stats["reached"]                         # opaque rays dropped out before their last round
    assert stats["emitted"] >= int(np.minimum(counts, 16).sum())       # ... but every ray took part in the first


def test_occupancy_kernels(cuda, nb, orc):
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    res, levels, casc = (32, 32, 32), 4, 2
    sc = _scene(nb, res, casc, levels, 1)
    G, S = sc.cells_per_cascade, sc.pyramid_cells
    N = casc * G
    amin, amax = [-.5] * 3, [.5] * 3
    f32, i32 = torch.float32, torch.int32
    # full-coverage samples of cascade 1 and random samples of the whole grid: cell ids exact, positions to float error
    smp = torch.zeros((G, 4), dtype=f32, device="cuda")
    nb.check(lib.nb_occ_sample_cells(ctypes.byref(sc), P(smp), G, G, G, 77, st), "nb_occ_sample_cells")
    torch.cuda.synchronize()
    ref = orc.sample_aabb(amin, amax, res, G, G, G, 77)
    got = smp.cpu().numpy()
    assert np.array_equal(got[:, 3].copy().view(np.int32), ref[:, 3].copy().view(np.int32))
    assert np.allclose(got[:, :3], ref[:, :3], atol=2e-6)
    smp2 = torch.zeros((5000, 4), dtype=f32, device="cuda")
    nb.check(lib.nb_occ_sample_cells(ctypes.byref(sc), P(smp2), 5000, N, 0, 78, st), "nb_occ_sample_cells")
    torch.cuda.synchronize()
    ref2 = orc.sample_aabb(amin, amax, res, 5000, N, 0, 78)
    got2 = smp2.cpu().numpy()
    assert np.mean(got2[:, 3].copy().view(np.int32) != ref2[:, 3].copy().view(np.int32)) < 1e-3      # (int)(u * N) at a boundary
    # density maximum per cell, master grid decay + sum
    rng = np.random.default_rng(1)
    dens = np.zeros((G, 16), np.float32); dens[:, 0] = rng.normal(0, 2, G)
    tmp = torch.zeros(N, dtype=f32, device="cuda")
    nb.check(lib.nb_occ_update_tmp_grid(P(smp), up.f(dens), P(tmp), 1.0, G, st), "nb_occ_update_tmp_grid")
    master0 = np.abs(rng.normal(0, 1, N)).astype(np.float32); master0[3] = -1.0
    master = torch.from_numpy(master0.copy()).cuda()
    scratch = torch.zeros(int(lib.nb_occ_scratch_bytes(N)) // 8 + 1, dtype=torch.float64, device="cuda"); dsum = torch.zeros(1, dtype=f32, device="cuda")
    nb.check(lib.nb_occ_update_master_grid(P(tmp), P(master), 0.95, N, P(scratch), P(dsum), st), "nb_occ_update_master_grid")
    torch.cuda.synchronize()
    tmp_ref = np.zeros(N, np.float32); orc.update_tmp_grid(got, dens, tmp_ref, 1.0)
    assert np.allclose(tmp.cpu().numpy(), tmp_ref, rtol=1e-5)
    m_ref = master0.copy(); orc.update_master_grid(tmp.cpu().numpy(), m_ref, 0.95)
    m_got = master.cpu().numpy()
    assert np.allclose(m_got, m_ref, rtol=1e-6) and m_got[3] == -1.0
    assert abs(dsum.item() - m_got.astype(np.float64).sum()) <= 1e-6 * abs(m_got.astype(np.float64).sum())
    # bits and pyramid from the GPU's own master grid and sum: bit-exact
    bits = torch.zeros(casc * S // 8, dtype=torch.uint8, device="cuda")
    nb.check(lib.nb_occ_update_bitfield(ctypes.byref(sc), P(bits), P(master), P(dsum), 0.01, st), "nb_occ_update_bitfield")
    torch.cuda.synchronize()
    b_ref = np.zeros(casc * S // 8, np.uint8)
    orc.update_occupancy_bits(b_ref, m_got, dsum.item(), G, S, 0.01, 1.0 / 32)
    orc.build_mipmaps(b_ref, res, levels, casc)
    b_got = bits.cpu().numpy()
    assert np.array_equal(b_got, b_ref), "%d of %d occupancy bytes differ" % ((b_got != b_ref).sum(), b_ref.size)
    assert 0 < np.unpackbits(b_got).sum() < 8 * b_got.size
    # occupied-cell list: same set
    act = torch.zeros(N, dtype=i32, device="cuda"); nact = torch.zeros(1, dtype=i32, device="cuda")
    nb.check(lib.nb_occ_extract_active(ctypes.byref(sc), P(bits), P(act), P(nact), st), "nb_occ_extract_active")
    torch.cuda.synchronize()
    a_ref = orc.extract_active_cells(b_got, N, G, S)
    a_got = act.cpu().numpy()[:nact.item()]
    assert nact.item() == len(a_ref) and np.array_equal(np.sort(a_got), a_ref)
    smp3 = torch.zeros((4096, 4), dtype=f32, device="cuda")
    nb.check(lib.nb_occ_sample_occupied(ctypes.byref(sc), P(smp3), P(act), P(nact), 4096, 79, st), "nb_occ_sample_occupied")
    torch.cuda.synchronize()
    ref3 = orc.sample_occupied(a_got, amin, amax, res, 4096, 79)
    got3 = smp3.cpu().numpy()
    same = got3[:, 3].copy().view(np.int32) == ref3[:, 3].copy().view(np.int32)
    assert same.mean() > 0.999 and np.allclose(got3[same, :3], ref3[same, :3], atol=2e-6)


def test_generated_rays_plain_and_tiled(cuda, nb):
    """nb_generate_rays against the pinhole formula, and nb_generate_rays_tiled (all tiles of a rank in one launch)
    against nb_generate_rays per tile: the same bits, ragged last tile included."""
    import importlib
    torch = cuda
    syn = importlib.import_module("3dmaker_b200.synthetic"); D = importlib.import_module("3dmaker_b200.distributed")
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    W, H, tile, world = 50, 37, 128, 3                       # 1850 pixels: 15 tiles, the last one 58 pixels
    focal = syn.focal_from_fov(W, 50.0)
    c2w = np.ascontiguousarray(syn.orbit_c2w(25.0, 10.0, 1.5), np.float32)
    cp = c2w.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
    o = torch.zeros((W * H, 3), device="cuda"); d = torch.zeros((W * H, 3), device="cuda")
    nb.check(lib.nb_generate_rays(W, H, focal, cp, 0, W * H, P(o), P(d), st), "nb_generate_rays")
    torch.cuda.synchronize()
    wo, wd = syn.frame_rays(torch, c2w, W, H, 50.0)
    assert torch.allclose(o, wo, atol=1e-6) and torch.allclose(d, wd, atol=1e-5)
    for rank in range(world):
        tiles = D.pixel_tiles(W * H, rank, world, tile)
        total = sum(c for _, c in tiles)
        to = torch.full((total, 3), -7.0, device="cuda"); td = torch.full((total, 3), -7.0, device="cuda")
        nb.check(lib.nb_generate_rays_tiled(W, H, focal, cp, tile, rank, world, total, P(to), P(td), st), "nb_generate_rays_tiled")
        torch.cuda.synchronize()
        idx = torch.cat([torch.arange(f, f + c, device="cuda") for f, c in tiles])
        assert torch.equal(to, o[idx]) and torch.equal(td, d[idx])
    assert lib.nb_generate_rays_tiled(W, H, focal, cp, tile, 14, 1, 59, P(o), P(d), st) != 0     # one pixel past the frame


@pytest.mark.parametrize("world,tile,num_pixels", [(1, 64, 1000), (3, 64, 1000), (8, 16384, 1920 * 1080), (4, 128, 128 * 8 + 5)])
def test_undeal_tiles_rebuilds_the_frame(cuda, nb, world, tile, num_pixels):
    """nb_undeal_tiles: the blocks the ranks of a pixel-sharded frame send (tiles dealt round-robin, padded to equal
    size) back into frame order - bit for bit the strided copy it replaces."""
    torch = cuda
    lib, P = nb.load(), nb.ptr
    D = importlib.import_module("3dmaker_b200.distributed")
    num_tiles = (num_pixels + tile - 1) // tile
    rows = (num_tiles + world - 1) // world * tile
    frame_true = torch.rand((num_pixels, 3), device="cuda")
    blocks = torch.full((world, rows, 3), -7.0, device="cuda")
    for r in range(world):
        at = 0
        for first, count in D.pixel_tiles(num_pixels, r, world, tile):
            blocks[r, at:at + count] = frame_true[first:first + count]
            at += tile
    frame = torch.zeros((num_pixels, 3), device="cuda")
    nb.check(lib.nb_undeal_tiles(P(blocks), world, rows, tile, num_pixels, P(frame), nb.stream_ptr()), "nb_undeal_tiles")
    torch.cuda.synchronize()
    assert torch.equal(frame, frame_true)
    assert lib.nb_undeal_tiles(P(blocks), world, rows - 1, tile, num_pixels, P(frame), nb.stream_ptr()) == 1   # block too small
