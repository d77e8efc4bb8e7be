"""The opt-in half-precision gradient table (nb_set_tuning "grad_table_half"): the scatter kernels, the optimizer and
the peer optimizer against the default fp32 table on the same inputs.  The reference has no such mode; the fp32 path,
which is pinned against the reference elsewhere, is the yardstick here."""
import ctypes
import importlib

import numpy as np
import pytest

from helpers import half_bits, make_mlp, make_positions, make_table

pytestmark = pytest.mark.gpu


def _inputs(n, seed, rays=False):
    rng = np.random.default_rng(seed)
    if rays:
        # consecutive samples along rays: runs of samples in one cell on the coarse levels (the run-merging path)
        per = 64
        nr = (n + per - 1) // per
        o = rng.uniform(0.05, 0.95, (nr, 1, 3)).astype(np.float32)
        d = rng.normal(size=(nr, 1, 3)).astype(np.float32)
        d /= np.linalg.norm(d, axis=2, keepdims=True)
        t = (np.arange(per, dtype=np.float32) * 0.004)[None, :, None]
        p = np.clip(o + d * t, 0.0, 1.0).reshape(-1, 3)[:n]
        pos = np.zeros((n, 4), np.float32)
        pos[:, :3] = p
    else:
        pos = make_positions(n, seed)
    d = rng.normal(size=(n, 3)).astype(np.float32)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    tgt = np.zeros((n, 8), np.float32)
    tgt[:, :3] = rng.random((n, 3), dtype=np.float32)
    return pos, d, half_bits(tgt)


def _model(torch, pl, T):
    model = pl.FieldModel(torch, 16, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(16, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05))
    model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    return model


@pytest.fixture
def half_mode(nb):
    """Switches the mode on for the test body that asks for it and ALWAYS off again."""
    yield lambda on, scale_log2=None: nb.set_grad_table_half(on, scale_log2)
    nb.set_grad_table_half(False, 7)


@pytest.mark.parametrize("rays", [False, True])
@pytest.mark.parametrize("path", ["tc+scatter", "regs+scatter", "separate"])
@pytest.mark.parametrize("n", [129, 40000])
def test_half_table_gradient_matches_the_fp32_table(cuda, nb, half_mode, n, path, rays):
    """Same samples, same parameters: the table gradient accumulated in fp16 (times 2^7, divided again here) against
    the fp32 table.  Tolerance: 1e-2 of the level's largest gradient per entry (fp16 has 11 bits, an entry of a coarse
    level sums hundreds of contributions) and 2e-3 on the level's sum; the network gradients do not pass through the
    table and agree to accumulation order."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib = nb.load()
    T = 1 << 15
    model = _model(torch, pl, T)
    pos, dirs, tgt = _inputs(n, 21, rays)
    tcflag = {"tc+scatter": 1, "regs+scatter": 0, "separate": 2}[path]
    got = {}
    try:
        nb.check(lib.nb_set_tuning(b"backward_tc", tcflag), "nb_set_tuning")
        for mode in (False, True):
            half_mode(mode, 7)
            tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=(path != "separate"), ordered=False)
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            model.g.zero_()
            tr.forward_backward(n)
            nb.check(lib.nb_field_backward_tc_status(), "tensor-memory backward status")
            got[mode] = (model.hash_grad_f32().cpu().numpy().reshape(16, T, 2), model.g[model.hash_count:].cpu().numpy().copy())
    finally:
        nb.check(lib.nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
        half_mode(False, 7)
        model.g.zero_()
    (g32, tail32), (g16, tail16) = got[False], got[True]
    assert np.abs(g32).max() > 0
    for level in range(16):
        a, b = g32[level], g16[level]
        top = np.abs(a).max()
        assert np.isfinite(b).all()
        assert np.abs(b - a).max() <= 1e-2 * top + 1e-9, (level, np.abs(b - a).max(), top)
        assert abs(b.sum(dtype=np.float64) - a.sum(dtype=np.float64)) <= 2e-3 * np.abs(a).sum(dtype=np.float64) + 1e-9, level
    assert np.abs(tail16 - tail32).max() <= 2e-3 * np.abs(tail32).max()


def test_half_table_optimizer_consumes_and_clears_the_packed_gradient(cuda, nb, half_mode):
    """nb_adam_step with the half table: entry gradients are read as fp16 from the start of the arena, divided by the
    table scale on top of the loss scale, consumed (set to zero) - against the fp32 optimizer on the same VALUES, bit for
    bit, because the values chosen here are exact in fp16."""
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    H, total = 1 << 14, (1 << 14) + 512
    rng = np.random.default_rng(4)
    w0 = rng.uniform(-0.1, 0.1, total).astype(np.float32)
    g_true = (rng.integers(-64, 65, H) / 8.0 * (rng.random(H) < 0.3)).astype(np.float32)     # multiples of 1/8: exact in fp16, also times 2^7
    g_tail = rng.normal(0, 5, total - H).astype(np.float32)
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0)
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    ref = dict(w=dev(w0), h=dev(w0).half(), g=dev(np.concatenate([g_true, g_tail])), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
    nb.check(lib.nb_adam_step(P(ref["w"]), P(ref["h"]), P(ref["g"]), P(ref["m"]), P(ref["v"]), H, total, *hyper, 1, st), "nb_adam_step")
    got = dict(w=dev(w0), h=dev(w0).half(), g=torch.zeros(total, device="cuda"), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
    packed = got["g"][:H].view(torch.float16)
    packed[:H].copy_(dev(g_true * 128.0).half())
    got["g"][H:].copy_(dev(g_tail))
    try:
        half_mode(True, 7)
        nb.check(lib.nb_adam_step(P(got["w"]), P(got["h"]), P(got["g"]), P(got["m"]), P(got["v"]), H, total, *hyper, 1, st), "nb_adam_step")
        torch.cuda.synchronize()
    finally:
        half_mode(False, 7)
    for k in ("w", "h", "m", "v"):
        assert torch.equal(got[k], ref[k]), k
    # hash part consumed (a group of four that is all +-0 is left as it is: it reads as zero), dense tail cleared (zero_dense_grads = 1)
    assert float(got["g"][:H].view(torch.float16).abs().max().item()) == 0.0 and float(got["g"][H:].abs().max().item()) == 0.0
    # a sum that overflowed fp16 counts as zero, like any non-finite gradient
    got["g"][:H].view(torch.float16)[:4].copy_(torch.tensor([float("inf"), 1.0, float("-inf"), float("nan")], dtype=torch.float16))
    before = got["w"][:4].clone()
    try:
        half_mode(True, 7)
        nb.check(lib.nb_adam_step(P(got["w"]), P(got["h"]), P(got["g"]), P(got["m"]), P(got["v"]), H, total, *hyper, 1, st), "nb_adam_step")
        torch.cuda.synchronize()
    finally:
        half_mode(False, 7)
    assert torch.isfinite(got["w"]).all() and torch.isfinite(got["m"]).all() and torch.isfinite(got["v"]).all()
    assert float((got["w"][1] - before[1]).abs().item()) > 0


@pytest.mark.parametrize("world", [2, 4])
def test_half_table_peer_optimizer_equals_the_single_launch_on_the_sum(cuda, nb, half_mode, world):
    """nb_adam_step_peer with half-precision gradient slices (ranks played by buffers on one device): the slices are
    summed in fp32 in rank order, so the result equals one half-table launch on a gradient that holds that sum - chosen
    exact in fp16 here, which makes the comparison bit for bit."""
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    H, total = 1 << 15, (1 << 15) + 1024
    rng = np.random.default_rng(9)
    w0 = rng.uniform(-0.1, 0.1, total).astype(np.float32)
    grads, tails = [], []
    for r in range(world):
        grads.append((rng.integers(-8, 9, H) * (rng.random(H) < 0.2)).astype(np.float32))
        tails.append(rng.normal(0, 5, total - H).astype(np.float32))
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0)
    dev = lambda a: torch.from_numpy(a.copy()).cuda()

    def arena(gh, gt):
        g = torch.zeros(total, device="cuda")
        g[:H].view(torch.float16)[:H].copy_(dev(gh).half())
        g[H:].copy_(dev(gt))
        return g

    gsum, tsum = grads[0].copy(), tails[0].copy()
    for r in range(1, world):
        gsum += grads[r]; tsum += tails[r]
    ref = dict(w=dev(w0), h=dev(w0).half(), g=arena(gsum, tsum), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
    ranks = [dict(w=dev(w0), h=dev(w0).half(), g=arena(grads[r], tails[r]), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
             for r in range(world)]
    G = (ctypes.c_void_p * world)(*[t["g"].data_ptr() for t in ranks])
    W = (ctypes.c_void_p * world)(*[t["h"].data_ptr() for t in ranks])
    try:
        half_mode(True, 7)
        nb.check(lib.nb_adam_step(P(ref["w"]), P(ref["h"]), P(ref["g"]), P(ref["m"]), P(ref["v"]), H, total, *hyper, 1, st), "nb_adam_step")
        for r in range(world):
            nb.check(lib.nb_adam_step_peer(P(ranks[r]["w"]), P(ranks[r]["m"]), P(ranks[r]["v"]), G, W, r, world, H, total, *hyper, st), "nb_adam_step_peer")
        torch.cuda.synchronize()
    finally:
        half_mode(False, 7)
    shard = H // world
    for r in range(world):
        assert torch.equal(ranks[r]["h"], ref["h"]), "rank %d: fp16 parameters differ" % r
        lo, hi = r * shard, (r + 1) * shard
        for k in ("w", "m", "v"):
            assert torch.equal(ranks[r][k][lo:hi], ref[k][lo:hi]), (r, k)
            assert torch.equal(ranks[r][k][H:], ref[k][H:]), (r, k, "dense tail")


def test_half_table_training_tracks_fp32_table_training(cuda, nb, half_mode):
    """60 optimizer steps on a fixed batch with either table: both losses fall by two orders of magnitude and stay
    together - within 2 % over the first 20 steps and within 20 % to the end, where the loss has dropped a hundredfold and
    small differences in every step have steered the two trajectories apart (measured: 7.5 % at the widest)."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    n, T = 1 << 15, 1 << 15
    pos, dirs, tgt = _inputs(n, 33)
    curves = {}
    try:
        for mode in (False, True):
            half_mode(mode, 7)
            model = _model(torch, pl, T)
            tr = pl.SampleTrainer(model, n, lr=1e-2, loss_scale=128.0, density_bias=1.0, ordered=False)
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            losses = []
            for _ in range(60):
                tr.step_device(n)
                losses.append(float(tr.loss.item()))
            curves[mode] = np.array(losses)
    finally:
        half_mode(False, 7)
    a, b = curves[False], curves[True]
    assert a[-1] < 0.05 * a[0] and b[-1] < 0.05 * b[0]
    assert np.all(np.abs(b - a)[:20] <= 0.02 * a[:20]), float(np.max(np.abs(b - a)[:20] / a[:20]))
    assert np.all(np.abs(b - a) <= 0.2 * a), float(np.max(np.abs(b - a) / a))


def test_half_table_refuses_exchanges_that_need_one_fp32_arena(cuda, nb, half_mode):
    """A plain gradient callback between backward and optimizer would all-reduce fp16 bits as fp32: refused."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    model = _model(torch, pl, 1 << 14)
    n = 256
    pos, dirs, tgt = _inputs(n, 5)
    tr = pl.SampleTrainer(model, n, ordered=False)
    tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
    try:
        half_mode(True, 7)
        with pytest.raises(nb.NerfB200Error):
            tr.step_device(n, grad_sync=lambda g: None)
    finally:
        half_mode(False, 7)
        model.g.zero_()


def test_scene_engine_trains_with_the_half_table(cuda, nb, half_mode):
    """The scene engine (march, field, compositing, scatter, optimizer) for 300 optimizer steps on the same rays with
    either table, learning rate annealed 1e-2 -> 1e-3 by the reference trainer's cosine (at a constant 1e-2 two runs of
    ONE engine differ by a dB or more at this length: unordered atomics): the mean PSNR of two runs on a held-out view
    is within 1 dB and past the level that shows training worked."""
    import math
    torch = cuda
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    opts = nm.default_options(grid_resolution=(128,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=4, hash_table_size=1 << 19,
                              growth_factor=1.3819, color_hidden_dim=64, color_num_layers=3, batch_size=1 << 18, render_batch_size=1 << 18,
                              ray_chunk_size=1 << 16, lambda_dist=0.01, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
                              loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))
    scene = syn.SoftSphereScene(); poses = syn.sphere_cameras(100); bg = (1.0, 1.0, 1.0)
    psnr = {}
    try:
        for mode in (False, True):
            half_mode(mode, 7)
            runs = []
            for _ in range(2):
                eng = nm.InstantNerf(torch, opts)
                it = 0
                while eng.steps.value < 300:
                    eng.set_learning_rate(1e-3 + 0.5 * (1e-2 - 1e-3) * (1.0 + math.cos(math.pi * min(eng.steps.value / 300.0, 1.0))))
                    o, d = syn.random_training_rays(torch, poses, 1 << 16, 800, 800, 50.0, seed=700 + it)
                    eng.train_rays(o, d, syn.ground_truth(torch, scene, o, d, bg))
                    it += 1
                o, d = syn.frame_rays(torch, syn.orbit_c2w(33.0, 20.0, 1.5), 200, 200, 50.0)
                img = torch.zeros((200 * 200, 3), device="cuda")
                eng.render(o, d, img)
                torch.cuda.synchronize()
                runs.append(syn.psnr(torch, img, syn.ground_truth(torch, scene, o, d, bg)))
                eng.close()
            psnr[mode] = float(np.mean(runs))
    finally:
        half_mode(False, 7)
    print("PSNR after 300 steps: fp32 table %.2f dB, half table %.2f dB" % (psnr[False], psnr[True]))
    assert psnr[False] > 30.0 and psnr[True] > 30.0
    assert abs(psnr[True] - psnr[False]) <= 1.0
