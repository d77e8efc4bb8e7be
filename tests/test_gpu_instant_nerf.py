"""The C++ scene engine (InstantNerf host class through its C handle) on a B200: one optimizer step against
the oracle chain, training on the analytic soft-sphere scene, rendering in one and in several batches,
.inerf save / load."""
import importlib
import os

import numpy as np
import pytest

from helpers import ABS_RGB, REL_MLP, half_vals, make_mlp, make_table, rel_err
from oracle_pipeline import OracleField, oracle_ray_step

pytestmark = pytest.mark.gpu


def _mods():
    return importlib.import_module("3dmaker_b200.nerf"), importlib.import_module("3dmaker_b200.synthetic")


def _np(torch, nerf_mod, ptr, count, dtype):
    return nerf_mod.view_tensor(torch, ptr, count, dtype).cpu().numpy()


@pytest.mark.parametrize("fused", [False, True])
def test_one_step_matches_oracle_chain(cuda, nb, orc, fused):
    torch = cuda
    nm, syn = _mods()
    L, T = 16, 1 << 15
    opts = nm.default_options(grid_resolution=(64, 64, 64), aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=3, hash_table_size=T,
                              growth_factor=1.447, color_hidden_dim=64, color_num_layers=3, batch_size=1 << 16, render_batch_size=1 << 16,
                              ray_chunk_size=1 << 14, lambda_dist=0.1, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
                              loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))
    eng = nm.InstantNerf(torch, opts)
    assert eng.set_fused_field(fused) == fused
    table = make_table(L, T, seed=0, amp=0.5)
    dW, db = make_mlp(32, 64, 16, 2, seed=0, bias_amp=0.05)
    cW, cb = make_mlp(32, 64, 8, 3, seed=1, bias_amp=0.05)
    eng.load_params(table, (dW, db), (cW, cb))
    eng.rebuild_occupancy()
    poses = syn.sphere_cameras(8)
    R = 3000
    o, d = syn.random_training_rays(torch, poses, R, 200, 200, 50.0, seed=1)
    tgt = torch.rand((R, 3), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    captured = {}
    eng.set_grad_sync(lambda g: captured.__setitem__("g", g.clone()))
    w_before = eng.arena_tensor("w").clone()
    rgb_out = torch.zeros((R, 3), device="cuda")
    steps = eng.train_rays(o, d, tgt, rgb_out)
    torch.cuda.synchronize()
    assert steps >= 1
    v = eng.step_view()
    n = v.last_total_hits
    assert n > 1000
    # the step view holds the LAST step; make the test about a single step by checking it consumed all rays
    if steps != 1:
        pytest.skip("more than one step was needed for %d rays (%d): enlarge batch_size" % (R, steps))
    march = dict(num_steps=_np(torch, nm, v.num_steps, R, np.int32).view(np.uint32), ray_offsets=_np(torch, nm, v.ray_offsets, R, np.int32).view(np.uint32),
                 ray_indices=_np(torch, nm, v.ray_indices, n, np.int32).view(np.uint32), t=_np(torch, nm, v.t_sorted, n, np.float32),
                 pos4=_np(torch, nm, v.positions, 4 * n, np.float32).reshape(n, 4))
    assert march["num_steps"].sum() == n
    grid = nb.grid_setup(L, T, 16, 1.447)
    scales = np.array(list(grid.scales)[:L], np.float32)
    sscales = np.array(list(grid.scatter_scales)[:L], np.float32)
    field = OracleField(L, T, 16, 1.447, scales, grid.dense_level_start, (32, 64, 16, 2), (32, 64, 8, 3), table, dW, db, cW, cb, sscales)
    bg = np.ones(3, np.float32)
    r = oracle_ray_step(field, march, d.cpu().numpy(), tgt.cpu().numpy(), bg, 0.1, 128.0, 1.0, R)
    if v.logit_stride == 16:
        assert rel_err(_np(torch, nm, v.density_out, 16 * n, np.float32).reshape(n, 16), r["d_out"]) <= REL_MLP
    else:
        assert v.logit_stride == 1 and v.color_stride == 4
        assert rel_err(_np(torch, nm, v.density_out, n, np.float32), r["d_out"][:, 0]) <= REL_MLP
    assert rel_err(_np(torch, nm, v.sigma, n, np.float32), r["sigma"]) <= 2 * REL_MLP
    got_rgb = _np(torch, nm, v.render_rgb, 3 * R, np.float32).reshape(R, 3)
    assert np.max(np.abs(got_rgb - r["rgb"])) <= 3 * ABS_RGB            # fp16 network outputs feed the compositing
    assert np.array_equal(rgb_out.cpu().numpy(), got_rgb)
    assert rel_err(_np(torch, nm, v.dw, n, np.float32), r["dw"]) <= 3 * REL_MLP
    cg = half_vals(_np(torch, nm, v.color_grad, 8 * n, np.float16).view(np.uint16)).reshape(n, 8)
    assert rel_err(cg, half_vals(r["c_grad"])) <= 3 * REL_MLP
    assert rel_err(_np(torch, nm, v.tmp_dsigma, n, np.float32), r["dsig"]) <= 5 * REL_MLP
    g = captured["g"].cpu().numpy()
    a = eng.arena()
    H = a.sparse_count
    assert rel_err(g[a.color_weight_offset:a.color_weight_offset + a.color_weight_count], r["g_cW"]) <= 5 * REL_MLP
    assert rel_err(g[a.density_weight_offset:a.density_weight_offset + a.density_weight_count], r["g_dW"]) <= 8 * REL_MLP
    assert rel_err(g[:H], r["g_table"]) <= 8 * REL_MLP
    # the optimizer consumed the gradient and moved every touched parameter
    w_after = eng.arena_tensor("w")
    assert torch.all(eng.arena_tensor("g") == 0)
    touched = captured["g"][:H] != 0
    assert torch.all((w_after[:H] != w_before[:H])[touched]) and torch.all((w_after[:H] == w_before[:H])[~touched])
    eng.close()


def _train_soft_sphere(torch, nm, syn, steps_target, T=1 << 19, res=128, batch=1 << 18):
    opts = nm.default_options(grid_resolution=(res,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=4, hash_table_size=T,
                              growth_factor=1.3819, color_hidden_dim=64, color_num_layers=3, batch_size=batch, render_batch_size=batch,
                              ray_chunk_size=1 << 16, lambda_dist=0.01, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
                              loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))
    eng = nm.InstantNerf(torch, opts)
    scene = syn.SoftSphereScene()
    poses = syn.sphere_cameras(100)
    bg = (1.0, 1.0, 1.0)
    it = 0
    while eng.steps.value < steps_target:
        o, d = syn.random_training_rays(torch, poses, 1 << 16, 800, 800, 50.0, seed=100 + it)
        tgt = syn.ground_truth(torch, scene, o, d, bg)
        eng.train_rays(o, d, tgt)
        it += 1
    torch.cuda.synchronize()
    return eng, scene, bg


def test_training_converges_and_renders(cuda, nb, tmp_path):
    torch = cuda
    nm, syn = _mods()
    eng, scene, bg = _train_soft_sphere(torch, nm, syn, 400)
    W = H = 200
    c2w = syn.orbit_c2w(33.0, 20.0, 1.5)                               # a view outside the training lattice
    o, d = syn.frame_rays(torch, c2w, W, H, 50.0)
    img = torch.zeros((W * H, 3), device="cuda")
    eng.render(o, d, img)
    torch.cuda.synchronize()
    gt = syn.ground_truth(torch, scene, o, d, bg)
    p = syn.psnr(torch, img, gt)
    print("PSNR after %d steps: %.2f dB" % (eng.steps.value, p))
    assert p > 24.0
    # rendering in rounds stops evaluating rays behind the point where they turned opaque and still gives the picture that
    # evaluating every sample gives
    every = eng.last_render_samples()
    assert eng.set_render_rounds(True) is True
    part = torch.zeros_like(img)
    eng.render(o, d, part)
    torch.cuda.synchronize()
    assert 0 < eng.last_render_samples() < every
    assert eng.set_render_rounds(False) is False
    assert float((img - part).abs().max()) <= 1e-5
    bits, master = eng.occupancy()
    occ = np.unpackbits(bits.cpu().numpy()[:128 ** 3 // 8]).mean()
    assert 0.02 < occ < 0.6                                               # the grid has carved away empty space
    # several small render batches give the same image as one large one (rays never straddle a batch)
    opts2 = eng.options
    path = os.path.join(str(tmp_path), "model.inerf")
    eng.save(path)
    small = nm.default_options()
    eng2 = nm.InstantNerf(torch, nm.default_options(grid_resolution=(16,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=2,
                                                    hash_table_size=1 << 14, batch_size=1 << 12, render_batch_size=1 << 12, ray_chunk_size=1 << 10))
    eng2.load(path)                                                      # re-initialises with the stored options
    img2 = torch.zeros_like(img)
    eng2.render(o, d, img2)
    torch.cuda.synchronize()
    assert torch.equal(img, img2), "a reloaded model renders differently"
    assert os.path.getsize(path) > 16 * (1 << 19) * 2 * 4
    eng.close(); eng2.close()


def test_render_batching_is_invisible(cuda, nb):
    torch = cuda
    nm, syn = _mods()
    base = dict(grid_resolution=(64,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=3, hash_table_size=1 << 15,
                color_hidden_dim=64, color_num_layers=3, batch_size=1 << 16, ray_chunk_size=1 << 12, density_bias=-2.0)
    imgs = []
    o, d = syn.frame_rays(torch, syn.orbit_c2w(10.0, 5.0, 1.5), 96, 96, 50.0)
    for rb, rounds in ((1 << 20, True), (3000, True), (1 << 20, False), (3000, False)):
        eng = nm.InstantNerf(torch, nm.default_options(render_batch_size=rb, **base), inference=True)
        assert eng.set_render_rounds(rounds) is rounds
        img = torch.zeros((96 * 96, 3), device="cuda")
        eng.render(o, d, img)
        torch.cuda.synchronize()
        imgs.append(img)
        eng.close()
    assert torch.equal(imgs[0], imgs[1]) and torch.equal(imgs[2], imgs[3])
    assert imgs[0].std() > 1e-3
    # rendering in rounds sums each ray in pieces: the same picture up to fp32 rounding
    assert float((imgs[0] - imgs[2]).abs().max()) <= 1e-5
    # the kernel-by-kernel sequence (which evaluates every sample) renders the same picture as the single field kernel
    # does on every sample, bit for bit
    eng = nm.InstantNerf(torch, nm.default_options(render_batch_size=1 << 20, **base), inference=True)
    assert eng.set_fused_field(False) is False
    img = torch.zeros((96 * 96, 3), device="cuda")
    eng.render(o, d, img)
    torch.cuda.synchronize()
    eng.close()
    assert torch.equal(imgs[2], img)


def test_gradient_arena_in_caller_memory(cuda, nb):
    """set_grad_buffer: the engine accumulates its gradient in a tensor the caller owns (what data-parallel training
    hands to the communicator), through mode switches, and returns to its own allocation on request."""
    torch = cuda
    nm, syn = _mods()
    opts = nm.default_options(grid_resolution=(64,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=3, hash_table_size=1 << 15,
                              color_hidden_dim=64, color_num_layers=3, batch_size=1 << 16, ray_chunk_size=1 << 12, density_bias=1.0)
    eng = nm.InstantNerf(torch, opts)
    total = eng.arena().total
    buf = torch.full((total + 8,), 3.0, dtype=torch.float32, device="cuda")
    seen = []

    def sync(g):
        seen.append((g.data_ptr(), g.numel(), float(g.abs().sum().item())))
    eng.set_grad_sync(sync)
    scene, poses = syn.SoftSphereScene(), syn.sphere_cameras(20)

    def one_call(seed):
        o, d = syn.random_training_rays(torch, poses, 1 << 12, 200, 200, 50.0, seed=seed)
        eng.train_rays(o, d, syn.ground_truth(torch, scene, o, d, (1.0, 1.0, 1.0)))
        torch.cuda.synchronize()
    one_call(1)
    own_ptr = seen[-1][0]
    assert own_ptr != buf.data_ptr() and seen[-1][2] > 0
    eng.set_grad_buffer(buf)
    assert float(buf[:total].abs().sum().item()) == 0.0 and float(buf[total:].min().item()) == 3.0   # zeroed, nothing written past the arena
    one_call(2)
    assert seen[-1][0] == buf.data_ptr() and seen[-1][1] == total and seen[-1][2] > 0
    assert float(buf[:total].abs().sum().item()) == 0.0                                              # Adam cleared it again
    eng.set_memory_mode(True); eng.set_memory_mode(False)                                            # inference and back
    one_call(3)
    assert seen[-1][0] == buf.data_ptr() and seen[-1][2] > 0
    with pytest.raises(nb.NerfB200Error):
        eng.set_grad_buffer(torch.zeros(total - 4, dtype=torch.float32, device="cuda"))
    eng.set_grad_buffer(None)
    one_call(4)
    assert seen[-1][0] != buf.data_ptr() and seen[-1][2] > 0
    assert float(buf[total:].min().item()) == 3.0
    eng.close()


def test_fixed_steps_per_call_survive_a_ray_that_does_not_fit_the_batch(cuda, nb):
    """Data parallelism fixes the number of optimizer steps (gradient exchanges) per call.  A sample batch too small for
    one of the rays must not make this rank leave the loop early - the other ranks would wait in their collective for
    ever: the ray is dropped, every exchange still happens, and the per-step hit counts stay inside their array."""
    torch = cuda
    nm, syn = _mods()
    opts = nm.default_options(grid_resolution=(64,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=3, hash_table_size=1 << 15,
                              color_hidden_dim=64, color_num_layers=3, batch_size=16, ray_chunk_size=1 << 10, density_bias=1.0)
    eng = nm.InstantNerf(torch, opts)
    calls = []
    eng.set_grad_sync(lambda g: calls.append(1))
    eng.set_steps_per_call(5)
    scene, poses = syn.SoftSphereScene(), syn.sphere_cameras(20)
    o, d = syn.random_training_rays(torch, poses, 1 << 10, 200, 200, 50.0, seed=1)
    # rays through the sphere carry more than 16 samples on a 64^3 grid, rays past it none
    steps = eng.train_rays(o, d, syn.ground_truth(torch, scene, o, d, (1.0, 1.0, 1.0)))
    torch.cuda.synchronize()
    assert steps == 5 and len(calls) == 5
    assert torch.isfinite(eng.arena_tensor("w")).all()
    eng.close()
