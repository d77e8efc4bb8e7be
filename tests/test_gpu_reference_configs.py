"""Parity against the reference's OWN CUDA code (oracle/_ref/libref3dmaker.so) at the shapes the benchmark configurations
name, and for the parts the kernel-level comparisons of test_gpu_vs_reference.py leave open:

  * the optimizer alone, fed identical gradients, three steps (hash-table rule and dense rule), rel 1e-5;
  * the field step at the benchmark shape: 2^20 samples, T = 2^19, growth 1.447;
  * the config-5 grid: T = 2^22 per level - indices bit-exact against the oracle, encoded features against the reference;
  * compositing and its gradients with depth priors switched on;
  * .inerf files written by either engine and read by the other, and 1920x1080 frames rendered by both engines from the
    same file (composited RGB within 1e-3).

Skipped when the reference build is not present."""
import ctypes
import importlib
import os

import numpy as np
import pytest

from helpers import ABS_RGB, REL_ENCODE, REL_MLP, Uploader, dev_half_bits, half_bits, half_vals, make_mlp, make_positions, make_table, mlp_dims, rel_err
from test_gpu_vs_reference import _dirs, _field_pair

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import ref_cuda
    if not ref_cuda.available():
        pytest.skip("reference CUDA build (oracle/_ref) not present")
    ref_cuda.lib()
    return ref_cuda


def _view(torch, ptr, count, dtype=np.float32):
    nm = importlib.import_module("3dmaker_b200.nerf")
    return nm.view_tensor(torch, ptr, count, dtype)


def _layer_slices(model):
    """(net, layer, what, arena offset, count) of every dense parameter block, in the arena's order."""
    out = []
    for net, (off_w, off_b, dims) in enumerate(((model.off_dw, model.off_db, mlp_dims(32, 64, 16, 2)), (model.off_cw, model.off_cb, mlp_dims(32, 64, 8, 3)))):
        wo, bo = off_w, off_b
        for l, (ki, ko) in enumerate(dims):
            out.append((net, l, 0, wo, ki * ko)); out.append((net, l, 1, bo, ko))
            wo += ki * ko; bo += ko
    return out


def test_optimizer_alone_against_the_reference_optimizer(cuda, nb, ref):
    """Both optimizers get the SAME gradient written into their buffers, three steps in a row (so the moments matter):
    sparse hash-table rule (untouched entries keep parameters AND moments), dense rule, loss-scale division, the
    non-finite self-heal.  Parameters must agree to rel 1e-5 (fp32, same operation order)."""
    torch = cuda
    L, T = 16, 1 << 16
    model, tr, rf, params = _field_pair(torch, nb, ref, L, T, 1.447, 1024)
    H, total = model.hash_count, model.total
    lib, st = ref.lib(), nb.stream_ptr()
    r_hash_g = _view(torch, lib.ref_field_hash_grads(rf), H)
    rng = np.random.default_rng(42)
    for step in range(3):
        g = np.zeros(total, np.float32)
        touched = rng.random(H) < (0.3 if step < 2 else 0.05)             # step 3 touches few: the rest must not decay
        g[:H] = (rng.normal(0, 3.0, H) * touched).astype(np.float32)
        g[H:] = rng.normal(0, 20.0, total - H).astype(np.float32)
        if step == 1:                                                       # non-finite gradients are dropped, not spread
            g[5] = np.inf; g[H + 7] = np.nan
        dg = torch.from_numpy(g).cuda()
        model.g.copy_(dg)
        r_hash_g.copy_(dg[:H])
        for net, l, what, off, cnt in _layer_slices(model):
            _view(torch, lib.ref_field_layer_grads(rf, net, l, what), cnt).copy_(dg[off:off + cnt])
        tr.optimizer_step()
        lib.ref_field_step(rf, 128.0, 1e-2, 0.9, 0.99, 1e-15, st)
        torch.cuda.synchronize()
        assert float(model.g.abs().sum().item()) == 0.0                    # consumed and cleared
    table, dW, db, cW, cb = params
    r_hash = np.zeros(H, np.float32); r_dW, r_db, r_cW, r_cb = (np.zeros_like(x) for x in (dW, db, cW, cb))
    lib.ref_field_save(rf, ref.hptr(r_hash), ref.hptr(r_dW), ref.hptr(r_db), ref.hptr(r_cW), ref.hptr(r_cb))
    w = model.w.cpu().numpy()
    assert np.isfinite(w).all() and np.isfinite(r_hash).all()
    assert rel_err(w[:H], r_hash) <= 1e-5
    moved = r_hash != table.ravel()
    assert 0.3 < moved.mean() < 0.7 and np.array_equal(moved, w[:H] != table.ravel())      # the same entries were touched
    for name, off, cnt, r in (("dW", model.off_dw, dW.size, r_dW), ("db", model.off_db, db.size, r_db), ("cW", model.off_cw, cW.size, r_cW),
                              ("cb", model.off_cb, cb.size, r_cb)):
        assert rel_err(w[off:off + cnt], r) <= 1e-5, name
    # the fp16 copy the forward reads is the rounded master copy
    assert np.array_equal(dev_half_bits(model.w_h[:H]), half_bits(w[:H]))
    lib.ref_field_destroy(rf)


def test_field_step_at_the_benchmark_shape_against_reference(cuda, nb, ref):
    """2^20 samples, T = 2^19, growth 1.447 - the shape of the headline measurement: encoded features, outputs, every
    gradient, then one whole optimizer step of each implementation."""
    torch = cuda
    L, T, n = 16, 1 << 19, 1 << 20
    model, tr, rf, params = _field_pair(torch, nb, ref, L, T, 1.447, n, fused=True)
    rng = np.random.default_rng(3)
    pos = make_positions(n, 3); dirs = _dirs(n, 4)
    tgt3 = rng.random((n, 3), dtype=np.float32)
    tgt8 = np.zeros((n, 8), np.float32); tgt8[:, :3] = tgt3
    tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(half_bits(tgt8).view(np.float16)))
    d_t3 = torch.from_numpy(half_bits(tgt3).view(np.float16)).cuda()
    lib, st = ref.lib(), nb.stream_ptr()
    tr.forward_backward(n)
    lib.ref_field_forward_backward(rf, nb.ptr(tr.pos), nb.ptr(tr.dirs), nb.ptr(d_t3), n, 1.0, 128.0, st)
    torch.cuda.synchronize()
    r_enc = _view(torch, lib.ref_field_grid_activation(rf, 0), n * 32, np.float16).view(n, 32)
    assert torch.equal(tr.encoded(n).view(torch.int16), r_enc.view(torch.int16)), "encoded features differ from the reference's"
    r_dout = _view(torch, lib.ref_field_density_out(rf), n * 16).view(n, 16)
    r_cout = _view(torch, lib.ref_field_color_out(rf), n * 3).view(n, 3)
    assert float((tr.c_out[:, :3] - r_cout).abs().max().item()) <= 1e-2
    assert float((tr.logit0 - r_dout[:, 0]).abs().max().item()) <= REL_MLP * float(r_dout[:, 0].abs().max().item())
    H = model.hash_count
    r_hash = _view(torch, lib.ref_field_hash_grads(rf), H)
    scale = float(r_hash.abs().max().item())
    assert float((model.g[:H] - r_hash).abs().max().item()) <= 3 * REL_MLP * scale
    assert float(((model.g[:H] != 0) != (r_hash != 0)).float().mean().item()) < 1e-3
    g = model.g.cpu().numpy()
    for net, l, what, off, cnt in _layer_slices(model):
        r = _view(torch, lib.ref_field_layer_grads(rf, net, l, what), cnt).cpu().numpy()
        assert rel_err(g[off:off + cnt], r) <= 3 * REL_MLP, (net, l, what)
    # one whole step of each.  The first Adam step moves every touched entry by lr * sign(g) (m / sqrt(v) = +-1), so the
    # parameters agree to fp32 rounding wherever the two gradients have the same sign - everywhere but at gradients that
    # round to zero on one side.
    model.g.zero_()
    tr.step_device(n)
    lib.ref_field_train_step(rf, nb.ptr(tr.pos), nb.ptr(tr.dirs), nb.ptr(d_t3), n, 1.0, 128.0, 1e-2, 0.9, 0.99, 1e-15, st)
    torch.cuda.synchronize()
    r_hash_w = np.zeros(H, np.float32)
    lib.ref_field_save(rf, ref.hptr(r_hash_w), None, None, None, None)
    w = model.w[:H].cpu().numpy()
    off_by = np.abs(w - r_hash_w) > 1e-5 * np.abs(r_hash_w).max()
    print("benchmark shape: table entries that moved differently after one step: %.2e" % off_by.mean())
    assert off_by.mean() < 2e-3
    lib.ref_field_destroy(rf)


@pytest.mark.parametrize("b", [1.447, 1.3819])
def test_config5_grid_indices_and_encoding(cuda, nb, ref, orc, b):
    """T = 2^22 per level (config 5): corner indices bit-exact against the oracle in both clamp conventions, first hashed
    level as the reference's launcher computes it, encoded features identical to the reference kernel's."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    L, T, n = 16, 1 << 22, 1 << 17
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    model = pl.FieldModel(torch, L, T, 16, b, 64, 2, 64, 3, training=False)
    assert model.grid.dense_level_start == orc.dense_level_start(T, 16, b, L) == (7 if b == 1.447 else 8)
    pos = make_positions(n, 9)
    pos[:8, :3] = [[0, 0, 0], [1, 1, 1], [1, 0, 0.5], [0.999999, 0.5, 0.25], [0.5, 1, 0], [0, 1, 1], [0.25, 0.75, 1.0], [1.0, 1e-7, 0.3]]
    d_pos = torch.from_numpy(pos).cuda()
    sub = 1 << 14
    idx = torch.zeros((sub, L, 8), dtype=torch.int32, device="cuda")
    scales = np.array(list(model.grid.scales)[:L], np.float32)
    for mode in (0, 1):
        nb.check(lib.nb_hash_indices(ctypes.byref(model.grid), P(d_pos), sub, mode, P(idx), st), "nb_hash_indices")
        torch.cuda.synchronize()
        want = orc.hash_indices(pos[:sub], scales if mode == 0 else np.array(list(model.grid.scatter_scales)[:L], np.float32), T,
                                model.grid.dense_level_start, mode)
        assert np.array_equal(idx.cpu().numpy().view(np.uint32), want), "corner indices differ from the oracle's (clamp mode %d)" % mode
    # encoded features and the grid network's output against the reference's classes at the same table size
    table = make_table(L, T, seed=1, amp=0.1)
    dW, db = make_mlp(32, 64, 16, 2, seed=2, bias_amp=0.02)
    cW, cb = make_mlp(32, 64, 8, 3, seed=3, bias_amp=0.02)
    model.load_hashgrid(table); model.load_density_weights(dW, db); model.load_color_weights(cW, cb)
    rf = ref.lib().ref_field_create(L, T, 16, b, 64, 2, 64, 3, n)
    ref.lib().ref_field_load(rf, ref.hptr(np.ascontiguousarray(table.ravel())), ref.hptr(dW), ref.hptr(db), ref.hptr(cW), ref.hptr(cb))
    dirs = torch.from_numpy(_dirs(n, 5)).cuda()
    enc = torch.zeros((n, 32), dtype=torch.float16, device="cuda"); sigma = torch.zeros(n, device="cuda"); logit = torch.zeros(n, device="cuda")
    rgb = torch.zeros((n, 4), device="cuda")
    m = model
    nb.check(lib.nb_field_forward(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(d_pos), m.ptr("w_h", 0), P(dirs), None, 0,
                                  m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, 1.0, P(enc),
                                  P(sigma), P(logit), P(rgb), 4, st), "nb_field_forward")
    ref.lib().ref_field_forward(rf, P(d_pos), P(dirs), n, 1.0, st)
    torch.cuda.synchronize()
    r_enc = _view(torch, ref.lib().ref_field_grid_activation(rf, 0), n * 32, np.float16).view(n, 32)
    e, r = half_vals(dev_half_bits(enc)), half_vals(dev_half_bits(r_enc))
    assert rel_err(e, r) <= REL_ENCODE
    assert np.array_equal(dev_half_bits(enc), dev_half_bits(r_enc)), "encoded features are within tolerance but not bit-identical"
    r_cout = _view(torch, ref.lib().ref_field_color_out(rf), n * 3).view(n, 3)
    assert float((rgb[:, :3] - r_cout).abs().max().item()) <= 1e-2
    ref.lib().ref_field_destroy(rf)


def test_compositing_with_depth_priors_against_reference(cuda, nb, ref, orc):
    """lambda_depth > 0 and real per-ray priors (a third of the rays carry none: depth -1): rendered colour, depth,
    dL/dw with the depth term, per-ray weight sums and the loss gradients that consume them, against
    render_rays_distortion_kernel / compute_color_grad of the reference - and the oracle against the same outputs."""
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    from test_gpu_nerf import _random_ray_samples
    counts, off, t, dens, col, target = _random_ray_samples(4000, 19)
    R, n = len(counts), len(t)
    rng = np.random.default_rng(23)
    prior_depth = rng.uniform(0.6, 2.9, R).astype(np.float32)
    prior_depth[rng.random(R) < 0.33] = -1.0
    prior_sigma = rng.uniform(0.02, 0.5, R).astype(np.float32)
    bias, lam, lam_depth, scale = 1.0, 0.1, 0.05, 128.0
    sigma = np.exp(np.minimum(dens[:, 0] - np.float32(bias), 8)).astype(np.float32)
    bgn = np.array([1.0, 0.5, 0.25], np.float32); bg = (ctypes.c_float * 3)(*bgn)
    Z = lambda *shape, dt=torch.float32: torch.zeros(shape, dtype=dt, device="cuda")
    d_off, d_cnt, d_t, d_sig, d_col8, d_col3, d_tgt, d_dens, d_pd, d_ps = (
        up.f(off.view(np.int32)), up.f(counts.view(np.int32)), up.f(t), up.f(sigma), up.f(col), up.f(np.ascontiguousarray(col[:, :3])), up.f(target),
        up.f(dens), up.f(prior_depth), up.f(prior_sigma))
    m = dict(rgb=Z(R, 3), depth=Z(R), phi=Z(R, 3), dw=Z(n), ws=Z(R), grad=Z(n, 8, dt=torch.float16), dsig=Z(n))
    r = dict(rgb=Z(R, 3), depth=Z(R), phi=Z(R, 3), dw=Z(n), ws=Z(R), grad=Z(n, 3, dt=torch.float16), dsig=Z(n))
    nb.check(lib.nb_composite_train(R, 0, d_off, d_cnt, d_t, d_sig, d_pd, d_ps, d_col8, 8, d_tgt, P(m["rgb"]), P(m["depth"]), P(m["phi"]), P(m["dw"]),
                                    P(m["ws"]), lam, lam_depth, bg, st), "nb_composite_train")
    nb.check(lib.nb_color_grad(R, 0, d_cnt, d_off, d_t, d_dens, 16, d_col8, 8, P(m["phi"]), P(m["rgb"]), P(m["dw"]), P(m["ws"]), P(m["grad"]), 8,
                               P(m["dsig"]), scale, bias, R, st), "nb_color_grad")
    ref.lib().ref_volume_rendering_priors(R, d_off, d_cnt, d_t, d_sig, d_pd, d_ps, d_col3, d_tgt, P(r["rgb"]), P(r["depth"]), P(r["phi"]), P(r["dw"]),
                                          P(r["ws"]), lam, lam_depth, ref.hptr(bgn), st)
    ref.lib().ref_color_grad(R, d_cnt, d_off, d_t, d_dens, d_col3, P(r["phi"]), P(r["rgb"]), P(r["dw"]), P(r["ws"]), P(r["grad"]), P(r["dsig"]), scale,
                             bias, R, st)
    # the priors must have mattered: the same call without them gives a different dL/dw
    plain = Z(n); plain_ws = Z(R); scratch = dict(rgb=Z(R, 3), depth=Z(R), phi=Z(R, 3))
    nb.check(lib.nb_composite_train(R, 0, d_off, d_cnt, d_t, d_sig, None, None, d_col8, 8, d_tgt, P(scratch["rgb"]), P(scratch["depth"]),
                                    P(scratch["phi"]), P(plain), P(plain_ws), lam, 0.0, bg, st), "nb_composite_train")
    torch.cuda.synchronize()
    assert float((plain - m["dw"]).abs().max().item()) > 1e-3 * float(m["dw"].abs().max().item())
    assert (m["rgb"] - r["rgb"]).abs().max().item() <= 1e-5 and (m["phi"] - r["phi"]).abs().max().item() <= 2e-5
    assert rel_err(m["depth"].cpu().numpy(), r["depth"].cpu().numpy()) <= 1e-5
    assert rel_err(m["dw"].cpu().numpy(), r["dw"].cpu().numpy()) <= 1e-4 and rel_err(m["ws"].cpu().numpy(), r["ws"].cpu().numpy()) <= 1e-4
    assert rel_err(half_vals(dev_half_bits(m["grad"]))[:, :3], half_vals(dev_half_bits(r["grad"]))) <= 1e-3
    assert rel_err(m["dsig"].cpu().numpy(), r["dsig"].cpu().numpy()) <= 1e-3
    # the oracle's restatement of the same kernel, pinned here by the reference's output
    o_rgb, o_depth, o_phi, o_dw, o_ws = orc.render_rays_distortion(R, off, counts, t, sigma, col[:, :3].copy(), target, lam, lam_depth, bgn,
                                                                   depth_prior=prior_depth, sigma_prior=prior_sigma)
    assert np.max(np.abs(o_rgb - r["rgb"].cpu().numpy())) <= ABS_RGB
    assert rel_err(o_dw, r["dw"].cpu().numpy()) <= REL_MLP and rel_err(o_ws, r["ws"].cpu().numpy()) <= REL_MLP


def _scene_options(nm, T=1 << 19):
    return nm.default_options(grid_resolution=(128,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=4, hash_table_size=T,
                              growth_factor=1.3819, color_hidden_dim=64, color_num_layers=3, batch_size=1 << 18, render_batch_size=1 << 18,
                              ray_chunk_size=1 << 16, lambda_dist=0.01, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
                              loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))


def test_inerf_files_cross_the_engines_and_their_frames_agree(cuda, nb, ref, tmp_path):
    """A model trained and saved by this engine loads in the reference's InstantNerf, and the other way round; the file
    carries parameters, master occupancy grid and bit pyramid.  From the same file both engines render the same
    1920x1080 orbit frame: composited RGB within 1e-3 (config 4's frame, InstantNerf.cu:713-864)."""
    torch = cuda
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    lib, st = ref.lib(), nb.stream_ptr()
    opts = _scene_options(nm)
    eng = nm.InstantNerf(torch, opts)
    scene, poses, bg = syn.SoftSphereScene(), syn.sphere_cameras(100), (1.0, 1.0, 1.0)
    R, it = 1 << 16, 0
    while eng.steps.value < 200:
        o, d = syn.random_training_rays(torch, poses, R, 800, 800, 50.0, seed=700 + it)
        eng.train_rays(o, d, syn.ground_truth(torch, scene, o, d, bg))
        it += 1
    torch.cuda.synchronize()
    ours_path = os.path.join(str(tmp_path), "ours.inerf")
    eng.save(ours_path)
    rh = lib.ref_nerf_create(ctypes.byref(opts), 0)
    assert lib.ref_nerf_load(rh, ours_path.encode()) == 0, "the reference could not read a file this engine wrote"

    def frames(W, H, az):
        o, d = syn.frame_rays(torch, syn.orbit_c2w(az, 20.0, 1.5), W, H, 50.0)
        a = torch.zeros((W * H, 3), device="cuda"); b = torch.zeros_like(a)
        eng.render(o, d, a)
        lib.ref_nerf_render(rh, nb.ptr(o), nb.ptr(d), W * H, nb.ptr(b), st)
        torch.cuda.synchronize()
        return a, b, syn.ground_truth(torch, scene, o[:: 7], d[:: 7], bg), None

    a, b, gt, _ = frames(1920, 1080, 33.0)
    diff = (a - b).abs()
    print("ours-written file, 1920x1080: max |dRGB| %.2e, mean %.2e, PSNR ours %.2f dB" % (diff.max().item(), diff.mean().item(),
                                                                                            syn.psnr(torch, a[:: 7], gt)))
    assert syn.psnr(torch, a[:: 7], gt) > 28.0                               # a real picture, not two equal blanks
    assert diff.max().item() <= ABS_RGB
    # ---- the other direction: the reference trains on, writes, we read ---------------------------------------
    depth = torch.full((R,), -1.0, device="cuda"); sig = torch.ones(R, device="cuda")
    for k in range(3):
        o, d = syn.random_training_rays(torch, poses, R, 800, 800, 50.0, seed=900 + k)
        tgt = syn.ground_truth(torch, scene, o, d, bg)
        lib.ref_nerf_train(rh, nb.ptr(o), nb.ptr(d), nb.ptr(depth), nb.ptr(sig), nb.ptr(tgt), R, None, None, st)
    torch.cuda.synchronize()
    ref_path = os.path.join(str(tmp_path), "reference.inerf")
    assert lib.ref_nerf_save(rh, ref_path.encode()) == 0
    eng.load(ref_path)
    av = eng.arena()
    w = eng.arena_tensor("w").cpu().numpy()
    H = av.sparse_count
    r_hash = np.zeros(H, np.float32)
    r_dW = np.zeros(av.density_weight_count, np.float32); r_db = np.zeros(av.density_bias_count, np.float32)
    lib.ref_nerf_save_params(rh, ref.hptr(r_hash), ref.hptr(r_dW), ref.hptr(r_db), None, None)
    assert np.array_equal(w[:H], r_hash) and np.array_equal(w[av.density_weight_offset:av.density_weight_offset + av.density_weight_count], r_dW)
    bits, master = eng.occupancy()
    nbytes = ctypes.c_long()
    r_bits = _view(torch, lib.ref_nerf_bitfield(rh, ctypes.byref(nbytes)), bits.numel(), np.uint8)
    assert nbytes.value == bits.numel() and torch.equal(bits, r_bits)
    assert torch.equal(master, _view(torch, lib.ref_nerf_master_grid(rh), master.numel()))
    a, b, gt, _ = frames(1920, 1080, 117.0)
    diff = (a - b).abs()
    print("reference-written file, 1920x1080: max |dRGB| %.2e, mean %.2e" % (diff.max().item(), diff.mean().item()))
    assert diff.max().item() <= ABS_RGB
    lib.ref_nerf_destroy(rh)
    eng.close()
