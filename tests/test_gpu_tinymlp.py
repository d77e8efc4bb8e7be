"""GPU parity of the TinyMLP-level kernels (hash grid, fused MLPs, loss, Adam) against the CPU oracle.

Every call goes through the C ABI of libnerf_b200.so.  Integer results (hash indices) and the encoded
fp16 features are compared bit for bit; MLP outputs and gradients within the stated relative tolerance."""
import ctypes

import numpy as np
import pytest

from helpers import (REL_ENCODE, REL_MLP, Uploader, dev_half_bits, half_bits, half_to_dev, half_vals, make_mlp, make_positions,
                     make_table, mlp_dims, rel_err, to_dev)

pytestmark = pytest.mark.gpu


def _grid(nb, L=16, T=1 << 14, base=16, b=1.447):
    d = nb.grid_setup(L, T, base, b)
    scales = np.array(list(d.scales)[:L], np.float32)
    d.np_scatter_scales = np.array(list(d.scatter_scales)[:L], np.float32)
    return d, scales


@pytest.mark.parametrize("b", [1.447, 1.3819])
@pytest.mark.parametrize("T", [1 << 14, 1 << 19])
def test_grid_setup_matches_oracle(cuda, nb, orc, b, T):
    d, scales = _grid(nb, T=T, b=b)
    assert d.dense_level_start == orc.dense_level_start(T, 16, b, 16)
    ref = orc.level_scales(16, b, 16)
    # the device evaluates the power with its approximate intrinsic: a few ulp from libm, same integer part
    assert np.allclose(scales, ref, rtol=2e-6)
    assert np.array_equal(np.floor(scales), np.floor(ref))
    # the scatter's own expression lands within a few ulp of the same values
    assert np.allclose(d.np_scatter_scales, ref, rtol=4e-6) and np.array_equal(np.floor(d.np_scatter_scales), np.floor(ref))


@pytest.mark.parametrize("clamp_mode", [0, 1])
@pytest.mark.parametrize("n", [0, 1, 1000, 65536])
def test_hash_indices_bit_exact(cuda, nb, orc, clamp_mode, n):
    torch = cuda
    up = Uploader(torch, nb)
    d, scales = _grid(nb, T=1 << 19)
    pos = make_positions(n, seed=0)
    if n >= 3:
        pos[0, :3] = 0.0; pos[1, :3] = 1.0; pos[2, :3] = [1.0, 0.0, 0.999999]
    out = torch.zeros((max(n, 1), 16, 8), dtype=torch.int32, device="cuda")
    nb.check(nb.load().nb_hash_indices(ctypes.byref(d), up.f(pos) if n else nb.ptr(out), n, clamp_mode,
                                       nb.ptr(out), nb.stream_ptr()), "nb_hash_indices")
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint32)[:n]
    ref = orc.hash_indices(pos, d.np_scatter_scales if clamp_mode else scales, 1 << 19, d.dense_level_start, clamp_mode)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("n", [1, 127, 128, 1000, 65536])
@pytest.mark.parametrize("b", [1.447, 1.3819])
def test_encode_forward_bit_exact(cuda, nb, orc, n, b):
    torch = cuda
    up = Uploader(torch, nb)
    T = 1 << 19
    d, scales = _grid(nb, T=T, b=b)
    pos = make_positions(n, seed=0)
    table = half_bits(make_table(16, T, seed=0, amp=1e-4))
    enc = torch.zeros((n, 32), dtype=torch.float16, device="cuda")
    nb.check(nb.load().nb_hash_encode_forward(ctypes.byref(d), up.f(pos), up.h(table), n,
                                              nb.ptr(enc), nb.stream_ptr()), "nb_hash_encode_forward")
    torch.cuda.synchronize()
    ref = orc.encode_forward(pos, table, scales, T, d.dense_level_start)
    got = dev_half_bits(enc)
    assert rel_err(half_vals(got), half_vals(ref)) <= REL_ENCODE
    assert np.array_equal(got, ref), "encoded features differ in %d of %d halves" % ((got != ref).sum(), got.size)


@pytest.mark.parametrize("dims", [(32, 64, 16, 2), (32, 32, 16, 2), (32, 64, 16, 3)])
@pytest.mark.parametrize("n", [16, 1000, 65536])
def test_grid_mlp_forward(cuda, nb, orc, dims, n):
    """Config 1: encode + density MLP forward, N = 2^16 points, T = 2^19, table U[-1e-4, 1e-4], Xavier weights."""
    torch = cuda
    up = Uploader(torch, nb)
    i, h, o, nl = dims
    T = 1 << 19
    d, scales = _grid(nb, T=T)
    mlp = nb.mlp_desc(i, h, o, nl)
    pos = make_positions(n, seed=0)
    table = half_bits(make_table(16, T, seed=0, amp=0.1 if n < 65536 else 1e-4))
    W, bias = make_mlp(i, h, o, nl, seed=0, bias_amp=0.05)
    Wh = half_bits(W)
    out = torch.zeros((n, o), dtype=torch.float32, device="cuda")
    enc = torch.zeros((n, i), dtype=torch.float16, device="cuda")
    acts = torch.zeros((max(nl - 1, 1), n, h), dtype=torch.float16, device="cuda")
    args = (ctypes.byref(d), ctypes.byref(mlp), up.f(pos), up.h(table),
            up.h(Wh), up.f(bias), n, nb.ptr(out))
    nb.check(nb.load().nb_grid_mlp_forward(*args, nb.ptr(enc), nb.ptr(acts), nb.stream_ptr()), "nb_grid_mlp_forward")
    torch.cuda.synchronize()
    enc_ref = orc.encode_forward(pos, table, scales, T, d.dense_level_start)
    assert np.array_equal(dev_half_bits(enc), enc_ref)
    out_ref, acts_ref = orc.mlp_forward(enc_ref, dims, Wh, bias, save_acts=True)
    assert rel_err(out.cpu().numpy(), out_ref) <= REL_MLP
    if nl > 1:
        assert rel_err(half_vals(dev_half_bits(acts)[:nl - 1]), half_vals(acts_ref)) <= REL_MLP
    # inference variant (nothing saved) gives the same output bits
    out2 = torch.zeros_like(out)
    nb.check(nb.load().nb_grid_mlp_forward(*args[:-1], nb.ptr(out2), None, None, nb.stream_ptr()), "nb_grid_mlp_forward")
    torch.cuda.synchronize()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dims,act", [((32, 64, 16, 2), 0), ((32, 64, 8, 3), 1), ((32, 64, 8, 2), 1), ((32, 32, 8, 3), 1),
                                      ((64, 64, 64, 2), 0), ((64, 64, 64, 4), 0), ((32, 32, 32, 2), 0), ((16, 16, 16, 2), 0),
                                      ((32, 64, 16, 1), 0)])
@pytest.mark.parametrize("n", [1, 100, 4096 + 17])
def test_mlp_forward(cuda, nb, orc, dims, act, n):
    torch = cuda
    up = Uploader(torch, nb)
    i, h, o, nl = dims
    rng = np.random.default_rng(21)
    x = half_bits(rng.normal(0, 1, size=(n, i)).astype(np.float32))
    W, bias = make_mlp(i, h, o, nl, seed=1, bias_amp=0.1)
    Wh = half_bits(W)
    mlp = nb.mlp_desc(i, h, o, nl, act)
    out = torch.full((n, o), 7.0, dtype=torch.float32, device="cuda")
    acts = torch.zeros((max(nl - 1, 1), n, h), dtype=torch.float16, device="cuda")
    nb.check(nb.load().nb_mlp_forward(ctypes.byref(mlp), up.h(x), up.h(Wh),
                                      up.f(bias), n, nb.ptr(out), nb.ptr(acts), nb.stream_ptr()), "nb_mlp_forward")
    torch.cuda.synchronize()
    out_ref, acts_ref = orc.mlp_forward(x, dims, Wh, bias, out_act=act, save_acts=True)
    assert rel_err(out.cpu().numpy(), out_ref) <= REL_MLP
    if nl > 1:
        assert rel_err(half_vals(dev_half_bits(acts)[:nl - 1]), half_vals(acts_ref)) <= REL_MLP


def test_mlp_unsupported_shape_is_an_error_not_a_noop(cuda, nb):
    torch = cuda
    up = Uploader(torch, nb)
    mlp = nb.mlp_desc(48, 64, 16, 2)
    buf = torch.zeros(4096, dtype=torch.float32, device="cuda")
    rc = nb.load().nb_mlp_forward(ctypes.byref(mlp), nb.ptr(buf), nb.ptr(buf), nb.ptr(buf), 16, nb.ptr(buf), None, nb.stream_ptr())
    assert rc == 2 and b"shape" in nb.load().nb_last_error()
    rc = nb.load().nb_mlp_forward(ctypes.byref(mlp), None, nb.ptr(buf), nb.ptr(buf), 16, nb.ptr(buf), None, nb.stream_ptr())
    assert rc == 1


@pytest.mark.parametrize("dims", [(32, 64, 16, 2), (32, 64, 8, 3), (32, 64, 8, 2), (32, 32, 8, 3), (64, 64, 64, 2), (16, 16, 16, 2),
                                  (32, 64, 16, 1)])
@pytest.mark.parametrize("n", [1, 100, 128 * 300 + 5])
@pytest.mark.parametrize("want_dx", [False, True])
def test_mlp_backward(cuda, nb, orc, dims, n, want_dx):
    torch = cuda
    up = Uploader(torch, nb)
    i, h, o, nl = dims
    rng = np.random.default_rng(22)
    x = half_bits(rng.normal(0, 1, size=(n, i)).astype(np.float32))
    W, bias = make_mlp(i, h, o, nl, seed=2, bias_amp=0.05)
    Wh = half_bits(W)
    _, acts_ref = orc.mlp_forward(x, dims, Wh, bias, save_acts=True)
    dL = half_bits(rng.normal(0, 1e-2, size=(n, o)).astype(np.float32))
    mlp = nb.mlp_desc(i, h, o, nl)
    dW = torch.zeros(mlp.weight_count, dtype=torch.float32, device="cuda")
    db = torch.zeros(mlp.bias_count, dtype=torch.float32, device="cuda")
    dX = torch.zeros((n, i), dtype=torch.float16, device="cuda") if want_dx else None
    acts_dev = half_to_dev(torch, acts_ref) if nl > 1 else torch.zeros(8, dtype=torch.float16, device="cuda")
    call = lambda: nb.check(nb.load().nb_mlp_backward(
        ctypes.byref(mlp), up.h(dL), up.h(Wh), up.h(x),
        nb.ptr(acts_dev), n, nb.ptr(dW), nb.ptr(db), nb.ptr(dX), nb.stream_ptr()), "nb_mlp_backward")
    call()
    torch.cuda.synchronize()
    dW_ref, db_ref, dX_ref = orc.mlp_backward(dL, dims, Wh, x, acts_ref, want_dx=want_dx)
    assert rel_err(dW.cpu().numpy(), dW_ref) <= REL_MLP
    assert rel_err(db.cpu().numpy(), db_ref) <= REL_MLP
    if want_dx:
        assert rel_err(half_vals(dev_half_bits(dX)), half_vals(dX_ref)) <= REL_MLP
    # gradients accumulate: a second call doubles them
    call()
    torch.cuda.synchronize()
    assert rel_err(dW.cpu().numpy(), 2 * dW_ref) <= REL_MLP


@pytest.mark.parametrize("n", [1, 1000, 65536])
@pytest.mark.parametrize("T", [1 << 14, 1 << 19])
def test_scatter_backward(cuda, nb, orc, n, T):
    """Config 1 backward: upstream gradients fp16 N(0, 1e-2)."""
    torch = cuda
    up = Uploader(torch, nb)
    d, scales = _grid(nb, T=T)
    rng = np.random.default_rng(0)
    pos = make_positions(n, seed=0)
    denc = half_bits(rng.normal(0, 1e-2, size=(n, 32)).astype(np.float32))
    grads = torch.zeros(16 * T * 2, dtype=torch.float32, device="cuda")
    nb.check(nb.load().nb_hash_scatter_backward(ctypes.byref(d), up.f(pos), up.h(denc), n,
                                                nb.ptr(grads), nb.stream_ptr()), "nb_hash_scatter_backward")
    torch.cuda.synchronize()
    ref = orc.scatter_backward(pos, denc, d.np_scatter_scales, T, d.dense_level_start)
    got = grads.cpu().numpy()
    assert rel_err(got, ref) <= REL_MLP
    assert np.array_equal(got != 0, ref != 0) or n > 1000   # same touched set (tiny products may cancel at scale)
    # mass conservation: per level and feature the table gradient sums to the sum of the upstream gradient
    per = got.astype(np.float64).reshape(16, T, 2).sum(axis=1)
    assert np.allclose(per, half_vals(denc).astype(np.float64).reshape(n, 16, 2).sum(axis=0), rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("n", [4000, 70000])
def test_scatter_of_ray_ordered_samples(cuda, nb, orc, n):
    """Samples in ray order (a short step between neighbours, as the marcher emits them): most warps take the path that
    sums runs of samples in one cell before reducing.  Against the oracle, and against the direct path switched on by
    nb_set_tuning - the two differ by fp32 summation order only.  Some gradient rows are exactly zero (skipped)."""
    torch = cuda
    up = Uploader(torch, nb)
    T = 1 << 17
    d, scales = _grid(nb, T=T, b=1.3819)
    rng = np.random.default_rng(5)
    per_ray = 40
    rays = (n + per_ray - 1) // per_ray
    o = rng.uniform(0.3, 0.7, (rays, 1, 3)); dirs = rng.normal(size=(rays, 1, 3)); dirs /= np.linalg.norm(dirs, axis=2, keepdims=True)
    pts = (o + dirs * (np.arange(per_ray)[None, :, None] * 0.004)).reshape(-1, 3)[:n]
    pos = np.zeros((n, 4), np.float32); pos[:, :3] = np.clip(pts, 0.0, 0.999)
    g = rng.normal(0, 1e-2, size=(n, 32)).astype(np.float32)
    g[rng.random(n) < 0.1] = 0.0
    denc = half_bits(g)
    out = {}
    lib = nb.load()
    for merge in (1, 0):
        nb.check(lib.nb_set_tuning(b"scatter_run_merge", 32 if merge else 0), "nb_set_tuning")
        grads = torch.zeros(16 * T * 2, dtype=torch.float32, device="cuda")
        nb.check(lib.nb_hash_scatter_backward(ctypes.byref(d), up.f(pos), up.h(denc), n, nb.ptr(grads), nb.stream_ptr()), "nb_hash_scatter_backward")
        torch.cuda.synchronize()
        out[merge] = grads.cpu().numpy()
    nb.check(lib.nb_set_tuning(b"scatter_run_merge", 20), "nb_set_tuning")
    ref = orc.scatter_backward(pos, denc, d.np_scatter_scales, T, d.dense_level_start)
    assert rel_err(out[1], ref) <= REL_MLP and rel_err(out[0], ref) <= REL_MLP
    assert rel_err(out[1], out[0]) <= 1e-5
    per = out[1].astype(np.float64).reshape(16, T, 2).sum(axis=1)
    assert np.allclose(per, half_vals(denc).astype(np.float64).reshape(n, 16, 2).sum(axis=0), rtol=1e-3, atol=1e-5)


def test_mse_loss_grad(cuda, nb, orc):
    torch = cuda
    up = Uploader(torch, nb)
    rng = np.random.default_rng(23)
    n, padded, valid = 4099, 8, 3
    pred = rng.random((n, padded)).astype(np.float32)
    tgt = half_bits(rng.random((n, padded)).astype(np.float32))
    for act in (0, 1):
        grad = torch.zeros((n, padded), dtype=torch.float16, device="cuda")
        total = torch.zeros(1, dtype=torch.float32, device="cuda")
        nb.check(nb.load().nb_mse_loss_grad(up.f(pred), up.h(tgt), nb.ptr(grad), nb.ptr(total),
                                            n, padded, valid, 128.0, act, nb.stream_ptr()), "nb_mse_loss_grad")
        torch.cuda.synchronize()
        total_ref, grad_ref = orc.mse_loss_grad(pred, tgt, valid, 128.0, out_act=act)
        assert abs(total.item() - total_ref) <= 1e-4 * total_ref          # fp32, reference tolerance 1e-4
        assert rel_err(half_vals(dev_half_bits(grad)), half_vals(grad_ref)) <= 1e-3   # fp16, reference tolerance 1e-3


def test_adam_step_arena(cuda, nb, orc):
    torch = cuda
    up = Uploader(torch, nb)
    rng = np.random.default_rng(24)
    sparse, total = 1 << 16, (1 << 16) + 3152
    w = rng.normal(0, 0.1, total).astype(np.float32)
    g = rng.normal(0, 1, total).astype(np.float32)
    g[:sparse][rng.random(sparse) < 0.6] = 0.0
    g[sparse + 7] = 0.0
    m = rng.normal(0, 0.01, total).astype(np.float32)
    v = np.abs(rng.normal(0, 0.01, total)).astype(np.float32)
    g[11] = np.inf; m[12] = np.nan; w[13] = np.nan; g[13] = 1.0; g[sparse + 3] = np.nan
    wh0 = half_bits(np.nan_to_num(w))
    bc1, bc2 = orc.adam_bias_corrections(1, 0.9, 0.99)
    hyper = (1e-2, 0.9, 0.99, 1e-15, bc1, bc2, 1.0 / 128.0)
    d_w, d_g, d_m, d_v = (to_dev(torch, a.copy()) for a in (w, g, m, v))
    d_wh = half_to_dev(torch, wh0.copy())
    nb.check(nb.load().nb_adam_step(nb.ptr(d_w), nb.ptr(d_wh), nb.ptr(d_g), nb.ptr(d_m), nb.ptr(d_v), sparse, total, *hyper, 1,
                                    nb.stream_ptr()), "nb_adam_step")
    torch.cuda.synchronize()
    # oracle: sparse rule on the first part, dense on the rest
    ws, gs, ms, vs, whs = w[:sparse].copy(), g[:sparse].copy(), m[:sparse].copy(), v[:sparse].copy(), wh0[:sparse].copy()
    orc.adam_hash(ws, whs, gs, ms, vs, *hyper)
    wd, md, vd = w[sparse:].copy(), m[sparse:].copy(), v[sparse:].copy()
    whd = orc.adam_dense(wd, g[sparse:], md, vd, *hyper)
    got_w, got_m, got_v, got_g = (t.cpu().numpy() for t in (d_w, d_m, d_v, d_g))
    for got, ref in ((got_w, np.concatenate([ws, wd])), (got_m, np.concatenate([ms, md])), (got_v, np.concatenate([vs, vd]))):
        assert np.allclose(got, ref, rtol=1e-5, atol=1e-9, equal_nan=True)     # "rel 1e-5 after one step"
    assert np.all(got_g == 0)
    untouched = g[:sparse] == 0
    assert np.array_equal(got_w[:sparse][untouched], w[:sparse][untouched], equal_nan=True)   # no decay, no write
    got_wh = dev_half_bits(d_wh)
    assert np.array_equal(got_wh[:sparse][untouched], wh0[:sparse][untouched])
    ref_wh = np.concatenate([whs, whd])
    assert np.mean(got_wh != ref_wh) < 1e-3 and rel_err(half_vals(got_wh), half_vals(ref_wh)) < 2e-3
