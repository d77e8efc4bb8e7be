"""CPU checks of the oracle itself: each C function against an independent numpy statement of the same
formula, plus the structural properties the reference's design implies.  No GPU needed."""
import numpy as np
import pytest

from helpers import half_bits, half_vals, make_mlp, make_positions, make_table, mlp_dims, rel_err


def np_hash(cx, cy, cz, T):
    with np.errstate(over="ignore"):
        return ((cx.astype(np.uint32) * np.uint32(1)) ^ (cy.astype(np.uint32) * np.uint32(2654435761)) ^
                (cz.astype(np.uint32) * np.uint32(805459861))) & np.uint32(T - 1)


def test_dense_level_start_matches_known_values(orc):
    # T = 2^19: levels 0..4 are dense for both growth factors; T = 2^22: 7 (b=1.447) and 8 (b=1.3819)
    assert orc.dense_level_start(1 << 19, 16, 1.447, 16) == 5
    assert orc.dense_level_start(1 << 19, 16, 1.3819, 16) == 5
    assert orc.dense_level_start(1 << 22, 16, 1.447, 16) == 7
    assert orc.dense_level_start(1 << 22, 16, 1.3819, 16) == 8
    assert orc.dense_level_start(4, 16, 1.5, 16) == 0          # clamps at 0
    assert orc.dense_level_start(1 << 30, 2, 1.1, 4) == 4       # clamps at numLevels


def test_level_scales_restart_every_four_levels(orc):
    s = orc.level_scales(16, 1.3819, 16)
    assert s[0] == 16.0
    for l in range(16):
        start = (l // 4) * 4
        v = np.float32(16) * np.float32(np.power(np.float32(1.3819), np.float32(start)))
        for _ in range(start, l):
            v = np.float32(v * np.float32(1.3819))
        assert abs(s[l] - v) <= 2e-6 * v
    assert int(np.floor(s[15])) in (2046, 2047, 2048)          # default growth reaches ~2048


@pytest.mark.parametrize("clamp_mode", [0, 1])
def test_hash_indices_against_numpy(orc, clamp_mode):
    L, T = 16, 1 << 14
    scales = orc.level_scales(16, 1.447, L)
    dls = orc.dense_level_start(T, 16, 1.447, L)
    pos = make_positions(777, seed=3)
    pos[0, :3] = 0.0
    pos[1, :3] = 1.0           # the only place the two clamps differ
    pos[2, :3] = [1.0, 0.0, 0.5]
    idx, w = orc.hash_indices(pos, scales, T, dls, clamp_mode, want_weights=True)
    for l in range(L):
        s = scales[l]
        N = int(np.floor(s))
        xl = pos[:, :3] * s
        c0 = np.floor(xl).astype(np.int64)
        hi = N - 1 if clamp_mode else N
        c0 = np.clip(c0, 0, hi)
        c1 = np.minimum(c0 + 1, N)
        w1 = (np.float32(1.0) - xl) + np.floor(xl)
        for k in range(8):
            ix, iy, iz = k & 1, (k >> 1) & 1, (k >> 2) & 1
            cx = np.where(ix, c1[:, 0], c0[:, 0]); cy = np.where(iy, c1[:, 1], c0[:, 1]); cz = np.where(iz, c1[:, 2], c0[:, 2])
            if l < dls:
                ti = (cx + cy * (N + 1) + cz * (N + 1) * (N + 1)).astype(np.uint32)
                assert ti.max() < T                                  # dense levels fit the table
            else:
                ti = np_hash(cx, cy, cz, T)
            expect = np.uint32(l * T * 2) + ti * np.uint32(2)
            assert np.array_equal(idx[:, l, k], expect)
            wx = np.where(ix, np.float32(1) - w1[:, 0], w1[:, 0]); wy = np.where(iy, np.float32(1) - w1[:, 1], w1[:, 1])
            wz = np.where(iz, np.float32(1) - w1[:, 2], w1[:, 2])
            assert np.array_equal(w[:, l, k], (wx * wy).astype(np.float32) * wz)
    # trilinear weights sum to one
    assert np.allclose(w.sum(axis=2), 1.0, atol=1e-5)


def test_encode_is_interpolation_of_the_table(orc):
    L, T = 16, 1 << 12
    scales = orc.level_scales(16, 1.3819, L)
    dls = orc.dense_level_start(T, 16, 1.3819, L)
    table = make_table(L, T, seed=1, amp=0.1)
    tb = half_bits(table)
    pos = make_positions(300, seed=4)
    enc = half_vals(orc.encode_forward(pos, tb, scales, T, dls))
    idx, w = orc.hash_indices(pos, scales, T, dls, 0, want_weights=True)
    flat = half_vals(tb).ravel().astype(np.float64)
    for f in range(2):
        expect = (flat[idx.astype(np.int64) + f] * w).sum(axis=2)            # [n][L]
        got = enc.reshape(300, L, 2)[:, :, f]
        assert np.max(np.abs(got - expect)) <= 1e-3 * np.max(np.abs(expect)) + 1e-7
    # a constant table encodes to that constant at every point
    const = np.full((L, T, 2), 0.03125, np.float32)
    enc_c = half_vals(orc.encode_forward(pos, half_bits(const), scales, T, dls))
    assert np.allclose(enc_c, 0.03125, rtol=2e-3)
    # empty batch
    assert orc.encode_forward(np.zeros((0, 4), np.float32), tb, scales, T, dls).shape == (0, 32)


def test_scatter_is_the_transpose_of_encode(orc):
    """<encode(table), dEnc> == <table, scatter(dEnc)> away from the upper boundary (where the two clamps agree)."""
    L, T = 16, 1 << 12
    scales = orc.level_scales(16, 1.447, L)
    dls = orc.dense_level_start(T, 16, 1.447, L)
    rng = np.random.default_rng(7)
    pos = make_positions(500, seed=5)
    pos[:, :3] *= 0.93   # x * scale < floor(scale) at every level, so both clamps agree
    table = make_table(L, T, seed=2, amp=0.5)
    tq = half_vals(half_bits(table)).astype(np.float64)
    denc = rng.normal(0, 1e-2, size=(500, 2 * L)).astype(np.float32)
    dq = half_vals(half_bits(denc)).astype(np.float64)
    grads = orc.scatter_backward(pos, half_bits(denc), scales, T, dls).astype(np.float64)
    idx, w = orc.hash_indices(pos, scales, T, dls, 0, want_weights=True)
    flat = tq.ravel()
    enc_exact = np.stack([(flat[idx.astype(np.int64) + f] * w).sum(axis=2) for f in range(2)], axis=2).reshape(500, 2 * L)
    lhs = float((enc_exact * dq).sum())
    rhs = float((flat * grads).sum())
    assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), abs(rhs), 1e-9) + 1e-9
    # linearity and accumulation into an existing table
    g2 = orc.scatter_backward(pos, half_bits(denc), scales, T, dls, grads=grads.astype(np.float32).copy())
    assert np.allclose(g2, 2 * grads, rtol=1e-5, atol=1e-9)
    # total mass per level/feature: sum of the table gradient equals the sum of dEnc (weights sum to 1)
    per = grads.reshape(L, T, 2).sum(axis=1)
    assert np.allclose(per, dq.reshape(500, L, 2).sum(axis=0), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dims,act", [((32, 64, 16, 2), 0), ((32, 64, 8, 3), 1), ((64, 64, 64, 4), 0), ((32, 64, 16, 1), 0)])
def test_mlp_forward_against_numpy(orc, dims, act):
    i, h, o, nl = dims
    rng = np.random.default_rng(11)
    n = 257
    W, b = make_mlp(i, h, o, nl, seed=1, bias_amp=0.1)
    x = rng.normal(0, 1, size=(n, i)).astype(np.float32)
    out, acts = orc.mlp_forward(half_bits(x), dims, half_bits(W), b, out_act=act, save_acts=True)
    cur = half_vals(half_bits(x)).astype(np.float64)
    Wq = half_vals(half_bits(W)).astype(np.float64)
    wo = bo = 0
    for l, (ki, ko) in enumerate(mlp_dims(i, h, o, nl)):
        Wl = Wq[wo:wo + ki * ko].reshape(ko, ki); wo += ki * ko
        z = cur @ Wl.T + b[bo:bo + ko]; bo += ko
        if l < nl - 1:
            z = np.maximum(z, 0)
            got = half_vals(acts[l])
            assert rel_err(got, z) < 2e-3
            cur = got.astype(np.float64)           # continue from the oracle's own rounding
        else:
            if act == 1:
                z = 1.0 / (1.0 + np.exp(-z))
            assert rel_err(out, z) < 1e-5


@pytest.mark.parametrize("dims", [(32, 64, 16, 2), (32, 64, 8, 3)])
def test_mlp_backward_against_numpy(orc, dims):
    i, h, o, nl = dims
    rng = np.random.default_rng(12)
    n = 200
    W, b = make_mlp(i, h, o, nl, seed=2, bias_amp=0.05)
    x = rng.normal(0, 1, size=(n, i)).astype(np.float32)
    _, acts = orc.mlp_forward(half_bits(x), dims, half_bits(W), b, save_acts=True)
    dL = rng.normal(0, 1e-2, size=(n, o)).astype(np.float32)
    dW, db, dX = orc.mlp_backward(half_bits(dL), dims, half_bits(W), half_bits(x), acts, want_dx=True)
    Wq = half_vals(half_bits(W)).astype(np.float64)
    layers = mlp_dims(i, h, o, nl)
    offs = np.cumsum([0] + [ki * ko for ki, ko in layers])
    boffs = np.cumsum([0] + [ko for _, ko in layers])
    dz = half_vals(half_bits(dL)).astype(np.float64)
    for l in range(nl - 1, -1, -1):
        ki, ko = layers[l]
        A = (half_vals(half_bits(x)) if l == 0 else half_vals(acts[l - 1])).astype(np.float64)
        assert rel_err(dW[offs[l]:offs[l + 1]].reshape(ko, ki), dz.T @ A) < 1e-5
        assert rel_err(db[boffs[l]:boffs[l + 1]], dz.sum(axis=0)) < 1e-5
        dA = dz @ Wq[offs[l]:offs[l + 1]].reshape(ko, ki)
        dA = half_vals(half_bits(dA.astype(np.float32))).astype(np.float64)
        if l > 0:
            dz = np.where(A > 0, dA, 0.0)
        else:
            assert rel_err(half_vals(dX), dA) < 2e-3


def test_mse_loss_grad_against_numpy(orc):
    rng = np.random.default_rng(13)
    n, padded, valid = 100, 8, 3
    pred = rng.random((n, padded)).astype(np.float32)
    tgt = rng.random((n, padded)).astype(np.float32)
    for act in (0, 1):
        total, grad = orc.mse_loss_grad(pred, half_bits(tgt), valid, 128.0, out_act=act)
        diff = pred.astype(np.float64) - half_vals(half_bits(tgt))
        diff[:, valid:] = 0
        assert abs(total - (diff ** 2).sum()) < 1e-4 * (diff ** 2).sum()
        g = diff * (2.0 / (n * valid)) * 128.0
        if act:
            g = g * pred * (1 - pred)
        assert rel_err(half_vals(grad), g) < 2e-3
        assert np.all(half_vals(grad)[:, valid:] == 0)


def test_adam_rules(orc):
    rng = np.random.default_rng(14)
    cnt = 4096
    w = rng.normal(0, 0.1, cnt).astype(np.float32)
    g = rng.normal(0, 1, cnt).astype(np.float32)
    g[::3] = 0.0                                   # untouched entries
    m = rng.normal(0, 0.01, cnt).astype(np.float32)
    v = np.abs(rng.normal(0, 0.01, cnt)).astype(np.float32)
    g[5] = np.inf; m[6] = np.nan; w[9] = np.nan    # self-heal cases
    bc1, bc2 = orc.adam_bias_corrections(3, 0.9, 0.99)
    assert abs(bc1 - (1 - 0.9 ** 3)) < 1e-6 and abs(bc2 - (1 - 0.99 ** 3)) < 1e-6
    assert orc.adam_bias_corrections(10 ** 6, 0.9, 0.99) == orc.adam_bias_corrections(50000, 0.9, 0.99)

    def ref(dense):
        w2, m2, v2, g2 = w.astype(np.float64).copy(), m.astype(np.float64).copy(), v.astype(np.float64).copy(), g.astype(np.float64) / 128.0
        touched = np.ones(cnt, bool) if dense else (g != 0)
        g2 = np.where(np.isfinite(g2), g2, 0); m2 = np.where(np.isfinite(m2), m2, 0); v2 = np.where(np.isfinite(v2), v2, 0)
        w0 = np.where(np.isfinite(w2), w2, 0)
        mn = 0.9 * m2 + 0.1 * g2; vn = 0.99 * v2 + 0.01 * g2 * g2
        wn = w0 - 1e-2 * (mn / bc1) / (np.sqrt(vn / bc2) + 1e-15)
        return touched, wn, mn, vn

    # sparse rule
    ws, ms, vs, gs = w.copy(), m.copy(), v.copy(), g.copy()
    wh = half_bits(ws).copy()
    wh0 = wh.copy()
    orc.adam_hash(ws, wh, gs, ms, vs, 1e-2, 0.9, 0.99, 1e-15, bc1, bc2, 1.0 / 128.0)
    touched, wn, mn, vn = ref(False)
    assert np.all(gs == 0)
    assert np.array_equal(ws[~touched], w[~touched], equal_nan=True) and np.array_equal(ms[~touched], m[~touched], equal_nan=True)
    assert np.array_equal(wh[~touched], wh0[~touched])
    assert np.allclose(ws[touched], wn[touched], rtol=1e-5, atol=1e-8)
    assert np.allclose(ms[touched], mn[touched], rtol=1e-5, atol=1e-8) and np.allclose(vs[touched], vn[touched], rtol=1e-5, atol=1e-10)
    assert np.array_equal(wh[touched], half_bits(ws[touched]))
    assert np.all(np.isfinite(ws[touched]))
    # dense rule
    wd, md, vd = w.copy(), m.copy(), v.copy()
    whd = orc.adam_dense(wd, g, md, vd, 1e-2, 0.9, 0.99, 1e-15, bc1, bc2, 1.0 / 128.0)
    _, wn, mn, vn = ref(True)
    assert np.allclose(wd, wn, rtol=1e-5, atol=1e-8) and np.allclose(md, mn, rtol=1e-5, atol=1e-8)
    assert np.array_equal(whd, half_bits(wd)) and np.all(np.isfinite(wd))
