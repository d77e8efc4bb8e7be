"""CPU checks of the oracle's ray / march / compositing / occupancy functions: structural properties and,
for the analytic backward of compositing + distortion loss, finite differences of a float64 statement of
the loss.  No GPU needed."""
import numpy as np
import pytest

from helpers import half_vals


def sphere_bitfield(orc, res, levels, cascades, aabb=0.5, radius=0.3):
    """Level-0 bits set where the cell centre lies inside a sphere; mip pyramid built by the oracle."""
    S = orc.pyramid_cells(res, levels)
    G = res[0] * res[1] * res[2]
    bits = np.zeros(cascades * S // 8, np.uint8)
    zz, yy, xx = np.meshgrid(np.arange(res[2]), np.arange(res[1]), np.arange(res[0]), indexing="ij")
    for c in range(cascades):
        ext = 2 * aabb * (2 ** c)
        cx = ((xx + .5) / res[0] - .5) * ext; cy = ((yy + .5) / res[1] - .5) * ext; cz = ((zz + .5) / res[2] - .5) * ext
        inside = (cx ** 2 + cy ** 2 + cz ** 2 < radius ** 2).ravel()
        bits[c * S // 8: c * S // 8 + G // 8] = np.packbits(inside, bitorder="little")
    orc.build_mipmaps(bits, res, levels, cascades)
    return bits


def speckled_bitfield(orc, res, levels, cascades, p=0.02, seed=3):
    """The sphere plus stray finest-level cells set with probability p, pyramid rebuilt: empty-space skips keep
    running into isolated occupied cells, solid runs into holes' borders."""
    bits = sphere_bitfield(orc, res, levels, cascades)
    S = orc.pyramid_cells(res, levels)
    G = res[0] * res[1] * res[2]
    rng = np.random.default_rng(seed)
    for c in range(cascades):
        lvl0 = np.unpackbits(bits[c * S // 8: c * S // 8 + G // 8], bitorder="little")
        lvl0 |= (rng.random(G) < p).astype(np.uint8)
        bits[c * S // 8: c * S // 8 + G // 8] = np.packbits(lvl0, bitorder="little")
    orc.build_mipmaps(bits, res, levels, cascades)
    return bits


def camera_rays(n, radius=1.5, seed=0, jitter=0.25):
    rng = np.random.default_rng(seed)
    o = rng.normal(size=(n, 3)); o = (radius * o / np.linalg.norm(o, axis=1, keepdims=True)).astype(np.float32)
    target = rng.uniform(-jitter, jitter, size=(n, 3))
    d = target - o; d = (d / np.linalg.norm(d, axis=1, keepdims=True)).astype(np.float32)
    return o, d


def test_philox_is_uniform_and_counter_based(orc):
    u = np.stack([orc.philox_uniform4(7, i) for i in range(4096)])
    assert u.min() > 0 and u.max() <= 1
    assert abs(u.mean() - 0.5) < 0.01 and abs(u.std() - np.sqrt(1 / 12)) < 0.01
    assert np.array_equal(orc.philox_uniform4(7, 5), u[5])
    assert not np.array_equal(orc.philox_uniform4(8, 5), u[5])


def test_ray_aabb_and_contraction(orc):
    o = np.array([[0, 0, -1.5], [2, 2, 2], [0, 0, 0]], np.float32)
    d = np.array([[0, 0, 1], [0, 1, 0], [0, 0, 1]], np.float32)
    d_inv, n, f = orc.ray_aabb(o, d, [-.5] * 3, [.5] * 3, 1)
    assert np.allclose(n, [1.0, 0.0, 0.0]) and np.allclose(f, [2.0, 0.0, 0.5])
    assert d_inv[0, 2] == 1.0 and d_inv[0, 0] == np.float32(1.0) / np.float32(1e-8)
    _, n3, f3 = orc.ray_aabb(o, d, [-.5] * 3, [.5] * 3, 3)            # outermost cascade box is 4x larger
    assert np.allclose(n3[:1], [-0.0 + 0.0]) or n3[0] == 0.0
    assert np.isclose(f3[0], 3.5)
    p = orc.contract_pos(np.array([[-.5, 0, .5], [1.0, -2.0, 0.25], [1e6, 0, 0]], np.float32), [-.5] * 3, [.5] * 3)
    assert np.allclose(p[0], [0.25, 0.5, 0.75])                       # the box maps to [0.25, 0.75]
    assert np.allclose(p[1], [(2 - 1 / 2 + 2) / 4, (-(2 - 1 / 4) + 2) / 4, 0.625])
    assert np.isclose(p[2, 0], 1.0, atol=1e-6)


@pytest.mark.parametrize("cascades,spv", [(1, 1), (3, 1), (1, 2)])
def test_march_properties(orc, cascades, spv):
    res, levels = (32, 32, 32), 3
    bits = sphere_bitfield(orc, res, levels, cascades)
    o, d = camera_rays(500, seed=1)
    amin, amax = [-.5] * 3, [.5] * 3
    d_inv, nears, fars = orc.ray_aabb(o, d, amin, amax, cascades)
    cnt = orc.march_count(o, d, d_inv, nears, fars, bits, res, amin, amax, cascades, levels, spv)
    assert cnt.max() <= 1024 and cnt.sum() > 0
    off = orc.exclusive_sum(cnt)
    assert off[0] == 0 and np.array_equal(off[1:], np.cumsum(cnt)[:-1])
    t, ray, pos = orc.march_emit(o, d, d_inv, nears, fars, bits, res, amin, amax, cascades, levels, spv, off, 0, int(cnt.sum()))
    assert np.array_equal(np.bincount(ray, minlength=500).astype(np.uint32), cnt)      # emit agrees with count
    assert np.all(np.diff(ray.astype(np.int64)) >= 0)                                   # ray order
    for r in np.nonzero(cnt)[0][:50]:
        tr = t[off[r]:off[r] + cnt[r]]
        assert np.all(np.diff(tr) > 0) and tr[0] >= nears[r] and tr[-1] <= fars[r]
    # every sample lies in a set level-0 cell of cascade 0 (the sphere is inside the innermost box)
    world = o[ray] + t[:, None] * d[ray]
    cell = np.clip(np.floor((world + .5) * 32).astype(int), 0, 31)
    flat = cell[:, 2] * 1024 + cell[:, 1] * 32 + cell[:, 0]
    assert np.all((bits[flat >> 3] >> (flat & 7)) & 1)
    assert np.allclose(pos[:, :3], orc.contract_pos(world.astype(np.float32), amin, amax), atol=1e-6) and np.all(pos[:, 3] == 0)
    # an empty grid yields no samples
    assert orc.march_count(o, d, d_inv, nears, fars, np.zeros_like(bits), res, amin, amax, cascades, levels, spv).sum() == 0


def test_march_ends_on_far_rays_and_signed_zero_directions(orc):
    """8 cascades on a +-1 box reach t of several hundred, where the advance's +1e-5 is below half an ulp, and a
    direction component of -0.0 gives an exit distance of -inf on that axis: the walk must still end (the advance
    moves to the next float when its expression stalls, and the advances are bounded)."""
    res, levels, cascades = (16, 16, 16), 3, 8
    S = orc.pyramid_cells(res, levels)
    bits = np.zeros(cascades * S // 8, np.uint8)                       # empty space only: every advance is a skip
    rng = np.random.default_rng(11)
    n = 256
    o = rng.uniform(-120, 120, size=(n, 3)).astype(np.float32)
    d = rng.normal(size=(n, 3)); d = (d / np.linalg.norm(d, axis=1, keepdims=True)).astype(np.float32)
    d[:64, 0] = np.float32(-0.0); d[64:96, 1] = np.float32(0.0)        # axis-aligned planes, both zero signs
    amin, amax = [-1.0] * 3, [1.0] * 3
    d_inv, nears, fars = orc.ray_aabb(o, d, amin, amax, cascades)
    assert fars.max() > 256.0
    cnt = orc.march_count(o, d, d_inv, nears, fars, bits, res, amin, amax, cascades, levels, 1)
    assert cnt.sum() == 0
    # the same rays through a fully set grid are cut by the per-ray cap, not by the advance bound
    full = np.full_like(bits, 0xff)
    cnt = orc.march_count(o, d, d_inv, nears, fars, full, res, amin, amax, cascades, levels, 1)
    assert cnt.max() <= 1024 and cnt.sum() > 0


def test_cutoff_rule(orc):
    cnt = np.array([5, 0, 7, 3, 0, 9, 4], np.uint32)
    off = orc.exclusive_sum(cnt)
    assert orc.find_cutoff(off, cnt, 100) == 7
    assert orc.find_cutoff(off, cnt, 15) == 5            # 5+0+7+3+0 = 15 fits, the next ray (9) does not
    assert orc.find_cutoff(off, cnt, 14) == 3
    assert orc.find_cutoff(off, cnt, 4) == 0             # not even the first ray fits
    assert orc.find_cutoff(off, cnt, 9, rays_done=5) == 6
    assert orc.find_cutoff(off, cnt, 13, rays_done=5) == 7
    assert orc.find_cutoff(off, cnt, 8, rays_done=5) == 5  # nothing fits: stays at rays_done


def _loss64(t_list, logit0, cpre, target, bg, lam, bias):
    """float64 statement of the per-batch loss sum_rays [ |C - C*|^2 + lam * distortion ]."""
    total = 0.0
    k = 0
    for r, t in enumerate(t_list):
        n = len(t)
        z, c = logit0[k:k + n], 1 / (1 + np.exp(-cpre[k:k + n]))
        k += n
        tn = np.append(t[1:], t[-1] + 1e-3)
        dt = tn - t
        sig = np.exp(np.minimum(z - bias, 8.0))
        alpha = 1 - np.exp(-sig * dt)
        T = np.concatenate([[1.0], np.cumprod(1 - alpha)])
        w = alpha * T[:-1]
        C = (w[:, None] * c).sum(0) + T[-1] * bg
        total += ((C - target[r]) ** 2).sum()
        t_near = max(t[0], 1e-4); g_far = 1 - t_near / max(t[-1], t_near + 1e-4)
        inv = 1 / g_far if g_far > 1e-6 else 0.0
        s = (1 - t_near / np.maximum(t, 1e-4)) * inv; sn = (1 - t_near / np.maximum(tn, 1e-4)) * inv
        m = 0.5 * (s + sn); ds = np.maximum(sn - s, 0)
        total += lam * ((w[:, None] * w[None, :] * np.abs(m[:, None] - m[None, :])).sum() + (w * w * ds).sum() / 3)
    return total


def test_compositing_backward_matches_finite_differences(orc):
    rng = np.random.default_rng(3)
    counts = np.array([6, 1, 9, 0, 4], np.uint32)
    R, n = len(counts), int(counts.sum())
    off = orc.exclusive_sum(counts)
    t_list = [np.sort(rng.uniform(1.0, 2.0, c)) for c in counts]
    t = np.concatenate(t_list).astype(np.float32)
    t_list = [t[off[r]:off[r] + counts[r]].astype(np.float64) for r in range(R)]
    logit0 = rng.normal(2.0, 1.0, n).astype(np.float32)
    cpre = rng.normal(0, 1, (n, 3)).astype(np.float32)
    target = rng.random((R, 3)).astype(np.float32)
    bg = np.array([1.0, 0.5, 0.25], np.float32)
    lam, bias, scale = 0.1, 1.0, 128.0
    dens = np.zeros((n, 16), np.float32); dens[:, 0] = logit0
    col = np.zeros((n, 8), np.float32); col[:, :3] = 1 / (1 + np.exp(-cpre.astype(np.float64)))
    sigma = np.exp(np.minimum(logit0 - np.float32(bias), 8)).astype(np.float32)
    rgb, depth, phi, dw, wsum = orc.render_rays_distortion(R, off, counts, t, sigma, col[:, :3].copy(), target, lam, 0.0, bg)
    # forward agrees with the float64 statement and with the inference kernel's colour
    rgb_inf, _, phi_inf = orc.render_rays(R, 0, 0, off, counts, t, sigma, col[:, :3].copy(), target, bg)
    assert np.allclose(rgb, rgb_inf, atol=1e-4) and np.allclose(phi, 2 * (rgb - target), atol=1e-6)
    grad, dsig = orc.color_grad(R, counts, off, t, dens, col, phi, rgb, dw, wsum, scale, bias, R, grad_stride=8)
    grad = half_vals(grad)
    assert np.all(grad[:, 3:] == 0)
    live = [r for r in range(R) if counts[r] > 0]
    tl = [t_list[r] for r in live]
    tg = target[live].astype(np.float64)
    f0 = lambda z, c: _loss64(tl, z, c, tg, bg.astype(np.float64), lam, bias)
    z64, c64 = logit0.astype(np.float64), cpre.astype(np.float64)
    eps = 1e-5
    for i in range(n):
        zp, zm = z64.copy(), z64.copy(); zp[i] += eps; zm[i] -= eps
        num = (f0(zp, c64) - f0(zm, c64)) / (2 * eps) * scale / R
        assert abs(dsig[i] - num) <= 2e-3 * max(1.0, abs(num)), (i, dsig[i], num)
        for ch in range(3):
            cp, cm = c64.copy(), c64.copy(); cp[i, ch] += eps; cm[i, ch] -= eps
            num = (f0(z64, cp) - f0(z64, cm)) / (2 * eps) * scale / R
            assert abs(grad[i, ch] - num) <= 3e-3 * max(1.0, abs(num)), (i, ch, grad[i, ch], num)


def test_inference_compositing_terminates_early(orc):
    counts = np.array([50], np.uint32); off = np.array([0], np.uint32)
    t = np.linspace(1, 2, 50).astype(np.float32)
    sigma = np.full(50, 500.0, np.float32)
    rgb = np.tile(np.array([[0.2, 0.4, 0.6]], np.float32), (50, 1))
    out, depth, _ = orc.render_rays(1, 0, 0, off, counts, t, sigma, rgb, None, np.zeros(3, np.float32))
    assert np.allclose(out[0], [0.2, 0.4, 0.6], atol=1e-3) and depth[0] < 1.05


def test_occupancy_pipeline_properties(orc):
    res, levels, casc = (16, 16, 16), 3, 2
    G, S = 4096, orc.pyramid_cells(res, levels)
    amin, amax = [-.5] * 3, [.5] * 3
    samples = orc.sample_aabb(amin, amax, res, G, G, G, seed=11)          # every cell of cascade 1
    cells = samples[:, 3].copy().view(np.int32)
    assert np.array_equal(cells, np.arange(G, 2 * G))
    assert samples[:, :3].min() >= 0 and samples[:, :3].max() <= 1
    # cascade-1 samples outside the inner box are contracted beyond [0.25, 0.75] on at least one axis
    assert np.any((samples[:, :3] < 0.25) | (samples[:, :3] > 0.75))
    rnd = orc.sample_aabb(amin, amax, res, 1000, 2 * G, 0, seed=12)       # random cells of the whole grid
    rc = rnd[:, 3].copy().view(np.int32)
    assert rc.min() >= 0 and rc.max() < 2 * G and len(np.unique(rc)) > 800
    dens = np.zeros((G, 16), np.float32); dens[:, 0] = np.linspace(-3, 3, G)
    tmp = np.zeros(2 * G, np.float32)
    orc.update_tmp_grid(samples, dens, tmp, 1.0)
    assert np.allclose(tmp[G:], np.exp(dens[:, 0] - 1.0), rtol=1e-6) and np.all(tmp[:G] == 0)
    master = np.zeros(2 * G, np.float32); master[5] = 4.0; master[7] = -1.0
    orc.update_master_grid(tmp, master, 0.95)
    assert np.isclose(master[5], 3.8) and master[7] == -1.0 and np.allclose(master[G:], tmp[G:])
    bits = np.zeros(casc * S // 8, np.uint8)
    orc.update_occupancy_bits(bits, master, float(master.sum()), G, S, 0.01, 1.0 / 16)
    thr1 = min((0.01 / (1 / 16)) / 2, master.sum() / (2 * G))
    lvl0 = np.unpackbits(bits[S // 8: S // 8 + G // 8], bitorder="little")
    assert np.array_equal(lvl0.astype(bool), master[G:] > thr1)
    orc.build_mipmaps(bits, res, levels, casc)
    l0 = lvl0.reshape(16, 16, 16)
    l1 = np.unpackbits(bits[S // 8 + G // 8: S // 8 + G // 8 + 64], bitorder="little").reshape(8, 8, 8)
    assert np.array_equal(l1.astype(bool), l0.reshape(8, 2, 8, 2, 8, 2).max(axis=(1, 3, 5)).astype(bool))
    act = orc.extract_active_cells(bits, 2 * G, G, S)
    assert np.array_equal(act, np.nonzero(np.concatenate([np.unpackbits(bits[:G // 8], bitorder="little"), lvl0]))[0])
    occ = orc.sample_occupied(act, amin, amax, res, 500, seed=13)
    assert np.all(np.isin(occ[:, 3].copy().view(np.int32), act))
