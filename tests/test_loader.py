"""Ray batches from an image set: the oracle's restatement of the reference's streaming fetch kernel checked against
independent numpy statements of its rules (CPU), and nb_fetch_ray_chunk against the oracle (GPU)."""
import ctypes

import numpy as np
import pytest


def _image_set(n_img=24, w=20, h=12, seed=0):
    rng = np.random.default_rng(seed)
    imgs = rng.integers(0, 256, size=(n_img, h, w, 4), dtype=np.uint8)
    imgs[:, :, :, 3] = rng.choice([0, 128, 255], size=(n_img, h, w))
    T = np.zeros((n_img, 16), np.float32)
    for i in range(n_img):
        q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
        m = np.eye(4, dtype=np.float32); m[:3, :3] = q; m[:3, 3] = rng.normal(size=3)
        T[i] = m.ravel()
    return imgs, T


def _pcg_np(v):
    v = np.uint64(v) & np.uint64(0xffffffff)
    state = (v * np.uint64(747796405) + np.uint64(2891336453)) & np.uint64(0xffffffff)
    word = (((state >> ((state >> np.uint64(28)) + np.uint64(4))) ^ state) * np.uint64(277803737)) & np.uint64(0xffffffff)
    return int(((word >> np.uint64(22)) ^ word) & np.uint64(0xffffffff))


def test_pcg_hash_matches_an_independent_statement(orc):
    for v in (0, 1, 2, 12345, 0xffffffff, 0x9E3779B9, 747796405):
        assert orc.pcg_hash(v) == _pcg_np(v)
    vals = np.array([orc.pcg_hash(i) for i in range(4096)], np.uint64)
    assert len(np.unique(vals)) == 4096 and abs(float(vals.mean()) / 2 ** 32 - 0.5) < 0.02


def test_sequential_fetch_walks_the_pixels_in_order(orc):
    imgs, T = _image_set()
    n, h, w, _ = imgs.shape
    bg = (0.25, 0.5, 0.75)
    off, size = 3 * h * w - 5, 40                          # crosses an image boundary
    ro, rd, rgb, dep, sig, pick = orc.fetch_ray_chunk(off, size, 99, 0, w, h, 30.0, T, imgs, bg)
    assert np.array_equal(pick, np.arange(off, off + size, dtype=np.uint32))
    flat = imgs.reshape(-1, 4).astype(np.float32) / 255.0
    a = flat[pick, 3:4]
    assert np.allclose(rgb, flat[pick, :3] * a + np.array(bg, np.float32) * (1 - a), atol=1e-6)
    img, pix = pick // (h * w), pick % (h * w)
    px, py = (pix % w).astype(np.float32), (pix // w).astype(np.float32)
    d = np.stack([(px - w * 0.5) / 30.0, -(py - h * 0.5) / 30.0, -np.ones_like(px)], axis=1)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    R = T[img].reshape(-1, 4, 4)
    assert np.allclose(rd, np.einsum("nij,nj->ni", R[:, :3, :3], d), atol=1e-6) and np.allclose(ro, R[:, :3, 3])
    assert np.all(dep == -1) and np.all(sig == -1)


@pytest.mark.parametrize("holdout", [0, 2, 8])
def test_random_fetch_respects_the_hold_out(orc, holdout):
    imgs, T = _image_set()
    n, h, w, _ = imgs.shape
    size = 20000
    _, _, _, _, _, pick = orc.fetch_ray_chunk(100, size, 7, 1, w, h, 30.0, T, imgs, (1, 1, 1), holdout_every=holdout)
    img = pick // (h * w)
    if holdout:
        assert np.all(img % holdout != 0)
        assert set(np.unique(img)) == {i for i in range(n) if i % holdout != 0}
    else:
        assert len(np.unique(img)) == n
        assert np.array_equal(pick, np.array([_pcg_np(100 + i + 7) % (n * h * w) for i in range(64)] + list(pick[64:]), np.uint32))
    counts = np.bincount(img, minlength=n)[[i for i in range(n) if not holdout or i % holdout]]
    assert counts.min() > 0.7 * counts.mean()


def test_depth_prior_slots(orc):
    imgs, T = _image_set()
    n, h, w, _ = imgs.shape
    rng = np.random.default_rng(3)
    nrec = 50
    rec = (rng.integers(0, n, nrec).astype(np.int32), rng.uniform(0, 2 * w, nrec).astype(np.float32), rng.uniform(0, 2 * h, nrec).astype(np.float32),
           rng.uniform(1, 3, nrec).astype(np.float32), rng.uniform(0.01, 0.1, nrec).astype(np.float32))
    size = 8000
    ro, rd, rgb, dep, sig, pick = orc.fetch_ray_chunk(0, size, 11, 1, w, h, 30.0, T, imgs, (1, 1, 1), holdout_every=8, records=rec,
                                                      dense_fraction=0.25, prior_wh=(2 * w, 2 * h))
    dense = dep >= 0
    assert 0.2 < dense.mean() < 0.3
    assert np.all(np.isin(dep[dense], rec[3])) and np.all(sig[dense] > 0) and np.all(sig[~dense] == -1)
    assert np.all((pick[dense] // (h * w)) % 8 != 0)       # priors on held-out images are skipped
    # sequential mode never takes prior slots
    _, _, _, dep2, _, _ = orc.fetch_ray_chunk(0, 100, 11, 0, w, h, 30.0, T, imgs, (1, 1, 1), records=rec, dense_fraction=0.9)
    assert np.all(dep2 == -1)


@pytest.mark.gpu
@pytest.mark.parametrize("randomize,holdout,dense", [(0, 0, 0.0), (1, 0, 0.0), (1, 8, 0.0), (1, 8, 0.3)])
def test_gpu_fetch_matches_the_oracle(cuda, nb, orc, randomize, holdout, dense):
    torch = cuda
    imgs, T = _image_set(n_img=40, w=64, h=48, seed=5)
    n, h, w, _ = imgs.shape
    rng = np.random.default_rng(9)
    nrec = 200
    rec = (rng.integers(0, n, nrec).astype(np.int32), rng.uniform(0, w, nrec).astype(np.float32), rng.uniform(0, h, nrec).astype(np.float32),
           rng.uniform(1, 3, nrec).astype(np.float32), rng.uniform(0.01, 0.1, nrec).astype(np.float32))
    d_imgs, d_T = torch.from_numpy(imgs).cuda(), torch.from_numpy(T).cuda()
    d_rec = [torch.from_numpy(a).cuda() for a in rec]
    s = nb.ImageSet()
    s.d_images_rgba, s.d_transforms = d_imgs.data_ptr(), d_T.data_ptr()
    s.num_images, s.width, s.height, s.focal = n, w, h, 55.0
    s.d_rec_frame, s.d_rec_u, s.d_rec_v, s.d_rec_depth, s.d_rec_sigma = (t.data_ptr() for t in d_rec)
    s.num_records, s.dense_fraction, s.prior_width, s.prior_height = (nrec if dense > 0 else 0), dense, w, h
    size, off, seed = 50000, 1234, 42
    ro, rd, rgb = (torch.zeros((size, 3), device="cuda") for _ in range(3))
    dep, sig = torch.zeros(size, device="cuda"), torch.zeros(size, device="cuda")
    bg = (ctypes.c_float * 3)(0.1, 0.6, 0.9)
    nb.check(nb.load().nb_fetch_ray_chunk(ctypes.byref(s), off, size, seed, randomize, bg, holdout, nb.ptr(ro), nb.ptr(rd), nb.ptr(rgb), nb.ptr(dep),
                                          nb.ptr(sig), nb.stream_ptr()), "nb_fetch_ray_chunk")
    torch.cuda.synchronize()
    o_ro, o_rd, o_rgb, o_dep, o_sig, _ = orc.fetch_ray_chunk(off, size, seed, randomize, w, h, 55.0, T, imgs, (0.1, 0.6, 0.9), holdout_every=holdout,
                                                             records=rec if dense > 0 else None, dense_fraction=dense, prior_wh=(w, h))
    assert np.array_equal(ro.cpu().numpy(), o_ro)                             # origins are copies: the same image was picked
    assert np.array_equal(dep.cpu().numpy(), o_dep) and np.array_equal(sig.cpu().numpy(), o_sig)
    assert np.allclose(rgb.cpu().numpy(), o_rgb, atol=2e-6)                   # same pixel, division by 255 approximated on the GPU
    assert np.allclose(rd.cpu().numpy(), o_rd, atol=2e-6)
