"""The reference's own extern "C" launcher names exported by libnerf_b200.so (3dmaker_b200/host/ref_launchers.cu): each is
called with the reference's argument list - option structs, device arrays of per-layer device pointers, uint3 / float3
by value - and compared with the arena entry point it forwards to, or with the reference's launcher of the same name
(oracle/_ref build) where the ray march and volume rendering are concerned."""
import ctypes
import importlib

import numpy as np
import pytest

from helpers import Uploader, dev_half_bits, half_bits, make_mlp, mlp_dims, rel_err
from test_oracle_nerf_cpu import camera_rays, speckled_bitfield

pytestmark = pytest.mark.gpu

V, I, F, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_uint


class MLPOption(ctypes.Structure):
    _fields_ = [("inputDim", I), ("hiddenDim", I), ("outputDim", I), ("numLayers", I), ("activationType", I), ("outputActivation", I)]


class MLPGridOptions(ctypes.Structure):
    _fields_ = [("vectorDim", I), ("hiddenDim", I), ("outputDim", I), ("numLayers", I), ("activationType", I), ("tableSize", I), ("numLevels", I),
                ("b", F), ("lowestSize", I), ("featuresLevel", I)]


class uint3(ctypes.Structure):
    _fields_ = [("x", U), ("y", U), ("z", U)]


class float3(ctypes.Structure):
    _fields_ = [("x", F), ("y", F), ("z", F)]


def _pointer_array(torch, tensors):
    """Device array of the tensors' device pointers (what the reference's classes keep per network)."""
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def _layers(torch, flat, dims, kind):
    """Separate device tensors per layer from a flat host array (weights [out][in] or biases [out])."""
    out, at = [], 0
    for ki, ko in dims:
        cnt = ki * ko if kind == "w" else ko
        out.append(torch.from_numpy(np.ascontiguousarray(flat[at:at + cnt])).cuda())
        at += cnt
    return out


def test_plain_network_launchers_take_pointer_arrays(cuda, nb):
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    n, dims = 3000, mlp_dims(32, 64, 8, 3)
    W, B = make_mlp(32, 64, 8, 3, seed=7, bias_amp=0.05)
    opt = MLPOption(32, 64, 8, 3, 0, 1)
    desc = nb.mlp_desc(32, 64, 8, 3, 1)
    w_h = [t.half() for t in _layers(torch, W, dims, "w")]
    b_f = _layers(torch, B, dims, "b")
    wa, ba = _pointer_array(torch, w_h), _pointer_array(torch, b_f)
    x = torch.from_numpy(np.random.default_rng(1).normal(0, 0.5, (n, 32)).astype(np.float16)).cuda()
    got, want = torch.zeros((n, 8), device="cuda"), torch.zeros((n, 8), device="cuda")
    lib.launchNetworkFusionKernel.restype = None
    lib.launchNetworkFusionKernel.argtypes = [ctypes.POINTER(MLPOption), V, V, V, V, I, V]
    lib.launchNetworkFusionKernel(ctypes.byref(opt), P(x), P(wa), P(ba), P(got), n, st)
    flat_w = torch.cat([t.reshape(-1) for t in w_h]); flat_b = torch.cat(b_f)
    nb.check(lib.nb_mlp_forward(ctypes.byref(desc), P(x), P(flat_w), P(flat_b), n, P(want), None, st), "nb_mlp_forward")
    torch.cuda.synchronize()
    assert torch.equal(got, want) and float(want.abs().sum().item()) > 0
    # ---- optimizers and zero-grad over the same arrays ---------------------------------------------------------
    rng = np.random.default_rng(2)
    master = _layers(torch, W, dims, "w"); grads = [torch.from_numpy(rng.normal(0, 5, t.numel()).astype(np.float32)).cuda() for t in master]
    m = [torch.zeros_like(t) for t in master]; v = [torch.zeros_like(t) for t in master]
    fwd = [torch.zeros(t.numel(), dtype=torch.float16, device="cuda") for t in master]
    ref_w = [t.clone() for t in master]; ref_g = [t.clone() for t in grads]; ref_m = [torch.zeros_like(t) for t in master]
    ref_v = [torch.zeros_like(t) for t in master]; ref_h = [torch.zeros_like(t) for t in fwd]
    arrays = [_pointer_array(torch, a) for a in (master, fwd, grads, m, v)]
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0)
    lib.launchAdamWeightsOptim.restype = None
    lib.launchAdamWeightsOptim.argtypes = [ctypes.POINTER(MLPOption), V, V, V, V, V] + [F] * 7 + [V]
    lib.launchAdamWeightsOptim(ctypes.byref(opt), *[P(a) for a in arrays], *hyper, st)
    for l in range(3):
        nb.check(lib.nb_adam_step(P(ref_w[l]), P(ref_h[l]), P(ref_g[l]), P(ref_m[l]), P(ref_v[l]), 0, ref_w[l].numel(), *hyper, 0, st), "nb_adam_step")
    torch.cuda.synchronize()
    for l in range(3):
        assert torch.equal(master[l], ref_w[l]) and torch.equal(fwd[l], ref_h[l]) and torch.equal(m[l], ref_m[l]) and torch.equal(v[l], ref_v[l])
        assert torch.equal(grads[l], ref_g[l]) and float(grads[l].abs().sum().item()) > 0        # the dense rule leaves the gradient
    bias = _layers(torch, B, dims, "b"); bg = [torch.ones_like(t) for t in bias]; bm = [torch.zeros_like(t) for t in bias]; bv = [torch.zeros_like(t) for t in bias]
    before = [t.clone() for t in bias]
    lib.launchAdamBiasOptim.restype = None
    lib.launchAdamBiasOptim.argtypes = [ctypes.POINTER(MLPOption), V, V, V, V] + [F] * 7 + [V]
    bias_arrays = [_pointer_array(torch, a) for a in (bias, bg, bm, bv)]     # kept alive until the launches have run
    lib.launchAdamBiasOptim(ctypes.byref(opt), *[P(a) for a in bias_arrays], *hyper, st)
    lib.launchZeroGradients.restype = None
    lib.launchZeroGradients.argtypes = [ctypes.POINTER(MLPOption), V, V, V]
    lib.launchZeroGradients(ctypes.byref(opt), P(arrays[2]), P(bias_arrays[1]), st)
    torch.cuda.synchronize()
    assert all(not torch.equal(a, b) for a, b in zip(bias, before))
    assert all(float(g.abs().sum().item()) == 0.0 for g in grads + bg)


def test_loss_and_hash_optimizer_launchers(cuda, nb):
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    n = 5000
    rng = np.random.default_rng(3)
    pred = torch.from_numpy(rng.random((n, 8), dtype=np.float32)).cuda()
    tgt = torch.from_numpy(rng.random((n, 8), dtype=np.float32).astype(np.float16)).cuda()
    ga, gb = torch.zeros((n, 8), dtype=torch.float16, device="cuda"), torch.zeros((n, 8), dtype=torch.float16, device="cuda")
    la, lb = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    lib.launchMSELossGrad.restype = None
    lib.launchMSELossGrad.argtypes = [V, V, V, V, I, I, I, F, V, I]
    lib.launchMSELossGrad(P(pred), P(tgt), P(ga), P(la), n, 8, 3, 128.0, st, 1)
    nb.check(lib.nb_mse_loss_grad(P(pred), P(tgt), P(gb), P(lb), n, 8, 3, 128.0, 1, st), "nb_mse_loss_grad")
    torch.cuda.synchronize()
    assert torch.equal(ga, gb) and abs(la.item() - lb.item()) <= 1e-5 * lb.item() and lb.item() > 0
    opt = MLPGridOptions(4, 64, 16, 2, 0, 1 << 12, 16, 1.447, 16, 2)
    count = 16 * (1 << 12) * 2
    w = torch.from_numpy(rng.uniform(-0.1, 0.1, count).astype(np.float32)).cuda(); g = torch.from_numpy((rng.normal(0, 3, count) * (rng.random(count) < 0.4)).astype(np.float32)).cuda()
    sets = []
    for _ in range(2):
        sets.append([w.clone(), torch.zeros(count, dtype=torch.float16, device="cuda"), g.clone(), torch.zeros_like(w), torch.zeros_like(w)])
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0)
    lib.launchAdamHashGridOptim.restype = None
    lib.launchAdamHashGridOptim.argtypes = [ctypes.POINTER(MLPGridOptions), V, V, V, V, V] + [F] * 7 + [V]
    lib.launchAdamHashGridOptim(ctypes.byref(opt), *[P(t) for t in sets[0]], *hyper, st)
    nb.check(lib.nb_adam_step(*[P(t) for t in sets[1]], count, count, *hyper, 0, st), "nb_adam_step")
    torch.cuda.synchronize()
    for a, b in zip(sets[0], sets[1]):
        assert torch.equal(a, b)
    assert float(sets[0][2].abs().sum().item()) == 0.0 and not torch.equal(sets[0][0], w)      # gradient consumed, parameters moved


def test_grid_network_inference_launcher(cuda, nb):
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    from helpers import make_positions, make_table
    L, T, n = 16, 1 << 14, 4000
    opt = MLPGridOptions(4, 64, 16, 2, 0, T, L, 1.447, 16, 2)
    dims = mlp_dims(32, 64, 16, 2)
    W, B = make_mlp(32, 64, 16, 2, seed=9, bias_amp=0.05)
    w_h = [t.half() for t in _layers(torch, W, dims, "w")]; b_f = _layers(torch, B, dims, "b")
    table = torch.from_numpy(make_table(L, T, seed=1, amp=0.3)).cuda().half()
    pos = torch.from_numpy(make_positions(n, 5)).cuda()
    got, want = torch.zeros((n, 16), device="cuda"), torch.zeros((n, 16), device="cuda")
    lib.launchNetworkFusionHashTableKernel.restype = None
    lib.launchNetworkFusionHashTableKernel.argtypes = [ctypes.POINTER(MLPGridOptions), V, V, V, V, V, I, V]
    wa, ba = _pointer_array(torch, w_h), _pointer_array(torch, b_f)
    lib.launchNetworkFusionHashTableKernel(ctypes.byref(opt), P(table), P(pos), P(wa), P(ba), P(got), n, st)
    grid = nb.grid_setup(L, T, 16, 1.447)
    desc = nb.mlp_desc(32, 64, 16, 2, 0)
    flat_w = torch.cat([t.reshape(-1) for t in w_h]); flat_b = torch.cat(b_f)
    nb.check(lib.nb_grid_mlp_forward(ctypes.byref(grid), ctypes.byref(desc), P(pos), P(table), P(flat_w), P(flat_b), n, P(want), None, None, st))
    torch.cuda.synchronize()
    assert torch.equal(got, want) and float(want.abs().sum().item()) > 0


def test_ray_march_and_volume_rendering_launchers_against_the_reference(cuda, nb, orc):
    """processRaysHitLinear and launchVolumeRendering under their reference names, next to the reference's own functions
    of the same names: counts, offsets, ray ids, distances and positions bit for bit; composited colour to 1e-5."""
    from oracle import ref_cuda
    if not ref_cuda.available():
        pytest.skip("reference CUDA build (oracle/_ref) not present")
    ref = ref_cuda
    torch = cuda
    up = Uploader(torch, nb)
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    res, levels, cascades, spv, R, batch = (64, 64, 64), 3, 2, 1, 20000, 1 << 17
    bits = speckled_bitfield(orc, res, levels, cascades)
    o, d = camera_rays(R, seed=11)
    d_o, d_d, d_bits = up.f(o), up.f(d), torch.from_numpy(bits).cuda()
    i32, f32 = torch.int32, torch.float32
    Z = lambda *shape, dt=f32: torch.zeros(shape, dtype=dt, device="cuda")
    sc = nb.scene_desc(res, [-.5] * 3, [.5] * 3, cascades, levels, spv)
    dinv, near, far = Z(R, 3), Z(R), Z(R)
    nb.check(lib.nb_ray_aabb(ctypes.byref(sc), d_o, d_d, R, P(dinv), P(near), P(far), st))
    mine = dict(steps=Z(R, dt=i32), offs=Z(R, dt=i32), t=Z(batch), ray=Z(batch, dt=i32), pos=Z(batch, 4), bs=Z(64, dt=i32), act=Z(1, dt=i32))
    theirs = dict(steps=Z(R, dt=i32), offs=Z(R, dt=i32), t=Z(batch), ray=Z(batch, dt=i32), pos=Z(batch, 4), bs=Z(64, dt=i32), act=Z(1, dt=i32))
    lib.processRaysHitLinear.restype = I
    lib.processRaysHitLinear.argtypes = [U, V, V, V, V, V, V, uint3, float3, float3, I, I, I, I, ctypes.POINTER(U), V, V, V, V, V, V, V, V]
    total = U(0)
    active = lib.processRaysHitLinear(R, d_o, d_d, P(dinv), P(near), P(far), P(d_bits), uint3(*res), float3(-.5, -.5, -.5), float3(.5, .5, .5), cascades,
                                      levels, spv, batch, ctypes.byref(total), P(mine["act"]), P(mine["steps"]), P(mine["offs"]), P(mine["pos"]),
                                      P(mine["ray"]), P(mine["t"]), P(mine["bs"]), st)
    amin = np.array([-.5] * 3, np.float32); amax = np.array([.5] * 3, np.float32); r3 = np.array(res, np.uint32)
    r_total = U(0)
    r_active = ref.lib().ref_process_rays_hit_linear(R, d_o, d_d, P(dinv), P(near), P(far), P(d_bits), ref.hptr(r3), ref.hptr(amin), ref.hptr(amax),
                                                     cascades, levels, spv, batch, ctypes.byref(r_total), P(theirs["act"]), P(theirs["steps"]),
                                                     P(theirs["offs"]), P(theirs["pos"]), P(theirs["ray"]), P(theirs["t"]), P(theirs["bs"]), st)
    torch.cuda.synchronize()
    assert active == r_active and total.value == r_total.value and 0 < active < R
    assert int(mine["act"].item()) == active
    nn = total.value
    assert torch.equal(mine["steps"], theirs["steps"]) and torch.equal(mine["offs"][:active], theirs["offs"][:active])
    assert torch.equal(mine["ray"][:nn], theirs["ray"][:nn]) and torch.equal(mine["t"][:nn], theirs["t"][:nn])
    assert torch.equal(mine["pos"][:nn, :3], theirs["pos"][:nn, :3])
    # ---- volume rendering on those samples, both variants ----------------------------------------------------------
    rng = np.random.default_rng(4)
    sigma = torch.from_numpy(rng.uniform(0, 30, nn).astype(np.float32)).cuda()
    rgb3 = torch.from_numpy(rng.random((nn, 3), dtype=np.float32)).cuda()
    tgt = torch.from_numpy(rng.random((active, 3), dtype=np.float32)).cuda()
    bgn = np.array([1.0, 0.5, 0.25], np.float32)
    lib.launchVolumeRendering.restype = None
    lib.launchVolumeRendering.argtypes = [U, V, V, V, V, V, V, V, V, V, V, V, V, V, F, F, float3, U, U, V]
    for train in (False, True):
        a = dict(rgb=Z(active, 3), depth=Z(active), phi=Z(active, 3), dw=Z(nn), ws=Z(active))
        b = dict(rgb=Z(active, 3), depth=Z(active), phi=Z(active, 3), dw=Z(nn), ws=Z(active))
        lib.launchVolumeRendering(active, P(mine["offs"]), P(mine["steps"]), P(mine["t"]), P(sigma), None, None, P(rgb3), P(tgt), P(a["rgb"]),
                                  P(a["depth"]), P(a["phi"]), P(a["dw"]) if train else None, P(a["ws"]) if train else None, 0.1, 0.0,
                                  float3(*bgn), 0, 0, st)
        ref.lib().ref_volume_rendering(active, P(mine["offs"]), P(mine["steps"]), P(mine["t"]), P(sigma), P(rgb3), P(tgt), P(b["rgb"]), P(b["depth"]),
                                       P(b["phi"]), P(b["dw"]) if train else None, P(b["ws"]) if train else None, 0.1, 0.0, ref.hptr(bgn), 0, 0, st)
        torch.cuda.synchronize()
        assert (a["rgb"] - b["rgb"]).abs().max().item() <= 1e-5 and (a["phi"] - b["phi"]).abs().max().item() <= 2e-5
        if train:
            assert rel_err(a["dw"].cpu().numpy(), b["dw"].cpu().numpy()) <= 1e-4 and rel_err(a["ws"].cpu().numpy(), b["ws"].cpu().numpy()) <= 1e-4
