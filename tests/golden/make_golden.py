"""Generates tests/golden/reference_vectors.npz: outputs of the REFERENCE's own CUDA code (its sources compiled where
they lie into oracle/_ref/libref3dmaker.so by oracle/build_ref.py) on small seeded inputs - reference output only.
A second file, tests/golden/device_level_scales.npz, holds what is NOT reference output: the per-level grid
resolutions as this library's set-up kernel evaluates them on the device (the reference never materialises them).

Run on a machine with a CUDA GPU, from the repository root, after the reference build exists:

    python tests/golden/make_golden.py [copy-to-directory]

The inputs are not stored: tests/test_golden_cpu.py rebuilds them from the same seeded generators (golden_inputs
below, pure numpy) and checks the CPU oracle against these vectors without a GPU.  The file stays small (a few
hundred KB): hash-table gradients are stored sparse.
"""
import ctypes
import importlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

from helpers import half_bits, make_mlp, make_positions, make_table  # noqa: E402

FIELD = dict(L=16, T=1 << 14, base=16, n=200, density=(32, 64, 16, 2), color=(32, 64, 8, 3), density_bias=1.0, loss_scale=128.0)
MARCH = dict(res=(32, 32, 32), levels=3, rays=300, batch=1 << 15, aabb=0.5)


def golden_inputs():
    """Everything the reference was fed, from seeds (numpy only)."""
    from test_oracle_nerf_cpu import camera_rays
    f = FIELD
    rng = np.random.default_rng(77)
    dirs = rng.normal(size=(f["n"], 3)).astype(np.float32)
    dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    tgt3 = rng.random((f["n"], 3), dtype=np.float32)
    field = dict(table=make_table(f["L"], f["T"], seed=0, amp=0.1), dens=make_mlp(*f["density"], seed=0, bias_amp=0.02),
                 col=make_mlp(*f["color"], seed=1, bias_amp=0.02), pos=make_positions(f["n"], 3), dirs=dirs, tgt3=tgt3)
    o, d = camera_rays(MARCH["rays"], seed=12)
    # compositing: random sorted sample distances per ray
    rng = np.random.default_rng(5)
    R = 120
    counts = rng.integers(0, 50, R).astype(np.uint32)
    counts[:4] = [0, 1, 33, 49]
    n = int(counts.sum())
    off = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    t = np.concatenate([np.sort(rng.uniform(0.5, 3.0, c)) for c in counts]).astype(np.float32)
    dens = rng.normal(1.5, 1.5, (n, 16)).astype(np.float32)
    col = rng.random((n, 3), dtype=np.float32)
    target = rng.random((R, 3), dtype=np.float32)
    comp = dict(R=R, counts=counts, off=off, t=t, dens=dens, col=col, target=target, bias=1.0, lam=0.1, scale=128.0,
                bg=np.array([1.0, 0.5, 0.25], np.float32))
    return dict(field=field, rays_o=o, rays_d=d, comp=comp)


def main():
    import torch
    from oracle import ref_cuda as ref
    import oracle as orc
    from test_oracle_nerf_cpu import speckled_bitfield
    nb = importlib.import_module("3dmaker_b200")
    nm = importlib.import_module("3dmaker_b200.nerf")
    if not ref.available():
        raise SystemExit("oracle/_ref/libref3dmaker.so is missing: run oracle/build_ref.py where the reference tree is mounted")
    lib = ref.lib()
    P, st = nb.ptr, nb.stream_ptr()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    inp = golden_inputs()
    out, aux = {}, {}
    V = lambda p, cnt, dt=np.float32: nm.view_tensor(torch, p, cnt, dt).cpu().numpy().copy()

    # ---- field forward + backward, both growth factors ----------------------------------------------------
    f, fi = FIELD, inp["field"]
    n = f["n"]
    for tag, b in (("b1447", 1.447), ("b13819", 1.3819)):
        rf = lib.ref_field_create(f["L"], f["T"], f["base"], b, 64, 2, 64, 3, n)
        lib.ref_field_load(rf, ref.hptr(np.ascontiguousarray(fi["table"].ravel())), ref.hptr(fi["dens"][0]), ref.hptr(fi["dens"][1]),
                           ref.hptr(fi["col"][0]), ref.hptr(fi["col"][1]))
        d_pos, d_dirs = dev(fi["pos"]), dev(fi["dirs"])
        d_t3 = torch.from_numpy(half_bits(fi["tgt3"]).view(np.float16)).cuda()
        lib.ref_field_forward_backward(rf, P(d_pos), P(d_dirs), P(d_t3), n, f["density_bias"], f["loss_scale"], st)
        torch.cuda.synchronize()
        out["field_%s_density_out" % tag] = V(lib.ref_field_density_out(rf), n * 16).reshape(n, 16)
        out["field_%s_color_out" % tag] = V(lib.ref_field_color_out(rf), n * 3).reshape(n, 3)
        out["field_%s_color_in" % tag] = V(lib.ref_field_color_in(rf), n * 32, np.float16).view(np.uint16).reshape(n, 32)
        g = V(lib.ref_field_hash_grads(rf), f["L"] * f["T"] * 2)
        nz = np.nonzero(g)[0].astype(np.uint32)
        out["field_%s_hash_grad_idx" % tag] = nz
        out["field_%s_hash_grad_val" % tag] = g[nz]
        for net, dims in ((0, f["density"]), (1, f["color"])):
            i, h, o, nl = dims
            for l in range(nl):
                ki, ko = (i if l == 0 else h), (o if l == nl - 1 else h)
                out["field_%s_dW_%d_%d" % (tag, net, l)] = V(lib.ref_field_layer_grads(rf, net, l, 0), ki * ko)
                out["field_%s_db_%d_%d" % (tag, net, l)] = V(lib.ref_field_layer_grads(rf, net, l, 1), ko)
        lib.ref_field_destroy(rf)
        # NOT a reference output, hence a file of its own: the per-level resolutions as evaluated on the device by this
        # library's set-up kernel with the reference's expressions.  The reference never materialises them; that the two
        # agree is what tests/test_gpu_vs_reference.py checks.  Stored so the CPU test indexes the same cells as the GPU did.
        gd = nb.grid_setup(f["L"], f["T"], f["base"], b)
        aux["%s_scales" % tag] = np.array(list(gd.scales)[:f["L"]], np.float32)
        aux["%s_scatter_scales" % tag] = np.array(list(gd.scatter_scales)[:f["L"]], np.float32)
        aux["%s_dense_level_start" % tag] = np.array([gd.dense_level_start], np.int32)

    # ---- ray / box, march, compaction ------------------------------------------------------------------------
    m = MARCH
    R, batch = m["rays"], m["batch"]
    amin = np.array([-m["aabb"]] * 3, np.float32); amax = np.array([m["aabb"]] * 3, np.float32); r3 = np.array(m["res"], np.uint32)
    d_o, d_d = dev(inp["rays_o"]), dev(inp["rays_d"])
    Z = lambda *shape, dt=torch.float32: torch.zeros(shape, dtype=dt, device="cuda")
    for tag, cascades, spv in (("c1", 1, 1), ("c2", 2, 1), ("k2", 1, 2)):
        bits = speckled_bitfield(orc, m["res"], m["levels"], cascades)
        d_bits = dev(bits)
        t = dict(dinv=Z(R, 3), near=Z(R), far=Z(R), steps=Z(R, dt=torch.int32), offs=Z(R, dt=torch.int32), t=Z(batch), ray=Z(batch, dt=torch.int32),
                 pos=Z(batch, 4), bs=Z(64, dt=torch.int32), act=Z(1, dt=torch.int32))
        lib.ref_ray_aabb(R, P(d_o), P(d_d), ref.hptr(amin), ref.hptr(amax), cascades, P(t["dinv"]), P(t["near"]), P(t["far"]), st)
        total = ctypes.c_uint(0)
        active = lib.ref_process_rays_hit_linear(R, P(d_o), P(d_d), P(t["dinv"]), P(t["near"]), P(t["far"]), P(d_bits), ref.hptr(r3), ref.hptr(amin),
                                                 ref.hptr(amax), cascades, m["levels"], spv, batch, ctypes.byref(total), P(t["act"]), P(t["steps"]),
                                                 P(t["offs"]), P(t["pos"]), P(t["ray"]), P(t["t"]), P(t["bs"]), st)
        torch.cuda.synchronize()
        nn = total.value
        assert active == R, "the golden march case is meant to fit one batch"
        out["march_%s_dinv" % tag] = t["dinv"].cpu().numpy(); out["march_%s_near" % tag] = t["near"].cpu().numpy()
        out["march_%s_far" % tag] = t["far"].cpu().numpy()
        out["march_%s_steps" % tag] = t["steps"].cpu().numpy().view(np.uint32); out["march_%s_offs" % tag] = t["offs"].cpu().numpy().view(np.uint32)
        out["march_%s_t" % tag] = t["t"].cpu().numpy()[:nn]; out["march_%s_ray" % tag] = t["ray"].cpu().numpy().view(np.uint32)[:nn]
        out["march_%s_pos" % tag] = t["pos"].cpu().numpy()[:nn, :3]

    # ---- compositing (training and inference variants) and loss gradients ------------------------------------------
    c = inp["comp"]
    R, n = c["R"], len(c["t"])
    sigma = np.exp(np.minimum(c["dens"][:, 0] - np.float32(c["bias"]), 8)).astype(np.float32)
    d_off, d_cnt, d_t, d_sig, d_col, d_tgt, d_dens = (dev(x) for x in (c["off"].view(np.int32), c["counts"].view(np.int32), c["t"], sigma, c["col"],
                                                                        c["target"], c["dens"]))
    r = dict(rgb=Z(R, 3), depth=Z(R), phi=Z(R, 3), dw=Z(n), ws=Z(R), grad=torch.zeros((n, 3), dtype=torch.float16, device="cuda"), dsig=Z(n))
    lib.ref_volume_rendering(R, P(d_off), P(d_cnt), P(d_t), P(d_sig), P(d_col), P(d_tgt), P(r["rgb"]), P(r["depth"]), P(r["phi"]), P(r["dw"]), P(r["ws"]),
                             c["lam"], 0.0, ref.hptr(c["bg"]), 0, 0, st)
    lib.ref_color_grad(R, P(d_cnt), P(d_off), P(d_t), P(d_dens), P(d_col), P(r["phi"]), P(r["rgb"]), P(r["dw"]), P(r["ws"]), P(r["grad"]), P(r["dsig"]),
                       c["scale"], c["bias"], R, st)
    rgb_i, dep_i = Z(R, 3), Z(R)
    lib.ref_volume_rendering(R, P(d_off), P(d_cnt), P(d_t), P(d_sig), P(d_col), None, P(rgb_i), P(dep_i), None, None, None, 0.0, 0.0, ref.hptr(c["bg"]),
                             0, 0, st)
    torch.cuda.synchronize()
    for k in ("rgb", "depth", "phi", "dw", "ws", "dsig"):
        out["comp_" + k] = r[k].cpu().numpy()
    out["comp_grad"] = r["grad"].cpu().numpy().view(np.uint16)
    out["comp_infer_rgb"] = rgb_i.cpu().numpy()

    # ---- occupancy sample jitter (cuRAND Philox) ---------------------------------------------------------------
    res16 = np.array([16, 16, 16], np.uint32)
    G = 16 ** 3
    s = Z(G, 4)
    lib.ref_sample_aabb(P(s), ref.hptr(amin), ref.hptr(amax), ref.hptr(res16), G, G, 0, 5, st)
    torch.cuda.synchronize()
    out["occ_samples"] = s.cpu().numpy()

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    aux_path = os.path.join(HERE, "device_level_scales.npz")
    np.savez_compressed(aux_path, **aux)
    print("wrote %s (%d arrays, %.0f KB) and %s" % (path, len(out), os.path.getsize(path) / 1024, aux_path))
    if len(sys.argv) > 1:                      # optional second copy, e.g. into a folder that is collected from the GPU machine
        import shutil
        os.makedirs(sys.argv[1], exist_ok=True)
        shutil.copy(path, os.path.join(sys.argv[1], "reference_vectors.npz"))
        shutil.copy(aux_path, os.path.join(sys.argv[1], "device_level_scales.npz"))


if __name__ == "__main__":
    main()
