"""Generates tests/golden/psnr_runs.json: PSNR of this engine and of the reference's InstantNerf (oracle/_ref build)
after a fixed number of optimizer steps on the analytic soft-sphere scene, several paired runs.

    python tests/golden/make_psnr_runs.py [--runs 16] [--steps 2000] [--schedule cosine|constant] [--out DIR]

Protocol (the single-GPU training configuration of the benchmark: 100 cameras 800x800, 128^3 occupancy grid with one
cascade, T = 2^19, growth 1.3819, batch 2^18 samples, 65536-ray chunks, Adam beta = (0.9, 0.99), eps 1e-15, distortion
weight 0.1, loss scale 128, white background; learning rate 1e-2 annealed to 1e-3 over the run by the half cosine of
the reference's own trainer, INerfTrainer::currentLR, NerfTrainer.cu:131-135, set before every call - or held at 1e-2
with --schedule constant, where either engine ends anywhere within several dB): run k draws its training rays from seeds
10000 k + call index, the SAME rays go to both engines call by call, both start from the parameters their
constructors draw from std::mt19937(42) (identical, checked), training stops at the first call boundary at or past
`steps` optimizer steps, and the PSNR is the mean over four held-out 200x200 views against the analytic ground truth.
Needs a GPU and the reference build.  tests/test_psnr_fixture_cpu.py reads the file without a GPU."""
import argparse
import ctypes
import importlib
import json
import math
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

VIEWS = ((33.0, 20.0), (117.0, 20.0), (250.0, -30.0), (190.0, 45.0))
OPTIONS = dict(grid_resolution=(128,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=4, hash_table_size=1 << 19,
               growth_factor=1.3819, color_hidden_dim=64, color_num_layers=3, batch_size=1 << 18, render_batch_size=1 << 18,
               ray_chunk_size=1 << 16, lambda_dist=0.1, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
               loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--runs", type=int, default=16)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--lambda-dist", type=float, default=OPTIONS["lambda_dist"])
    ap.add_argument("--schedule", default="cosine", choices=["cosine", "constant"])
    ap.add_argument("--name", default="psnr_runs.json", help="file name of the fixture")
    ap.add_argument("--out", default=None, help="also copy the file into this directory")
    args = ap.parse_args()
    import torch
    from oracle import ref_cuda as ref
    nb = importlib.import_module("3dmaker_b200")
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    if not ref.available():
        raise SystemExit("oracle/_ref/libref3dmaker.so is missing: run oracle/build_ref.py where the reference tree is mounted")
    lib, st = ref.lib(), nb.stream_ptr()
    opts = nm.default_options(**dict(OPTIONS, lambda_dist=args.lambda_dist))
    scene, poses, bg = syn.SoftSphereScene(), syn.sphere_cameras(100), (1.0, 1.0, 1.0)
    R = 1 << 16
    depth = torch.full((R,), -1.0, device="cuda"); sig = torch.ones(R, device="cuda")
    views = []
    for az, el in VIEWS:
        o, d = syn.frame_rays(torch, syn.orbit_c2w(az, el, 1.5), 200, 200, 50.0)
        views.append((o, d, syn.ground_truth(torch, scene, o, d, bg)))
    runs = []
    t_start = time.time()
    for k in range(args.runs):
        eng = nm.InstantNerf(torch, opts)
        rh = lib.ref_nerf_create(ctypes.byref(opts), 0)
        ref_steps, call = 0, 0

        def lr_at(step):
            if args.schedule == "constant":
                return 1e-2
            x = min(step / float(args.steps), 1.0)
            return 1e-3 + 0.5 * (1e-2 - 1e-3) * (1.0 + math.cos(math.pi * x))

        while eng.steps.value < args.steps or ref_steps < args.steps:
            o, d = syn.random_training_rays(torch, poses, R, 800, 800, 50.0, seed=10000 * k + call)
            tgt = syn.ground_truth(torch, scene, o, d, bg)
            if eng.steps.value < args.steps:
                eng.set_learning_rate(lr_at(eng.steps.value))
                eng.train_rays(o, d, tgt)
            if ref_steps < args.steps:
                lib.ref_nerf_set_learning_rate(rh, lr_at(ref_steps))
                ref_steps += lib.ref_nerf_train(rh, nb.ptr(o), nb.ptr(d), nb.ptr(depth), nb.ptr(sig), nb.ptr(tgt), R, None, None, st)
            call += 1
        torch.cuda.synchronize()
        ours, theirs = [], []
        for o, d, gt in views:
            a = torch.zeros_like(gt); b = torch.zeros_like(gt)
            eng.render(o, d, a)
            lib.ref_nerf_render(rh, nb.ptr(o), nb.ptr(d), o.shape[0], nb.ptr(b), st)
            torch.cuda.synchronize()
            ours.append(syn.psnr(torch, a, gt)); theirs.append(syn.psnr(torch, b, gt))
        runs.append({"run": k, "ours_db": float(np.mean(ours)), "reference_db": float(np.mean(theirs)), "ours_steps": int(eng.steps.value),
                     "reference_steps": int(ref_steps), "calls": call})
        print("run %2d: ours %.2f dB (%d steps), reference %.2f dB (%d steps)  [%.0f s]" % (k, runs[-1]["ours_db"], eng.steps.value,
                                                                                            runs[-1]["reference_db"], ref_steps, time.time() - t_start),
              flush=True)
        eng.close()
        lib.ref_nerf_destroy(rh)
    doc = {"protocol": {"steps": args.steps, "schedule": args.schedule, "views": list(VIEWS), "view_size": [200, 200], "rays_per_call": R,
                        "options": {k: (list(v) if isinstance(v, tuple) else v) for k, v in dict(OPTIONS, lambda_dist=args.lambda_dist).items()},
                        "device": torch.cuda.get_device_name(0)},
           "runs": runs}
    path = os.path.join(HERE, args.name)
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)
    if args.out:
        os.makedirs(args.out, exist_ok=True)
        with open(os.path.join(args.out, args.name), "w") as f:
            json.dump(doc, f, indent=1)
    d = np.array([r["ours_db"] - r["reference_db"] for r in runs])
    print("paired difference ours - reference: mean %.3f dB, sd %.3f, n %d" % (d.mean(), d.std(ddof=1) if len(d) > 1 else 0.0, len(d)))


if __name__ == "__main__":
    main()
