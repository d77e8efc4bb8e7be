#!/usr/bin/env python
"""Benchmark of the NeRF field-training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = hash-grid encode + density MLP + SH + colour MLP forward, MSE loss, both MLPs backward, gradient
scatter and the fused Adam update, on one batch of 2^20 synthetic samples per GPU (grid L=16, F=2, T=2^19,
base 16, growth 1.447; density 32->64->16, colour 32->64->64->3(pad 8), fp16 weights/activations with fp32
accumulation).  Prints ONE JSON line (rank 0).  Under torchrun each rank trains on its own batch and the
gradient arena is all-reduced with NCCL before Adam (weak scaling).
"""
import argparse
import importlib
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

BATCH = 1 << 20
L, T, BASE, GROWTH = 16, 1 << 19, 16, 1.447
DENSITY = (32, 64, 16, 2)
COLOR = (32, 64, 8, 3)
HYPER = dict(lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-15, loss_scale=128.0)
METRIC = "train samples/s (encode+MLP fwd/bwd+Adam)"
WORKLOAD = "cfg2+encode+Adam: 2^20 samples/GPU, L16 F2 T2^19 b1.447, density 32-64-16, colour 32-64-64-3, MSE, Adam"
L2_NOTE = "inputs and activations of one step (>1 GB) exceed the 126 MB L2; two input batches alternate"


def common_config(world):
    """The `config` object of the line: identical in both arms (what ran it goes under `notes`)."""
    return {"workload": WORKLOAD, "per_gpu_batch": BATCH, "l2": L2_NOTE, "parallelism": "dp%d" % world}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_batch(n, seed):
    rng = np.random.default_rng(seed)
    pos = np.zeros((n, 4), np.float32)
    pos[:, :3] = rng.random((n, 3), dtype=np.float32)
    d = rng.normal(size=(n, 3)).astype(np.float32)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    tgt = np.zeros((n, 8), np.float16)
    tgt[:, :3] = rng.random((n, 3), dtype=np.float32).astype(np.float16)
    return pos, d, tgt


def init_params(seed_table=0):
    from helpers import make_mlp
    rng = np.random.default_rng(seed_table)
    table = rng.uniform(-1e-4, 1e-4, size=L * T * 2).astype(np.float32)
    dW, db = make_mlp(*DENSITY, seed=1)
    cW, cb = make_mlp(*COLOR, seed=1)
    return table, dW, db, cW, cb


class ClockSampler:
    """Reads SM clock and throttle reasons through NVML (read-only queries) every few milliseconds from a
    thread while the timed region runs; falls back to polling nvidia-smi when NVML is not importable."""

    def __init__(self, gpu_index):
        self.gpu, self.samples, self.stop_flag, self.thread = gpu_index, [], threading.Event(), None
        self.max_mhz = None

    def _loop_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        phys = self.gpu
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                phys = int(vis.split(",")[self.gpu])
            except (ValueError, IndexError):
                phys = self.gpu
        h = pynvml.nvmlDeviceGetHandleByIndex(phys)
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
        while not self.stop_flag.is_set():
            mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
            try:
                r = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
            except Exception:
                r = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
            self.samples.append((mhz, [k for k, b in bits.items() if r & b]))
            time.sleep(0.002)

    def _loop_smi(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=10).stdout
                f = [x.strip() for x in out.strip().split(",")]
                self.max_mhz = float(f[1])
                self.samples.append((float(f[0]), [nm for k, nm in enumerate(names) if f[2 + k].lower().startswith("active")]))
            except Exception:
                return

    def _loop(self):
        try:
            self._loop_nvml()
        except Exception:
            self._loop_smi()

    def start(self):
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def mark(self):
        """Index of the next sample: brackets the timed region inside a longer sampling window."""
        return len(self.samples)

    def stop(self, lo=0, hi=None):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=15)
        window = self.samples[lo:hi] if self.samples[lo:hi] else self.samples
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no clock samples"], "samples": 0}
        reasons = sorted({r for _, rs in window for r in rs})
        return {"sm_mhz": float(np.median([m for m, _ in window])), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(window)}


def cpu_baseline(sample, repeats=1):
    """The oracle's restatement of the same step on `sample` samples, OpenMP over all host cores."""
    import oracle as orc
    from oracle_pipeline import OracleField
    table, dW, db, cW, cb = init_params()
    scales = orc.level_scales(BASE, GROWTH, L)
    dls = orc.dense_level_start(T, BASE, GROWTH, L)
    field = OracleField(L, T, BASE, GROWTH, scales, dls, DENSITY, COLOR, table, dW, db, cW, cb)
    pos, dirs, tgt = make_batch(sample, 123)
    tgt_bits = tgt.view(np.uint16)
    H = L * T * 2
    m, v = np.zeros(H, np.float32), np.zeros(H, np.float32)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        r = field.forward_backward(pos, dirs, tgt_bits, HYPER["loss_scale"])
        bc1, bc2 = orc.adam_bias_corrections(1, HYPER["beta1"], HYPER["beta2"])
        wh = orc.half_bits(field.table).copy()
        orc.adam_hash(field.table, wh, r["g_table"], m, v, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], bc1, bc2,
                      1.0 / HYPER["loss_scale"])
        for w, g in ((field.dW, r["g_dW"]), (field.db, r["g_db"]), (field.cW, r["g_cW"]), (field.cb, r["g_cb"])):
            orc.adam_dense(w, g, np.zeros_like(w), np.zeros_like(w), HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], bc1, bc2,
                           1.0 / HYPER["loss_scale"])
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample / best, best


def run_reference_cuda(args, rank, world, local_rank):
    """Reference arm, CUDA: the reference's own TinyMLPHashGrid / TinyMLP classes and kernels, compiled unmodified
    for sm_100a into oracle/_ref (oracle/build_ref.py), driven through the same step on the same workload:
    zero_grad, grid forward, SH gather, colour forward, MSE loss, colour backward (dX), density gradient, grid
    backward + scatter, Adam of both networks.  The reference is single-GPU: under torchrun rank 0 measures one
    GPU and reports N ideal replicas."""
    if rank != 0:
        return
    import torch
    from oracle import ref_cuda as ref
    nb = importlib.import_module("3dmaker_b200")
    torch.cuda.set_device(local_rank)
    lib = ref.lib()
    rf = lib.ref_field_create(L, T, BASE, GROWTH, DENSITY[1], DENSITY[3], COLOR[1], COLOR[3], BATCH)
    table, dW, db, cW, cb = init_params()
    lib.ref_field_load(rf, ref.hptr(table), ref.hptr(dW), ref.hptr(db), ref.hptr(cW), ref.hptr(cb))
    host, dev = [], []
    for k in range(2):
        pos, dirs, tgt = make_batch(BATCH, 1000 + k)
        t3 = np.ascontiguousarray(tgt[:, :3])
        hp = tuple(torch.from_numpy(a).pin_memory() for a in (pos, dirs, t3))
        host.append(hp)
        dev.append(tuple(t.cuda() for t in hp))
    st = nb.stream_ptr()
    P = nb.ptr

    def step(bufs):
        lib.ref_field_train_step(rf, P(bufs[0]), P(bufs[1]), P(bufs[2]), BATCH, 0.0, HYPER["loss_scale"], HYPER["lr"], HYPER["beta1"],
                                 HYPER["beta2"], HYPER["eps"], st)

    warm = max(args.warmup, 3)
    for i in range(warm):
        step(dev[i % 2])
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.05)
    for i in range(3):
        step(dev[i % 2])
    torch.cuda.synchronize()
    mark0 = sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(dev[i % 2])
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(mark0, sampler.mark())
    ms = e0.elapsed_time(e1) / args.steps
    # e2e, harnessed exactly like ours: the copy of batch k + 1 runs on a copy stream into the input set the running step
    # does not use, and the 4 bytes read back per step (one colour value: the reference's step leaves no loss scalar on
    # the device) travel to pinned memory asynchronously and are read by the host one step late
    slots = [tuple(torch.empty_like(t) for t in dev[0]) for _ in range(2)]
    copy_stream = torch.cuda.Stream()
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    free = [torch.cuda.Event(), torch.cuda.Event()]
    probe = nm_view(torch, lib.ref_field_color_out(rf), 1)
    probe_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    probe_done = [torch.cuda.Event(), torch.cuda.Event()]
    cur = torch.cuda.current_stream()

    def prefetch(k, src):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[k])
            for dst, a in zip(slots[k], src):
                dst.copy_(a, non_blocking=True)
            ready[k].record(copy_stream)

    def e2e_loop(count):
        """`count` steps; slot 0 holds the first batch already (primed outside the timed region, as in the other arm),
        every step copies the next batch in and reads the value of the step before."""
        reads = 0
        for i in range(count):
            k = i % 2
            prefetch(1 - k, host[(i + 1) % 2])
            cur.wait_event(ready[k])
            step(slots[k])
            free[k].record(cur)
            probe_host[k].copy_(probe, non_blocking=True)
            probe_done[k].record(cur)
            if i > 0:
                probe_done[1 - k].synchronize(); float(probe_host[1 - k].item()); reads += 1
        probe_done[(count - 1) % 2].synchronize(); float(probe_host[(count - 1) % 2].item()); reads += 1
        return reads

    prefetch(0, host[0])
    e2e_loop(2)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    reads = e2e_loop(args.steps)
    e1.record()
    torch.cuda.synchronize()
    assert reads == args.steps
    e2e_ms = e0.elapsed_time(e1) / args.steps
    h2d = sum(a.numel() * a.element_size() for a in host[0])
    value = world * BATCH / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": common_config(world),
        "notes": {"reference": "reference CUDA classes/kernels recompiled for sm_100a (oracle/_ref); single-GPU code, value = %d ideal replicas" % world,
                  "e2e": "copy stream + loss read one step late, the same harness as the other arm"},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": 0, "kind": "reference",
                         "sample": "full 2^20-sample step on the GPU: the reference has no CPU implementation of this path"},
        "e2e": {"value": world * BATCH / (e2e_ms / 1000.0), "unit": "samples/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4},
        "gpu_launches": 0, "clocks": clocks,
    }
    lib.ref_field_destroy(rf)
    del dev, slots
    torch.cuda.empty_cache()
    if not args.no_extras:
        # the reference is single-GPU: its render and config-5 numbers are one GPU's, whatever --gpus says
        line.update(run_extras(args, 0, 1, local_rank))
    print(json.dumps(line))
    return


def nm_view(torch, ptr, count):
    nm = importlib.import_module("3dmaker_b200.nerf")
    return nm.view_tensor(torch, ptr, count, np.float32)


def run_reference(args, rank, world=1, local_rank=0):
    """Reference arm.  With the reference's CUDA build present (oracle/_ref) and a GPU, its own kernels are timed;
    otherwise the oracle's CPU restatement of them (kind "port") on all host cores, each step a bounded sample."""
    try:
        import torch
        from oracle import ref_cuda
        if ref_cuda.available() and torch.cuda.is_available() and not args.reference_cpu:
            return run_reference_cuda(args, rank, world, local_rank)
    except ImportError:
        pass
    if rank != 0:
        return
    total = args.steps + args.warmup
    sample = 1 << 16 if total <= 8 else (1 << 15 if total <= 20 else (1 << 14 if total <= 60 else 1 << 13))
    cores = os.cpu_count() or 1
    times = []
    for i in range(total):
        _, dt = cpu_baseline(sample)
        if i >= args.warmup:
            times.append(dt)
    ms = 1000.0 * float(np.mean(times))
    value = sample / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": common_config(args.gpus), "notes": {"sample_per_step": sample},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port",
                         "sample": "%d samples per step of the 2^20-sample workload, full T=2^19 table and Adam over it" % sample},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def time_kernels(torch, tr, n, iters=5):
    """Per-kernel device time of one step (CUDA events around each launch on the launching stream)."""
    import ctypes
    nb = importlib.import_module("3dmaker_b200")
    m, lib, P = tr.model, tr.lib, nb.ptr
    st = nb.stream_ptr()
    if tr.fused and tr.ordered:
        # the step as it runs: brick order of the samples, then the two field kernels in that order
        calls = {
            "sample_order": lambda: lib.nb_sample_order(P(tr.pos), n, P(tr.order), P(tr.order_scratch), st),
            "field_forward": lambda: lib.nb_field_forward_ordered(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(tr.pos),
                                                                  m.ptr("w_h", 0), P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db),
                                                                  m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, P(tr.order), tr.density_bias,
                                                                  P(tr.enc), P(tr.sigma), P(tr.logit0), P(tr.c_out), 8, st),
            "mse_loss_grad": lambda: lib.nb_mse_loss_grad(P(tr.c_out), P(tr.target), P(tr.c_grad), P(tr.loss), n, 8, 3, tr.loss_scale, 1, st),
            "field_backward": lambda: lib.nb_field_backward_ordered(ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0,
                                                                    m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                                                    m.ptr("w", m.off_cb), n, P(tr.order), P(tr.c_grad), None, m.ptr("g", m.off_dw),
                                                                    m.ptr("g", m.off_db), m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(tr.d_enc),
                                                                    None, None, None, st),
            "scatter_backward": lambda: lib.nb_hash_scatter_backward(ctypes.byref(m.grid), P(tr.pos), P(tr.d_enc), n, m.ptr("g", 0), st),
        }
        if tr.fused_scatter:
            calls["field_backward_scatter"] = lambda: lib.nb_field_backward_ordered(
                ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db),
                m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, P(tr.order), P(tr.c_grad), None, m.ptr("g", m.off_dw), m.ptr("g", m.off_db),
                m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(tr.d_enc), ctypes.byref(m.grid), P(tr.pos), m.ptr("g", 0), st)
    elif tr.fused:
        calls = {}
        if tr.fused_loss:
            # the step's forward: loss and colour gradient taken in its epilogue
            calls["field_forward_mse"] = lambda: lib.nb_field_forward_mse(
                ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(tr.pos), m.ptr("w_h", 0), P(tr.dirs), m.ptr("w_h", m.off_dw),
                m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, tr.density_bias, P(tr.enc), P(tr.sigma), P(tr.logit0),
                P(tr.c_out), 8, P(tr.target), P(tr.c_grad), P(tr.loss), tr.loss_scale, st)
        calls.update({
            "field_forward": lambda: lib.nb_field_forward(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(tr.pos),
                                                          m.ptr("w_h", 0), P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db),
                                                          m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, tr.density_bias, P(tr.enc),
                                                          P(tr.sigma), P(tr.logit0), P(tr.c_out), 8, st),
            "mse_loss_grad": lambda: lib.nb_mse_loss_grad(P(tr.c_out), P(tr.target), P(tr.c_grad), P(tr.loss), n, 8, 3, tr.loss_scale, 1, st),
            "field_backward": lambda: lib.nb_field_backward(ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0,
                                                            m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                                            m.ptr("w", m.off_cb), n, P(tr.c_grad), None, m.ptr("g", m.off_dw),
                                                            m.ptr("g", m.off_db), m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(tr.d_enc),
                                                            None, None, None, st),
            "scatter_backward": lambda: lib.nb_hash_scatter_backward(ctypes.byref(m.grid), P(tr.pos), P(tr.d_enc), n, m.ptr("g", 0), st),
        })
        if tr.fused_scatter:
            calls["field_backward_scatter"] = lambda: lib.nb_field_backward(
                ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db),
                m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, P(tr.c_grad), None, m.ptr("g", m.off_dw), m.ptr("g", m.off_db),
                m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(tr.d_enc), ctypes.byref(m.grid), P(tr.pos), m.ptr("g", 0), st)
    else:
        calls = {
            "grid_mlp_forward": lambda: lib.nb_grid_mlp_forward(ctypes.byref(m.grid), ctypes.byref(m.density), P(tr.pos), m.ptr("w_h", 0),
                                                                m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), n, P(tr.d_out), P(tr.enc),
                                                                P(tr.d_acts), st),
            "sh_gather": lambda: lib.nb_sh_gather(P(tr.dirs), P(tr.ray_idx), 0, n, tr.density_bias, P(tr.d_out), P(tr.c_in), P(tr.sigma), st),
            "mlp_forward_color": lambda: lib.nb_mlp_forward(ctypes.byref(m.color), P(tr.c_in), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb),
                                                            n, P(tr.c_out), P(tr.c_acts), st),
            "mse_loss_grad": lambda: lib.nb_mse_loss_grad(P(tr.c_out), P(tr.target), P(tr.c_grad), P(tr.loss), n, 8, 3, tr.loss_scale, 1, st),
            "mlp_backward_color": lambda: lib.nb_mlp_backward(ctypes.byref(m.color), P(tr.c_grad), m.ptr("w_h", m.off_cw), P(tr.c_in),
                                                              P(tr.c_acts), n, m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(tr.c_dx), st),
            "density_grad": lambda: lib.nb_density_grad(n, None, P(tr.c_dx), P(tr.d_grad), st),
            "mlp_backward_density": lambda: lib.nb_mlp_backward(ctypes.byref(m.density), P(tr.d_grad), m.ptr("w_h", m.off_dw), P(tr.enc),
                                                                P(tr.d_acts), n, m.ptr("g", m.off_dw), m.ptr("g", m.off_db), P(tr.d_enc), st),
            "scatter_backward": lambda: lib.nb_hash_scatter_backward(ctypes.byref(m.grid), P(tr.pos), P(tr.d_enc), n, m.ptr("g", 0), st),
        }
    out = {}
    for name, fn in calls.items():
        ts = []
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            nb.check(fn(), name)
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b))
        out[name] = float(np.median(ts))
    # Adam on the gradient the calls above left behind (first call touches everything, later ones nothing:
    # time the first)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    tr.optimizer_step()
    b.record()
    b.synchronize()
    out["adam_step"] = float(a.elapsed_time(b))
    return out


# algorithmic bytes per sample of the HBM/L2-bound kernels (encode: 16 B position + 16 levels x 8 corners x 4 B
# gathers + 64 B features out; field forward: the same + 12 B direction + 4 B sigma + 4 B logit + 32 B colour row;
# scatter: 16 B + 64 B gradient in + 16 x 8 x 2 x 4 B adds counted once)
# field backward with the scatter inside: 64 B features + 12 B direction + 16 B colour gradient + 16 B position in,
# 16 x 8 x 2 x 4 B adds counted once)
ALGO_BYTES = {"grid_mlp_forward": 592.0, "field_forward": 644.0, "scatter_backward": 1104.0, "field_backward_scatter": 1132.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch at 2^20 samples, from the ncu capture summarised in
# profiles/field_step_kernels_2p20_ncu.md (same workload, same sizes)
NCU_TRAFFIC = {"field_forward": 159.7e6, "field_backward_scatter": 190.9e6 + 33.7e6}   # backward kernel + the levels 0-1 kernel


def bind_to_gpu_numa_node(torch, local_rank):
    """Several ranks on one host: keeps this process (and so the pinned staging buffers it allocates next: first touch)
    on the NUMA node its GPU hangs off, so that eight ranks do not pull their input through one socket.  Best effort;
    returns the node or None."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bus = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bus).read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


# L1TEX lane requests of one field_forward launch and L2 reduction requests of one backward launch at 2^20 samples, from the
# ncu captures summarised in profiles/field_step_kernels_2p20_ncu.md
NCU_REQUESTS = {"field_forward": 105.0e6, "field_backward_scatter": 92.0e6}


def random_access_rates(torch, nb):
    """What the memory system gives a kernel that does nothing but scattered accesses to an L2-resident table the size
    of ours (nb_probe_random_access): 4-byte gathers from 2^23 entries (the 32 MiB fp16 table), 8-byte fp32-pair
    reductions into 2^23 entries (the 64 MiB gradient table).  G operations per second, best of 3."""
    lib = nb.load()
    table = torch.zeros(1 << 24, dtype=torch.float32, device="cuda")
    blocks, per_thread = 148 * 16, 128
    out = {}
    for name, kind in (("gather_gops", 0), ("reduction_gops", 1)):
        nb.check(lib.nb_probe_random_access(kind, 23, blocks, per_thread, nb.ptr(table), nb.stream_ptr()), "nb_probe_random_access")
        best = None
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            nb.check(lib.nb_probe_random_access(kind, 23, blocks, per_thread, nb.ptr(table), nb.stream_ptr()), "nb_probe_random_access")
            b.record(); b.synchronize()
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
        out[name] = blocks * 256 * per_thread / best / 1e6
    return out


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nb = importlib.import_module("3dmaker_b200")
    pl = importlib.import_module("3dmaker_b200.pipeline")
    nb.load()
    for kv in args.tune:
        k, v = kv.split("=")
        nb.check(nb.load().nb_set_tuning(k.encode(), int(v)), "nb_set_tuning")
    if args.grad_half:
        nb.set_grad_table_half(True, args.grad_scale_log2)

    buffers = None
    if world > 1 and args.dp == "allreduce" and not args.plain_buffers:
        # the gradient lives in memory registered with the communicator: all-reduced in place through NVSwitch
        D = importlib.import_module("3dmaker_b200.distributed")
        buffers = D.CollectiveBuffers(torch, dist, "cuda:%d" % local_rank)
    model = pl.FieldModel(torch, L, T, BASE, GROWTH, DENSITY[1], DENSITY[3], COLOR[1], COLOR[3],
                          grad_alloc=buffers.zeros if buffers is not None else None, exportable=(world > 1 and args.dp == "peer"))
    if buffers is not None:
        buffers.register()
    table, dW, db, cW, cb = init_params()
    model.load_hashgrid(table); model.load_density_weights(dW, db); model.load_color_weights(cW, cb)
    tr = pl.SampleTrainer(model, BATCH, fused=False if args.unfused else None, fused_scatter=False if args.separate_scatter else None,
                          ordered=True if args.ordered else None, fused_loss=False if args.separate_loss else None, **HYPER)

    # two distinct seeded batches per rank: resident on the device in the kernels' layouts (`value`), and pinned on the
    # host in the compact layout they travel in (`e2e`: position float3, direction float3, target three halves = 30 B)
    numa_node = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None
    host, dev = [], []
    for k in range(2):
        pos, dirs, tgt = make_batch(BATCH, 1000 + 10 * rank + k)
        dev.append(tuple(torch.from_numpy(a).cuda() for a in (pos, dirs, tgt)))
        host.append(tuple(torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in (pos[:, :3], dirs, tgt[:, :3])))
    own = (tr.pos, tr.dirs, tr.target)

    grad_sync = None
    if world > 1:
        if args.dp == "allreduce":
            def grad_sync(g):
                dist.all_reduce(g, op=dist.ReduceOp.SUM)
        else:
            # "sharded": reduce-scatter, Adam on this rank's slice of the table, all-gather of the fp16 slice;
            # "sliced": allreduce and Adam pipelined over 4 slices (SampleTrainer.optimizer_step_sharded / _synced)
            grad_sync = dist
            tr.dp_mode = args.dp

    def step_resident(i):
        tr.pos, tr.dirs, tr.target = dev[i % 2]
        tr.step_device(BATCH, None, grad_sync)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: inputs resident in HBM ------------------------------------------------------------------
    for i in range(max(args.warmup, 3)):
        step_resident(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    for i in range(3):          # every rank (the step holds a collective): GPU under load while the sampler spins up
        step_resident(i)
    launches0 = nb.load().nb_launch_count()
    barrier()
    mark0 = sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step_resident(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = nb.load().nb_launch_count() - launches0
    clocks = sampler.stop(mark0, sampler.mark()) if rank == 0 else None
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = world * BATCH / (ms_step / 1000.0)

    # ---- e2e: pinned host inputs copied in every step, loss read back every step ---------------------------
    # The public entry is prefetch() + step_prefetched(): the copy of batch k+1 runs on a copy stream while the
    # step on batch k computes; every step still copies its own inputs and reads its own loss inside the timed region.
    tr.pos, tr.dirs, tr.target = own
    tr.prefetch(*host[0])
    for i in range(2):
        tr.prefetch(*host[(i + 1) % 2])
        tr.step_prefetched(None, grad_sync)
    tr.flush_loss()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss, losses_read = 0.0, 0
    for i in range(args.steps):
        tr.prefetch(*host[(i + 1) % 2])
        got = tr.step_prefetched(None, grad_sync)      # the loss of the previous step: its 4-byte copy has landed by now
        if got is not None:
            loss, losses_read = got, losses_read + 1
    loss, losses_read = tr.flush_loss(), losses_read + 1   # the last step's loss, still inside the timed region
    e1.record()
    tr.step_prefetched(None, grad_sync, lag=False)      # drain the last prefetched batch (outside the timed region)
    barrier()
    assert losses_read == args.steps, "every timed step's loss must have been read back"
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / args.steps
    e2e_value = world * BATCH / (e2e_ms / 1000.0)
    h2d = sum(a.numel() * a.element_size() for a in host[0])

    line = None
    if rank == 0:
        peak, peak_src = load_peaks()
        kt = time_kernels(torch, tr, BATCH)
        # kernels timed only for the A/B split are not part of the step when the backward scatters itself
        in_step = [k for k in ALGO_BYTES if k in kt and not (tr.fused_scatter and k in ("scatter_backward", "field_backward"))]
        dom = max(in_step, key=lambda k: kt[k])
        achieved = ALGO_BYTES[dom] * BATCH / (kt[dom] / 1000.0) / 1e9
        roofline = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(dom),
                    "note": "achieved = %.0f algorithmic B/sample x 2^20 samples / %.3f ms (CUDA events); the fp16 table (32 MiB) and "
                            "its fp32 gradient (64 MiB) are L2-resident, so the kernel is bound by L2 reductions and the L1TEX request "
                            "rate, not by HBM: DRAM traffic per launch (ncu) is far below the algorithmic bytes"
                            % (ALGO_BYTES[dom], kt[dom])}
        # the roof these kernels actually run under: scattered accesses to L2-resident tables
        rates = random_access_rates(torch, nb)
        scale = BATCH / float(1 << 20)
        fwd_rate = NCU_REQUESTS["field_forward"] * scale / (kt["field_forward"] / 1000.0) / 1e9 if "field_forward" in kt else None
        bwd_key = "field_backward_scatter" if "field_backward_scatter" in kt else None
        bwd_rate = NCU_REQUESTS["field_backward_scatter"] * scale / (kt[bwd_key] / 1000.0) / 1e9 if bwd_key else None
        roofline["l2_random_access"] = {
            "probe": rates, "unit": "G operations/s",
            "field_forward": None if fwd_rate is None else {"gather_requests_gops": fwd_rate, "frac_of_probe": fwd_rate / rates["gather_gops"]},
            "field_backward_scatter": None if bwd_rate is None else {"reduction_requests_gops": bwd_rate,
                                                                      "frac_of_probe": bwd_rate / rates["reduction_gops"]},
            "note": "request counts per launch from ncu (profiles/field_step_kernels_2p20_ncu.md); probe = nb_probe_random_access on "
                    "tables of the same size, a kernel that does nothing else"}
        line = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": common_config(world),
            "notes": {"exchange": None if world == 1 else args.dp,
                      "field_kernels": (("fused+scatter" if tr.fused_scatter else "fused") + ("+ordered" if tr.ordered else "") + ("+loss" if tr.fused_loss else "")) if tr.fused else "sequence",
                      "tuning": args.tune, "grad_table": ("fp16 x 2^%d (opt-in A/B)" % args.grad_scale_log2) if args.grad_half else "fp32",
                      "host_batch_layout": "pos float3 + dir float3 + target half3 (30 B/sample), widened on the device",
                      "numa_node": numa_node},
            "e2e": {"value": e2e_value, "unit": "samples/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "last_loss": loss},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "kernel_ms": kt,
        }
        if world == 1 and not args.no_cpu_baseline:
            sample = 1 << 16
            v, dt = cpu_baseline(sample)
            line["cpu_baseline"] = {"value": v, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": "one step on %d samples (%.1f s) of the 2^20-sample workload, full T=2^19 table" % (sample, dt)}
    # ---- the rest of the metric (render Mrays/s) and config 5, on the same ranks ----------------------------------
    if world > 1 and args.dp == "peer":
        tr.close_peers(dist)
    del tr, model, dev, own
    if buffers is not None:
        del buffers
    torch.cuda.empty_cache()
    if not args.no_extras:
        extras = run_extras(args, rank, world, local_rank)
        if rank == 0:
            line.update(extras)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------
# Secondary workloads (not the driver's line): the full NeRF step on the analytic soft-sphere scene and
# frame rendering along an orbit, both through the scene engine, with the reference's engine as the other arm.
# ---------------------------------------------------------------------------------------------------------
SCENE_OPTS = dict(grid_resolution=(128,) * 3, aabb_min=(-.5,) * 3, aabb_max=(.5,) * 3, levels_mipmap=4, hash_table_size=1 << 19,
                  growth_factor=1.3819, color_hidden_dim=64, color_num_layers=3, batch_size=1 << 18, render_batch_size=1 << 20,
                  ray_chunk_size=1 << 16, lambda_dist=0.01, lambda_depth=0.0, learning_rate=1e-2, beta2=0.99, epsilon=1e-15,
                  loss_scale=128.0, density_bias=1.0, bg_color=(1.0, 1.0, 1.0))
SCENE_WORKLOAD = ("cfg3: analytic soft sphere, 100 cameras 800x800, 128^3 occupancy x1 cascade, L16 F2 T2^19, batch 2^18 samples, "
                  "ray chunk 65536, distortion loss, Adam")
RENDER_WORKLOAD = "cfg4: 1920x1080 orbit frames of the cfg3 model after %d training steps, <=1024 samples/ray, early termination"


# config 5: 32 seeded soft spheres in a box of scale 4, 3 cascades of 128^3, T = 2^22 per level, 300 cameras 1280x720,
# 2^21 samples per optimizer step over ALL ranks, split evenly (strong scaling): a rank's sample batch is 2^21 / N and
# it gets 524288 / N rays per call, about six optimizer steps' worth
SCENE5_GLOBAL_BATCH = 1 << 21
SCENE5_GLOBAL_RAYS = 1 << 19
SCENE5_OPTS = dict(SCENE_OPTS, hash_table_size=1 << 22, num_cascades=3)
SCENE5_WORKLOAD = ("cfg5: 32 soft spheres in a scale-4 box, 300 cameras 1280x720, 128^3 occupancy x3 cascades, L16 F2 T2^22, "
                   "2^21 samples per optimizer step over all GPUs (2^21/N per GPU), 2^19 rays per call over all GPUs, distortion loss, Adam")


class _RefEngine:
    """The reference's InstantNerf (oracle/_ref build) behind the few methods the workloads call."""

    def __init__(self, torch, opts):
        import ctypes
        from oracle import ref_cuda as ref
        self.torch, self.ref, self.nb = torch, ref, importlib.import_module("3dmaker_b200")
        self.h = ref.lib().ref_nerf_create(ctypes.byref(opts), 0)
        self.steps = 0
        self._depth = self._sig = None
        self.hits = torch.zeros(64, dtype=torch.int32).numpy()

    def set_learning_rate(self, lr):
        self.ref.lib().ref_nerf_set_learning_rate(self.h, float(lr))

    def train_rays(self, o, d, rgb):
        n = o.shape[0]
        if self._depth is None or self._depth.shape[0] < n:
            self._depth = self.torch.full((n,), -1.0, device="cuda"); self._sig = self.torch.ones(n, device="cuda")
        P = self.nb.ptr
        self.hits[:] = 0
        k = self.ref.lib().ref_nerf_train(self.h, P(o), P(d), P(self._depth), P(self._sig), P(rgb), n, None, self.ref.hptr(self.hits),
                                          self.nb.stream_ptr())
        self.steps += k
        return self.steps

    def samples_last_call(self):
        return int(self.hits.astype("int64").sum())

    def render(self, o, d, out):
        self.ref.lib().ref_nerf_render(self.h, self.nb.ptr(o), self.nb.ptr(d), o.shape[0], self.nb.ptr(out), self.nb.stream_ptr())

    def close(self):
        self.ref.lib().ref_nerf_destroy(self.h)


def _scene_batches(torch, syn, count, rays, seed0, config=3):
    bg = (1.0, 1.0, 1.0)
    if config == 5:
        scene, poses, wh = syn.MultiSphereScene(), syn.sphere_cameras(300, radius=4.5), (1280, 720)
        extent = scene.extent
    else:
        scene, poses, wh, extent = syn.SoftSphereScene(), syn.sphere_cameras(100), (800, 800), None
    out = []
    for k in range(count):
        o, d = syn.random_training_rays(torch, poses, rays, wh[0], wh[1], 50.0, seed=seed0 + k)
        out.append((o, d, syn.ground_truth(torch, scene, o, d, bg, extent=extent, chunk=(1 << 14) if config == 5 else (1 << 18))))
    return out


def run_scene(args, rank, world, local_rank, embedded=False):
    """Full training step (march + field + compositing + loss + backward + scatter + Adam) on the analytic scene.
    scene (config 3): every rank trains 65536 rays per call, one gradient allreduce per optimizer step (weak scaling).
    scene5 (config 5): 2^21 samples per optimizer step and 2^19 rays per call over ALL ranks (strong scaling).
    embedded: called from the default run - the process group exists already, the line is returned, not printed."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    reference = args.impl == "reference"
    if reference and rank != 0:
        return None
    if world > 1 and not reference and not embedded:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nb = importlib.import_module("3dmaker_b200")
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    D = importlib.import_module("3dmaker_b200.distributed")
    cfg5 = args.workload == "scene5"
    nranks = 1 if reference else world
    if args.grad_half and not reference:
        nb.set_grad_table_half(True, args.grad_scale_log2)
    if cfg5:
        rays = SCENE5_GLOBAL_RAYS // nranks
        opts = nm.default_options(**dict(SCENE5_OPTS, batch_size=SCENE5_GLOBAL_BATCH // nranks, ray_chunk_size=rays))
    else:
        rays = 1 << 16
        opts = nm.default_options(**SCENE_OPTS)
    if reference:
        from oracle import ref_cuda as ref
        if not ref.available():
            line = {"impl": "reference", "unavailable": "oracle/_ref/libref3dmaker.so not built (no reference tree at build time)"}
            if not embedded:
                print(json.dumps(line))
            return line
        eng, trainer = _RefEngine(torch, opts), None
    else:
        eng = nm.InstantNerf(torch, opts)
        # data parallel: every rank takes DP_STEPS optimizer steps on its rays of a call (one occupancy walk per call)
        # config 3: 65536 rays per rank and call hold 6-7 batches of 2^18 samples; config 5: a rank's share of the 2^19 rays
        # holds 17 batches of its share of the 2^21 samples at every N.  Rays walked but not trained on are wasted march time.
        trainer = D.DataParallelTrainer(torch, eng, dist if world > 1 else None, steps_per_call=16 if cfg5 else 6,
                                        registered_gradient=not args.plain_buffers,
                                        exchange=args.exchange or ("levels" if cfg5 else "peer"))
    batches = _scene_batches(torch, syn, 4 if cfg5 else 8, rays * nranks, 9000, config=5 if cfg5 else 3)

    used = [0]

    def step(i):
        o, d, c = batches[i % len(batches)]
        if trainer is not None:
            used[0] += trainer.train_rays(o, d, c)
        else:
            eng.train_rays(o, d, c)
            used[0] += o.shape[0]
        return eng.samples_last_call()

    warm = max(args.warmup, args.scene_warm)   # default: past the 256 steps of whole-grid occupancy updates
    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    if world > 1 and not reference:
        dist.barrier()
    if args.phases and not reference:
        eng.set_profiling(True)      # every phase is waited for: the per-phase times add up, the step gets slower
        p0, s0 = eng.phase_times()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    samples = 0
    steps_before = eng.steps if reference else eng.steps.value
    used[0] = 0
    e0.record()
    for i in range(args.steps):
        samples += step(warm + i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1), float(samples), float(used[0])], dtype=torch.float64, device="cuda")
    if world > 1 and not reference:
        tm = t[:1].clone(); dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ts = t[1:].clone(); dist.all_reduce(ts, op=dist.ReduceOp.SUM)
        t = torch.cat([tm, ts])
    ms, total, rays_used = float(t[0].item()), float(t[1].item()), float(t[2].item())
    opt_steps = (eng.steps if reference else eng.steps.value) - steps_before
    line = None
    in_sync = None
    if trainer is not None and world > 1:
        in_sync = bool(trainer.replicas_in_sync())
    if rank == 0:
        line = {"metric": "train samples/s (full NeRF step)", "value": total / (ms / 1000.0), "unit": "samples/s", "n_gpus": nranks,
                "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong" if cfg5 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": SCENE5_WORKLOAD if cfg5 else SCENE_WORKLOAD, "rays_per_call_per_gpu": rays, "optimizer_steps": opt_steps,
                           "samples_per_call": total / args.steps, "rays_per_s": rays_used / (ms / 1000.0),
                           "samples_per_optimizer_step": total / max(opt_steps, 1),
                           "ms_per_optimizer_step": ms / max(opt_steps, 1)}}
        if reference:
            line["impl"] = "reference"
        elif trainer is not None:
            line["config"]["replicas_in_sync"] = in_sync
            line["config"]["exchange"] = trainer.exchange if world > 1 else None
            if args.grad_half:
                line["config"]["grad_table"] = "fp16 x 2^%d (opt-in A/B)" % args.grad_scale_log2
            if args.phases:
                p1, s1 = eng.phase_times()
                line["config"]["phase_ms_per_optimizer_step"] = {k: round((p1[k] - p0[k]) / max(s1 - s0, 1), 4) for k in p1}
            if world > 1:
                line["config"]["exchange_stats"] = trainer.exchange_stats()
        if not embedded:
            print(json.dumps(line))
    if trainer is not None:
        trainer.close()          # peer exchange: meets the other ranks before it unmaps their memory
    if trainer is not None and world > 1 and not embedded:
        dist.barrier(); dist.destroy_process_group()
    eng.close()
    return line


def run_render(args, rank, world, local_rank, embedded=False):
    """Frames of the trained scene along an orbit, pixels sharded over the ranks, one gather per frame."""
    import ctypes
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    reference = args.impl == "reference"
    if reference and rank != 0:
        return None
    if world > 1 and not reference and not embedded:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nb = importlib.import_module("3dmaker_b200")
    nm = importlib.import_module("3dmaker_b200.nerf"); syn = importlib.import_module("3dmaker_b200.synthetic")
    D = importlib.import_module("3dmaker_b200.distributed")
    lib = nb.load()
    opts = nm.default_options(**SCENE_OPTS)
    train_steps = args.render_train_steps
    if reference:
        from oracle import ref_cuda as ref
        if not ref.available():
            line = {"impl": "reference", "unavailable": "oracle/_ref/libref3dmaker.so not built (no reference tree at build time)"}
            if not embedded:
                print(json.dumps(line))
            return line
        eng = _RefEngine(torch, opts)
    else:
        eng = nm.InstantNerf(torch, opts)
    # every rank trains the same model from the same seeded batches (replicated, no exchange needed for the benchmark)
    # learning rate annealed from 1e-2 to 1e-3 over the training by the reference trainer's cosine (NerfTrainer.cu:131-135):
    # at a constant 1e-2 the PSNR a few hundred steps in moves by several dB from run to run, for either engine
    i = 0
    while (eng.steps if reference else eng.steps.value) < train_steps:
        done = (eng.steps if reference else eng.steps.value) / float(train_steps)
        eng.set_learning_rate(1e-3 + 0.5 * (1e-2 - 1e-3) * (1.0 + math.cos(math.pi * min(done, 1.0))))
        eng.train_rays(*_scene_batches(torch, syn, 1, 1 << 16, 9000 + i)[0]); i += 1
    torch.cuda.synchronize()
    # frames are rendered in inference mode, as INerfTrainer::renderC2W does (NerfTrainer.cu:302-328): the sample batch
    # is renderBatchSize and the training buffers are released
    if reference:
        eng.ref.lib().ref_nerf_set_memory_mode(eng.h, 1)
    else:
        eng.set_memory_mode(True)
        if args.render_rounds:
            eng.set_render_rounds(True)
    W, H = 1920, 1080
    focal = syn.focal_from_fov(W, 50.0)
    pose = {}

    def ray_fn(first, count, o, d):
        c2w = np.ascontiguousarray(pose["c2w"], np.float32)
        nb.check(lib.nb_generate_rays(W, H, focal, c2w.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), first, count, nb.ptr(o), nb.ptr(d),
                                      nb.stream_ptr()), "nb_generate_rays")

    def tiled_ray_fn(tile, first_tile, stride, count, o, d):
        c2w = np.ascontiguousarray(pose["c2w"], np.float32)
        nb.check(lib.nb_generate_rays_tiled(W, H, focal, c2w.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), tile, first_tile, stride, count,
                                            nb.ptr(o), nb.ptr(d), nb.stream_ptr()), "nb_generate_rays_tiled")

    def undeal_fn(blocks, ranks, rows, tile, num_pixels, frame):
        nb.check(lib.nb_undeal_tiles(nb.ptr(blocks), ranks, rows, tile, num_pixels, nb.ptr(frame), nb.stream_ptr()), "nb_undeal_tiles")

    r = D.ShardedRenderer(torch, eng, ray_fn, dist if (world > 1 and not reference) else None, tile=1 << 14, tiled_ray_fn=tiled_ray_fn,
                          undeal_fn=undeal_fn)
    nranks = 1 if reference else world

    def frame(k):
        pose["c2w"] = syn.orbit_c2w(3.0 * k, 20.0, 1.5)
        return r.render_frame(W * H, "cuda")

    frames = args.render_frames if embedded else args.steps
    for k in range(max(args.warmup, 3)):
        img = frame(k)
    torch.cuda.synchronize()
    if nranks > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(frames):
        img = frame(10 + k)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    if nranks > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / frames
    line = None
    if rank == 0:
        frame_samples = None if reference else eng.last_render_samples() * nranks   # this rank's share of the last frame, scaled
        frame_mean = float(img.mean().item())
        scene = syn.SoftSphereScene()
        o, d = syn.frame_rays(torch, pose["c2w"], W // 4, H // 4, 50.0)
        gt = syn.ground_truth(torch, scene, o, d, (1.0, 1.0, 1.0))
        small = torch.zeros_like(gt)
        eng.render(o, d, small)
        torch.cuda.synchronize()
        line = {"metric": "render Mrays/s", "value": W * H / (ms / 1000.0) / 1e6, "unit": "Mrays/s", "n_gpus": nranks, "steps": frames,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16", "data": "synthetic",
                "config": {"workload": RENDER_WORKLOAD % train_steps, "frame": [W, H], "tile_pixels": 1 << 14,
                           "gather_bytes_per_frame": D.gathered_bytes(W * H, nranks, 1 << 14),
                           "psnr_quarter_res_db": float(syn.psnr(torch, small, gt)), "frame_mean": frame_mean,
                           "field_samples_per_frame": frame_samples}}
        if reference:
            line["impl"] = "reference"
        if not embedded:
            print(json.dumps(line))
    if nranks > 1 and not embedded:
        dist.barrier(); dist.destroy_process_group()
    eng.close()
    return line


def run_extras(args, rank, world, local_rank):
    """The other half of the metric and the multi-GPU configuration, measured in the same process (and process group)
    as the headline line: `render` = 1920x1080 orbit frames of the config-3 model, pixels sharded over the ranks
    (config 4, Mrays/s); `scene5` = the full training step of config 5 (T = 2^22, 3 cascades, 2^21 samples per
    optimizer step split over the ranks: strong scaling).  Returns {"render": {...}, "scene5": {...}} on rank 0."""
    import copy
    import torch
    out = {}
    for key, workload, fn in (("render", "render", run_render), ("scene5", "scene5", run_scene)):
        a = copy.copy(args)
        a.workload = workload
        a.warmup, a.steps, a.scene_warm = 3, args.extra_steps, args.extra_scene_warm
        try:
            line = fn(a, rank, world, local_rank, embedded=True)
        except Exception as e:            # an extra must never cost the headline line
            if world > 1:
                raise                     # ... but ranks of a collective job have to fail together
            line = {"error": "%s: %s" % (type(e).__name__, e)}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        if rank == 0 and line is not None:
            if "metric" in line:
                out[key] = {"value": line["value"], "unit": line["unit"], "metric": line["metric"], "n_gpus": line["n_gpus"],
                            "ms_per_step": line["ms_per_step"], "scaling": line["scaling"], "steps": line["steps"], "warmup": line["warmup"],
                            "workload": line["config"]["workload"], "detail": {k: v for k, v in line["config"].items() if k != "workload"}}
                if key == "render":
                    out[key]["ms_per_frame"] = line["ms_per_step"]
            else:
                out[key] = line
    return out


def run_partition_kernels(args):
    """The kernels of the level-partitioned step on ONE GPU, at config-5 sizes: this device plays rank 0 of `--ranks`
    (it owns levels 0, R, 2R, ...), the other ranks' samples are random positions in their slots, the exchanges are
    skipped (their buffers are simply there).  Per-kernel CUDA-event times next to the replicated path's fused kernels
    on the same number of own samples.  Not a throughput claim for the multi-GPU step: it times what one rank computes."""
    import ctypes
    import torch
    torch.cuda.set_device(0)
    nb = importlib.import_module("3dmaker_b200")
    pl = importlib.import_module("3dmaker_b200.pipeline")
    from helpers import make_mlp
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    R, Tp = args.ranks, 1 << 22
    cap = SCENE5_GLOBAL_BATCH // R
    own = L // R
    model = pl.FieldModel(torch, L, Tp, BASE, 1.3819, DENSITY[1], DENSITY[3], COLOR[1], COLOR[3])
    model.w[:model.hash_count].uniform_(-1e-4, 1e-4)
    model.w_h[:model.hash_count].copy_(model.w[:model.hash_count].half())
    model.load_density_weights(*make_mlp(*DENSITY, seed=1)); model.load_color_weights(*make_mlp(*COLOR, seed=1))
    G, D, C = ctypes.byref(model.grid), ctypes.byref(model.density), ctypes.byref(model.color)
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    pos_all = torch.rand((R, cap + 1, 4), generator=g, device="cuda")
    for q in range(R):
        nb.check(lib.nb_part_stamp_count(ctypes.c_void_p(pos_all[q].data_ptr()), cap, cap, st), "nb_part_stamp_count")
    pos = pos_all[0, :cap].contiguous()
    dirs = torch.nn.functional.normalize(torch.randn((cap, 3), generator=g, device="cuda"), dim=1).contiguous()
    pieces = torch.zeros((R, own, cap), dtype=torch.int32, device="cuda")
    pieces2 = torch.zeros_like(pieces)
    enc = torch.zeros((cap, 32), dtype=torch.float16, device="cuda")
    denc = torch.zeros((cap, 32), dtype=torch.float16, device="cuda")
    sigma, logit = torch.zeros(cap, device="cuda"), torch.zeros(cap, device="cuda")
    rgb = torch.zeros((cap, 4), device="cuda")
    dcol = (torch.randn((cap, 8), generator=g, device="cuda") * 1e-3).half()
    w = (model.ptr("w_h", model.off_dw), model.ptr("w", model.off_db), model.ptr("w_h", model.off_cw), model.ptr("w", model.off_cb))
    gw = (model.ptr("g", model.off_dw), model.ptr("g", model.off_db), model.ptr("g", model.off_cw), model.ptr("g", model.off_cb))
    level = model.hash_count // L
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0, 1, st)

    def owned_adam():
        rc = 0
        for l in range(0, L, R):
            off = l * level
            rc |= lib.nb_adam_step(model.ptr("w", off), model.ptr("w_h", off), model.ptr("g", off), model.ptr("m", off), model.ptr("v", off), level, level, *hyper)
        return rc

    calls = [
        ("part_encode (own levels, all ranks' samples)", lambda: lib.nb_part_encode(G, R, 0, cap, P(pos_all), model.ptr("w_h", 0), P(pieces), st),
         R * cap * own * (16.0 / own + 8 * 4 + 4)),
        ("part_field_forward (networks from pieces)", lambda: lib.nb_part_field_forward(G, D, C, R, cap, P(pieces), P(dirs), None, 0, *w, cap, 1.0, P(enc), P(sigma),
                                                                                       P(logit), P(rgb), 4, st), cap * (64.0 + 12 + 64 + 24)),
        ("field_backward (no table gradient)", lambda: lib.nb_field_backward(D, C, P(enc), P(dirs), None, 0, *w, cap, P(dcol), None, *gw, P(denc), None, None, None, st),
         cap * (64.0 + 12 + 16 + 64)),
        ("part_pack_denc", lambda: lib.nb_part_pack_denc(G, R, cap, P(denc), cap, P(pieces2), st), cap * 128.0),
        ("part_scatter (own levels, all ranks' samples)", lambda: lib.nb_part_scatter(G, R, 0, cap, P(pos_all), P(pieces2), model.ptr("g", 0), st),
         R * cap * own * (16.0 / own + 4 + 8 * 8)),
        ("adam on the owned levels", owned_adam, None),
        ("replicated: field_forward on the own samples", lambda: lib.nb_field_forward(G, D, C, P(pos), model.ptr("w_h", 0), P(dirs), None, 0, *w, cap, 1.0, P(enc), P(sigma),
                                                                                       P(logit), P(rgb), 4, st), cap * ALGO_BYTES["field_forward"]),
        ("replicated: field_backward with the scatter", lambda: lib.nb_field_backward(D, C, P(enc), P(dirs), None, 0, *w, cap, P(dcol), None, *gw, P(denc), G, P(pos),
                                                                                       model.ptr("g", 0), st), cap * ALGO_BYTES["field_backward_scatter"]),
        ("replicated: adam on the whole arena", lambda: lib.nb_adam_step(model.ptr("w", 0), model.ptr("w_h", 0), model.ptr("g", 0), model.ptr("m", 0), model.ptr("v", 0),
                                                                        model.hash_count, model.total, *hyper), None),
    ]
    peak, peak_source = load_peaks()
    out = {}
    for name, fn, nbytes in calls:
        ts = []
        for i in range(args.warmup + args.steps):
            if "adam" in name:
                model.g[:model.hash_count].uniform_(-1e-3, 1e-3)          # every entry touched, as a config-5 step leaves it
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            nb.check(fn(), name)
            b.record(); b.synchronize()
            if i >= args.warmup:
                ts.append(a.elapsed_time(b))
        ms = float(np.median(ts))
        out[name] = {"ms": round(ms, 4)}
        if nbytes:
            out[name]["algorithmic_GBs"] = round(nbytes / ms / 1e6, 1)
            if peak:
                out[name]["frac_of_%s_hbm" % peak_source] = round(nbytes / ms / 1e6 / peak, 3)
    print(json.dumps({"metric": "kernel ms of one rank's share of a level-partitioned step", "n_gpus": 1, "ranks_played": R, "dtype": "f16",
                      "data": "synthetic", "config": {"workload": "cfg5 grid (L16 F2 T2^22 b1.3819), 2^21 / ranks samples per rank, uniformly scattered",
                                                       "samples_per_rank": cap, "owned_levels": own}, "kernel_ms": out}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="field", choices=["field", "scene", "scene5", "render", "partition"],
                    help="field: the headline step on explicit samples (default, the driver's line); scene / scene5: full NeRF training step on the "
                         "analytic scene of config 3 / config 5; render: 1920x1080 orbit frames, pixels sharded over the ranks")
    ap.add_argument("--batch-log2", type=int, default=20, help="field workload: log2 of the samples per GPU and step (20 = the benchmark's; "
                    "smaller values are for profiling small cases, their lines are not benchmark results)")
    ap.add_argument("--scene-warm", type=int, default=272, help="scene workload: untimed train_rays calls before the timed ones")
    ap.add_argument("--render-train-steps", type=int, default=400, help="render workload: optimizer steps the model is trained for first")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="field workload: leave the `render` and `scene5` keys out of the line")
    ap.add_argument("--extra-steps", type=int, default=10, help="timed train_rays calls of the embedded scene5 measurement")
    ap.add_argument("--extra-scene-warm", type=int, default=48, help="untimed train_rays calls of the embedded scene5 measurement "
                    "(six optimizer steps each: past the 256 steps of whole-grid occupancy updates)")
    ap.add_argument("--render-frames", type=int, default=12, help="timed frames of the embedded render measurement")
    ap.add_argument("--exchange", default=None, choices=["allreduce", "sharded", "peer", "levels"],
                    help="scene workloads at N > 1: all-reduce + replicated Adam; reduce-scatter + Adam on a table slice + all-gather of fp16 "
                         "parameters; the same three stages as one kernel over peer memory (default for config 3); or the table "
                         "partitioned by level, encodings exchanged instead of the table (default for config 5, whose table outweighs "
                         "a step's samples)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE", help="nb_set_tuning switch for A/B runs, e.g. pair_ops=0")
    ap.add_argument("--separate-loss", action="store_true", help="keep the MSE loss a launch of its own instead of the forward's epilogue (A/B)")
    ap.add_argument("--separate-scatter", action="store_true", help="keep the gradient scatter a launch of its own (A/B)")
    ap.add_argument("--dp", default="peer", choices=["peer", "sharded", "allreduce", "sliced"],
                    help="N > 1: how the gradient is exchanged (peer: one kernel per rank that sums the ranks' gradients of its table slice "
                         "from peer memory, applies Adam and stores the fp16 slice into every rank; sharded: reduce-scatter + Adam on a slice + "
                         "all-gather of fp16 parameters; allreduce: one allreduce + one full Adam; sliced: both pipelined over 4 slices)")
    ap.add_argument("--render-rounds", action="store_true", help="render workload: render in rounds of samples per ray (A/B; off by default)")
    ap.add_argument("--plain-buffers", action="store_true", help="N > 1: keep the gradient in ordinary device memory instead of memory "
                    "registered with the communicator (A/B)")
    ap.add_argument("--ranks", type=int, default=8, help="partition workload: how many ranks the one device pretends to be one of")
    ap.add_argument("--phases", action="store_true", help="scene workloads: per-phase device times of the engine (waits after every phase: "
                                                          "the line's throughput is NOT a benchmark value then)")
    ap.add_argument("--grad-half", action="store_true", help="keep the table gradient in half precision (A/B; off by default: the reference keeps fp32)")
    ap.add_argument("--grad-scale-log2", type=int, default=7, help="with --grad-half: contributions are multiplied by 2^this before they are rounded to fp16")
    ap.add_argument("--ordered", action="store_true", help="sort every batch by brick and run the field kernels in that order (A/B; off by default)")
    ap.add_argument("--unfused", action="store_true", help="run the kernel-by-kernel sequence instead of the two field kernels (A/B)")
    ap.add_argument("--reference-cpu", action="store_true", help="reference arm: time the CPU port even when the CUDA build exists")
    args = ap.parse_args()
    global BATCH, WORKLOAD
    if args.batch_log2 != 20:
        BATCH = 1 << args.batch_log2
        WORKLOAD = WORKLOAD.replace("2^20 samples/GPU", "2^%d samples/GPU (NOT the benchmark size)" % args.batch_log2)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "partition":
        run_partition_kernels(args)
    elif args.workload in ("scene", "scene5"):
        run_scene(args, rank, world, local_rank)
    elif args.workload == "render":
        run_render(args, rank, world, local_rank)
    elif args.impl == "reference":
        run_reference(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
