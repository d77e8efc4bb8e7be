"""One full field-training step (encode + both MLPs fwd/bwd + scatter + Adam) through the C ABI, compared
stage by stage with the same step restated from oracle calls."""
import ctypes
import importlib

import numpy as np
import pytest

from helpers import REL_MLP, dev_half_bits, half_bits, half_vals, make_mlp, make_positions, make_table, rel_err
from oracle_pipeline import OracleField

pytestmark = pytest.mark.gpu


def _inputs(n, seed):
    rng = np.random.default_rng(seed)
    pos = make_positions(n, seed)
    d = rng.normal(size=(n, 3)).astype(np.float32)
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    tgt = np.zeros((n, 8), np.float32)
    tgt[:, :3] = rng.random((n, 3), dtype=np.float32)
    return pos, d, half_bits(tgt)


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("n", [300, 8192])
def test_sample_training_step_matches_oracle(cuda, nb, orc, n, fused):
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    L, T = 16, 1 << 15
    model = pl.FieldModel(torch, L, T, 16, 1.447, 64, 2, 64, 3)
    table = make_table(L, T, seed=0, amp=0.1)
    dW, db = make_mlp(32, 64, 16, 2, seed=0)
    cW, cb = make_mlp(32, 64, 8, 3, seed=1)
    model.load_hashgrid(table); model.load_density_weights(dW, db); model.load_color_weights(cW, cb)
    tr = pl.SampleTrainer(model, n, lr=1e-2, loss_scale=128.0, fused=fused)
    assert tr.fused == fused
    pos, dirs, tgt = _inputs(n, 5)
    tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
    tr.forward_backward(n)
    torch.cuda.synchronize()

    scales = np.array(list(model.grid.scales)[:L], np.float32)
    sscales = np.array(list(model.grid.scatter_scales)[:L], np.float32)
    ref = OracleField(L, T, 16, 1.447, scales, model.grid.dense_level_start, (32, 64, 16, 2), (32, 64, 8, 3), table, dW, db, cW, cb, sscales)
    r = ref.forward_backward(pos, dirs, tgt, 128.0)
    assert np.array_equal(dev_half_bits(tr.encoded(n)), r["enc"])
    if fused:
        assert rel_err(tr.logit0.cpu().numpy(), r["d_out"][:, 0]) <= REL_MLP
    else:
        assert rel_err(tr.d_out.cpu().numpy(), r["d_out"]) <= REL_MLP
        assert rel_err(half_vals(dev_half_bits(tr.c_in)), half_vals(r["c_in"])) <= REL_MLP
    assert rel_err(tr.sigma.cpu().numpy(), r["sigma"]) <= 2 * REL_MLP
    assert np.max(np.abs(tr.c_out.cpu().numpy()[:, :3] - r["c_out"][:, :3])) <= 1e-2
    assert abs(tr.loss.item() - r["loss_sum"]) <= 1e-2 * r["loss_sum"]
    assert rel_err(half_vals(dev_half_bits(tr.c_grad)), half_vals(r["c_grad"])) <= 2 * REL_MLP
    g = model.g.cpu().numpy()
    H = model.hash_count
    # gradients of a chain of fp16 stages: each stage is within 1e-2 of the oracle GIVEN the same inputs; end to end
    # the bound is looser because upstream roundings differ
    assert rel_err(g[model.off_cw:model.off_cw + model.color.weight_count], r["g_cW"]) <= 3 * REL_MLP
    assert rel_err(g[model.off_cb:model.off_cb + model.color.bias_count], r["g_cb"]) <= 3 * REL_MLP
    assert rel_err(g[model.off_dw:model.off_dw + model.density.weight_count], r["g_dW"]) <= 5 * REL_MLP
    assert rel_err(g[model.off_db:model.off_db + model.density.bias_count], r["g_db"]) <= 5 * REL_MLP
    assert rel_err(g[:H], r["g_table"]) <= 5 * REL_MLP

    # optimizer: feed the GPU's own gradient to the oracle rule and compare the update exactly-ish
    w0, g0 = model.w.cpu().numpy().copy(), g.copy()
    tr.optimizer_step()
    torch.cuda.synchronize()
    bc1, bc2 = orc.adam_bias_corrections(1, 0.9, 0.99)
    hyper = (1e-2, 0.9, 0.99, 1e-15, bc1, bc2, 1.0 / 128.0)
    ws, gs = w0[:H].copy(), g0[:H].copy()
    ms, vs, whs = np.zeros(H, np.float32), np.zeros(H, np.float32), half_bits(ws).copy()
    orc.adam_hash(ws, whs, gs, ms, vs, *hyper)
    wd = w0[H:].copy(); md = np.zeros_like(wd); vd = np.zeros_like(wd)
    orc.adam_dense(wd, g0[H:], md, vd, *hyper)
    w1 = model.w.cpu().numpy()
    assert np.allclose(w1[:H], ws, rtol=1e-5, atol=1e-7)
    assert np.allclose(w1[H:], wd, rtol=1e-5, atol=1e-7)
    assert np.all(model.g.cpu().numpy() == 0)
    assert np.array_equal(dev_half_bits(model.w_h)[:H][g0[:H] == 0], half_bits(w0[:H])[g0[:H] == 0])


def test_training_reduces_loss(cuda, nb):
    """Size-independent property: repeated steps on a fixed batch drive the loss down."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    model = pl.FieldModel(torch, 16, 1 << 15, 16, 1.3819, 64, 2, 64, 3)
    rng = np.random.default_rng(0)
    model.load_hashgrid(make_table(16, 1 << 15, seed=0, amp=1e-4))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=0)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=1))
    n = 4096
    tr = pl.SampleTrainer(model, n)
    pos, dirs, tgt = _inputs(n, 9)
    tgt_f = np.zeros((n, 8), np.float32); tgt_f[:, :3] = pos[:, :3]      # learn colour = position
    P = lambda a: torch.from_numpy(a).pin_memory()
    losses = [tr.step_host(P(pos), P(dirs), P(half_bits(tgt_f).view(np.float16))) for _ in range(60)]
    assert np.isfinite(losses).all()
    assert losses[-1] < 0.5 * losses[0]


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000, 40000])
def test_fused_field_kernels_agree_with_the_kernel_sequence(cuda, nb, n):
    """The two-kernel field path against the kernel-by-kernel one on the same parameters and inputs: every fp16
    intermediate has the same rounding points, so the encoding, the outputs and the encoding gradient are
    bit-identical; weight gradients differ by fp32 summation order only."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    L, T = 16, 1 << 15
    model = pl.FieldModel(torch, L, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 11)
    out = {}
    modes = {"sequence": dict(fused=False), "fused": dict(fused=True, fused_scatter=False),
             "fused+scatter": dict(fused=True, fused_scatter=True, ordered=False)}
    # the bit-for-bit claims hold for the mma.sync backward, which accumulates in the sequence's order; the tensor-memory
    # backward (the default) has its own test below
    nb.check(nb.load().nb_set_tuning(b"backward_tc", 0), "nb_set_tuning")
    for name, kw in modes.items():
        tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, **kw)
        tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
        model.g.zero_()
        tr.forward_backward(n)
        torch.cuda.synchronize()
        out[name] = dict(enc=dev_half_bits(tr.encoded(n)), sigma=tr.sigma.cpu().numpy(), c_out=tr.c_out.cpu().numpy()[:, :3].copy(),
                         logit=(tr.logit0 if tr.fused else tr.d_out[:, 0]).cpu().numpy(), d_enc=dev_half_bits(tr.d_enc), g=model.g.cpu().numpy().copy(),
                         loss=tr.loss.item())
    model.g.zero_()
    nb.check(nb.load().nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
    a = out["sequence"]
    H = model.hash_count
    for name in ("fused", "fused+scatter"):
        b = out[name]
        assert np.array_equal(a["enc"], b["enc"])
        assert np.array_equal(a["logit"], b["logit"])
        assert np.array_equal(a["sigma"], b["sigma"])
        assert np.array_equal(a["c_out"], b["c_out"])
        assert abs(a["loss"] - b["loss"]) <= 1e-5 * abs(a["loss"])          # one atomic sum, order differs
        if name == "fused":
            assert np.array_equal(a["d_enc"], b["d_enc"])
        assert np.allclose(a["g"][:H], b["g"][:H], rtol=1e-4, atol=1e-6 * np.abs(a["g"][:H]).max()), name
        assert np.array_equal(a["g"][:H] != 0, b["g"][:H] != 0), name
        for off, cnt in ((model.off_dw, model.density.weight_count), (model.off_db, model.density.bias_count),
                         (model.off_cw, model.color.weight_count), (model.off_cb, model.color.bias_count)):
            assert rel_err(b["g"][off:off + cnt], a["g"][off:off + cnt]) <= 1e-4, name


def test_fused_field_rejects_other_shapes(cuda, nb):
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    model = pl.FieldModel(torch, 16, 1 << 14, 16, 1.3819, 32, 2, 32, 3)
    assert pl.SampleTrainer(model, 64).fused is False
    with pytest.raises(nb.NerfB200Error):
        pl.SampleTrainer(model, 64, fused=True)


def test_pipelined_allreduce_and_adam_equal_the_single_launch(cuda, nb):
    """optimizer_step_synced (allreduce and Adam over slices of the arena) on a one-rank NCCL group against
    optimizer_step: identical parameters, moments and fp16 copy, and the gradient is consumed."""
    torch = cuda
    import socket
    import torch.distributed as dist
    pl = importlib.import_module("3dmaker_b200.pipeline")
    if dist.is_initialized():
        pytest.skip("a process group already exists in this process")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        n, out = 4096, {}
        pos, dirs, tgt = _inputs(n, 21)
        for mode in ("single", "sliced", "sharded"):
            model = pl.FieldModel(torch, 16, 1 << 14, 16, 1.3819, 64, 2, 64, 3)
            model.load_hashgrid(make_table(16, 1 << 14, seed=2, amp=0.1))
            model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=3)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=4))
            tr = pl.SampleTrainer(model, n)
            tr.dp_mode = mode
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            for _ in range(2):
                tr.step_device(n, None, dist if mode != "single" else (lambda g: dist.all_reduce(g)))
            if mode == "sharded":
                tr.gather_master(dist)
            torch.cuda.synchronize()
            out[mode] = [getattr(model, k).clone() for k in ("w", "w_h", "m", "v", "g")]
        # the gradient itself differs run to run in its last bits (unordered atomics), so compare loosely but completely
        for other in ("sliced", "sharded"):
            for a, b in zip(out["single"][:4], out[other][:4]):
                assert torch.allclose(a.float(), b.float(), rtol=1e-3, atol=1e-6), other
            assert torch.all(out[other][4] == 0)
        assert torch.all(out["single"][4] == 0)
        assert (out["sliced"][0] != torch.from_numpy(make_table(16, 1 << 14, seed=2, amp=0.1).ravel()).cuda()[:1].new_zeros(1)).any()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000, 70000])
def test_tensor_memory_backward_agrees_with_the_register_formulation(cuda, nb, n):
    """nb_field_backward with tcgen05.mma / tensor-memory accumulators against the mma.sync formulation: same rounding
    points, so dL/d(encoding) and every gradient agree to accumulation order (an fp16 value may differ in its last bit
    where the fp32 sums straddle a rounding boundary)."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib = nb.load()
    L, T = 16, 1 << 15
    model = pl.FieldModel(torch, L, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 13)
    out = {}
    try:
        for name, tcflag, fs in (("regs", 0, False), ("tc", 1, False), ("regs+scatter", 0, True), ("tc+scatter", 1, True)):
            nb.check(lib.nb_set_tuning(b"backward_tc", tcflag), "nb_set_tuning")
            tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=fs, ordered=False)
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            model.g.zero_()
            tr.forward_backward(n)
            nb.check(lib.nb_field_backward_tc_status(), "tensor-memory backward status")
            out[name] = dict(d_enc=half_vals(dev_half_bits(tr.d_enc)), g=model.g.cpu().numpy().copy())
    finally:
        nb.check(lib.nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
        model.g.zero_()
    H = model.hash_count
    assert rel_err(out["tc"]["d_enc"], out["regs"]["d_enc"]) <= 2e-3
    assert np.mean(out["tc"]["d_enc"] != out["regs"]["d_enc"]) < 2e-2
    for name in ("tc", "tc+scatter"):
        a, b = out["regs+scatter" if "scatter" in name else "regs"]["g"], out[name]["g"]
        assert rel_err(b[:H], a[:H]) <= 2e-3, name
        for off, cnt in ((model.off_dw, model.density.weight_count), (model.off_db, model.density.bias_count),
                         (model.off_cw, model.color.weight_count), (model.off_cb, model.color.bias_count)):
            assert rel_err(b[off:off + cnt], a[off:off + cnt]) <= 2e-3, (name, off)


def test_tensor_memory_backward_wait_that_runs_out_is_reported_and_recoverable(cuda, nb):
    """With the wait limit set to 0 a chain warp gives up as soon as its MMA barrier is not ready: the kernel must return
    (nothing hangs, nothing faults), the condition must surface - nb_field_backward refuses to go on, the status call
    reports and clears it - and the next launch with the normal limit must work and give the register kernel's gradients."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib = nb.load()
    L, T, n = 16, 1 << 15, 5000
    model = pl.FieldModel(torch, L, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 17)
    tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=True, ordered=False)
    tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
    try:
        nb.check(lib.nb_set_tuning(b"backward_tc", 0), "nb_set_tuning")
        model.g.zero_(); tr.forward_backward(n); torch.cuda.synchronize()
        want = model.g.cpu().numpy().copy()
        nb.check(lib.nb_set_tuning(b"backward_tc", 1), "nb_set_tuning")
        nb.check(lib.nb_set_tuning(b"backward_tc_wait_us", 0), "nb_set_tuning")
        model.g.zero_(); tr.forward_backward(n); torch.cuda.synchronize()          # the launch itself succeeds and returns
        with pytest.raises(nb.NerfB200Error):                                       # ... but the next call is refused
            tr.forward_backward(n)
        assert lib.nb_field_backward_tc_status() == 3                               # NB_ERR_CUDA, and cleared
        assert b"ran out" in lib.nb_last_error()
        assert lib.nb_field_backward_tc_status() == 0
        nb.check(lib.nb_set_tuning(b"backward_tc_wait_us", 1000000), "nb_set_tuning")
        model.g.zero_(); tr.forward_backward(n)
        nb.check(lib.nb_field_backward_tc_status(), "status after recovery")
        got = model.g.cpu().numpy()
        assert rel_err(got[:model.hash_count], want[:model.hash_count]) <= 2e-3
        assert rel_err(got[model.off_cw:model.off_cw + model.color.weight_count], want[model.off_cw:model.off_cw + model.color.weight_count]) <= 2e-3
    finally:
        lib.nb_set_tuning(b"backward_tc_wait_us", 1000000)
        lib.nb_set_tuning(b"backward_tc", 2)
        lib.nb_field_backward_tc_status()
        model.g.zero_()


def test_field_backward_with_8_byte_aligned_weight_gradients_uses_the_register_kernel(cuda, nb):
    """Weight-gradient pointers that are 8- but not 16-byte aligned: the default mode must not pick the tensor-memory
    kernel (16-byte reductions); the register kernel runs and the gradients equal the aligned call's."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib, P = nb.load(), nb.ptr
    L, T, n = 16, 1 << 14, 3000
    model = pl.FieldModel(torch, L, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 19)
    tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=False)
    tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
    model.g.zero_(); tr.forward_backward(n); torch.cuda.synchronize()
    m = model
    dense = m.total - m.hash_count
    want = m.g[m.hash_count:].cpu().numpy().copy()
    shifted = torch.zeros(dense + 8, dtype=torch.float32, device="cuda")
    base = shifted[2:]                                                    # 8 bytes past a 16-byte boundary
    assert base.data_ptr() % 16 == 8
    off = lambda o: ctypes.c_void_p(base.data_ptr() + (o - m.hash_count) * 4)
    nb.check(lib.nb_field_backward(ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw),
                                   m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n, P(tr.c_grad), None, off(m.off_dw),
                                   off(m.off_db), off(m.off_cw), off(m.off_cb), P(tr.d_enc), None, None, None, nb.stream_ptr()), "nb_field_backward")
    torch.cuda.synchronize()
    assert rel_err(base[:dense].cpu().numpy(), want) <= 2e-3
    model.g.zero_()


def _brick_keys(pos):
    """12-bit Morton key of the 16^3 brick of every position (numpy restatement of the ordering's key)."""
    q = np.clip(np.floor(pos[:, :3] * np.float32(16.0)).astype(np.int64), 0, 15)
    spread = lambda v: (v & 1) | ((v & 2) << 2) | ((v & 4) << 4) | ((v & 8) << 6)
    return spread(q[:, 0]) | (spread(q[:, 1]) << 1) | (spread(q[:, 2]) << 2)


@pytest.mark.parametrize("n", [1, 255, 2048, 2049, 100000])
def test_sample_order_is_a_permutation_sorted_by_brick(cuda, nb, n):
    torch = cuda
    lib, P = nb.load(), nb.ptr
    pos = make_positions(n, 31)
    pos[: min(n, 4), :3] = np.array([[0, 0, 0], [1, 1, 1], [-3.0, 0.5, 2.0], [0.999999, 0.0625, 0.5]], np.float32)[: min(n, 4)]
    d_pos = torch.from_numpy(pos).cuda()
    order = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(int(lib.nb_sample_order_scratch_bytes()) // 4, dtype=torch.int32, device="cuda")
    for _ in range(2):                                   # the scratch is reused call after call
        nb.check(lib.nb_sample_order(P(d_pos), n, P(order), P(scratch), nb.stream_ptr()), "nb_sample_order")
    torch.cuda.synchronize()
    o = order.cpu().numpy().astype(np.int64)
    assert np.array_equal(np.sort(o), np.arange(n))      # every sample exactly once
    keys = _brick_keys(pos)[o]
    assert np.all(np.diff(keys) >= 0)                    # brick after brick, in Morton order


@pytest.mark.parametrize("order_kind", ["bricks", "random", "identity"])
@pytest.mark.parametrize("n", [1, 127, 513, 5000, 70000])
def test_ordered_field_kernels_agree_with_the_unordered_ones(cuda, nb, n, order_kind):
    """nb_field_forward_ordered / nb_field_backward_ordered against nb_field_forward / nb_field_backward on the same
    inputs: the forward's outputs are identical bit for bit whatever the order (levels staged in shared memory hold the
    same table entries), the saved encoding is the same rows permuted, and every gradient agrees to fp32 summation
    order - with the brick order (boxes small, many levels staged), a random permutation (boxes cover the whole grid,
    nothing or little staged) and the identity."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib, P = nb.load(), nb.ptr
    L, T = 16, 1 << 15
    model = pl.FieldModel(torch, L, T, 16, 1.447, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 23)
    if n > 8:
        pos[:4, :3] = [[0, 0, 0], [1, 1, 1], [1.0, 0.0, 0.999999], [0.5, 0.5, 0.5]]
    out = {}
    try:
        nb.check(lib.nb_set_tuning(b"backward_tc", 1), "nb_set_tuning")
        for name in ("plain", "ordered"):
            tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=True, ordered=(name == "ordered"))
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            model.g.zero_()
            if name == "ordered" and order_kind != "bricks":
                # drive the two ordered entry points with an order of our own
                rng = np.random.default_rng(5)
                o = rng.permutation(n) if order_kind == "random" else np.arange(n)
                tr.order.copy_(torch.from_numpy(o.astype(np.int32)))
                st, m = nb.stream_ptr(), model
                nb.check(lib.nb_zero_async(P(tr.loss), 4, st))
                nb.check(lib.nb_field_forward_ordered(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(tr.pos), m.ptr("w_h", 0),
                                                      P(tr.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                                      m.ptr("w", m.off_cb), n, P(tr.order), tr.density_bias, P(tr.enc), P(tr.sigma), P(tr.logit0),
                                                      P(tr.c_out), 8, st), "nb_field_forward_ordered")
                nb.check(lib.nb_mse_loss_grad(P(tr.c_out), P(tr.target), P(tr.c_grad), P(tr.loss), n, 8, 3, tr.loss_scale, 1, st))
                nb.check(lib.nb_field_backward_ordered(ctypes.byref(m.density), ctypes.byref(m.color), P(tr.enc), P(tr.dirs), None, 0,
                                                       m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n,
                                                       P(tr.order), P(tr.c_grad), None, m.ptr("g", m.off_dw), m.ptr("g", m.off_db), m.ptr("g", m.off_cw),
                                                       m.ptr("g", m.off_cb), P(tr.d_enc), ctypes.byref(m.grid), P(tr.pos), m.ptr("g", 0), st),
                         "nb_field_backward_ordered")
            else:
                tr.forward_backward(n)
            nb.check(lib.nb_field_backward_tc_status(), "tensor-memory backward status")
            out[name] = dict(enc=dev_half_bits(tr.encoded(n)), sigma=tr.sigma.cpu().numpy(), logit=tr.logit0.cpu().numpy(),
                             c_out=tr.c_out.cpu().numpy().copy(), g=model.g.cpu().numpy().copy(), loss=tr.loss.item())
    finally:
        nb.check(lib.nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
        model.g.zero_()
    a, b = out["plain"], out["ordered"]
    for k in ("enc", "sigma", "logit", "c_out"):
        assert np.array_equal(a[k], b[k]), k
    assert abs(a["loss"] - b["loss"]) <= 1e-5 * abs(a["loss"])
    H = model.hash_count
    assert rel_err(b["g"][:H], a["g"][:H]) <= 2e-3
    assert np.mean((a["g"][:H] != 0) != (b["g"][:H] != 0)) < 1e-4
    for off, cnt in ((model.off_dw, model.density.weight_count), (model.off_db, model.density.bias_count),
                     (model.off_cw, model.color.weight_count), (model.off_cb, model.color.bias_count)):
        assert rel_err(b["g"][off:off + cnt], a["g"][off:off + cnt]) <= 2e-3, off


def test_ordered_backward_without_the_fused_scatter_writes_the_encoding_gradient_by_sample(cuda, nb):
    """d_table_grads == NULL: dL/d(encoding) comes back as a matrix indexed by SAMPLE, ready for nb_hash_scatter_backward."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    lib = nb.load()
    L, T, n = 16, 1 << 15, 3000
    model = pl.FieldModel(torch, L, T, 16, 1.447, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 29)
    res = {}
    try:
        nb.check(lib.nb_set_tuning(b"backward_tc", 1), "nb_set_tuning")
        for name, ordered in (("plain", False), ("ordered", True)):
            tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, fused_scatter=False, ordered=ordered)
            tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
            model.g.zero_()
            tr.forward_backward(n)
            torch.cuda.synchronize()
            res[name] = (half_vals(dev_half_bits(tr.d_enc)), model.g.cpu().numpy().copy())
    finally:
        nb.check(lib.nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
        model.g.zero_()
    assert rel_err(res["ordered"][0], res["plain"][0]) <= 2e-3
    assert rel_err(res["ordered"][1][:model.hash_count], res["plain"][1][:model.hash_count]) <= 2e-3


def test_compact_host_batches_train_like_full_layout_ones(cuda, nb):
    """prefetch() with the compact host layout (position float3, target three halves: 30 bytes per sample instead of
    44) widens the batch on the device with nb_unpack_samples; the step's inputs, and so its loss, are bit-identical."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    L, T, n = 16, 1 << 14, 3000
    pos, dirs, tgt = _inputs(n, 37)
    losses = {}
    for layout in ("full", "compact"):
        model = pl.FieldModel(torch, L, T, 16, 1.447, 64, 2, 64, 3)
        model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
        model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
        tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, ordered=False)
        nb.check(nb.load().nb_set_tuning(b"backward_tc", 0), "nb_set_tuning")      # one summation order for both runs is not needed: only the loss is compared
        P = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
        t16 = tgt.view(np.float16)
        batch = (P(pos), P(dirs), P(t16)) if layout == "full" else (P(pos[:, :3]), P(dirs), P(t16[:, :3]))
        tr.prefetch(*batch)
        losses[layout] = tr.step_prefetched(lag=False)
        if layout == "compact":
            assert torch.equal(tr.pos[:n].cpu(), torch.from_numpy(pos)) and torch.equal(tr.target[:n].cpu().view(torch.int16), torch.from_numpy(tgt.view(np.int16)))
    nb.check(nb.load().nb_set_tuning(b"backward_tc", 2), "nb_set_tuning")
    # the loss is one atomic sum over the batch: equal up to its summation order
    assert abs(losses["full"] - losses["compact"]) <= 1e-6 * losses["full"] and losses["full"] > 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_peer_optimizer_kernel_equals_reduce_then_adam(cuda, nb, world):
    """nb_adam_step_peer with the ranks played by separate buffers on ONE device (the kernel never waits for another rank,
    so the ranks' launches simply run one after the other): every rank's fp16 parameters end up equal to what one Adam
    launch on the summed gradient gives, each slice's master copy and moments are right on its owner, the dense tail on
    everybody; untouched entries keep parameters and moments."""
    torch = cuda
    lib, P, st = nb.load(), nb.ptr, nb.stream_ptr()
    H, total = 1 << 16, (1 << 16) + 1024
    rng = np.random.default_rng(8)
    w0 = rng.uniform(-0.1, 0.1, total).astype(np.float32)
    grads = []
    for r in range(world):
        g = np.zeros(total, np.float32)
        g[:H] = (rng.normal(0, 3, H) * (rng.random(H) < 0.2)).astype(np.float32)
        g[H:] = rng.normal(0, 5, total - H).astype(np.float32)
        grads.append(g)
    hyper = (1e-2, 0.9, 0.99, 1e-15, 0.1, 0.01, 1.0 / 128.0)
    dev = lambda a: torch.from_numpy(a.copy()).cuda()
    # reference: one launch on the sum (added in rank order, as the kernel adds)
    gsum = grads[0].copy()
    for r in range(1, world):
        gsum += grads[r]
    ref = dict(w=dev(w0), h=dev(w0).half(), g=dev(gsum), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
    nb.check(lib.nb_adam_step(P(ref["w"]), P(ref["h"]), P(ref["g"]), P(ref["m"]), P(ref["v"]), H, total, *hyper, 1, st), "nb_adam_step")
    ranks = [dict(w=dev(w0), h=dev(w0).half(), g=dev(grads[r]), m=torch.zeros(total, device="cuda"), v=torch.zeros(total, device="cuda"))
             for r in range(world)]
    G = (ctypes.c_void_p * world)(*[t["g"].data_ptr() for t in ranks])
    W = (ctypes.c_void_p * world)(*[t["h"].data_ptr() for t in ranks])
    for r in range(world):
        nb.check(lib.nb_adam_step_peer(P(ranks[r]["w"]), P(ranks[r]["m"]), P(ranks[r]["v"]), G, W, r, world, H, total, *hyper, st), "nb_adam_step_peer")
    torch.cuda.synchronize()
    shard = H // world
    for r in range(world):
        assert torch.equal(ranks[r]["h"], ref["h"]), "rank %d: fp16 parameters differ" % r
        lo, hi = r * shard, (r + 1) * shard
        for k in ("w", "m", "v"):
            assert torch.equal(ranks[r][k][lo:hi], ref[k][lo:hi]), (r, k)
            assert torch.equal(ranks[r][k][H:], ref[k][H:]), (r, k, "dense tail")
        untouched = torch.from_numpy(gsum[:H] == 0).cuda()
        assert torch.equal(ranks[r]["h"][:H][untouched], dev(w0).half()[:H][untouched])
        assert torch.equal(ranks[r]["g"], dev(grads[r]))            # the kernel leaves the gradients alone: the caller clears them
    assert lib.nb_adam_step_peer(P(ranks[0]["w"]), P(ranks[0]["m"]), P(ranks[0]["v"]), G, W, 0, 9, H, total, *hyper, st) == 4     # NB_ERR_LIMIT


def test_random_access_probe_counts_its_operations(cuda, nb):
    """nb_probe_random_access: the reduction kind adds (1, 2) to an entry per operation, so the table's sums give the
    operation count back; the gather kind leaves the table alone."""
    torch = cuda
    lib, P = nb.load(), nb.ptr
    table = torch.zeros((1 << 12, 2), dtype=torch.float32, device="cuda")
    nb.check(lib.nb_probe_random_access(1, 12, 8, 16, P(table), nb.stream_ptr()), "nb_probe_random_access")
    torch.cuda.synchronize()
    ops = 8 * 256 * 16
    assert float(table[:, 0].sum().item()) == ops and float(table[:, 1].sum().item()) == 2 * ops
    before = table.clone()
    nb.check(lib.nb_probe_random_access(0, 13, 8, 16, P(table), nb.stream_ptr()), "nb_probe_random_access")
    torch.cuda.synchronize()
    assert torch.equal(table, before)
    assert lib.nb_probe_random_access(2, 12, 8, 16, P(table), nb.stream_ptr()) == 1


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000, 70000])
def test_forward_with_the_loss_in_its_epilogue_equals_forward_then_loss_kernel(cuda, nb, n):
    """nb_field_forward_mse against nb_field_forward + nb_mse_loss_grad: same colours, sigma, saved encoding (bit for
    bit: the same code ran), the same fp16 colour gradient (the same expression on the same fp32 colour; the compiler may
    contract it differently in the two kernels, so a last-bit difference in a few values is allowed) and the same loss
    up to summation order."""
    torch = cuda
    pl = importlib.import_module("3dmaker_b200.pipeline")
    L, T = 16, 1 << 15
    model = pl.FieldModel(torch, L, T, 16, 1.3819, 64, 2, 64, 3)
    model.load_hashgrid(make_table(L, T, seed=3, amp=0.3))
    model.load_density_weights(*make_mlp(32, 64, 16, 2, seed=4, bias_amp=0.05)); model.load_color_weights(*make_mlp(32, 64, 8, 3, seed=5, bias_amp=0.05))
    pos, dirs, tgt = _inputs(n, 17)
    got = {}
    for fused_loss in (False, True):
        tr = pl.SampleTrainer(model, n, loss_scale=128.0, density_bias=1.0, fused=True, ordered=False, fused_loss=fused_loss)
        assert tr.fused_loss == fused_loss
        tr.pos.copy_(torch.from_numpy(pos)); tr.dirs.copy_(torch.from_numpy(dirs)); tr.target.copy_(torch.from_numpy(tgt.view(np.float16)))
        tr.c_grad.fill_(7.0)
        model.g.zero_()
        tr.forward_backward(n)
        torch.cuda.synchronize()
        got[fused_loss] = dict(rgb=tr.c_out[:n].cpu().numpy().copy(), sigma=tr.sigma[:n].cpu().numpy().copy(), enc=dev_half_bits(tr.enc[:n]).copy(),
                               grad=half_vals(dev_half_bits(tr.c_grad[:n])).copy(), loss=float(tr.loss.item()), g=model.g.cpu().numpy().copy())
    model.g.zero_()
    a, b = got[False], got[True]
    assert np.array_equal(a["rgb"], b["rgb"]) and np.array_equal(a["sigma"], b["sigma"]) and np.array_equal(a["enc"], b["enc"])
    assert np.all(b["grad"][:, 3:] == 0)
    assert np.mean(a["grad"] != b["grad"]) < 1e-3 and rel_err(b["grad"], a["grad"]) <= 1e-3
    assert abs(a["loss"] - b["loss"]) <= 1e-5 * max(a["loss"], 1e-30)
    assert rel_err(b["g"], a["g"]) <= 2e-3
