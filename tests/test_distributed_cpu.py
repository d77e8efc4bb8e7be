"""Data-parallel training and pixel-sharded rendering logic (3dmaker_b200/distributed.py) on two CPU ranks over gloo,
with a stand-in engine: the partitioning, the one-exchange-per-step rule, replica agreement and the frame gather are
host logic that needs no GPU."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

D = importlib.import_module("3dmaker_b200.distributed")


class FakeEngine:
    """A linear 'field': prediction = P[3, 6] @ [o, d]; squared error against the target; the gradient is normalised
    by (local rays x global scale) the way the scene engine normalises by the global ray count, summed over rays,
    handed to the sync hook, then applied with plain SGD.  max_rays mimics the sample batch that bounds one step."""

    SPARSE = 16     # the first 16 of the 18 parameters play the hash table (updated shard-wise by the sharded optimizer)

    def __init__(self, max_rays=1 << 30):
        self.w = torch.linspace(-0.5, 0.5, 18, dtype=torch.float32)
        self.w_h = self.w.half()          # the copy the "forward" reads, as in the real engine
        self.g = torch.zeros(18, dtype=torch.float32)
        self.scale, self.sync, self.single, self.steps, self.max_rays, self.consumed = 1, None, 0, 0, max_rays, 0
        self.shard, self.param_sync = None, None
        self.part = None

    def arena(self):
        class View:
            sparse_count, total = FakeEngine.SPARSE, 18
        return View()

    def set_optimizer_shard(self, rank, world, fn):
        self.shard, self.param_sync = ((rank, world), fn) if world > 1 and fn is not None else (None, None)

    def set_level_partition(self, rank, world, gather, exchange, reduce):
        self.part = (rank, world, gather, exchange, reduce) if world > 1 else None

    def sync_levels(self, master=False):
        """Owned table parameters to every rank (the real engine all-gathers whole levels)."""
        rank, world, gather, _, _ = self.part
        for arr in ([self.w_h, self.w] if master else [self.w_h]):
            mine = arr[rank:FakeEngine.SPARSE:world].contiguous()
            everybody = torch.zeros(world * mine.numel(), dtype=arr.dtype)
            gather(mine, everybody)
            for q in range(world):
                arr[q:FakeEngine.SPARSE:world] = everybody[q * mine.numel():(q + 1) * mine.numel()]

    def _partitioned_step(self, x, target, n_global):
        """The level partition's protocol on the linear field: table parameter j belongs to rank j % world.  Inputs of
        all ranks are gathered, every owner computes ITS parameters' share of every rank's prediction, the shares travel
        to the samples' ranks (all-to-all), the errors travel back (all-to-all), every owner forms the gradient of its
        parameters from all ranks' samples; the two dense parameters are reduced and updated by everybody."""
        rank, world, gather, exchange, reduce = self.part
        k, cap = x.shape[0], 64                                       # cap: fixed slot size, as the engine's batch capacity
        slot = torch.zeros((cap + 1, 6)); slot[:k] = x; slot[cap, 0] = k
        slots = torch.zeros((world, cap + 1, 6))
        gather(slot.view(-1), slots.view(-1))
        W = self.w_h.float().view(3, 6)
        own = torch.zeros(18, dtype=torch.bool); own[rank:FakeEngine.SPARSE:world] = True
        dense = torch.zeros(18, dtype=torch.bool); dense[FakeEngine.SPARSE:] = True
        W_own = torch.where(own.view(3, 6), W, torch.zeros_like(W))
        send = torch.stack([slots[q, :cap] @ W_own.t() for q in range(world)])          # [world][cap][3]: piece q for rank q
        recv = torch.zeros_like(send)
        exchange(send.view(-1), recv.view(-1))
        W_dense = torch.where(dense.view(3, 6), W, torch.zeros_like(W))
        pred = recv.sum(0)[:k] + x @ W_dense.t()
        err = torch.zeros((cap, 3)); err[:k] = pred - target
        back = torch.stack([err] * world)                                                # every owner needs this rank's errors
        got = torch.zeros_like(back)
        exchange(back.view(-1), got.view(-1))
        g = torch.zeros(3, 6)
        for q in range(world):
            cnt = int(slots[q, cap, 0].item())
            g += 2.0 * got[q, :cnt].t() @ slots[q, :cnt] / n_global
        self.g += torch.where(own, g.reshape(-1), torch.zeros(18))
        g_dense = (2.0 * err[:k].t() @ x / n_global).reshape(-1)
        tail = g_dense[FakeEngine.SPARSE:].clone()
        reduce(tail)
        self.g[FakeEngine.SPARSE:] += tail
        upd = own | dense
        self.w[upd] -= 0.1 * self.g[upd]
        self.w_h[upd] = self.w[upd].half()
        self.g.zero_()

    def set_global_ray_scale(self, s):
        self.scale = s

    def set_steps_per_call(self, k):
        self.single = k

    def set_grad_sync(self, fn):
        self.sync = fn

    def rays_consumed(self):
        return self.consumed

    def arena_tensor(self, name):
        return {"w": self.w, "g": self.g, "w_h": self.w_h}[name]

    def train_rays(self, o, d, rgb):
        n, done, taken = o.shape[0], 0, 0
        while (taken < self.single) if self.single else (done < n):
            k = min(self.max_rays, n - done)
            x = torch.cat([o[done:done + k], d[done:done + k]], dim=1)
            if self.part is not None:
                self._partitioned_step(x, rgb[done:done + k], n * self.scale)
                self.steps += 1; done += k; taken += 1; self.consumed = done
                continue
            err = x @ self.w_h.float().view(3, 6).t() - rgb[done:done + k]
            self.g += (2.0 * err.t() @ x / (n * self.scale)).reshape(-1)
            if self.sync is not None:
                self.sync(self.g)
            if self.shard is None:
                self.w -= 0.1 * self.g
                self.w_h.copy_(self.w.half())
            else:                          # this rank's slice of the table and the dense tail; then the slices are gathered
                (r, world), H = self.shard, FakeEngine.SPARSE
                lo, hi = r * H // world, (r + 1) * H // world
                for a, b in ((lo, hi), (H, 18)):
                    self.w[a:b] -= 0.1 * self.g[a:b]
                    self.w_h[a:b] = self.w[a:b].half()
                self.param_sync(self.w_h)
            self.g.zero_()
            self.steps += 1
            done += k
            taken += 1
            self.consumed = done
        return self.steps

    def render(self, o, d, out):
        out.copy_(o * 0.25 + d)


def _batch(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.rand((n, 3), generator=g), torch.rand((n, 3), generator=g), torch.rand((n, 3), generator=g)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, case):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        if case == "train":
            eng = FakeEngine()
            tr = D.DataParallelTrainer(torch, eng, dist)
            used = []
            for step in range(5):
                o, d, c = _batch(64, 100 + step)
                used.append(tr.train_rays(o, d, c))
            np.save(os.path.join(out_dir, "w%d.npy" % rank), eng.w.numpy())
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([tr.sync_calls, eng.steps, int(tr.replicas_in_sync())] + used))
        elif case == "sharded":
            # reduce-scatter + slice update + all-gather of the fp16 copy, with uneven per-rank sample batches
            eng = FakeEngine(max_rays=20 if rank == 1 else 1 << 30)
            tr = D.DataParallelTrainer(torch, eng, dist, steps_per_call=2, exchange="sharded")
            for c in range(4):
                tr.train_rays(*_batch(64, 40 + c))
            in_sync = int(tr.replicas_in_sync())
            stale = eng.w.clone()
            tr.gather_master()
            np.save(os.path.join(out_dir, "w%d.npy" % rank), eng.w.numpy())
            np.save(os.path.join(out_dir, "wh%d.npy" % rank), eng.w_h.float().numpy())
            np.save(os.path.join(out_dir, "stale%d.npy" % rank), stale.numpy())
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([tr.sync_calls, eng.steps, in_sync]))
            tr.close()
            assert eng.sync is None and eng.shard is None
        elif case == "sharded_vs_allreduce":
            eng = FakeEngine(max_rays=20 if rank == 1 else 1 << 30)
            tr = D.DataParallelTrainer(torch, eng, dist, steps_per_call=2, exchange="allreduce")
            for c in range(4):
                tr.train_rays(*_batch(64, 40 + c))
            np.save(os.path.join(out_dir, "ar_w%d.npy" % rank), eng.w.numpy())
        elif case == "levels":
            # table partitioned over the ranks: positions gathered, shares exchanged, errors exchanged back, dense tail reduced
            eng = FakeEngine(max_rays=20 if rank == 1 else 1 << 30)
            tr = D.DataParallelTrainer(torch, eng, dist, steps_per_call=2, exchange="levels")
            for c in range(4):
                tr.train_rays(*_batch(64, 40 + c))
            stale = eng.w_h.clone()
            in_sync = int(tr.replicas_in_sync())            # makes the table whole first
            tr.gather_master()
            np.save(os.path.join(out_dir, "lv_w%d.npy" % rank), eng.w.numpy())
            np.save(os.path.join(out_dir, "lv_stale%d.npy" % rank), stale.float().numpy())
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([eng.steps, in_sync]))
            tr.close()
            assert eng.part is None
        elif case == "overflow":
            # rank 1's sample batch holds only 20 of its 32 rays: it still takes ONE step and ONE exchange
            eng = FakeEngine(max_rays=20 if rank == 1 else 1 << 30)
            tr = D.DataParallelTrainer(torch, eng, dist)
            o, d, c = _batch(64, 7)
            used = tr.train_rays(o, d, c)
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([tr.sync_calls, eng.steps, int(tr.replicas_in_sync()), used]))
        elif case == "multistep":
            # three steps per call on every rank: rank 0 needs one step for its 32 rays, rank 1 two (20 + 12); the
            # steps a rank has no rays left for still exchange and update
            eng = FakeEngine(max_rays=20 if rank == 1 else 1 << 30)
            tr = D.DataParallelTrainer(torch, eng, dist, steps_per_call=3)
            used = [tr.train_rays(*_batch(64, 40 + c)) for c in range(2)]
            np.save(os.path.join(out_dir, "w%d.npy" % rank), eng.w.numpy())
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([tr.sync_calls, eng.steps, int(tr.replicas_in_sync())] + used))
        elif case == "drift":
            eng = FakeEngine()
            tr = D.DataParallelTrainer(torch, eng, dist)
            if rank == 1:
                eng.w[3] += 1e-7
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([int(tr.replicas_in_sync())]))
        elif case == "render":
            W, H = 50, 37                                     # 1850 pixels, tile 128 -> 15 tiles, ragged last tile
            def ray_fn(first, count, o, d):
                idx = torch.arange(first, first + count, dtype=torch.float32)
                o.copy_(torch.stack([idx, idx * 2, idx * 3], dim=1))
                d.copy_(torch.stack([idx % W, idx // W, torch.ones_like(idx)], dim=1))
            r = D.ShardedRenderer(torch, FakeEngine(), ray_fn, dist, tile=128)
            frame = r.render_frame(W * H, "cpu")
            assert (frame is None) == (rank != 0)

            def tiled_ray_fn(tile, first_tile, stride, count, o, d):      # all tiles of the rank in one call
                i = torch.arange(count)
                ray_fn_at = ((first_tile + (i // tile) * stride) * tile + i % tile).float()
                o.copy_(torch.stack([ray_fn_at, ray_fn_at * 2, ray_fn_at * 3], dim=1))
                d.copy_(torch.stack([ray_fn_at % W, ray_fn_at // W, torch.ones_like(ray_fn_at)], dim=1))
            frame2 = D.ShardedRenderer(torch, FakeEngine(), None, dist, tile=128, tiled_ray_fn=tiled_ray_fn).render_frame(W * H, "cpu")
            if rank == 0:
                assert torch.equal(frame, frame2)
                np.save(os.path.join(out_dir, "frame.npy"), frame.numpy())
            np.save(os.path.join(out_dir, "meta%d.npy" % rank), np.array([r.local_pixels(W * H)]))
    finally:
        dist.destroy_process_group()


def _run(case, tmp_path, world=2):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), case), nprocs=world, join=True)


def test_ray_and_pixel_partitions_cover_everything_once():
    for n, world in ((64, 2), (65537, 8), (7, 8), (0, 4)):
        spans = [D.ray_shard(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == n
        assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    for n, world, tile in ((1850, 2, 128), (1920 * 1080, 8, 4096), (5, 4, 4096), (4096 * 3, 3, 4096)):
        seen = np.zeros(n, np.int32)
        for r in range(world):
            for first, count in D.pixel_tiles(n, r, world, tile):
                seen[first:first + count] += 1
        assert np.all(seen == 1)
    assert D.gathered_bytes(1920 * 1080, 1) == 0
    assert D.gathered_bytes(1920 * 1080, 8) == 7 * 64 * 4096 * 12


def test_two_ranks_reproduce_the_single_process_gradient(tmp_path):
    _run("train", tmp_path)
    single = FakeEngine()
    tr = D.DataParallelTrainer(torch, single, None)
    for step in range(5):
        tr.train_rays(*_batch(64, 100 + step))
    w0, w1 = np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy")
    assert np.array_equal(w0, w1)                                   # replicas bit-identical after every rank's update
    assert np.allclose(w0, single.w.numpy(), rtol=1e-5, atol=1e-6)  # and equal to the one-GPU result (fp32 sum order aside)
    for r in range(2):
        meta = np.load(tmp_path / ("meta%d.npy" % r))
        assert meta[0] == 5 and meta[1] == 5 and meta[2] == 1       # one exchange per step
        assert list(meta[3:]) == [32] * 5


def test_a_rank_that_overflows_its_batch_still_exchanges_once(tmp_path):
    _run("overflow", tmp_path)
    m0, m1 = np.load(tmp_path / "meta0.npy"), np.load(tmp_path / "meta1.npy")
    assert list(m0) == [1, 1, 1, 32]
    assert list(m1) == [1, 1, 1, 20]


def test_fixed_number_of_steps_per_call_keeps_ranks_in_lock_step(tmp_path):
    _run("multistep", tmp_path)
    m0, m1 = np.load(tmp_path / "meta0.npy"), np.load(tmp_path / "meta1.npy")
    assert list(m0) == [6, 6, 1, 32, 32] and list(m1) == [6, 6, 1, 32, 32]
    assert np.array_equal(np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy"))


def test_sharded_optimizer_equals_the_allreduce_exchange(tmp_path):
    """Reduce-scatter, update of the own table slice, all-gather of the fp16 copy: every rank ends with the parameters the
    all-reduce + full update gives; before gather_master() a rank's master copy of the OTHER slice is stale, after it
    every rank holds all of it."""
    _run("sharded", tmp_path)
    _run("sharded_vs_allreduce", tmp_path)
    w0, w1 = np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy")
    assert np.array_equal(w0, w1)
    assert np.array_equal(np.load(tmp_path / "wh0.npy"), np.load(tmp_path / "wh1.npy"))
    assert np.allclose(w0, np.load(tmp_path / "ar_w0.npy"), rtol=1e-5, atol=1e-6)
    assert np.array_equal(np.load(tmp_path / "wh0.npy"), w0.astype(np.float16).astype(np.float32))
    s0, s1 = np.load(tmp_path / "stale0.npy"), np.load(tmp_path / "stale1.npy")
    assert np.array_equal(s0[:8], w0[:8]) and not np.array_equal(s0[8:16], w0[8:16])      # rank 0 owns the first half
    assert np.array_equal(s1[8:16], w0[8:16]) and not np.array_equal(s1[:8], w0[:8])
    assert np.array_equal(s0[16:], w0[16:]) and np.array_equal(s1[16:], w0[16:])            # the dense tail is replicated
    for r in range(2):
        meta = np.load(tmp_path / ("meta%d.npy" % r))
        assert list(meta) == [8, 8, 1]


def test_level_partition_equals_the_allreduce_exchange(tmp_path):
    """exchange="levels" through gloo: the three collectives deliver the right blocks (the fake engine runs the engine's
    protocol on a linear field), every rank ends with the parameters the all-reduce exchange gives, and before the table
    is made whole a rank's copy of the parameters it does not own is stale."""
    _run("levels", tmp_path)
    _run("sharded_vs_allreduce", tmp_path)
    w0, w1 = np.load(tmp_path / "lv_w0.npy"), np.load(tmp_path / "lv_w1.npy")
    assert np.array_equal(w0, w1)
    assert np.allclose(w0, np.load(tmp_path / "ar_w0.npy"), rtol=1e-4, atol=1e-5)
    s0 = np.load(tmp_path / "lv_stale0.npy")
    half = w0.astype(np.float16).astype(np.float32)
    assert np.array_equal(s0[0:16:2], half[0:16:2]) and not np.array_equal(s0[1:16:2], half[1:16:2])   # rank 0 owns the even ones
    for r in range(2):
        assert list(np.load(tmp_path / ("meta%d.npy" % r))) == [8, 1]


def test_replica_drift_is_detected(tmp_path):
    _run("drift", tmp_path)
    assert np.load(tmp_path / "meta0.npy")[0] == 0 and np.load(tmp_path / "meta1.npy")[0] == 0


def test_sharded_frame_equals_the_single_process_frame(tmp_path):
    _run("render", tmp_path)
    W, H = 50, 37
    idx = np.arange(W * H, dtype=np.float32)
    o = np.stack([idx, idx * 2, idx * 3], axis=1)
    d = np.stack([idx % W, idx // W, np.ones_like(idx)], axis=1)
    assert np.array_equal(np.load(tmp_path / "frame.npy"), o * 0.25 + d)
    assert np.load(tmp_path / "meta0.npy")[0] + np.load(tmp_path / "meta1.npy")[0] == W * H


def test_uneven_global_batch_is_rejected():
    tr = D.DataParallelTrainer(torch, FakeEngine(), None)
    tr.world = 2
    with pytest.raises(ValueError):
        tr.train_rays(*_batch(63, 1))


def test_collective_buffers_fall_back_to_plain_tensors_without_a_nccl_allocator():
    # no process group / a backend without its own allocator: ordinary tensors, nothing to register
    b = D.CollectiveBuffers(torch, dist, "cpu")
    t = b.zeros(12, torch.float32)
    assert t.shape == (12,) and t.dtype == torch.float32 and float(t.abs().sum()) == 0.0
    assert b.register() is False
