"""Host-side driver of the field-training hot path (encode -> density MLP -> SH -> colour MLP -> loss ->
backward -> scatter -> Adam) over the C ABI.

This is the orchestration the reference spreads over TinyMLPHashGrid::forward/backward/step,
TinyMLP::forward/calculate_loss_and_grad/backward/step and the glue kernels of InstantNerf::trainWithRaysHit
(modules/NeRF/InstantNerf.cu:506-571), restated for one flat parameter arena:

    arena = [ hash table L*T*2 | density W, b | colour W, b ]     (fp32 master, fp16 copy, grad, m, v)

so the gradient of the whole model is one contiguous buffer (one allreduce under data parallelism) and one
Adam launch updates everything.  torch is used for device memory, streams and the process group only; every
kernel on the path is launched through libnerf_b200.so.
"""
import ctypes
import importlib

import numpy as np

nb = importlib.import_module("3dmaker_b200")


def _pad4(x):
    return (x + 3) // 4 * 4


class FieldModel:
    """Parameters of hash grid + density network + colour network in one arena, with Adam state."""

    def __init__(self, torch, num_levels=16, table_size=1 << 19, base_resolution=16, growth=1.3819, density_hidden=64,
                 density_layers=2, color_hidden=64, color_layers=3, training=True, stream=None, grad_alloc=None, exportable=False):
        """exportable: the gradient and the fp16 parameter copy are cudaMalloc allocations of their own (nb_device_alloc)
        instead of torch tensors, so that other ranks can map them (distributed.PeerMemory) for nb_adam_step_peer."""
        self.torch = torch
        self.lib = nb.load()
        self.grid = nb.grid_setup(num_levels, table_size, base_resolution, growth, stream)
        self.density = nb.mlp_desc(2 * num_levels, density_hidden, 16, density_layers, 0)
        self.color = nb.mlp_desc(32, color_hidden, 8, color_layers, 1)
        self.hash_count = num_levels * table_size * 2
        # arena offsets (elements)
        o = self.hash_count
        self.off_dw = o; o += self.density.weight_count
        self.off_db = o; o += self.density.bias_count
        self.off_cw = o; o += self.color.weight_count
        self.off_cb = o; o += self.color.bias_count
        self.total = _pad4(o)
        dev = "cuda"
        self.w = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self._own = []          # base addresses of nb_device_alloc allocations, freed with the model
        self.w_h = self._exportable(self.total, np.float16) if exportable else torch.zeros(self.total, dtype=torch.float16, device=dev)
        self.training = training
        if training:
            # grad_alloc(count, dtype): where the gradient lives, e.g. distributed.CollectiveBuffers.zeros for data parallelism
            if exportable:
                self.g = self._exportable(self.total, np.float32)
            else:
                self.g = grad_alloc(self.total, torch.float32) if grad_alloc is not None else torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.m = torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.v = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.step_count = 0

    def _exportable(self, count, dtype):
        nm = importlib.import_module("3dmaker_b200.nerf")
        ptr = ctypes.c_void_p()
        nb.check(self.lib.nb_device_alloc(count * np.dtype(dtype).itemsize, ctypes.byref(ptr)), "nb_device_alloc")
        self._own.append(ptr.value)
        return nm.view_tensor(self.torch, ptr.value, count, dtype)

    def __del__(self):
        try:
            for p in getattr(self, "_own", []):
                self.lib.nb_device_free(ctypes.c_void_p(p))
            self._own = []
        except Exception:
            pass

    # ---- parameter I/O (host numpy <-> arena), mirrors loadHashgrid / loadWeights of the reference classes
    def load_hashgrid(self, table_f32):
        t = self.torch.from_numpy(np.ascontiguousarray(table_f32, np.float32).ravel()).cuda()
        assert t.numel() == self.hash_count
        self.w[:self.hash_count].copy_(t)
        self.w_h[:self.hash_count].copy_(t.half())

    def load_density_weights(self, W, b):
        self._load(self.off_dw, self.density.weight_count, W)
        self._load(self.off_db, self.density.bias_count, b)

    def load_color_weights(self, W, b):
        self._load(self.off_cw, self.color.weight_count, W)
        self._load(self.off_cb, self.color.bias_count, b)

    def _load(self, off, count, arr):
        t = self.torch.from_numpy(np.ascontiguousarray(arr, np.float32).ravel()).cuda()
        assert t.numel() == count
        self.w[off:off + count].copy_(t)
        self.w_h[off:off + count].copy_(t.half())

    def view(self, which, off, count):
        return getattr(self, which)[off:off + count]

    def ptr(self, which, off):
        t = getattr(self, which)
        return ctypes.c_void_p(t.data_ptr() + off * t.element_size())

    # ---- the table gradient in the precision the library currently keeps it in (nb.set_grad_table_half) ------------
    def hash_grad(self):
        """The hash part of the gradient as the library wrote it: fp32 [hash_count], or with the half-precision table
        fp16 [hash_count] packed at the start of the same memory and scaled by nb.grad_table_scale()."""
        if nb.grad_table_half():
            return self.g[:self.hash_count].view(self.torch.float16)[:self.hash_count]
        return self.g[:self.hash_count]

    def hash_grad_f32(self):
        """The table gradient as fp32 values without the half-precision table's extra scale (a copy)."""
        return self.hash_grad().float() / nb.grad_table_scale()

    def hash_grad_ptr(self, off):
        t = self.hash_grad()
        return ctypes.c_void_p(t.data_ptr() + off * t.element_size())


class SampleTrainer:
    """One optimizer step on explicit samples (position, view direction, target colour):
    the 'encode + MLP fwd/bwd + Adam' step of the benchmark.  Buffers are sized once for max_batch."""

    def __init__(self, model, max_batch, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-15, loss_scale=128.0, density_bias=0.0, fused=None, fused_scatter=None,
                 ordered=None, fused_loss=None):
        """fused=None picks the two-kernel field path (nb_field_forward / nb_field_backward) when it is built for
        the model's shapes, else the kernel-by-kernel sequence; True / False force one of them.  fused_scatter
        (default: on with the fused path) lets the backward kernel scatter the table gradient itself.  ordered
        (default: off) sorts the samples of every step by brick first (nb_sample_order) and runs the field kernels in
        that order (nb_field_forward_ordered / nb_field_backward_ordered); measured on uniformly scattered samples it
        does not pay - the eleven hashed levels, whose entries have no locality in any order, set the pace.  fused_loss
        (default: on with the fused, unordered path) takes the MSE loss and its gradient in the forward kernel's epilogue
        (nb_field_forward_mse) instead of a launch of its own."""
        torch = model.torch
        self.model, self.torch, self.lib = model, torch, model.lib
        self.max_batch = max_batch
        self.lr, self.beta1, self.beta2, self.eps, self.loss_scale, self.density_bias = lr, beta1, beta2, eps, loss_scale, density_bias
        supported = bool(self.lib.nb_field_supported(ctypes.byref(model.grid), ctypes.byref(model.density), ctypes.byref(model.color)))
        if fused and not supported:
            raise nb.NerfB200Error("the fused field kernels are not built for these network shapes")
        self.fused = supported if fused is None else bool(fused)
        self.fused_scatter = self.fused if fused_scatter is None else (bool(fused_scatter) and self.fused)
        self.ordered = False if ordered is None else (bool(ordered) and self.fused)
        self.fused_loss = (self.fused and not self.ordered) if fused_loss is None else (bool(fused_loss) and self.fused and not self.ordered)
        n, dev = max_batch, "cuda"
        d, c = model.density, model.color
        f16, f32 = torch.float16, torch.float32
        self.pos = torch.zeros((n, 4), dtype=f32, device=dev)
        self.dirs = torch.zeros((n, 3), dtype=f32, device=dev)
        self.target = torch.zeros((n, 8), dtype=f16, device=dev)
        self.enc = torch.zeros((n, d.input_dim), dtype=f16, device=dev)
        self.sigma = torch.zeros(n, dtype=f32, device=dev)
        self.c_out = torch.zeros((n, 8), dtype=f32, device=dev)
        self.c_grad = torch.zeros((n, 8), dtype=f16, device=dev)
        self.d_enc = torch.zeros((n, d.input_dim), dtype=f16, device=dev)
        self.loss = torch.zeros(1, dtype=f32, device=dev)
        if self.ordered:
            self.order = torch.zeros(n, dtype=torch.int32, device=dev)
            self.order_scratch = torch.zeros(int(self.lib.nb_sample_order_scratch_bytes()) // 4, dtype=torch.int32, device=dev)
        if self.fused:
            self.logit0 = torch.zeros(n, dtype=f32, device=dev)
        else:
            self.ray_idx = torch.arange(n, dtype=torch.int32, device=dev)
            self.d_acts = torch.zeros((max(d.num_layers - 1, 1), n, d.hidden_dim), dtype=f16, device=dev)
            self.d_out = torch.zeros((n, 16), dtype=f32, device=dev)
            self.c_in = torch.zeros((n, 32), dtype=f16, device=dev)
            self.c_acts = torch.zeros((max(c.num_layers - 1, 1), n, c.hidden_dim), dtype=f16, device=dev)
            self.c_dx = torch.zeros((n, 32), dtype=f16, device=dev)
            self.d_grad = torch.zeros((n, 16), dtype=f16, device=dev)

    def forward_backward(self, n, stream=None):
        """Everything of a step except the optimizer, on inputs already in self.pos / dirs / target."""
        m, lib, P = self.model, self.lib, nb.ptr
        st = nb.stream_ptr(stream)
        if n > self.max_batch:
            raise nb.NerfB200Error("batch exceeds max_batch")
        nb.check(lib.nb_zero_async(P(self.loss), 4, st), "nb_zero_async")
        if self.fused and self.ordered:
            gs = ctypes.byref(m.grid) if self.fused_scatter else None
            nb.check(lib.nb_sample_order(P(self.pos), n, P(self.order), P(self.order_scratch), st), "nb_sample_order")
            nb.check(lib.nb_field_forward_ordered(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(self.pos), m.ptr("w_h", 0),
                                                  P(self.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                                  m.ptr("w", m.off_cb), n, P(self.order), self.density_bias, P(self.enc), P(self.sigma),
                                                  P(self.logit0), P(self.c_out), 8, st), "nb_field_forward_ordered")
            nb.check(lib.nb_mse_loss_grad(P(self.c_out), P(self.target), P(self.c_grad), P(self.loss), n, 8, 3, self.loss_scale, 1, st),
                     "nb_mse_loss_grad")
            nb.check(lib.nb_field_backward_ordered(ctypes.byref(m.density), ctypes.byref(m.color), P(self.enc), P(self.dirs), None, 0,
                                                   m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n,
                                                   P(self.order), P(self.c_grad), None, m.ptr("g", m.off_dw), m.ptr("g", m.off_db),
                                                   m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(self.d_enc), gs,
                                                   P(self.pos) if self.fused_scatter else None, m.ptr("g", 0) if self.fused_scatter else None, st),
                     "nb_field_backward_ordered")
            if self.fused_scatter:
                return
        elif self.fused:
            if self.fused_loss:
                nb.check(lib.nb_field_forward_mse(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(self.pos), m.ptr("w_h", 0),
                                                  P(self.dirs), m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                                  m.ptr("w", m.off_cb), n, self.density_bias, P(self.enc), P(self.sigma), P(self.logit0),
                                                  P(self.c_out), 8, P(self.target), P(self.c_grad), P(self.loss), self.loss_scale, st),
                         "nb_field_forward_mse")
            else:
                nb.check(lib.nb_field_forward(ctypes.byref(m.grid), ctypes.byref(m.density), ctypes.byref(m.color), P(self.pos), m.ptr("w_h", 0),
                                              P(self.dirs), None, 0, m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw),
                                              m.ptr("w", m.off_cb), n, self.density_bias, P(self.enc), P(self.sigma), P(self.logit0),
                                              P(self.c_out), 8, st), "nb_field_forward")
                nb.check(lib.nb_mse_loss_grad(P(self.c_out), P(self.target), P(self.c_grad), P(self.loss), n, 8, 3, self.loss_scale, 1, st),
                         "nb_mse_loss_grad")
            nb.check(lib.nb_field_backward(ctypes.byref(m.density), ctypes.byref(m.color), P(self.enc), P(self.dirs), None, 0,
                                           m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n,
                                           P(self.c_grad), None, m.ptr("g", m.off_dw), m.ptr("g", m.off_db), m.ptr("g", m.off_cw),
                                           m.ptr("g", m.off_cb), P(self.d_enc), ctypes.byref(m.grid) if self.fused_scatter else None,
                                           P(self.pos) if self.fused_scatter else None, m.ptr("g", 0) if self.fused_scatter else None,
                                           st), "nb_field_backward")
            if self.fused_scatter:
                return
        else:
            nb.check(lib.nb_grid_mlp_forward(ctypes.byref(m.grid), ctypes.byref(m.density), P(self.pos), m.ptr("w_h", 0),
                                             m.ptr("w_h", m.off_dw), m.ptr("w", m.off_db), n, P(self.d_out), P(self.enc), P(self.d_acts),
                                             st), "nb_grid_mlp_forward")
            nb.check(lib.nb_sh_gather(P(self.dirs), P(self.ray_idx), 0, n, self.density_bias, P(self.d_out), P(self.c_in), P(self.sigma),
                                      st), "nb_sh_gather")
            nb.check(lib.nb_mlp_forward(ctypes.byref(m.color), P(self.c_in), m.ptr("w_h", m.off_cw), m.ptr("w", m.off_cb), n,
                                        P(self.c_out), P(self.c_acts), st), "nb_mlp_forward")
            nb.check(lib.nb_mse_loss_grad(P(self.c_out), P(self.target), P(self.c_grad), P(self.loss), n, 8, 3, self.loss_scale, 1, st),
                     "nb_mse_loss_grad")
            nb.check(lib.nb_mlp_backward(ctypes.byref(m.color), P(self.c_grad), m.ptr("w_h", m.off_cw), P(self.c_in), P(self.c_acts), n,
                                         m.ptr("g", m.off_cw), m.ptr("g", m.off_cb), P(self.c_dx), st), "nb_mlp_backward(colour)")
            nb.check(lib.nb_density_grad(n, None, P(self.c_dx), P(self.d_grad), st), "nb_density_grad")
            nb.check(lib.nb_mlp_backward(ctypes.byref(m.density), P(self.d_grad), m.ptr("w_h", m.off_dw), P(self.enc), P(self.d_acts), n,
                                         m.ptr("g", m.off_dw), m.ptr("g", m.off_db), P(self.d_enc), st), "nb_mlp_backward(density)")
        nb.check(lib.nb_hash_scatter_backward(ctypes.byref(m.grid), P(self.pos), P(self.d_enc), n, m.ptr("g", 0), st),
                 "nb_hash_scatter_backward")

    def encoded(self, n):
        """The encoded features the last forward saved, in SAMPLE order (the ordered kernels keep them in the order they
        visited the samples).  For tests; allocates."""
        if not (self.fused and self.ordered):
            return self.enc[:n]
        out = self.torch.empty_like(self.enc[:n])
        out[self.order[:n].long()] = self.enc[:n]
        return out

    def optimizer_step(self, stream=None):
        """Fused Adam over the whole arena; bias corrections as TinyMLPHashGrid::step (step counter capped at 50000)."""
        m = self.model
        if m.step_count < 50000:
            m.step_count += 1
        bc1 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta1), np.float32(m.step_count)))
        bc2 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta2), np.float32(m.step_count)))
        nb.check(self.lib.nb_adam_step(m.ptr("w", 0), m.ptr("w_h", 0), m.ptr("g", 0), m.ptr("m", 0), m.ptr("v", 0), m.hash_count,
                                       m.total, self.lr, self.beta1, self.beta2, self.eps, float(bc1), float(bc2),
                                       1.0 / self.loss_scale, 1, nb.stream_ptr(stream)), "nb_adam_step")

    def optimizer_step_sharded(self, dist, stream=None):
        """Data-parallel tail of a step with the hash table's optimizer state used shard-wise: reduce-scatter of the table
        gradient (each rank receives the summed gradient of its 1/N slice), Adam on that slice only, all-gather of the
        updated fp16 slice - the copy the forward reads.  Against allreduce + full Adam this moves 3/4 of the bytes over
        NVLink (fp32 gradient one way, fp16 parameters back) and divides the Adam launch by N.  The small dense tail
        (network weights and biases) is allreduced and updated by every rank.  Every rank ends with identical fp16
        parameters; the fp32 master copy, m and v of a slice are current on its owner only (gather_master() collects them)."""
        m = self.model
        world, rank = dist.get_world_size(), dist.get_rank()
        H = m.hash_count
        if H % (4 * world) != 0:
            raise nb.NerfB200Error("hash table size must be divisible by 4 x ranks")
        shard = H // world
        lo, hi = rank * shard, (rank + 1) * shard
        if m.step_count < 50000:
            m.step_count += 1
        bc1 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta1), np.float32(m.step_count)))
        bc2 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta2), np.float32(m.step_count)))
        hyper = (self.lr, self.beta1, self.beta2, self.eps, float(bc1), float(bc2), 1.0 / self.loss_scale, 1, nb.stream_ptr(stream))
        gh = m.hash_grad()                                                      # fp32, or fp16 with the half-precision table
        dist.reduce_scatter_tensor(gh[lo:hi], gh, op=dist.ReduceOp.SUM)         # in place: the output is this rank's slice
        dist.all_reduce(m.g[H:], op=dist.ReduceOp.SUM)
        nb.check(self.lib.nb_adam_step(m.ptr("w", lo), m.ptr("w_h", lo), m.hash_grad_ptr(lo), m.ptr("m", lo), m.ptr("v", lo), shard, shard, *hyper),
                 "nb_adam_step(table slice)")
        nb.check(self.lib.nb_adam_step(m.ptr("w", H), m.ptr("w_h", H), m.ptr("g", H), m.ptr("m", H), m.ptr("v", H), 0, m.total - H, *hyper),
                 "nb_adam_step(networks)")
        # the other slices still hold this rank's unreduced gradient: clear them for the next step's accumulation
        gb = gh.element_size()
        if lo > 0:
            nb.check(self.lib.nb_zero_async(m.hash_grad_ptr(0), lo * gb, nb.stream_ptr(stream)), "nb_zero_async")
        if hi < H:
            nb.check(self.lib.nb_zero_async(m.hash_grad_ptr(hi), (H - hi) * gb, nb.stream_ptr(stream)), "nb_zero_async")
        dist.all_gather_into_tensor(m.w_h[:H], m.w_h[lo:hi])                        # in place as well

    def optimizer_step_peer(self, dist, stream=None):
        """Data-parallel tail of a step as one kernel per rank (nb_adam_step_peer): the model must be `exportable`.  The
        first call maps the other ranks' gradient and fp16 parameter arrays (distributed.PeerMemory).  Per step: a
        one-element all-reduce as barrier, the kernel, the barrier again, then this rank's gradient is cleared."""
        m = self.model
        if not hasattr(self, "_peers"):
            D = importlib.import_module("3dmaker_b200.distributed")
            if not m._own:
                raise nb.NerfB200Error("optimizer_step_peer needs FieldModel(exportable=True)")
            self._peers = (D.PeerMemory(nb, dist, m.g.data_ptr()), D.PeerMemory(nb, dist, m.w_h.data_ptr()))
            self._token = self.torch.zeros(1, dtype=self.torch.float32, device=m.g.device)
            world = dist.get_world_size()
            self._peer_arrays = ((ctypes.c_void_p * world)(*self._peers[0].pointers), (ctypes.c_void_p * world)(*self._peers[1].pointers))
        world, rank = dist.get_world_size(), dist.get_rank()
        if m.step_count < 50000:
            m.step_count += 1
        bc1 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta1), np.float32(m.step_count)))
        bc2 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta2), np.float32(m.step_count)))
        dist.all_reduce(self._token)
        nb.check(self.lib.nb_adam_step_peer(m.ptr("w", 0), m.ptr("m", 0), m.ptr("v", 0), self._peer_arrays[0], self._peer_arrays[1], rank, world,
                                            m.hash_count, m.total, self.lr, self.beta1, self.beta2, self.eps, float(bc1), float(bc2),
                                            1.0 / self.loss_scale, nb.stream_ptr(stream)), "nb_adam_step_peer")
        dist.all_reduce(self._token)
        nb.check(self.lib.nb_zero_async(m.ptr("g", 0), m.total * 4, nb.stream_ptr(stream)), "nb_zero_async")

    def close_peers(self, dist):
        """Unmaps the other ranks' arrays (after a barrier: nobody's kernel may still be using them)."""
        if hasattr(self, "_peers"):
            self.torch.cuda.synchronize()
            dist.barrier()
            for p in self._peers:
                p.close()
            del self._peers

    def gather_master(self, dist):
        """After sharded steps: brings the fp32 master table of every slice to every rank (e.g. before saving)."""
        m = self.model
        world, rank = dist.get_world_size(), dist.get_rank()
        shard = m.hash_count // world
        dist.all_gather_into_tensor(m.w[:m.hash_count], m.w[rank * shard:(rank + 1) * shard])

    def optimizer_step_synced(self, dist, chunks=4, stream=None):
        """Data-parallel tail of a step: SUM-allreduce of the gradient arena and Adam, pipelined over `chunks` slices of
        the arena - the allreduce of slice c+1 (NCCL's stream) runs while Adam updates slice c, so only the first
        exchange and the last update are exposed.  Same result as one allreduce followed by optimizer_step()."""
        m = self.model
        if nb.grad_table_half():
            raise nb.NerfB200Error("the half-precision gradient table cannot be all-reduced as one fp32 array: use dp_mode 'peer' or 'sharded'")
        if m.step_count < 50000:
            m.step_count += 1
        bc1 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta1), np.float32(m.step_count)))
        bc2 = np.float32(1.0) - np.float32(np.power(np.float32(self.beta2), np.float32(m.step_count)))
        step = (m.total // chunks + 3) // 4 * 4
        bounds = [min(c * step, m.total) for c in range(chunks)] + [m.total]
        works = [dist.all_reduce(m.g[bounds[c]:bounds[c + 1]], op=dist.ReduceOp.SUM, async_op=True) for c in range(chunks)]
        for c in range(chunks):
            lo, hi = bounds[c], bounds[c + 1]
            if hi <= lo:
                continue
            works[c].wait()                                 # the current stream waits for this slice's exchange
            sparse = max(0, min(hi, m.hash_count) - lo)     # the slice's share of the hash table (sparse Adam rule)
            nb.check(self.lib.nb_adam_step(m.ptr("w", lo), m.ptr("w_h", lo), m.ptr("g", lo), m.ptr("m", lo), m.ptr("v", lo), sparse, hi - lo,
                                           self.lr, self.beta1, self.beta2, self.eps, float(bc1), float(bc2), 1.0 / self.loss_scale, 1,
                                           nb.stream_ptr(stream)), "nb_adam_step")

    def step_device(self, n, stream=None, grad_sync=None):
        """One full step on device-resident inputs.  grad_sync: a callable grad_sync(grad_tensor) that runs between
        backward and Adam, or torch.distributed itself (initialised) for the pipelined allreduce + Adam."""
        self.forward_backward(n, stream)
        if grad_sync is not None and hasattr(grad_sync, "all_reduce"):
            # a torch.distributed module: sharded optimizer (default) or the pipelined allreduce + Adam
            mode = getattr(self, "dp_mode", "sharded")
            if mode == "peer":
                self.optimizer_step_peer(grad_sync, stream=stream)
            elif mode == "sharded":
                self.optimizer_step_sharded(grad_sync, stream=stream)
            else:
                self.optimizer_step_synced(grad_sync, stream=stream)
            return
        if grad_sync is not None:
            if nb.grad_table_half():
                raise nb.NerfB200Error("the half-precision gradient table cannot be exchanged as one fp32 array: use dp_mode 'peer' or 'sharded'")
            grad_sync(self.model.g)
        self.optimizer_step(stream)

    # ---- pipelined host input: the copy of the next batch overlaps the step on the current one -----------------
    def prefetch(self, pos4, dirs3, target_h8):
        """Enqueues the host->device copy of one batch (pinned tensors) on a copy stream into the input slot that
        the running step is not using.  Pair every call with one step_prefetched().  The batch comes either in the
        kernels' own layouts (positions [n, 4] float32, targets [n, 8] float16: 44 bytes per sample with the directions) or
        compact (positions [n, 3], targets [n, 3]: 30 bytes), in which case nb_unpack_samples widens it on the device,
        on the copy stream."""
        torch = self.torch
        compact = pos4.shape[1] == 3
        if not hasattr(self, "_slots"):
            self._copy_stream = torch.cuda.Stream()
            self._slots = [(self.pos, self.dirs, self.target),
                           (torch.empty_like(self.pos), torch.empty_like(self.dirs), torch.empty_like(self.target))]
            self._ready = [torch.cuda.Event(), torch.cuda.Event()]
            self._free = [torch.cuda.Event(), torch.cuda.Event()]
            self._next, self._queued = 0, []
        k = self._next
        n = pos4.shape[0]
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(self._free[k])      # the step that last read this slot has finished
            p, d, t = self._slots[k]
            d[:n].copy_(dirs3, non_blocking=True)
            if compact:
                if not hasattr(self, "_compact"):
                    self._compact = [(torch.empty((self.max_batch, 3), dtype=torch.float32, device=p.device),
                                      torch.empty((self.max_batch, 3), dtype=torch.float16, device=p.device)) for _ in range(2)]
                p3, t3 = self._compact[k]
                p3[:n].copy_(pos4, non_blocking=True); t3[:n].copy_(target_h8, non_blocking=True)
                nb.check(self.lib.nb_unpack_samples(nb.ptr(p3), nb.ptr(t3), n, nb.ptr(p), nb.ptr(t), nb.stream_ptr(self._copy_stream)),
                         "nb_unpack_samples")
            else:
                p[:n].copy_(pos4, non_blocking=True); t[:n].copy_(target_h8, non_blocking=True)
            self._ready[k].record(self._copy_stream)
        self._queued.append((k, n))
        self._next = 1 - k

    def step_prefetched(self, stream=None, grad_sync=None, lag=True):
        """Runs one full step on the oldest prefetched batch.  The step's loss travels to pinned host memory by an
        asynchronous 4-byte copy enqueued behind the step; with lag=True (default) the call returns the mean squared error
        of the PREVIOUS step, whose copy has long finished, so the host never waits for the step it has just enqueued
        and the device never waits for the host (None on the first call; flush_loss() returns the last one).  lag=False
        waits for this step's own loss."""
        torch = self.torch
        k, n = self._queued.pop(0)
        cur = torch.cuda.current_stream()
        cur.wait_event(self._ready[k])
        self.pos, self.dirs, self.target = self._slots[k]
        self.step_device(n, stream, grad_sync)
        self._free[k].record(cur)
        if not hasattr(self, "_loss_host"):
            self._loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._loss_done = [torch.cuda.Event(), torch.cuda.Event()]
            self._loss_slot, self._loss_pending = 0, None
        j = self._loss_slot
        self._loss_host[j].copy_(self.loss, non_blocking=True)       # self.loss is re-zeroed by the next step, after this copy in stream order
        self._loss_done[j].record(cur)
        prev, self._loss_pending, self._loss_slot = self._loss_pending, (j, n), 1 - j
        if not lag:
            return self.flush_loss()
        if prev is None:
            return None
        self._loss_done[prev[0]].synchronize()
        return float(self._loss_host[prev[0]].item()) / (prev[1] * 3)

    def flush_loss(self):
        """Mean squared error of the last step enqueued by step_prefetched (waits for it)."""
        if getattr(self, "_loss_pending", None) is None:
            return None
        j, n = self._loss_pending
        self._loss_pending = None
        self._loss_done[j].synchronize()
        return float(self._loss_host[j].item()) / (n * 3)

    def step_host(self, pos4, dirs3, target_h8, stream=None, grad_sync=None):
        """One full step from pinned host tensors: copies inputs in, runs the step, returns the mean squared error
        (a device->host read of one float, which also synchronises)."""
        n = pos4.shape[0]
        self.pos[:n].copy_(pos4, non_blocking=True)
        self.dirs[:n].copy_(dirs3, non_blocking=True)
        self.target[:n].copy_(target_h8, non_blocking=True)
        self.step_device(n, stream, grad_sync)
        return float(self.loss.item()) / (n * 3)
