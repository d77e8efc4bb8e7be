"""One process per GPU: data-parallel training and pixel-sharded rendering over torch.distributed.

The reference is single-GPU.  Its training step normalises the loss gradients by the number of rays of the whole batch
(compute_color_grad, modules/NeRF/otherKernels.cu:370) and sums sample gradients into one table, so splitting the rays
of a batch over ranks and SUM-allreducing the flat gradient arena before the optimizer reproduces the single-GPU
gradient; every rank then applies the same Adam update to its replica.  Rendering needs no exchange at all: pixels are
independent, each rank renders its tiles and the frame is gathered once.

Nothing here launches a kernel: the engine (3dmaker_b200.nerf.InstantNerf, or any object with the same few methods)
does.  The partitioning, the step agreement and the gather are host logic and run on any backend (NCCL on GPUs, gloo
on CPU).
"""

def ray_shard(num_rays, rank, world):
    """Rays [start, start + count) of a global batch that `rank` trains on: contiguous, sizes differ by at most one."""
    start = rank * num_rays // world
    end = (rank + 1) * num_rays // world
    return start, end - start


def pixel_tiles(num_pixels, rank, world, tile=4096):
    """Runs of `tile` consecutive pixels dealt round-robin to the ranks: [(first_pixel, count), ...] of `rank`.
    Interleaving balances frames whose cost per pixel varies smoothly over the image (empty sky vs the object)."""
    out = []
    num_tiles = (num_pixels + tile - 1) // tile
    for t in range(rank, num_tiles, world):
        first = t * tile
        out.append((first, min(tile, num_pixels - first)))
    return out


def merge_runs(tiles):
    """Joins tiles that follow one another in the frame: [(first, count), ...] with as few entries as possible."""
    out = []
    for first, count in tiles:
        if out and out[-1][0] + out[-1][1] == first:
            out[-1] = (out[-1][0], out[-1][1] + count)
        else:
            out.append((first, count))
    return out


class CollectiveBuffers:
    """Device memory the communicator knows in advance: tensors come from NCCL's own allocator and the pool is
    registered with the process group, so that collectives work on them in place through NVSwitch instead of staging
    through NCCL's internal buffers (measured on 8 B200: the 67 MB gradient all-reduce 0.28 -> 0.20 ms).  Where the
    backend has no such allocator (gloo, older torch) the tensors are ordinary ones and everything still works."""

    def __init__(self, torch, dist, device):
        self.torch, self.device = torch, device
        self.pool = self.backend = None
        try:
            backend = dist.distributed_c10d._get_default_group()._get_backend(torch.device(device))
            self.pool = torch.cuda.MemPool(backend.mem_allocator)
            self.backend = backend
        except Exception:          # no NCCL allocator here: plain tensors
            self.pool = self.backend = None
        self.registered = False

    def zeros(self, count, dtype):
        torch = self.torch
        if self.pool is None:
            return torch.zeros(count, dtype=dtype, device=self.device)
        with torch.cuda.use_mem_pool(self.pool):
            t = torch.zeros(count, dtype=dtype, device=self.device)
        return t

    def register(self):
        """Call once after the last zeros(): makes the pool's memory known to the communicator."""
        if self.backend is not None and not self.registered:
            self.backend.register_mem_pool(self.pool)
            self.registered = True
        return self.registered


def _grad_table_half():
    """Whether the CUDA library keeps the table gradient in half precision (False when the library is not built: the
    host-side logic of this module is also exercised without it)."""
    import importlib
    nbm = importlib.import_module("3dmaker_b200")
    try:
        return nbm.grad_table_half()
    except nbm.NerfB200Error:
        return False


class PeerMemory:
    """Addresses of every rank's copy of an array, for kernels that read and write peer memory (nb_adam_step_peer):
    each rank exports its allocation (cudaIpcGetMemHandle through nb_ipc_export - the address must be the start of a
    cudaMalloc allocation), the handles travel through the process group, every rank opens the others'.  pointers[r] is
    rank r's array as THIS process addresses it.  One node only; needs peer access between the GPUs (NVLink)."""

    def __init__(self, nb, dist, base_ptr):
        import ctypes
        self.nb, self.lib = nb, nb.load()
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        handle = ctypes.create_string_buffer(64)
        nb.check(self.lib.nb_ipc_export(ctypes.c_void_p(int(base_ptr)), handle), "nb_ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw)
        self.pointers, self._opened = [], []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.pointers.append(int(base_ptr))
                continue
            p = ctypes.c_void_p()
            nb.check(self.lib.nb_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)), "nb_ipc_open")
            self.pointers.append(int(p.value))
            self._opened.append(int(p.value))

    def close(self):
        import ctypes
        for p in self._opened:
            self.lib.nb_ipc_close(ctypes.c_void_p(p))
        self._opened = []


class DataParallelTrainer:
    """Wraps a scene engine so that train_rays() takes the GLOBAL ray batch.

    engine needs: set_global_ray_scale(int), set_steps_per_call(int), set_grad_sync(fn), train_rays(o, d, rgb) -> total
    optimizer steps so far, rays_consumed(), arena_tensor(name), arena(); for exchange="sharded" also
    set_optimizer_shard(rank, world, fn).  dist is torch.distributed (already initialised) or None for a single process.
    registered_gradient (NCCL on GPUs): the engine's gradient arena is moved into CollectiveBuffers memory
    (engine.set_grad_buffer).

    exchange: how the ranks' gradients meet the optimizer.
      "allreduce"  one SUM all-reduce of the flat gradient arena, every rank runs Adam on everything (replicated state);
      "sharded"    reduce-scatter of the hash-table gradient in place, Adam on this rank's 1/N slice of the table (and
                   on the small dense tail, which is all-reduced), all-gather of the updated fp16 slices: 3/4 of the
                   all-reduce's bytes on the wire and 1/N of the optimizer's memory traffic - the part of a step that
                   does not shrink with the number of ranks when the batch is split (2^22-entry levels: 4.6 GB per
                   Adam launch).  The fp32 master copy and the moments of a slice live on its owner; gather_master()
                   collects the master copy (before saving);
      "peer"       the same three stages as ONE kernel per rank (nb_adam_step_peer): the slice's gradients are loaded
                   from every rank's memory over NVLink, the updated fp16 slice is stored into every rank's forward
                   copy, a one-element all-reduce before and after keeps the ranks together.  GPUs of one node only;
                   the engine's arenas must be its own allocations (no registered_gradient);
      "levels"     the table is not replicated at all: rank r OWNS levels r, r + N, ... (engine.set_level_partition).  Per
                   step one all-gather of the ranks' sample positions, one all-to-all of encodings, one all-to-all of
                   their gradients (128 bytes per sample in all) and an all-reduce of the networks' few thousand gradients;
                   no table gradient and no table parameter crosses the wire.  For tables that outweigh a step's samples
                   (T = 2^22: 805 MB of table traffic per step and rank against 34-270 MB of encodings).  The levels a
                   rank does not own go stale between occupancy updates: sync() before rendering, saving or comparing
                   (close() does it, fp32 master copy included; the Adam moments of a level stay with its owner)."""

    def __init__(self, torch, engine, dist=None, steps_per_call=1, registered_gradient=False, exchange="allreduce", shard_occupancy=True):
        self.torch, self.engine, self.dist = torch, engine, dist
        self.steps_per_call = steps_per_call
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self._steps_seen = 0
        self.sync_calls = 0
        self.buffers = None
        self._peer_g = self._peer_w = None
        if exchange not in ("allreduce", "sharded", "peer", "levels"):
            raise ValueError("unknown exchange %r" % (exchange,))
        if exchange not in ("peer", "levels") and dist is not None and dist.get_world_size() > 1 and _grad_table_half():
            raise ValueError("the half-precision gradient table needs exchange='peer' (the others treat the gradient arena as one fp32 array)")
        self.exchange = exchange
        self._bytes = {"gradient_out_per_step": 0, "parameters_out_per_step": 0}
        if self.world > 1:
            if exchange in ("peer", "levels"):
                registered_gradient = False      # peer: the kernel reads the engine's own allocation; levels: no table gradient travels
            if registered_gradient and hasattr(engine, "set_grad_buffer"):
                # the gradient arena moves into memory registered with the communicator
                self.buffers = CollectiveBuffers(torch, dist, "cuda:%d" % torch.cuda.current_device())
                count = (engine.arena().total + 3) // 4 * 4
                engine.set_grad_buffer(self.buffers.zeros(count, torch.float32))
                self.buffers.register()
            a = engine.arena()
            self._hash, self._total = int(a.sparse_count), int(a.total)
            if exchange == "sharded":
                if self._hash % (4 * self.world) != 0:
                    raise ValueError("the hash table (%d elements) does not split into %d aligned slices" % (self._hash, self.world))
                self._shard = self._hash // self.world
                engine.set_optimizer_shard(self.rank, self.world, self._allgather_params)
                engine.set_grad_sync(self._reduce_scatter)
                wire = (self.world - 1) / self.world
                self._bytes = {"gradient_out_per_step": int(self._hash * 4 * wire + (self._total - self._hash) * 4 * 2 * wire),
                               "parameters_out_per_step": int(self._hash * 2 * wire)}
            elif exchange == "peer":
                if self._hash % (4 * self.world) != 0:
                    raise ValueError("the hash table (%d elements) does not split into %d aligned slices" % (self._hash, self.world))
                self._shard = self._hash // self.world
                import importlib
                nbm = importlib.import_module("3dmaker_b200")
                self._peer_g = PeerMemory(nbm, dist, a.g)
                self._peer_w = PeerMemory(nbm, dist, a.w_h)
                self._token = torch.zeros(1, dtype=torch.float32, device="cuda:%d" % torch.cuda.current_device())
                engine.set_grad_sync(None)
                engine.set_peer_exchange(self.rank, self.world, self._peer_g.pointers, self._peer_w.pointers, self._barrier)
                wire = (self.world - 1) / self.world
                # what crosses NVLink per step: the other ranks read (N - 1) / N of this gradient table, this rank stores its
                # fp16 slice into N - 1 peers, and everybody reads everybody's dense tail
                gbytes = 2 if _grad_table_half() else 4
                self._bytes = {"gradient_out_per_step": int(self._hash * gbytes * wire + (self._total - self._hash) * 4 * (self.world - 1)),
                               "parameters_out_per_step": int(self._hash * 2 * wire)}
            elif exchange == "levels":
                engine.set_grad_sync(None)
                engine.set_level_partition(self.rank, self.world, self._gather_blocks, self._exchange_blocks, self._allreduce)
                self._bytes = {"gradient_out_per_step": int((self._total - self._hash) * 4 * 2 * (self.world - 1) / self.world),
                               "parameters_out_per_step": 0, "per_sample_out": 16 * (self.world - 1) + int(2 * 64 * (self.world - 1) / self.world)}
            else:
                engine.set_grad_sync(self._allreduce)
                self._bytes = {"gradient_out_per_step": int(self._total * 4 * 2 * (self.world - 1) / self.world), "parameters_out_per_step": 0}
            # occupancy updates: every rank evaluates its share of the density queries, the per-cell maxima are merged
            self._occupancy_sharded = hasattr(engine, "set_occupancy_shard") and shard_occupancy
            if self._occupancy_sharded:
                engine.set_occupancy_shard(self.rank, self.world, self._allreduce_max)
            # the same number of optimizer steps, hence exchanges, per call on every rank, whatever the local sample
            # counts are (steps_per_call > 1 lets one occupancy walk of a large ray shard serve several steps)
            engine.set_steps_per_call(steps_per_call)
        # with equal shards (num_rays a multiple of world) local_rays * world is exactly the global ray count
        engine.set_global_ray_scale(self.world)

    def _allreduce(self, grad):
        self.sync_calls += 1
        self.dist.all_reduce(grad, op=self.dist.ReduceOp.SUM)

    def _reduce_scatter(self, grad):
        self.sync_calls += 1
        lo = self.rank * self._shard
        self.dist.reduce_scatter_tensor(grad[lo:lo + self._shard], grad[:self._hash], op=self.dist.ReduceOp.SUM)   # in place
        self.dist.all_reduce(grad[self._hash:self._total], op=self.dist.ReduceOp.SUM)

    def _allreduce_max(self, t):
        self.sync_calls += 1
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)

    def _gather_blocks(self, send, recv):
        self.sync_calls += 1
        self.dist.all_gather_into_tensor(recv, send)

    def _exchange_blocks(self, send, recv):
        self.sync_calls += 1
        self.dist.all_to_all_single(recv, send)

    def sync(self, master=False):
        """exchange="levels": every rank's copy of the table is made whole again (all ranks call it)."""
        if self.world > 1 and self.exchange == "levels":
            self.engine.sync_levels(master)

    def _barrier(self):
        self.sync_calls += 1
        self.dist.all_reduce(self._token, op=self.dist.ReduceOp.SUM)

    def _allgather_params(self, w_h):
        lo = self.rank * self._shard
        self.dist.all_gather_into_tensor(w_h[:self._hash], w_h[lo:lo + self._shard])                                # in place

    def gather_master(self):
        """After sharded steps: every rank receives the fp32 master copy of every table slice (call before saving)."""
        if self.world > 1 and self.exchange in ("sharded", "peer"):
            w = self.engine.arena_tensor("w")
            lo = self.rank * self._shard
            self.dist.all_gather_into_tensor(w[:self._hash], w[lo:lo + self._shard])
        if self.world > 1 and self.exchange == "levels":
            self.sync(master=True)

    def exchange_stats(self):
        """Bytes this rank sends per optimizer step (ring accounting: (N - 1) / N of a buffer per reduce-scatter or
        all-gather, twice that per all-reduce)."""
        return dict(self._bytes, mode=self.exchange, ranks=self.world)

    def close(self):
        """Detaches the callbacks from the engine (they hold references to this object)."""
        if self.world > 1:
            if self.exchange == "sharded" and hasattr(self.engine, "set_optimizer_shard"):
                self.engine.set_optimizer_shard(0, 1, None)
            if self.exchange == "peer":
                self.torch.cuda.synchronize()
                self.dist.barrier()              # nobody unmaps memory a peer's kernel may still be using
                self.engine.set_peer_exchange(0, 1, None, None, None)
                self._peer_g.close(); self._peer_w.close()
            if self.exchange == "levels":
                self.engine.sync_levels(True)    # every rank leaves with the whole table, fp32 master included (all ranks close)
                if self.torch.cuda.is_available():
                    self.torch.cuda.synchronize()
                self.engine.set_level_partition(0, 1, None, None, None)
            if getattr(self, "_occupancy_sharded", False):
                self.engine.set_occupancy_shard(0, 1, None)
            self.engine.set_grad_sync(None)

    def train_rays(self, rays_o, rays_d, rgb_true):
        """steps_per_call optimizer steps on the global batch (which must split evenly over the ranks); returns the
        number of local rays that fitted this rank's sample batches and were trained on."""
        n = rays_o.shape[0]
        if n % self.world != 0:
            raise ValueError("global ray batch (%d) must be a multiple of the number of ranks (%d)" % (n, self.world))
        start, count = ray_shard(n, self.rank, self.world)
        before = self._steps_seen
        self._steps_seen = self.engine.train_rays(rays_o[start:start + count], rays_d[start:start + count], rgb_true[start:start + count])
        if self.world > 1 and self._steps_seen - before != self.steps_per_call:
            raise RuntimeError("the engine took %d optimizer steps instead of %d" % (self._steps_seen - before, self.steps_per_call))
        return self.engine.rays_consumed() if self.world > 1 else count

    def replicas_in_sync(self):
        """True when every rank holds bit-identical parameters: compares the 64-bit sum of the raw bits of the fp16 copy
        the forward reads (with the sharded optimizer the fp32 master copy of a slice is current on its owner only)."""
        owner_only = self.exchange in ("sharded", "peer", "levels")
        self.sync()                       # exchange="levels": make the table whole first (a collective: every rank is here)
        w = self.engine.arena_tensor("w_h" if owner_only else "w")
        s = w.view(self.torch.int16 if owner_only else self.torch.int32).to(self.torch.int64).sum().reshape(1)
        if self.world == 1:
            return True
        t = self.torch.stack([s[0], -s[0]])
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return int(t[0].item()) == -int(t[1].item())


class ShardedRenderer:
    """Renders one frame with the pixels split over the ranks and gathers it on rank 0.

    engine needs render(rays_o, rays_d, rgb_out); ray_fn(first_pixel, count, rays_o_out, rays_d_out) writes the rays of
    a pixel run into [count, 3] slices (nb_generate_rays on a GPU).  No collective touches the data path except the
    final gather."""

    def __init__(self, torch, engine, ray_fn, dist=None, tile=4096, tiled_ray_fn=None, undeal_fn=None):
        self.torch, self.engine, self.ray_fn, self.dist, self.tile = torch, engine, ray_fn, dist, tile
        # optional undeal_fn(blocks, ranks, rows_per_rank, tile, num_pixels, frame_out): frame assembly on rank 0 in one
        # launch (nb_undeal_tiles)
        self.undeal_fn = undeal_fn
        self._local = self._gathered = self._frame = None
        # optional tiled_ray_fn(tile, first_tile, tile_stride, count, rays_o_out, rays_d_out): all tiles of this rank in one
        # call (nb_generate_rays_tiled); without it ray_fn runs once per run of consecutive pixels
        self.tiled_ray_fn = tiled_ray_fn
        self.rank = dist.get_rank() if dist is not None else 0
        self.world = dist.get_world_size() if dist is not None else 1
        self._rays = None

    def local_pixels(self, num_pixels):
        return sum(c for _, c in pixel_tiles(num_pixels, self.rank, self.world, self.tile))

    def render_local(self, num_pixels, device, rows=0):
        """Renders this rank's tiles into one [max(local_pixels, rows), 3] tensor (tile order; rows behind the local pixels
        are padding and never read): the rays of all its tiles are generated into one buffer and rendered by ONE engine
        call, so the engine batches samples across tiles.  The buffers are kept between frames."""
        torch = self.torch
        tiles = pixel_tiles(num_pixels, self.rank, self.world, self.tile)
        total = sum(c for _, c in tiles)
        if self._rays is None or self._rays[0].shape[0] < max(1, total):
            self._rays = (torch.empty((max(1, total), 3), dtype=torch.float32, device=device),
                          torch.empty((max(1, total), 3), dtype=torch.float32, device=device))
        o, d = self._rays
        if self.tiled_ray_fn is not None and self.world > 1 and total > 0:
            # the last tile of the frame may be short, and it is the last of whichever rank holds it
            self.tiled_ray_fn(self.tile, self.rank, self.world, total, o[:total], d[:total])
        else:
            at = 0
            for first, count in merge_runs(tiles):
                self.ray_fn(first, count, o[at:at + count], d[at:at + count])
                at += count
        need = max(1, total, rows)
        if self._local is None or self._local.shape[0] < need:
            self._local = torch.zeros((need, 3), dtype=torch.float32, device=device)
        out = self._local[:need]
        if total > 0:
            self.engine.render(o[:total], d[:total], out[:total])
        return out, tiles

    def render_frame(self, num_pixels, device):
        """Returns the [num_pixels, 3] frame on rank 0 (None elsewhere).  The tensor is reused by the next call."""
        torch = self.torch
        num_tiles = (num_pixels + self.tile - 1) // self.tile
        max_tiles = (num_tiles + self.world - 1) // self.world
        rows = max_tiles * self.tile
        # with several ranks the local block is rendered straight into the equal-size block the gather sends
        local, tiles = self.render_local(num_pixels, device, rows=rows if self.world > 1 else 0)
        if self.world == 1:
            return local[:num_pixels]            # one rank holds every tile in frame order: the block IS the frame
        # equal-size gather: every rank's block padded to the largest one; rank 0 receives all blocks into one buffer and
        # un-deals the tiles into the frame with one launch (tile j of rank r is tile j * world + r of the frame)
        padded = local[:rows]
        if self.rank == 0:
            if self._gathered is None or self._gathered.shape[1] != rows or self._frame.shape[0] != num_pixels:
                self._gathered = torch.empty((self.world, rows, 3), dtype=torch.float32, device=device)
                self._frame = torch.empty((num_pixels, 3), dtype=torch.float32, device=device)
            buf = self._gathered
            self.dist.gather(padded, [buf[r] for r in range(self.world)], dst=0)
            if self.undeal_fn is not None:
                self.undeal_fn(buf, self.world, rows, self.tile, num_pixels, self._frame)
            else:   # no device kernel at hand (CPU ranks in the tests): the same permutation with a strided copy
                self._frame.copy_(buf.view(self.world, max_tiles, self.tile, 3).permute(1, 0, 2, 3).reshape(-1, 3)[:num_pixels])
            return self._frame
        self.dist.gather(padded, None, dst=0)
        return None


def gathered_bytes(num_pixels, world, tile=4096):
    """Bytes rank 0 receives per frame in render_frame (the only traffic of sharded rendering)."""
    num_tiles = (num_pixels + tile - 1) // tile
    max_tiles = (num_tiles + world - 1) // world
    return (world - 1) * max_tiles * tile * 3 * 4 if world > 1 else 0
