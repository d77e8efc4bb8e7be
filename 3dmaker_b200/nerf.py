"""Python handle on the C++ InstantNerf scene engine (include/nerf_b200.h, nb_nerf_*), used by the tests and
the benchmark.  torch tensors supply device memory; all work happens inside libnerf_b200.so."""
import ctypes
import importlib

import numpy as np

nb = importlib.import_module("3dmaker_b200")

PHASES = ("march", "occupancy", "density_fwd", "sh_gather", "color_fwd", "compositing", "loss_grad", "color_bwd", "density_grad",
          "density_bwd", "scatter", "optimizer")


def default_options(**overrides):
    o = nb.NerfOptions()
    nb.check(nb.load().nb_nerf_default_options(ctypes.byref(o)), "nb_nerf_default_options")
    for k, v in overrides.items():
        cur = getattr(o, k)
        if hasattr(cur, "__len__"):
            for i in range(len(cur)):
                cur[i] = v[i]
        else:
            setattr(o, k, v)
    return o


class InstantNerf:
    def __init__(self, torch, options, inference=False):
        self.torch, self.lib, self.options = torch, nb.load(), options
        self.h = self.lib.nb_nerf_create(ctypes.byref(options), 1 if inference else 0)
        if not self.h:
            raise nb.NerfB200Error("nb_nerf_create failed: " + self.lib.nb_last_error().decode())
        self._cb = None
        self.steps = ctypes.c_int(0)
        self._hits = np.zeros(4096, np.uint32)      # samples of every optimizer step of the last train_rays() call
        nb.check(self.lib.nb_nerf_set_hit_counts_capacity(self.h, self._hits.size), "nb_nerf_set_hit_counts_capacity")

    def close(self):
        if self.h:
            self.lib.nb_nerf_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def train_rays(self, rays_o, rays_d, rgb_true, rgb_out=None, depth=None, sigma=None, stream=None):
        n = rays_o.shape[0]
        before = self.steps.value
        nb.check(self.lib.nb_nerf_train_rays(self.h, nb.ptr(rays_o), nb.ptr(rays_d), nb.ptr(depth), nb.ptr(sigma), nb.ptr(rgb_true), n,
                                             ctypes.byref(self.steps), self._hits.ctypes.data_as(ctypes.c_void_p), nb.ptr(rgb_out),
                                             nb.stream_ptr(stream)), "nb_nerf_train_rays")
        self._last_steps = self.steps.value - before
        return self.steps.value

    def samples_last_call(self):
        """Samples (ray-march hits) the last train_rays() call trained on, over all its optimizer steps."""
        return int(self._hits[:min(self._last_steps, self._hits.size)].astype(np.int64).sum())

    def render(self, rays_o, rays_d, rgb_out, stream=None):
        nb.check(self.lib.nb_nerf_render(self.h, nb.ptr(rays_o), nb.ptr(rays_d), rays_o.shape[0], nb.ptr(rgb_out), nb.stream_ptr(stream)),
                 "nb_nerf_render")

    def set_learning_rate(self, lr):
        nb.check(self.lib.nb_nerf_set_learning_rate(self.h, lr))

    def set_bg_color(self, r, g, b):
        nb.check(self.lib.nb_nerf_set_bg_color(self.h, r, g, b))

    def set_profiling(self, on):
        nb.check(self.lib.nb_nerf_set_profiling(self.h, int(on)))

    def set_memory_mode(self, inference):
        nb.check(self.lib.nb_nerf_set_memory_mode(self.h, 1 if inference else 0), "nb_nerf_set_memory_mode")

    def set_global_ray_scale(self, scale):
        nb.check(self.lib.nb_nerf_set_global_ray_scale(self.h, scale))

    def set_single_step(self, on):
        """Exactly one optimizer step per train_rays() call (data parallelism); see rays_consumed()."""
        nb.check(self.lib.nb_nerf_set_single_step(self.h, 1 if on else 0))

    def set_steps_per_call(self, steps):
        """Exactly `steps` optimizer steps per train_rays() call on every rank (0: as many as the rays need)."""
        nb.check(self.lib.nb_nerf_set_steps_per_call(self.h, int(steps)))

    def rays_consumed(self):
        return self.step_view().rays_consumed

    def set_fused_field(self, on):
        """One kernel each way for the whole field (default) or the kernel-by-kernel sequence; returns the mode in effect."""
        return bool(self.lib.nb_nerf_set_fused_field(self.h, 1 if on else 0))

    def set_render_rounds(self, on):
        """Render in rounds of samples per ray, skipping what lies behind an opaque surface, or evaluate every sample of
        every ray (default); returns the mode in effect."""
        return bool(self.lib.nb_nerf_set_render_rounds(self.h, 1 if on else 0))

    def last_render_samples(self):
        """Samples the field was evaluated on during the last render() (waits for the device)."""
        n = ctypes.c_uint64(0)
        nb.check(self.lib.nb_nerf_last_render_samples(self.h, ctypes.byref(n)), "nb_nerf_last_render_samples")
        return int(n.value)

    def set_grad_sync(self, fn):
        """fn(grad_tensor) is called between backward and Adam with a float32 view of the gradient arena."""
        if fn is None:
            self._cb = None
            self._sync_fn = None
            nb.check(self.lib.nb_nerf_set_grad_sync(self.h, nb.GRAD_SYNC_FN(0), None))
            return
        self._sync_fn = fn
        grad = self._grad_buffer if getattr(self, "_grad_buffer", None) is not None else self.arena_tensor("g")

        def trampoline(user, ptr, count, stream):
            fn(grad)
        self._cb = nb.GRAD_SYNC_FN(trampoline)
        nb.check(self.lib.nb_nerf_set_grad_sync(self.h, self._cb, None))

    def set_optimizer_shard(self, rank, world, fn):
        """Sharded optimizer (see nb_nerf_set_optimizer_shard): this rank updates slice `rank` of `world` of the hash table;
        fn(w_h) runs after every update with a float16 view of the whole parameter arena and all-gathers the table slices.
        world <= 1 switches back."""
        if world <= 1 or fn is None:
            self._param_cb = None
            nb.check(self.lib.nb_nerf_set_optimizer_shard(self.h, 0, 1, nb.PARAM_SYNC_FN(0), None), "nb_nerf_set_optimizer_shard")
            return
        w_h = self.arena_tensor("w_h")

        def trampoline(user, ptr, count, stream):
            fn(w_h)
        self._param_cb = nb.PARAM_SYNC_FN(trampoline)
        nb.check(self.lib.nb_nerf_set_optimizer_shard(self.h, rank, world, self._param_cb, None), "nb_nerf_set_optimizer_shard")

    def set_peer_exchange(self, rank, world, grad_ptrs, param_ptrs, barrier):
        """Optimizer tail through nb_adam_step_peer (see nb_nerf_set_peer_exchange): grad_ptrs / param_ptrs are lists of
        `world` device addresses (ints), barrier() meets all ranks on the current stream.  world <= 1 switches back."""
        if world <= 1:
            nb.check(self.lib.nb_nerf_set_peer_exchange(self.h, 0, 1, None, None, nb.BARRIER_FN(0), None), "nb_nerf_set_peer_exchange")
            self._barrier_cb = None
            return
        G = (ctypes.c_void_p * world)(*[int(p) for p in grad_ptrs])
        W = (ctypes.c_void_p * world)(*[int(p) for p in param_ptrs])

        def trampoline(user, stream):
            barrier()
        self._barrier_cb = nb.BARRIER_FN(trampoline)
        nb.check(self.lib.nb_nerf_set_peer_exchange(self.h, rank, world, G, W, self._barrier_cb, None), "nb_nerf_set_peer_exchange")

    def set_level_partition(self, rank, world, gather, exchange, reduce):
        """Table partitioned by level over the ranks (see nb_nerf_set_level_partition).  The three collectives get torch
        views of the engine's buffers: gather(send_u8, recv_u8) - all-gather of equal blocks; exchange(send_u8, recv_u8) -
        all-to-all of equal blocks; reduce(grad_f32) - SUM over the ranks.  world <= 1 switches back."""
        if world <= 1:
            nb.check(self.lib.nb_nerf_set_level_partition(self.h, 0, 1, nb.BLOCK_FN(0), nb.BLOCK_FN(0), nb.GRAD_SYNC_FN(0), None),
                     "nb_nerf_set_level_partition")
            self._part_cbs = None
            return
        views = {}

        def view(ptr, count, dtype):
            key = (int(ptr), int(count), np.dtype(dtype).str)
            if key not in views:
                views[key] = view_tensor(self.torch, int(ptr), int(count), dtype)
            return views[key]

        def gather_cb(user, send, recv, nbytes, stream):
            gather(view(send, nbytes, np.uint8), view(recv, nbytes * world, np.uint8))

        def exchange_cb(user, send, recv, nbytes, stream):
            exchange(view(send, nbytes * world, np.uint8), view(recv, nbytes * world, np.uint8))

        def reduce_cb(user, ptr, count, stream):
            reduce(view(ptr, count, np.float32))
        self._part_cbs = (nb.BLOCK_FN(gather_cb), nb.BLOCK_FN(exchange_cb), nb.GRAD_SYNC_FN(reduce_cb))
        nb.check(self.lib.nb_nerf_set_level_partition(self.h, rank, world, *self._part_cbs, None), "nb_nerf_set_level_partition")

    def set_occupancy_shard(self, rank, world, reduce_max):
        """Occupancy updates split over the ranks (see nb_nerf_set_occupancy_shard): reduce_max(tensor_f32) must be an
        all-reduce with MAX over the ranks.  world <= 1 switches back."""
        if world <= 1 or reduce_max is None:
            nb.check(self.lib.nb_nerf_set_occupancy_shard(self.h, 0, 1, nb.GRAD_SYNC_FN(0), None), "nb_nerf_set_occupancy_shard")
            self._occ_cb = None
            return
        views = {}

        def trampoline(user, ptr, count, stream):
            key = (int(ptr), int(count))
            if key not in views:
                views[key] = view_tensor(self.torch, int(ptr), int(count), np.float32)
            reduce_max(views[key])
        self._occ_cb = nb.GRAD_SYNC_FN(trampoline)
        nb.check(self.lib.nb_nerf_set_occupancy_shard(self.h, rank, world, self._occ_cb, None), "nb_nerf_set_occupancy_shard")

    def sync_levels(self, master=False, stream=None):
        """Level-partitioned training: brings the levels this rank does not own up to date (all ranks must call it)."""
        nb.check(self.lib.nb_nerf_sync_levels(self.h, 1 if master else 0, nb.stream_ptr(stream)), "nb_nerf_sync_levels")

    def set_grad_buffer(self, tensor):
        """Moves the gradient arena into `tensor` (float32, CUDA, at least arena().total elements; the engine zeroes it and
        this object keeps it alive) - e.g. memory registered with the communicator so that the all-reduce of
        set_grad_sync() works on it in place.  None returns to the engine's own allocation."""
        if tensor is None:
            nb.check(self.lib.nb_nerf_set_grad_buffer(self.h, None, 0), "nb_nerf_set_grad_buffer")
            self._grad_buffer = None
        else:
            if tensor.dtype != self.torch.float32 or not tensor.is_cuda or not tensor.is_contiguous():
                raise ValueError("the gradient buffer must be a contiguous float32 CUDA tensor")
            nb.check(self.lib.nb_nerf_set_grad_buffer(self.h, nb.ptr(tensor), tensor.numel()), "nb_nerf_set_grad_buffer")
            self._grad_buffer = tensor[:self.arena().total]
        if getattr(self, "_sync_fn", None) is not None:
            self.set_grad_sync(self._sync_fn)

    def arena(self):
        v = nb.ArenaView()
        nb.check(self.lib.nb_nerf_get_arena(self.h, ctypes.byref(v)), "nb_nerf_get_arena")
        return v

    def arena_tensor(self, which):
        """Zero-copy torch view of one arena array ('w', 'g', 'm', 'v' float32; 'w_h' float16)."""
        v = self.arena()
        return _wrap(self.torch, getattr(v, which), v.total, np.float16 if which == "w_h" else np.float32)

    def load_params(self, hash_f32=None, density=None, color=None):
        P = lambda a: None if a is None else np.ascontiguousarray(a, np.float32).ctypes.data_as(ctypes.c_void_p)
        keep = [None if a is None else np.ascontiguousarray(a, np.float32) for a in
                (hash_f32, density[0] if density else None, density[1] if density else None, color[0] if color else None,
                 color[1] if color else None)]
        nb.check(self.lib.nb_nerf_load_params(self.h, *[None if a is None else a.ctypes.data_as(ctypes.c_void_p) for a in keep]),
                 "nb_nerf_load_params")

    def occupancy(self):
        """(bitfield uint8 tensor view, master grid float32 tensor view)."""
        bits, nbytes, master = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_void_p()
        nb.check(self.lib.nb_nerf_occupancy(self.h, ctypes.byref(bits), ctypes.byref(nbytes), ctypes.byref(master)))
        o = self.options
        cells = o.num_cascades * o.grid_resolution[0] * o.grid_resolution[1] * o.grid_resolution[2]
        return _wrap(self.torch, bits.value, nbytes.value, np.uint8), _wrap(self.torch, master.value, cells, np.float32)

    def rebuild_occupancy(self, stream=None):
        nb.check(self.lib.nb_nerf_rebuild_occupancy(self.h, nb.stream_ptr(stream)), "nb_nerf_rebuild_occupancy")

    def step_view(self):
        v = nb.StepView()
        nb.check(self.lib.nb_nerf_get_step_view(self.h, ctypes.byref(v)))
        return v

    def phase_times(self):
        arr = (ctypes.c_double * 12)()
        steps = ctypes.c_int64()
        nb.check(self.lib.nb_nerf_phase_times(self.h, arr, ctypes.byref(steps)))
        return dict(zip(PHASES, list(arr))), steps.value

    def save(self, path):
        nb.check(self.lib.nb_nerf_save(self.h, path.encode()), "nb_nerf_save")

    def load(self, path):
        nb.check(self.lib.nb_nerf_load(self.h, path.encode()), "nb_nerf_load")


class _CudaArrayView:
    """Minimal __cuda_array_interface__ holder so torch can alias library-owned device memory."""

    def __init__(self, ptr, count, dtype):
        self.__cuda_array_interface__ = {"shape": (int(count),), "typestr": np.dtype(dtype).str, "data": (int(ptr), False), "version": 3,
                                         "strides": None}


def _wrap(torch, ptr, count, dtype):
    return torch.as_tensor(_CudaArrayView(ptr, count, dtype), device="cuda")


def view_tensor(torch, ptr, count, dtype):
    return _wrap(torch, ptr, count, dtype)
