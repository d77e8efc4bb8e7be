"""Shared helpers of the parity tests: seeded inputs in the shapes of the benchmark configs, tolerances."""
import numpy as np

# Tolerances of the parity bar (max error relative to the largest reference magnitude):
REL_ENCODE = 1e-3   # encoded features
REL_MLP = 1e-2      # MLP outputs and gradients: fp16 operands, fp32 accumulate
ABS_RGB = 1e-3      # composited colour


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    scale = np.max(np.abs(b))
    if scale == 0:
        return float(np.max(np.abs(a)))
    return float(np.max(np.abs(a - b)) / scale)


def half_bits(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def half_vals(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def make_positions(n, seed=0):
    rng = np.random.default_rng(seed)
    p = np.zeros((n, 4), np.float32)
    p[:, :3] = rng.random((n, 3), dtype=np.float32)
    return p


def make_table(L, T, seed=0, amp=1e-4):
    rng = np.random.default_rng(seed)
    t = rng.uniform(-amp, amp, size=(L, T, 2)).astype(np.float32)
    return t


def mlp_dims(i, h, o, nl):
    return [((i if l == 0 else h), (o if l == nl - 1 else h)) for l in range(nl)]


def make_mlp(i, h, o, nl, seed=0, xavier=True, bias_amp=0.0):
    """Flat fp32 weights ([out][in] per layer) and biases."""
    rng = np.random.default_rng(seed)
    ws, bs = [], []
    for (ki, ko) in mlp_dims(i, h, o, nl):
        bound = np.sqrt(6.0 / (ki + ko)) if xavier else 1.0 / np.sqrt(ki)
        ws.append(rng.uniform(-bound, bound, size=(ko, ki)).astype(np.float32).ravel())
        bs.append(rng.uniform(-bias_amp, bias_amp, size=ko).astype(np.float32) if bias_amp else np.zeros(ko, np.float32))
    return np.concatenate(ws), np.concatenate(bs)


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def half_to_dev(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16)).cuda()


def dev_half_bits(t):
    return t.detach().cpu().numpy().view(np.uint16)


class Uploader:
    """Uploads numpy arrays and KEEPS the device tensors alive until the test ends (a temporary tensor
    whose pointer was taken would otherwise be recycled by the caching allocator before the kernel runs)."""

    def __init__(self, torch, nb):
        self.torch, self.nb, self.keep = torch, nb, []

    def f(self, a):
        t = to_dev(self.torch, a)
        self.keep.append(t)
        return self.nb.ptr(t)

    def h(self, bits):
        t = half_to_dev(self.torch, bits)
        self.keep.append(t)
        return self.nb.ptr(t)
