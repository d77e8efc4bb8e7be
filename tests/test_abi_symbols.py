"""The C-ABI library builds (nvcc cross-compiles without a GPU), loads, and exports every symbol that
include/*.h declares.  No compute call is made here."""
import ctypes
import glob
import importlib
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names |= set(re.findall(r"\b(nb_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_builds_and_exports_every_declared_symbol():
    build = importlib.import_module("3dmaker_b200.build")
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) >= 15
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, "declared in include/*.h but not exported: %s" % missing
    assert lib.nb_built_arch() == 100


def test_python_bindings_cover_the_header():
    nb = importlib.import_module("3dmaker_b200")
    assert set(nb.declared_symbols()) == _declared()
    nb.load()
    assert nb.load().nb_last_error() is not None


def test_missing_library_is_a_loud_error(monkeypatch):
    nb = importlib.import_module("3dmaker_b200")
    monkeypatch.setattr(nb, "_lib", None)
    monkeypatch.setattr(nb, "LIB_PATH", "/nonexistent/libnerf_b200.so")
    try:
        nb.load()
    except nb.NerfB200Error as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("load() must raise when the CUDA library is missing")


def test_forced_tensor_memory_backward_rejects_8_byte_aligned_weight_gradients():
    """Argument validation only (it returns before any CUDA call): the tensor-memory backward adds its weight gradients
    with 16-byte reductions, so forcing it with gradient pointers that are only 8-byte aligned is an error, not a fault."""
    nb = importlib.import_module("3dmaker_b200")
    lib = nb.load()
    density, color = nb.mlp_desc(32, 64, 16, 2, 0), nb.mlp_desc(32, 64, 8, 3, 1)
    A = ctypes.c_void_p(0x10000)             # any 16-byte aligned non-null address: never dereferenced
    G8 = ctypes.c_void_p(0x20008)            # 8- but not 16-byte aligned
    assert lib.nb_set_tuning(b"backward_tc", 1) == 0
    try:
        rc = lib.nb_field_backward(ctypes.byref(density), ctypes.byref(color), A, A, None, 0, A, A, A, A, 128, A, None, G8, A, G8, A, A,
                                   None, None, None, None)
        assert rc == 1 and b"16-byte aligned weight gradients" in lib.nb_last_error()
    finally:
        lib.nb_set_tuning(b"backward_tc", 2)
