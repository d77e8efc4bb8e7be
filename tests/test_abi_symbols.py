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
