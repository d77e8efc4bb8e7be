"""Builds the reference's own CUDA sources for sm_100a into oracle/_ref/ (test infrastructure).

The sources are compiled WHERE THEY LIE under the reference tree (nothing is copied), with the flags of the
reference's CMake files (modules/TinyMLP/CMakeLists.txt:38-59, modules/NeRF/CMakeLists.txt:57-74):
--use_fast_math --extra-device-vectorization --restrict -O3.  The reference's root CMake project is not
used (it downloads GLFW/FreeType/RmlUi).  Outputs:

  oracle/_ref/libref3dmaker.so   TinyMLP + NeRF kernels and classes, plus the C wrappers of oracle/ref_shim.cu
  oracle/_ref/libref_twin_*.so   the CPU check functions that live inside the reference's test programs
                                 (oracle/ref_twin_*.cu include the test source with main renamed)

oracle/_ref/ is git-ignored; the built files travel to the GPU box, the reference tree does not.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# Where the reference tree is mounted is always given by the caller: an argument of build() /
# build_if_reference_present(), the REFERENCE_ROOT environment variable, or the first command-line argument.
# Without any of them (or where the tree is absent, as on a GPU box) nothing is built and the prebuilt files are used.
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math", "--extra-device-vectorization",
         "--restrict", "-Xcompiler", "-fPIC", "-w"]

TINY_SRC = ["networkFusion.cu", "networkFusionBackward.cu", "networkFusionHashtable.cu", "networkFusionBackwardHashtable.cu",
            "optimizerKernel.cu", "TinyMLP.cu", "TinyMLPHashGrid.cu", "mlpKernel.cu"]
# InstantNerf.cu textually includes otherKernels.cu, so otherKernels.cu is not compiled on its own; the shim
# includes InstantNerf.cu to reach the kernels that have no launcher of their own.
NERF_SRC = ["processRays.cu", "compositing.cu"]
SHIM = os.path.join(HERE, "ref_shim.cu")


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target, sources):
    return os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in sources)


def _compile(src, obj, includes):
    if _newer(obj, [src]):
        return obj
    r = subprocess.run([_nvcc()] + FLAGS + includes + ["-c", src, "-o", obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference build failed for %s:\n%s" % (src, r.stderr[-4000:]))
    return obj


def _dirs(ref_root):
    return os.path.join(ref_root, "modules", "TinyMLP"), os.path.join(ref_root, "modules", "NeRF")


def build(ref_root, verbose=True):
    TINY, NERF = _dirs(ref_root)
    includes = ["-I", TINY, "-I", NERF]
    os.makedirs(OUT, exist_ok=True)
    jobs = [(os.path.join(TINY, s), os.path.join(OUT, "tiny_" + s[:-3] + ".o")) for s in TINY_SRC]
    jobs += [(os.path.join(NERF, s), os.path.join(OUT, "nerf_" + s[:-3] + ".o")) for s in NERF_SRC]
    if os.path.exists(SHIM):
        jobs.append((SHIM, os.path.join(OUT, "ref_shim.o")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda j: _compile(j[0], j[1], includes), jobs))
    lib = os.path.join(OUT, "libref3dmaker.so")
    if not _newer(lib, objs):
        r = subprocess.run([_nvcc(), "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference link failed:\n" + r.stderr[-4000:])
    if verbose:
        print("reference build in", OUT)
    return OUT


def build_if_reference_present(ref_root=None):
    """Called by __graft_entry__.build(): a no-op where the reference tree is absent (the GPU box)."""
    ref_root = ref_root or os.environ.get("REFERENCE_ROOT")
    if ref_root and all(os.path.isdir(d) for d in _dirs(ref_root)):
        return build(ref_root, verbose=False)
    return None


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: python oracle/build_ref.py <reference tree>   (or set REFERENCE_ROOT)")
    build(root)
