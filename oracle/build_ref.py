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
REF = os.environ.get("REFERENCE_ROOT", "/root/reference")
TINY = os.path.join(REF, "modules", "TinyMLP")
NERF = os.path.join(REF, "modules", "NeRF")

FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math", "--extra-device-vectorization",
         "--restrict", "-Xcompiler", "-fPIC", "-w", "-I", TINY, "-I", NERF]

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


def _compile(src, obj):
    if _newer(obj, [src]):
        return obj
    r = subprocess.run([_nvcc()] + FLAGS + ["-c", src, "-o", obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference build failed for %s:\n%s" % (src, r.stderr[-4000:]))
    return obj


def build(verbose=True):
    os.makedirs(OUT, exist_ok=True)
    jobs = [(os.path.join(TINY, s), os.path.join(OUT, "tiny_" + s[:-3] + ".o")) for s in TINY_SRC]
    jobs += [(os.path.join(NERF, s), os.path.join(OUT, "nerf_" + s[:-3] + ".o")) for s in NERF_SRC]
    if os.path.exists(SHIM):
        jobs.append((SHIM, os.path.join(OUT, "ref_shim.o")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda j: _compile(*j), jobs))
    lib = os.path.join(OUT, "libref3dmaker.so")
    if not _newer(lib, objs):
        r = subprocess.run([_nvcc(), "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference link failed:\n" + r.stderr[-4000:])
    if verbose:
        print("reference build in", OUT)
    return OUT


def build_if_reference_present():
    """Called by __graft_entry__.build(): a no-op where the reference tree is absent (the GPU box)."""
    if os.path.isdir(TINY) and os.path.isdir(NERF):
        return build(verbose=False)
    return None


if __name__ == "__main__":
    build()
