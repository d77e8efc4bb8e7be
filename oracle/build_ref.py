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


# The reference's own test programs, compiled UNMODIFIED against this repository's host classes instead of the
# reference's: (program name, module, path inside the module, the headers it reaches through "../").
COMPAT_TESTS = [("ref_testModes", "TinyMLP", os.path.join("tests_kernels", "testModes.cu"), ["TinyMLP.h", "TinyMLPHashGrid.h"]),
                ("ref_test_loading", "NeRF", os.path.join("test_kernels", "test_loading.cu"), ["InstantNerf.h"])]


def build_compat_tests(ref_root, verbose=True):
    """Source compatibility of 3dmaker_b200/host/*.h, shown with the reference's own programs: each test source is
    reached through a symbolic link placed in a scratch tree under oracle/_ref/compat/ whose parent directory holds
    one-line headers forwarding to this repository's classes, so the program's `#include "../TinyMLP.h"` finds OUR
    header; nothing of the reference is copied or edited.  The programs link against libnerf_b200.so (built first) and
    are run on the GPU by tests/test_gpu_host_classes.py."""
    repo = os.path.dirname(HERE)
    host = os.path.join(repo, "3dmaker_b200", "host")
    libdir = os.path.join(repo, "3dmaker_b200")
    if not os.path.exists(os.path.join(libdir, "libnerf_b200.so")):
        return []
    built = []
    for exe, module, rel, headers in COMPAT_TESTS:
        src = os.path.join(ref_root, "modules", module, rel)
        if not os.path.exists(src):
            continue
        mod_dir = os.path.join(OUT, "compat", module)
        link = os.path.join(mod_dir, rel)
        os.makedirs(os.path.dirname(link), exist_ok=True)
        if os.path.islink(link) or os.path.exists(link):
            os.remove(link)
        os.symlink(src, link)
        for h in headers:
            with open(os.path.join(mod_dir, h), "w") as f:
                f.write('#include "%s"\n' % os.path.join(host, h))
        out = os.path.join(OUT, exe)
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-w", link, "-o", out, "-I", os.path.join(repo, "include"),
               "-L", libdir, "-lnerf_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../3dmaker_b200"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("the reference's %s does not compile against 3dmaker_b200/host:\n%s" % (rel, r.stderr[-3000:]))
        built.append(out)
    # the scratch tree held only links and forwarding headers; the programs are what travels
    shutil.rmtree(os.path.join(OUT, "compat"), ignore_errors=True)
    if verbose:
        print("compatibility programs:", ", ".join(os.path.basename(b) for b in built))
    return built


def build_if_reference_present(ref_root=None):
    """Called by __graft_entry__.build(): a no-op where the reference tree is absent (the GPU box)."""
    ref_root = ref_root or os.environ.get("REFERENCE_ROOT")
    if ref_root and all(os.path.isdir(d) for d in _dirs(ref_root)):
        out = build(ref_root, verbose=False)
        build_compat_tests(ref_root, verbose=False)
        return out
    return None


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: python oracle/build_ref.py <reference tree>   (or set REFERENCE_ROOT)")
    build(root)
    build_compat_tests(root)
