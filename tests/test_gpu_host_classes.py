"""Builds and runs the C++ contract test of the host classes (tests/cpp/test_host_classes.cu) on the GPU."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_classes(cuda, tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available to build the C++ test")
    exe = os.path.join(str(tmp_path), "test_host_classes")
    libdir = os.path.join(ROOT, "3dmaker_b200")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", os.path.join(ROOT, "tests", "cpp", "test_host_classes.cu"), "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-L", libdir, "-lnerf_b200", "-Xlinker", "-rpath", "-Xlinker", libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "[SUCCESS] all host-class checks passed" in r.stdout
