"""The C ABI from a C++ host: the reference's launcher names (include/mc_sm100a_launchers.hpp)
compiled by g++ against the shared library, no Python objects involved in the calls."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
SRC = os.path.join(ROOT, "tests", "cpp", "abi_smoke.cpp")
LIBDIR = os.path.join(ROOT, "minicpm5-5080fast_b200")


def _build(tmp_path):
    exe = str(tmp_path / "abi_smoke")
    cmd = ["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), SRC, "-o", exe,
           "-L", LIBDIR, "-lmc_sm100a_linear", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + LIBDIR,
           "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime.h")),
                    reason="needs g++ and the CUDA runtime headers")
def test_launcher_header_compiles_and_links(pkg, tmp_path):
    """CPU: the header is valid C++ for a host compiler and every launcher it forwards to is exported."""
    assert os.path.exists(pkg.LIB_PATH)
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_abi_smoke_runs(pkg, tmp_path):
    exe = _build(tmp_path)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "ABI-SMOKE-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
