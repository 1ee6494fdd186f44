import importlib
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (ctypes view of the C-ABI library)."""
    return importlib.import_module("minicpm5-5080fast_b200")


@pytest.fixture(scope="session")
def cpu_ref_lib():
    """oracle/libcpu_ref.so, built on demand with gcc."""
    import ctypes
    so = os.path.join(ROOT, "oracle", "libcpu_ref.so")
    src = os.path.join(ROOT, "oracle", "cpu_ref.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "libcpu_ref.so"])
    return ctypes.CDLL(so)


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = os.path.join(ROOT, "tests", "golden")
    return {n: np.load(os.path.join(d, n + ".npz")) for n in ("codec", "small", "baseline")}
