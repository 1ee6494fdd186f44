"""Builds libmc_sm100a_linear.so (sm_100a only) next to this file.

    python minicpm5-5080fast_b200/build.py [--force] [--jobs N]

Every .cu under csrc/ is compiled with
`nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo` into build/*.o (in
parallel) and linked into one shared library with a static CUDA runtime, so
the library has no dependency beyond the driver.  nvcc cross-compiles without
a GPU.  Objects are rebuilt when a source or header is newer.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INC = os.path.join(HERE, "..", "include")
OUT = os.path.join(HERE, "libmc_sm100a_linear.so")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", CSRC, "-I", INC]


def _newest_header() -> float:
    t = 0.0
    for d in (CSRC, INC):
        for f in os.listdir(d):
            if f.endswith((".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def _compile(src: str, obj: str) -> tuple[str, int, str]:
    p = subprocess.run([NVCC, *FLAGS, "-c", src, "-o", obj], capture_output=True, text=True)
    return src, p.returncode, p.stdout + p.stderr


def build(force: bool = False, jobs: int | None = None, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_t = _newest_header()
    todo, objs = [], []
    for f in srcs:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            todo.append((src, obj))
    if todo:
        with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
            for src, rc, log in ex.map(lambda a: _compile(*a), todo):
                if verbose or rc != 0:
                    sys.stderr.write(log)
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src}")
    if todo or not os.path.exists(OUT) or any(os.path.getmtime(o) > os.path.getmtime(OUT) for o in objs):
        p = subprocess.run([NVCC, "-shared", "-o", OUT, *objs, "-cudart", "static"],
                           capture_output=True, text=True)
        if p.returncode != 0:
            sys.stderr.write(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.jobs, a.verbose))
