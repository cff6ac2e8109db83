"""Builds the sm_100a kernel library in-tree with nvcc (cross-compiles without a GPU).

    python -m xixi_vllm_b200.ops.build [--force] [--verbose]

Produces ``xixi_vllm_b200/ops/_xv_cuda.so``; the source list is every ``.cu`` under
``csrc/kernels``. The shared object carries only sm_100a code: there is no fallback arch.
"""

from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
LIB = os.path.join(_HERE, "_xv_cuda.so")
OBJ_DIR = os.path.join(_HERE, "_build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise FileNotFoundError("nvcc not found")
    return p


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def _headers() -> list[str]:
    return (glob.glob(os.path.join(CSRC, "common", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.cuh"))
            + glob.glob(os.path.join(CSRC, "kernels", "*.h")))


def _deps_mtime() -> float:
    files = sources() + _headers()
    return max(os.path.getmtime(f) for f in files)


def needs_build() -> bool:
    return not os.path.isfile(LIB) or os.path.getmtime(LIB) < _deps_mtime()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    hdr_time = max([os.path.getmtime(f) for f in _headers()] or [0.0])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.isfile(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", os.path.join(CSRC, "kernels"), "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed for {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    tmp = LIB + f".tmp{os.getpid()}"
    subprocess.run([nvcc, "-shared", "-o", tmp, *objs], check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
