"""Build librglru_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage:  python -m griffin_b200.build [--force]

The library has no dependency on PyTorch; it links the CUDA runtime statically
and resolves the one driver entry point it needs (tensor-map encoding) at run
time.  Object files go to griffin_b200/csrc/_build/.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(SRC_DIR, "_build")
LIB_PATH = os.path.join(PKG_DIR, "librglru_b200.so")
SOURCES = ["rglru_scan.cu", "rglru_conv.cu", "rglru_api.cu", "rglru_noalloc.cu"]
HEADERS = ["rglru_device.cuh", "rglru_internal.h", os.path.join("..", "..", "include", "rglru_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--threads", "2",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the RG-LRU kernels cannot be built")
    return found


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile whatever is out of date and return the path of the shared library."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(SRC_DIR, h) for h in HEADERS]
    jobs = []
    objects = []
    for src in SOURCES:
        src_path = os.path.join(SRC_DIR, src)
        obj_path = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objects.append(obj_path)
        if force or _stale(obj_path, [src_path] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src_path, "-o", obj_path]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
        return res.stderr

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        logs = list(pool.map(run, jobs))
    if verbose:
        for log in logs:
            sys.stderr.write(log)
    if force or jobs or _stale(LIB_PATH, objects):
        run([nvcc, "-shared", "-o", LIB_PATH, *objects, "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
