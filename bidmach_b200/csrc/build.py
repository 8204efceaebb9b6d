"""Builds libbidmachcuda-linux-x86_64.so (the C-ABI library) in-tree with nvcc.

The library name follows the reference's loader: base name ``bidmachcuda``
(src/main/java/edu/berkeley/bid/CUMACH.java:9) with the ``-<os>-<arch>`` suffix
its LibUtils appends.  Only sm_100a machine code is generated; the build needs
no GPU.

    python -m bidmach_b200.csrc.build [--force]
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_NAME = "libbidmachcuda-linux-x86_64.so"
LIB_PATH = os.path.join(PKG, LIB_NAME)
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = ["w2v_kernels.cu", "w2v_batch.cu", "w2v_noalloc.cu", "w2v_exchange.cu", "jni_shim.cpp",
           "matio_codec.cpp"]
# measuring aid of bench.py, a library of its own: nothing of it is in the C-ABI library
PROBE_SOURCE = "bench_rowprobe.cu"
PROBE_LIB_PATH = os.path.join(PKG, "libw2vrowprobe.so")
HEADERS = ["w2v_device.cuh", "w2v_internal.h", "w2v_rows.cuh", "jni_min.h",
           os.path.join("..", "..", "include", "bidmach_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=default",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    deps = [os.path.join(HERE, src)] + [os.path.join(HERE, h) for h in HEADERS] + [__file__]
    if force or _stale(obj, deps):
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        subprocess.check_call(cmd)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES) + 1) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), SOURCES + [PROBE_SOURCE]))
    probe_obj = objs.pop()
    if force or _stale(LIB_PATH, objs):
        subprocess.check_call([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                               *objs, "-o", LIB_PATH, "-ldl"])
    if force or _stale(PROBE_LIB_PATH, [probe_obj]):
        subprocess.check_call([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                               probe_obj, "-o", PROBE_LIB_PATH])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
