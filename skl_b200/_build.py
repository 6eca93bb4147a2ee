"""In-tree build of libskl_b200.so: nvcc for the sm_100a kernels, gcc -std=gnu99 for the host layer.

Run as ``python -m skl_b200._build`` or through ``__graft_entry__.build()``.  Cross-compiles without a
GPU.  Objects go to skl_b200/lib/obj/, the library to skl_b200/lib/libskl_b200.so; a file is rebuilt
only when it, or a header beside it, is newer than its object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "libskl_b200.so")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
CC = os.environ.get("CC", "gcc")
CFLAGS = ["-std=gnu99", "-O2", "-fPIC", "-Wall", "-Wextra", f"-I{CUDA_HOME}/include"]


def _newer(src: str, deps: list[str], out: str) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(p) > t for p in [src] + deps)


def _run(cmd: list[str], log: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.append("$ " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(log[-1])
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")


def build(verbose: bool = False, force: bool = False) -> str:
    if not os.path.exists(NVCC):
        raise RuntimeError(f"nvcc not found at {NVCC}")
    os.makedirs(OBJDIR, exist_ok=True)
    log: list[str] = []
    cu_dir = os.path.join(CSRC, "cuda")
    host_dir = os.path.join(CSRC, "host")
    headers = [os.path.join(CSRC, "abi.h"), os.path.join(ROOT, "include", "skl-b200.h")] + \
        [os.path.join(cu_dir, f) for f in sorted(os.listdir(cu_dir)) if f.endswith((".cuh", ".h"))]
    objs = []
    for f in sorted(os.listdir(cu_dir)):
        if not f.endswith(".cu"):
            continue
        src, obj = os.path.join(cu_dir, f), os.path.join(OBJDIR, f[:-3] + ".o")
        if force or _newer(src, headers, obj):
            _run([NVCC] + NVCC_FLAGS + ["-c", src, "-o", obj], log)
        objs.append(obj)
    for f in sorted(os.listdir(host_dir)):
        if not f.endswith(".c"):
            continue
        src, obj = os.path.join(host_dir, f), os.path.join(OBJDIR, f[:-2] + ".host.o")
        if force or _newer(src, headers, obj):
            _run([CC] + CFLAGS + ["-c", src, "-o", obj], log)
        objs.append(obj)
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        _run([NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                   "-cudart", "static"], log)
    with open(os.path.join(LIBDIR, "build.log"), "w") as fh:
        fh.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return LIB


def clean() -> None:
    shutil.rmtree(LIBDIR, ignore_errors=True)


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(LIB)
