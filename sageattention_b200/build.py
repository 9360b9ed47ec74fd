"""Builds libsage3_b200.so (sm_100a only) next to this file with nvcc.

Usage:  python -m sageattention_b200.build [--force]
The library is plain CUDA C++ behind a C ABI (include/sage3_b200.h); it links the CUDA runtime
statically and resolves the one driver entry point it needs at run time, so it has no link-time
dependency on libcuda or on PyTorch.
"""
from __future__ import annotations

import os
import pathlib
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libsage3_b200.so"
SOURCES = ["sage3_abi.cu", "sage3_prepass.cu", "sage3_attn.cu"]
HEADERS = ["sage3_common.cuh", "sage3_kernels.h"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [PKG.parent / "include" / "sage3_b200.h", pathlib.Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
    subprocess.check_call([nvcc, "-shared", "-o", str(LIB), *objs, "-Xcompiler", "-fvisibility=hidden"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
