"""Builds libinquant_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libinquant_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# Per-file flags: the codec must not contract a*b+c into an FMA (bit-exact bytes).
SOURCES = {
    "lib.cu": [],
    "codec.cu": ["-fmad=false"],
    "decode.cu": [],
    "append.cu": [],
    "prefill.cu": [],
    "decode_generic.cu": [],
    "exchange.cu": [],
    "pages.cu": [],
}


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    mtime = os.path.getmtime(target)
    return any(os.path.getmtime(d) > mtime for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "inquant_b200.h"))
    objects = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    running = []
    for name, extra in SOURCES.items():
        src = os.path.join(CSRC, name)
        obj = os.path.join(build_dir, name.replace(".cu", ".o"))
        if force or _stale(obj, [src, __file__] + headers):
            cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            # the translation units are independent: all stale ones compile at the same time (the
            # decode kernels alone take minutes), which bounds a build from scratch by the longest file
            running.append((cmd, subprocess.Popen(cmd)))
        objects.append(obj)
    failed = [cmd for cmd, process in running if process.wait() != 0]
    if failed:
        raise subprocess.CalledProcessError(1, failed[0])
    if force or _stale(LIB, objects):
        subprocess.run([nvcc, *ARCH, "-shared", "-o", LIB, *objects, "-cudart", "static"], check=True)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
