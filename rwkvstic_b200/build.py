"""Builds the CUDA library in-tree: ``python -m rwkvstic_b200.build``.

One nvcc call, sm_100a only.  The output ``rwkvstic_b200/libb200rwkv.so`` is what
``rwkvstic_b200._lib`` loads with ctypes.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["b200rwkv.cu"]
OUTPUT = os.path.join(HERE, "libb200rwkv.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    newest = max(os.path.getmtime(os.path.join(root, f)) for root, _, files in os.walk(CSRC) for f in files)
    newest = max(newest, os.path.getmtime(os.path.join(os.path.dirname(HERE), "include", "b200rwkv.h")))
    return newest > os.path.getmtime(OUTPUT)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUTPUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", OUTPUT, *[os.path.join(CSRC, s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
