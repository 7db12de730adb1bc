"""In-tree build of libmetile_b200.so with nvcc for sm_100a.

`python -m metile_b200.build [--force] [--verbose]`.  The shared object is written next to the
sources (metile_b200/csrc/libmetile_b200.so) so it travels with the tree; nothing is installed
into site-packages and there is no JIT cache.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUTPUT = os.path.join(CSRC, "libmetile_b200.so")
SOURCES = ("metile_b200.cu",)
HEADERS = ("common.cuh", "ptx.cuh", "affine_gemv.cuh", "affine_umma.cuh", "affine_mlp_fused.cuh", "add_rmsnorm.cuh", "attention_decode.cuh", "peer_reduce.cuh",
           "dense_rows.cuh", os.path.join("..", "..", "include", "metile_b200.h"))


def _nvcc():
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return found


def is_stale():
    if not os.path.exists(OUTPUT):
        return True
    built = os.path.getmtime(OUTPUT)
    inputs = [os.path.join(CSRC, name) for name in SOURCES + HEADERS]
    return any(os.path.getmtime(path) > built for path in inputs if os.path.exists(path))


def build(force=False, verbose=False):
    if not force and not is_stale():
        return OUTPUT
    command = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
        "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    ]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += [os.path.join(CSRC, name) for name in SOURCES]
    command += ["-o", OUTPUT]
    subprocess.run(command, check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
