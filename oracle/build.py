"""Compile oracle/affine_c.c into oracle/liboracle_affine.so (gcc + OpenMP).

Run as `python -m oracle.build`.  The flags avoid -march=native on purpose: the shared
object is built on one machine and carried to another, so it targets plain x86-64-v3
(AVX2 + FMA), which every host this runs on provides.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "affine_c.c")
OUTPUT = os.path.join(HERE, "liboracle_affine.so")


def build(force=False):
    if (not force and os.path.exists(OUTPUT)
            and os.path.getmtime(OUTPUT) >= os.path.getmtime(SOURCE)):
        return OUTPUT
    command = ["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-shared", "-fPIC", "-std=c11",
               SOURCE, "-o", OUTPUT, "-lm"]
    subprocess.run(command, check=True)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
