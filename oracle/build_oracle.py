"""Compile the C oracle into ``oracle/libkv_oracle.so`` (test infrastructure).

Usage: ``python oracle/build_oracle.py``.  The flags avoid ``-march=native`` so that
a library built in one container runs on another x86-64 host with AVX2.

The reference itself has no C, C++ or CUDA source for this path (its kernels are
WGSL strings dispatched through wgpu), so there is nothing to compile into
``oracle/_ref``; the oracle is a port, never the reference's own binary.
"""
import pathlib
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
SRC = HERE / "kv_oracle.c"
OUT = HERE / "libkv_oracle.so"


def build(force: bool = False) -> pathlib.Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-fPIC", "-shared", "-std=c11",
           "-Wall", "-o", str(OUT), str(SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
