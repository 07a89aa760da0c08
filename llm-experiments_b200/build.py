"""Build ``libb2kv.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

``python llm-experiments_b200/build.py [--force] [--verbose]``.  The library has no
dependency on torch or Python: it is loaded with ctypes.  Sources are compiled to
objects in parallel and linked with the static CUDA runtime.
"""
from __future__ import annotations

import concurrent.futures
import os
import pathlib
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
OUT = PKG / "libb2kv.so"
OBJ_DIR = PKG / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def sources():
    return sorted(CSRC.glob("*.cu"))


def _newest_input() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(f.stat().st_mtime for f in files)


def up_to_date() -> bool:
    return OUT.exists() and OUT.stat().st_mtime >= _newest_input()


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and up_to_date():
        return OUT
    OBJ_DIR.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: pathlib.Path) -> pathlib.Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    link = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(OUT), *map(str, objs)]
    subprocess.run(link, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
