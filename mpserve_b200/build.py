"""Builds libmpserve_b200.so in-tree with nvcc for sm_100a (no torch headers: seconds, not minutes).

    python -m mpserve_b200.build [--force] [--verbose]

Every source is compiled to its own object (in parallel, and only when it or a header changed),
then the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libmpserve_b200.so"
OBJ = PKG / "lib" / "obj"
SOURCES = ["decode_bucket.cu", "decode_shared.cu", "encode.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "--use_fast_math"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _headers() -> list[Path]:
    return list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "mpserve_b200.h"]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def needs_build() -> bool:
    return _stale(LIB, [CSRC / s for s in SOURCES] + _headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    OBJ.mkdir(parents=True, exist_ok=True)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    nvcc = nvcc_path()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: str) -> Path:
        obj = OBJ / (Path(src).stem + ".o")
        if force or _stale(obj, [CSRC / src] + _headers()):
            subprocess.run([nvcc, *CFLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)], check=True, env=env)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs)], check=True, env=env)
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
