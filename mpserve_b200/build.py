"""Builds libmpserve_b200.so in-tree with nvcc for sm_100a (no torch headers: seconds, not minutes).

    python -m mpserve_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libmpserve_b200.so"
SOURCES = ["decode_bucket.cu", "decode_shared.cu", "encode.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "mpserve_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc_path(), "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "--use_fast_math", "-o", str(LIB)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("MPS_EXTRA_NVCC_FLAGS", "").split()  # tuning experiments, e.g. -DMPS_LOOK=2
    cmd += [str(CSRC / s) for s in SOURCES]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.run(cmd, check=True, env=env)
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
