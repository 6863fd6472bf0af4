"""Build libcqa_b200.so (sm_100a) in-tree with nvcc.

    python certified-quantised-attention_b200/build.py [--force] [--verbose]

The library has no dependency on torch or Python: CUDA runtime only.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
LIB = HERE / "cqa_b200" / "libcqa_b200.so"
SOURCES = ["api.cu", "quantize.cu", "score.cu", "select.cu", "attend.cu", "hot_tier.cu", "peer.cu"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    cmd = [
        nvcc_path(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        # IEEE division / square root / no flush-to-zero: the canonical arithmetic depends on it
        "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
        "-I", str(INCLUDE), "-o", str(LIB),
    ] + [str(CSRC / s) for s in SOURCES]
    extra = os.environ.get("CQA_NVCC_FLAGS")
    if extra:
        cmd[1:1] = extra.split()
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libcqa_b200.so")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
