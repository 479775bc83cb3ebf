"""Builds libunholy_pkv.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m unholy_b200.build            # build if sources are newer than the library
    python -m unholy_b200.build --force

nvcc cross-compiles without a GPU. The flags matter for bit-exactness: no fast-math, no flush-to-zero, no fused
multiply-add contraction (-fmad=false), IEEE division.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libunholy_pkv.so"
SOURCES = [CSRC / "pkv_kernels.cu", CSRC / "pkv_topk.cu", CSRC / "pkv_topk_cluster.cu", CSRC / "pkv_topk_f32.cu", CSRC / "pkv_state.cu", CSRC / "pkv_shard.cu", CSRC / "page_pool.cpp", CSRC / "snapshot_store.cpp"]
HEADERS = [CSRC / "pkv_numeric.cuh", CSRC / "pkv_internal.hpp", CSRC / "page_pool.hpp", CSRC / "snapshot_store.hpp", PKG.parent / "include" / "unholy_pkv.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
    "-cudart", "static", "-Xcompiler", "-pthread",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in SOURCES + HEADERS + [Path(__file__)])


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    tmp = LIB.with_suffix(".so.tmp")  # linked beside the library and renamed: a reader never sees a half-written file
    cmd = [nvcc_path(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), *map(str, SOURCES), "-o", str(tmp)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    os.replace(tmp, LIB)
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    out = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(out)
