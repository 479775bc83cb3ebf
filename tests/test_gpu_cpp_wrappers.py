"""Builds and runs tests/cpp/kernel_test.cpp: the C++ wrappers that keep the reference's signatures
(unholy_b200/csrc/host/kernels.hpp), exercised the way the reference's standalone kernel tests do."""
import subprocess
from pathlib import Path

import pytest

from unholy_b200 import build

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "tests" / "cpp" / "kernel_test.bin"


def build_binary():
    lib = build.build_library()
    src = ROOT / "tests" / "cpp" / "kernel_test.cpp"
    if not BIN.exists() or BIN.stat().st_mtime < max(src.stat().st_mtime, lib.stat().st_mtime):
        cmd = [build.nvcc_path(), "-std=c++17", "-O2", "-x", "cu", "-gencode", "arch=compute_100a,code=sm_100a",
               str(src), "-o", str(BIN), f"-L{lib.parent}", "-lunholy_pkv", f"-Xlinker=-rpath={lib.parent}"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        assert res.returncode == 0, res.stdout + res.stderr
    return BIN


def test_wrappers_compile_against_the_library():
    """CPU: the header compiles and links (no GPU call is made)."""
    build_binary()


@pytest.mark.gpu
def test_wrappers_on_gpu(cuda):
    res = subprocess.run([str(build_binary())], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "all ok" in res.stdout, res.stdout + res.stderr
