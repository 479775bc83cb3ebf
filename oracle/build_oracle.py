"""Builds the CPU oracle libraries. TEST INFRASTRUCTURE ONLY.

    python oracle/build_oracle.py

  oracle/_build/libpkv_oracle.so   the scalar C++ restatement (oracle/pkv_oracle.cpp); always built.
  oracle/_ref/libref_numeric.so    the reference's own scalar helpers, compiled from <reference>/src/kernels/dev.hip.hpp
                                   where it lies (through oracle/hip_shim); only when the reference checkout exists.
  oracle/_ref/libref_engine.so     the reference's own engine.cpp + sampler.cpp with oracle/ref_engine_driver.cpp (a
                                   recording StepModel); only when the reference checkout exists.
  oracle/_ref/step_model_test      the reference's own engine.cpp + sampler.cpp driving the product library through its
                                   StepModel adaptor (tests/cpp/step_model_test.cpp); only when the reference checkout and
                                   the built product library exist. Needs a GPU to run.

No reference source is copied: the compiler reads it in place. The _ref outputs are git-ignored and travel to the GPU
box as binaries; when the checkout is absent the already-built files are used as they are.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REFERENCE = Path(os.environ.get("UNHOLY_REFERENCE", "/root/reference"))
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
ORACLE_LIB = BUILD / "libpkv_oracle.so"
REF_NUMERIC_LIB = REF_OUT / "libref_numeric.so"
REF_ENGINE_LIB = REF_OUT / "libref_engine.so"
STEP_MODEL_TEST = REF_OUT / "step_model_test"
ROOT = HERE.parent


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)


def _newer(target: Path, *deps: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists())


def build_oracle(force: bool = False) -> Path:
    src = HERE / "pkv_oracle.cpp"
    if force or not _newer(ORACLE_LIB, src):
        BUILD.mkdir(exist_ok=True)
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-fno-fast-math", "-ffp-contract=off",
              str(src), "-o", str(ORACLE_LIB)])
    return ORACLE_LIB


def build_reference(force: bool = False) -> dict:
    """Compiles the reference's own sources in place. Returns {name: path or None}."""
    out = {"numeric": None, "engine": None, "step_model_test": None}
    have = (REFERENCE / "src" / "kernels" / "dev.hip.hpp").exists()
    if have:
        REF_OUT.mkdir(exist_ok=True)
        drv = HERE / "ref_numeric_driver.cpp"
        if force or not _newer(REF_NUMERIC_LIB, drv, REFERENCE / "src/kernels/dev.hip.hpp"):
            _run(["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-w", "-fno-fast-math", "-ffp-contract=off",
                  f"-I{HERE / 'hip_shim'}", f"-I{REFERENCE / 'src'}", str(drv), "-o", str(REF_NUMERIC_LIB)])
        edrv = HERE / "ref_engine_driver.cpp"
        if edrv.exists() and (force or not _newer(REF_ENGINE_LIB, edrv, REFERENCE / "src/engine/engine.cpp")):
            _run(["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-pthread", f"-I{REFERENCE / 'src'}",
                  str(REFERENCE / "src/engine/engine.cpp"), str(REFERENCE / "src/engine/sampler.cpp"), str(edrv),
                  "-o", str(REF_ENGINE_LIB)])
        src = ROOT / "tests" / "cpp" / "step_model_test.cpp"
        hdr = ROOT / "unholy_b200" / "csrc" / "host" / "step_model.hpp"
        lib = ROOT / "unholy_b200" / "lib" / "libunholy_pkv.so"
        cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
        if src.exists() and lib.exists() and (force or not _newer(STEP_MODEL_TEST, src, hdr, lib, REFERENCE / "src/engine/engine.cpp")):
            _run(["g++", "-std=c++20", "-O2", "-pthread", f"-I{REFERENCE / 'src'}", f"-I{cuda / 'include'}", str(src),
                  str(REFERENCE / "src/engine/engine.cpp"), str(REFERENCE / "src/engine/sampler.cpp"), "-o", str(STEP_MODEL_TEST),
                  f"-L{lib.parent}", "-lunholy_pkv", f"-L{cuda / 'lib64'}", "-lcudart", "-Wl,-rpath,$ORIGIN/../../unholy_b200/lib"])
    if STEP_MODEL_TEST.exists():
        out["step_model_test"] = STEP_MODEL_TEST
    if REF_NUMERIC_LIB.exists():
        out["numeric"] = REF_NUMERIC_LIB
    if REF_ENGINE_LIB.exists():
        out["engine"] = REF_ENGINE_LIB
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_reference(force))
