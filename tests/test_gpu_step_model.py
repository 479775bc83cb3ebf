"""The host half of the drop-in boundary: the reference's unmodified Engine (src/engine/engine.cpp) drives the GPU path
through its own StepModel interface (src/engine/step.hpp:76-106), implemented by PkvStepModel
(unholy_b200/csrc/host/step_model.hpp) on the C-ABI library. The driver program (tests/cpp/step_model_test.cpp) is
compiled where the reference checkout exists — it contains the reference's engine, so it lives under oracle/_ref/ — and
travels to the GPU box as a binary."""
import subprocess

import pytest

from oracle import build_oracle


def binary():
    from unholy_b200 import build
    build.build_library()
    return build_oracle.build_reference()["step_model_test"]


def test_step_model_adaptor_compiles_against_the_reference_headers():
    if not (build_oracle.REFERENCE / "src" / "engine" / "step.hpp").exists():
        pytest.skip("no reference checkout here")
    assert binary() is not None


@pytest.mark.gpu
def test_reference_engine_drives_the_gpu_path(cuda):
    exe = binary()
    if exe is None:
        pytest.skip("oracle/_ref/step_model_test was not built (no reference checkout where the tree was prepared)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0 and "all ok" in res.stdout, res.stdout[-4000:] + res.stderr[-2000:]
