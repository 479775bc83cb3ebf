"""The C-ABI library builds, loads without a GPU, and exports exactly the functions include/unholy_pkv.h declares.
No compute call is made here."""
import ctypes as C
import re
from pathlib import Path

from unholy_b200 import capi

ROOT = Path(__file__).resolve().parent.parent


def declared():
    text = (ROOT / "include" / "unholy_pkv.h").read_text()
    return sorted(set(re.findall(r"^PKV_API [^;(]*?\b(pkv_\w+)\(", text, flags=re.M)))


def test_every_declared_symbol_is_exported_and_bound(pkv):
    names = declared()
    assert len(names) >= 40
    for n in names:
        assert hasattr(pkv, n), f"{n} declared in include/unholy_pkv.h but not exported"
    assert sorted(capi._SIGS) == names, "capi.py and the header disagree"


def test_struct_layouts_match_the_header():
    assert C.sizeof(capi.PkvChunk) == 16
    assert C.sizeof(capi.PkvLayer) == 64
    assert C.sizeof(capi.PkvStep) == 72
    assert C.sizeof(capi.PkvPoolDesc) == 24
    assert capi.PkvStep.tables.offset == 40 and capi.PkvStep.q_visible.offset == 64


def test_argument_errors_without_a_device(pkv):
    assert pkv.pkv_abi_version() == 1
    assert pkv.pkv_store_rows(None, 0, 576, None, None, 64, 576, 0, None) == capi.PKV_OK  # n <= 0 returns early
    assert pkv.pkv_store_rows(None, 4, 576, None, None, 64, 576, 0, None) == capi.PKV_ERR_ARG
    assert b"null pointer" in pkv.pkv_last_error()
    assert pkv.pkv_step_run(None, None, 1, 0, None) == capi.PKV_ERR_ARG
    st = capi.PkvStep()
    layers = (capi.PkvLayer * 1)()
    assert pkv.pkv_step_run(C.byref(st), layers, capi.PKV_MAX_LAYERS + 1, 8, None) == capi.PKV_ERR_LIMIT


def test_product_package_does_not_touch_the_oracle():
    for p in (ROOT / "unholy_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"):
            assert "oracle" not in p.read_text(), f"{p} mentions the oracle"
