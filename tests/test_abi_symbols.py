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
    assert C.sizeof(capi.PkvStep) == 80
    assert C.sizeof(capi.PkvPoolDesc) == 24
    assert capi.PkvStep.max_slots.offset == 40 and capi.PkvStep.tables.offset == 48 and capi.PkvStep.q_visible.offset == 72


def test_argument_errors_without_a_device(pkv):
    assert pkv.pkv_abi_version() == 2
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


def test_step_run_validates_before_touching_the_device(pkv):
    """Shape, pointer and alignment errors are reported by the host code, so they can be checked without a GPU."""
    st = capi.PkvStep()
    layers = (capi.PkvLayer * 1)()
    st.width, st.row_stride, st.rows_per_page, st.max_pages_per_seq = 576, 576, 64, 8
    st.nchunks, st.T, st.Q, st.k = 1, 1, 1, 8
    assert pkv.pkv_step_run(C.byref(st), layers, 1, capi.PKV_DO_ROWS | capi.PKV_DO_GATHER, None) == capi.PKV_ERR_ARG
    assert b"num_pages and max_slots" in pkv.pkv_last_error()                              # ids are checked against them
    st.num_pages, st.max_slots = 16, 2
    flags = capi.PKV_DO_ROWS | capi.PKV_DO_GATHER
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags, None) == capi.PKV_ERR_ARG       # no tables / chunks
    assert b"tables and chunks" in pkv.pkv_last_error()
    st.tables = st.chunks = 4096
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags, None) == capi.PKV_ERR_ARG       # gather without q arrays
    st.q_chunk = st.q_visible = 4096
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags, None) == capi.PKV_ERR_ARG       # layer lacks idx / gathered
    st.width = 570
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags, None) == capi.PKV_ERR_ARG       # width not a multiple of 8
    st.width = 576
    layers[0].rows = layers[0].row_pool = layers[0].idx = layers[0].gathered = 4096
    layers[0].row_pool = 4100                                                                  # off the 16-byte grid
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags, None) == capi.PKV_ERR_ARG
    assert b"16-byte aligned" in pkv.pkv_last_error()
    st.fp8_block = 48
    layers[0].row_pool = 4096
    assert pkv.pkv_step_run(C.byref(st), layers, 1, flags | capi.PKV_DO_KEYS_FP8, None) == capi.PKV_ERR_ARG
    assert pkv.pkv_step_run(C.byref(st), layers, 0, flags, None) == capi.PKV_OK            # nothing to do
    assert pkv.pkv_copy_pages(None, 0, None, None, 0, 0, 0, None) == capi.PKV_OK
    descs = (capi.PkvPoolDesc * 1)()
    descs[0].src_base = descs[0].dst_base = 4096
    descs[0].page_bytes = 100                                                                  # not a multiple of 16
    assert pkv.pkv_copy_pages(descs, 1, 4096, 4096, 1, 0, 0, None) == capi.PKV_ERR_ARG
    assert pkv.pkv_tune(99, 0) == capi.PKV_ERR_ARG


def test_host_objects_validate_their_arguments(pkv):
    """The sharded host and the snapshot store refuse bad configurations before touching a device or a file."""
    cfg = capi.PkvShardConfig(0, 16, 64, 576, 576, 2, 4, 8, 64, 0)          # no shards
    assert not pkv.pkv_shards_create(C.byref(cfg), (C.c_int * 1)(0)) and b"bad configuration" in pkv.pkv_last_error()
    cfg = capi.PkvShardConfig(1, 16, 64, 570, 570, 2, 4, 8, 64, 0)          # width not a multiple of 8
    assert not pkv.pkv_shards_create(C.byref(cfg), (C.c_int * 1)(0))
    cfg = capi.PkvShardConfig(1, 16, 64, 576, 576, 100, 4, 8, 64, 1)        # 200 pools: more than one migration launch takes
    assert not pkv.pkv_shards_create(C.byref(cfg), (C.c_int * 1)(0))
    assert pkv.pkv_shards_owner(None, 0) == -1 and pkv.pkv_shards_migrate_pending(None) == -1
    assert pkv.pkv_shards_step(None, None) == capi.PKV_ERR_ARG
    assert not pkv.pkv_snap_create(-1, None, 0, None, 0, capi.SNAP_IO_HOOK(0), None)
    s = pkv.pkv_snap_create(2, None, 0, b"/nonexistent-dir/x", 4, capi.SNAP_IO_HOOK(0), None)   # snapshots not in host memory: tier off
    assert s and pkv.pkv_snap_disk_on(s) == 0
    assert pkv.pkv_snap_take(s) == 0 and pkv.pkv_snap_take(s) == 1 and pkv.pkv_snap_take(s) == -1   # slot 0 first (engine.cpp:90)
    pkv.pkv_snap_destroy(s)
