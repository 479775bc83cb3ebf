"""ctypes binding of include/unholy_pkv.h. One declaration per exported function; no logic."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "lib" / "libunholy_pkv.so"

PKV_OK, PKV_ERR_ARG, PKV_ERR_CUDA, PKV_ERR_DEVICE, PKV_ERR_LIMIT = range(5)
PKV_MAX_LAYERS = 48
PKV_DO_ROWS, PKV_DO_KEYS_FP4, PKV_DO_KEYS_FP8, PKV_DO_GATHER, PKV_VARIANT_BULK = 1, 2, 4, 8, 256
PKV_KEYS_HADAMARD = 32

c_i32p = C.POINTER(C.c_int32)
c_u8p = C.POINTER(C.c_uint8)


class PkvError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"pkv error {code}: {msg}")
        self.code = code


class PkvChunk(C.Structure):
    _fields_ = [("slot", C.c_int32), ("s0", C.c_int32), ("n", C.c_int32), ("t0", C.c_int32)]


class PkvLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("rows", "row_pool", "keys", "key_pool_fp4", "key_fp8_codes", "key_fp8_scales", "idx", "gathered")]


class PkvStep(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("width", "row_stride", "rows_per_page", "max_pages_per_seq", "num_pages", "fp8_block", "nchunks", "T",
                 "Q", "k", "max_slots", "reserved")] + [(n, C.c_void_p) for n in ("tables", "chunks", "q_chunk", "q_visible")]


class PkvStateSeg(C.Structure):
    _fields_ = [("dev", C.c_void_p), ("bytes", C.c_size_t), ("off", C.c_size_t)]


class PkvStateOp(C.Structure):
    _fields_ = [("slot", C.c_int32), ("snapshot", C.c_int32)]


class PkvTopkGroup(C.Structure):
    _fields_ = [("off", C.c_size_t), ("rows", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("idx_off", C.c_int32)]


class PkvShardConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("ngpus", "num_pages", "rows_per_page", "width", "row_stride", "layers", "max_slots",
                                         "max_pages_per_seq", "k", "key_pools")]


class PkvShardIo(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("rows", "keys", "idx", "gathered")]


class PkvSnapHit(C.Structure):
    _fields_ = [("pages", C.c_int32), ("snap", C.c_int32), ("disk_slot", C.c_int32), ("reserved", C.c_int32), ("hash", C.c_uint64)]


class PkvSnapDone(C.Structure):
    _fields_ = [("write", C.c_int32), ("ok", C.c_int32), ("snap", C.c_int32), ("reserved", C.c_int32), ("load_id", C.c_uint64)]


class PkvSnapCounters(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("cached", "free_or_evictable", "on_disk", "io_pending")] + \
               [(n, C.c_uint64) for n in ("spills", "disk_hits", "disk_read_bytes", "disk_write_bytes")]


SNAP_IO_HOOK = C.CFUNCTYPE(None, C.c_int, C.c_void_p)


class PkvPoolDesc(C.Structure):
    _fields_ = [("src_base", C.c_void_p), ("dst_base", C.c_void_p), ("page_bytes", C.c_uint64)]


_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_SIGS = {
    "pkv_last_error": (C.c_char_p, []),
    "pkv_abi_version": (_i, []),
    "pkv_tune": (_i, [_i, _i]),
    "pkv_device_status": (_i, [C.POINTER(C.c_int)]),
    "pkv_stream_check": (_i, [_vp]),
    "pkv_store_rows": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_store_rows_fp4": (_i, [_vp, _i, _vp, _vp, _i, _i, _vp]),
    "pkv_load_rows_fp4": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "pkv_act_quant_fp8": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_fake_quant_fp8": (_i, [_vp, _i, _i, _i, _i, _vp]),
    "pkv_fake_quant_fp4": (_i, [_vp, _i, _i, _i, _i, _vp]),
    "pkv_store_rows_fp8": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "pkv_copy": (_i, [_vp, _vp, _sz, _vp]),
    "pkv_gather_rows": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp]),
    "pkv_gather_rows_fp8": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp, _vp]),
    "pkv_step_run": (_i, [C.POINTER(PkvStep), C.POINTER(PkvLayer), _i, _i, _vp]),
    "pkv_step_gather_fp8": (_i, [C.POINTER(PkvStep), _vp, _vp, _i, _i, _vp, _vp, _vp]),
    "pkv_step_gather_fp8_pools": (_i, [C.POINTER(PkvStep), _vp, _vp, _i, _i, _vp, _vp, _i, _i, _vp, _vp]),
    "pkv_hadamard128": (_i, [_vp, _sz, _vp]),
    "pkv_store_rows_fake_fp8": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_store_rows_kv_chain": (_i, [_vp, _vp, _vp, _i, _i, C.c_float, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_topk_scratch_words": (_sz, [_i, _i, _i]),
    "pkv_topk_bf16": (_i, [_vp, _i, _i, C.c_longlong, _i, _vp, _vp, _sz, _vp]),
    "pkv_topk_static_scratch_words": (_sz, []),
    "pkv_topk_bf16_static": (_i, [_vp, _i, _i, C.c_longlong, _i, _vp, _vp]),
    "pkv_topk_batch_scratch_words": (_sz, [C.POINTER(PkvTopkGroup), _i]),
    "pkv_topk_bf16_batch": (_i, [_vp, C.POINTER(PkvTopkGroup), _i, _vp, _vp, _sz, _vp]),
    "pkv_topk_f32": (_i, [_vp, _i, _i, C.c_longlong, _i, _vp, _vp]),
    "pkv_state_copies": (_i, [C.POINTER(PkvStateSeg), _i, C.POINTER(PkvStateOp), _i, _vp, _sz, _i, _i, _i, _vp]),
    "pkv_idx_expand": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_copy_pages": (_i, [C.POINTER(PkvPoolDesc), _i, _vp, _vp, _i, _i, _i, _vp]),
    "pkv_device_alloc": (_i, [C.POINTER(_vp), _sz]),
    "pkv_device_free": (_i, [_vp]),
    "pkv_ipc_export": (_i, [_vp, c_u8p]),
    "pkv_ipc_open": (_i, [c_u8p, C.POINTER(_vp)]),
    "pkv_ipc_close": (_i, [_vp]),
    "pkv_shards_create": (_vp, [C.POINTER(PkvShardConfig), C.POINTER(C.c_int)]),
    "pkv_shards_destroy": (None, [_vp]),
    "pkv_shards_add": (_i, [_vp, _i, _i, _i]),
    "pkv_shards_remove": (_i, [_vp, _i]),
    "pkv_shards_owner": (_i, [_vp, _i]),
    "pkv_shards_length": (_i, [_vp, _i]),
    "pkv_shards_slot": (_i, [_vp, _i]),
    "pkv_shards_local": (_i, [_vp, _i, c_i32p, _i]),
    "pkv_shards_free_pages": (_i, [_vp, _i]),
    "pkv_shards_row_pool": (_vp, [_vp, _i, _i]),
    "pkv_shards_key_pool": (_vp, [_vp, _i, _i]),
    "pkv_shards_tables": (_vp, [_vp, _i]),
    "pkv_shards_stream": (_vp, [_vp, _i]),
    "pkv_shards_step": (_i, [_vp, C.POINTER(PkvShardIo)]),
    "pkv_shards_mark": (_i, [_vp, _i]),
    "pkv_shards_elapsed_ms": (_i, [_vp, C.POINTER(C.c_float)]),
    "pkv_shards_sync": (_i, [_vp]),
    "pkv_shards_migrate_begin": (_i, [_vp, c_i32p, c_i32p, _i]),
    "pkv_shards_migrate_end": (_i, [_vp, _i]),
    "pkv_shards_migrate_pending": (_i, [_vp]),
    "pkv_shards_migrate_landed": (_i, [_vp]),
    "pkv_shards_migrate_stats": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_float)]),
    "pkv_snap_create": (_vp, [_i, _vp, _sz, C.c_char_p, _i, SNAP_IO_HOOK, _vp]),
    "pkv_snap_destroy": (None, [_vp]),
    "pkv_snap_disk_on": (_i, [_vp]),
    "pkv_snap_match": (_i, [_vp, C.POINTER(C.c_uint64), _i, c_u8p, C.POINTER(PkvSnapHit)]),
    "pkv_snap_start_load": (C.c_uint64, [_vp, C.POINTER(PkvSnapHit)]),
    "pkv_snap_cancel_load": (None, [_vp, C.POINTER(PkvSnapHit)]),
    "pkv_snap_take": (_i, [_vp]),
    "pkv_snap_put": (None, [_vp, _i]),
    "pkv_snap_commit": (None, [_vp, _i, C.c_uint64, _i, C.POINTER(C.c_int), C.POINTER(C.c_uint64)]),
    "pkv_snap_spare": (_i, [_vp]),
    "pkv_snap_spill": (None, [_vp]),
    "pkv_snap_poll": (_i, [_vp, C.POINTER(PkvSnapDone), _i]),
    "pkv_snap_clear": (None, [_vp]),
    "pkv_snap_wait_idle": (None, [_vp]),
    "pkv_snap_counters": (_i, [_vp, C.POINTER(PkvSnapCounters)]),
    "pkv_pool_create": (_vp, [_i, _i, _i, _i, _i]),
    "pkv_pool_destroy": (None, [_vp]),
    "pkv_pool_seq_open": (_i, [_vp]),
    "pkv_pool_seq_close": (_i, [_vp, _i]),
    "pkv_pool_match_prefix": (_i, [_vp, _i, c_i32p, _i, c_u8p]),
    "pkv_token_keys": (_i, [c_i32p, _i, c_i32p, c_i32p, C.POINTER(C.c_uint64), _i, C.POINTER(C.c_uint64)]),
    "pkv_pool_match_prefix_keys": (_i, [_vp, _i, C.POINTER(C.c_uint64), _i, c_u8p]),
    "pkv_pool_register_keys": (_i, [_vp, _i, C.POINTER(C.c_uint64), _i, _i]),
    "pkv_pool_cached_prefix_keys": (_i, [_vp, C.POINTER(C.c_uint64), _i]),
    "pkv_page_hash_keys": (C.c_uint64, [C.POINTER(C.c_uint64), _i, _i]),
    "pkv_pool_assign_slot": (_i, [_vp, _i]),
    "pkv_pool_alloc": (_i, [_vp, _i, _i]),
    "pkv_pool_register": (_i, [_vp, _i, c_i32p, _i, _i]),
    "pkv_pool_release": (_i, [_vp, _i]),
    "pkv_pool_drop_prefix": (_i, [_vp, _i]),
    "pkv_pool_fork": (_i, [_vp, _i, _i]),
    "pkv_pool_cow": (_i, [_vp, _i, _i, _i, c_i32p, c_i32p, _i]),
    "pkv_pool_cow_pairs": (_i, [_vp, _i, _i, _i]),
    "pkv_pool_compact_pairs": (_i, [_vp]),
    "pkv_pool_free_lru": (_i, [_vp, _i, c_i32p, _i]),
    "pkv_pool_compact": (_i, [_vp, c_i32p, c_i32p, _i]),
    "pkv_pool_migrate": (_i, [_vp, _i, _vp, C.POINTER(C.c_int), c_i32p, c_i32p, _i]),
    "pkv_pool_available": (_i, [_vp]),
    "pkv_pool_free_count": (_i, [_vp]),
    "pkv_pool_evictable_count": (_i, [_vp]),
    "pkv_pool_cached_count": (_i, [_vp]),
    "pkv_pool_seq_pages": (_i, [_vp, _i, c_i32p, _i]),
    "pkv_pool_seq_slot": (_i, [_vp, _i]),
    "pkv_pool_page_refs": (_i, [_vp, _i]),
    "pkv_pool_page_hash": (C.c_uint64, [_vp, _i]),
    "pkv_pool_dirty": (_i, [_vp]),
    "pkv_pool_tables": (c_i32p, [_vp]),
    "pkv_pool_free_list": (_i, [_vp, c_i32p, _i]),
    "pkv_pool_evictable_list": (_i, [_vp, c_i32p, _i]),
    "pkv_page_hash": (C.c_uint64, [c_i32p, _i, _i]),
}

_lib = None


def library_path() -> Path:
    return _LIB_PATH


def lib() -> C.CDLL:
    """The loaded library. Raises when it has not been built: there is nothing to fall back to."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise FileNotFoundError(
                f"{_LIB_PATH} is missing: build it with `python -m unholy_b200.build` (needs nvcc). "
                "There is no CPU or Python fallback for this library.")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(rc: int) -> None:
    if rc != PKV_OK:
        raise PkvError(rc, lib().pkv_last_error().decode())
