"""ctypes + numpy front end of the CPU oracle (oracle/pkv_oracle.cpp). TEST INFRASTRUCTURE ONLY: imported by tests/,
by __graft_entry__.smoke() and by bench.py's CPU-baseline legs, never by the product package."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import build_oracle as _b  # noqa: E402

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_SIGS = {
    "orc_bf16_to_f32": (C.c_float, [C.c_uint16]),
    "orc_f32_to_bf16": (C.c_uint16, [C.c_float]),
    "orc_e4m3_to_f32": (C.c_float, [C.c_uint8]),
    "orc_f32_to_e4m3": (C.c_uint8, [C.c_float]),
    "orc_e8m0_to_f32": (C.c_float, [C.c_uint8]),
    "orc_e2m1_to_f32": (C.c_float, [C.c_uint32]),
    "orc_round_e2m1": (C.c_float, [C.c_float]),
    "orc_pow2_ceil_e8m0": (C.c_uint8, [C.c_float]),
    "orc_e2m1_code": (C.c_uint32, [C.c_float]),
    "orc_store_rows": (None, [_vp, _i, _i, _vp, _vp, _i, _i, _i]),
    "orc_store_rows_fp4": (None, [_vp, _i, _i, _vp, _vp, _i, _i]),
    "orc_load_rows_fp4": (None, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "orc_fake_quant_fp4": (None, [_vp, _i, _i, _i, _i]),
    "orc_act_quant_fp8": (None, [_vp, _i, _vp, _vp, _i, _i, _i]),
    "orc_fake_quant_fp8": (None, [_vp, _i, _i, _i, _i]),
    "orc_kv_chain": (None, [_vp, _vp, _i, _i, C.c_float, _vp, _vp, _i, _i]),
    "orc_store_rows_fp8": (None, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _i]),
    "orc_gather_rows": (None, [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _i]),
    "orc_store_rows_chunks": (None, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _i, _i]),
    "orc_store_rows_fp4_chunks": (None, [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _i]),
    "orc_store_rows_fp8_chunks": (None, [_vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _i]),
    "orc_copy_pages": (None, [_vp, _sz, _vp, _vp, _i, _i]),
    "orc_move_pages": (None, [_vp, _vp, _sz, _vp, _vp, _i, _i]),
    "orc_copy": (None, [_vp, _vp, _sz]),
    "orc_topk_bf16": (None, [_vp, _i, _i, C.c_longlong, _i, _vp, _i]),
    "orc_topk_f32": (None, [_vp, _i, _i, C.c_longlong, _i, _vp, _i]),
    "orc_idx_expand": (None, [_vp, _vp, _vp, _i, _i, _i]),
    "orc_hadamard128": (None, [_vp, C.c_size_t]),
    "orc_state_copies": (None, [_vp, _vp, _vp, _i, _vp, _vp, _i, _vp, C.c_size_t, _i]),
    "orc_gather_rows_fp8": (None, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "orc_hardware_threads": (_i, []),
}
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = _b.ORACLE_LIB if _b.ORACLE_LIB.exists() else _b.build_oracle()
        h = C.CDLL(str(path))
        for name, (res, args) in _SIGS.items():
            fn = getattr(h, name)
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data


# ---- bf16 helpers on numpy (bit patterns in uint16) ----
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---- operations (arrays are modified in place where the C function does so) ----
def store_rows(rows, pool, table, rows_per_page, row_stride, row0):
    n, width = rows.shape
    lib().orc_store_rows(_p(rows), n, width, _p(pool), _p(table), rows_per_page, row_stride, row0)


def store_rows_fp4(rows, pool, table, rows_per_page, row0):
    n, dim = rows.shape
    lib().orc_store_rows_fp4(_p(rows), n, dim, _p(pool), _p(table), rows_per_page, row0)


def load_rows_fp4(pool, table, rows_per_page, dim, row0, n):
    out = np.empty((n, dim), np.uint16)
    lib().orc_load_rows_fp4(_p(pool), _p(table), rows_per_page, dim, row0, n, _p(out))
    return out


def fake_quant_fp4(x, cols, block):
    lib().orc_fake_quant_fp4(_p(x), x.shape[1], x.shape[0], cols, block)


def act_quant_fp8(x, cols, block):
    rows = x.shape[0]
    q = np.empty((rows, cols), np.uint8)
    s = np.empty((rows, cols // block), np.uint8)
    lib().orc_act_quant_fp8(_p(x), x.shape[1], _p(q), _p(s), rows, cols, block)
    return q, s


def fake_quant_fp8(x, cols, block):
    lib().orc_fake_quant_fp8(_p(x), x.shape[1], x.shape[0], cols, block)


def kv_chain(x, w, eps, pos, freqs, npair, quant=True):
    """In place on x [rows][dim] (bf16 bits); freqs float32 [positions][npair][2] = (cos, sin)."""
    rows, dim = x.shape
    lib().orc_kv_chain(_p(x), _p(w), rows, dim, eps, _p(pos), _p(freqs), npair, 1 if quant else 0)


def store_rows_fp8(rows, block, codes, scales, table, rows_per_page, s0):
    n, width = rows.shape
    lib().orc_store_rows_fp8(_p(rows), n, width, block, _p(codes), _p(scales), _p(table), rows_per_page, s0)


def gather_rows(pool, tables, rows_per_page, row_stride, width, idx, q_slot, q_visible, threads=1):
    T, k = idx.shape
    out = np.empty((T, k, width), np.uint16)
    lib().orc_gather_rows(_p(pool), _p(tables), tables.shape[1], rows_per_page, row_stride, width, _p(idx), _p(q_slot),
                          _p(q_visible), T, k, _p(out), threads)
    return out


def store_rows_chunks(rows, pool, tables, rows_per_page, row_stride, chunks, threads=1):
    lib().orc_store_rows_chunks(_p(rows), rows.shape[1], _p(pool), _p(tables), tables.shape[1], rows_per_page,
                                row_stride, _p(chunks), chunks.shape[0], threads)


def store_rows_fp4_chunks(rows, pool, tables, rows_per_page, chunks, threads=1):
    lib().orc_store_rows_fp4_chunks(_p(rows), rows.shape[1], _p(pool), _p(tables), tables.shape[1], rows_per_page,
                                    _p(chunks), chunks.shape[0], threads)


def store_rows_fp8_chunks(rows, block, codes, scales, tables, rows_per_page, chunks, threads=1):
    lib().orc_store_rows_fp8_chunks(_p(rows), rows.shape[1], block, _p(codes), _p(scales), _p(tables), tables.shape[1],
                                    rows_per_page, _p(chunks), chunks.shape[0], threads)


def copy_pages(pool, page_bytes, src, dst, threads=1):
    lib().orc_copy_pages(_p(pool), page_bytes, _p(src), _p(dst), len(src), threads)


def move_pages(src_pool, dst_pool, page_bytes, src, dst, threads=1):
    lib().orc_move_pages(_p(src_pool), _p(dst_pool), page_bytes, _p(src), _p(dst), len(src), threads)


def topk_bf16(scores, n, k, threads=1):
    T, ld = scores.shape
    idx = np.empty((T, k), np.int32)
    lib().orc_topk_bf16(_p(scores), T, n, ld, k, _p(idx), threads)
    return idx


def topk_f32(scores, n, k, threads=1):
    T, ld = scores.shape
    assert scores.dtype == np.float32
    idx = np.empty((T, k), np.int32)
    lib().orc_topk_f32(_p(scores), T, n, ld, k, _p(idx), threads)
    return idx


def state_copies(bufs, seg_off, ops, snap, snap_bytes, save):
    """bufs: uint8 arrays [slots][bytes per slot] (modified in place when save is false); seg_off: each one's offset in
    a snapshot; ops: (slot, snapshot) pairs; snap: uint8 [snapshots * snap_bytes] (modified in place when save)."""
    n = len(bufs)
    dev = np.array([b.ctypes.data for b in bufs], np.uint64)
    nbytes = np.array([b.shape[1] for b in bufs], np.uint64)
    off = np.array(seg_off, np.uint64)
    slot = np.array([o[0] for o in ops], np.int32)
    sn = np.array([o[1] for o in ops], np.int32)
    lib().orc_state_copies(_p(dev), _p(nbytes), _p(off), n, _p(slot), _p(sn), len(ops), _p(snap), snap_bytes, int(save))


def hadamard128(x):
    """In place on a contiguous uint16 (bf16 bits) array whose size is a multiple of 128."""
    assert x.dtype == np.uint16 and x.flags.c_contiguous and x.size % 128 == 0
    lib().orc_hadamard128(_p(x), x.size // 128)
    return x


def idx_expand(pools, pos, pool):
    n, k = pools.shape
    idx = np.empty((n, k * pool + pool - 1), np.int32)
    lib().orc_idx_expand(_p(pools), _p(pos), _p(idx), n, k, pool)
    return idx


def gather_rows_fp8(codes, scales, table, rows_per_page, block, idx, q_visible):
    T, k = idx.shape
    width = codes.shape[1]
    out = np.empty((T, k, width), np.uint16)
    lib().orc_gather_rows_fp8(_p(codes), _p(scales), _p(table), rows_per_page, width, block, _p(idx), _p(q_visible), T, k, _p(out))
    return out


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())
