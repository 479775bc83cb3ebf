"""Shared helpers of the parity tests: seeded synthetic inputs in the shapes of the benchmark configurations, and
device buffers (torch is used only to own device memory)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import oracle_lib as orc
from unholy_b200 import capi

W, KEY_DIM, RPP = 576, 128, 64
ROW_BYTES = W * 2
PAGE_BYTES = RPP * ROW_BYTES
FP4_PAGE_BYTES = RPP * 68


def rng(seed):
    return np.random.Generator(np.random.MT19937(seed))


def normal_bf16(g, shape, scale=1.0):
    return orc.f32_to_bf16_bits((g.standard_normal(shape, dtype=np.float32) * np.float32(scale)))


def key_rows(g, n, dim=KEY_DIM):
    """Keys N(0,1) with a per-row magnitude 2^U{-3..3} (the spread of the reference's indexer test)."""
    mag = np.ldexp(np.float32(1.0), g.integers(-3, 4, size=(n, 1))).astype(np.float32)
    return orc.f32_to_bf16_bits(g.standard_normal((n, dim), dtype=np.float32) * mag)


def outlier_rows(g, n, width):
    """N(0,1) rows with 1 % of the entries replaced by +-20."""
    x = g.standard_normal((n, width), dtype=np.float32)
    m = g.random((n, width)) < 0.01
    x[m] = np.where(g.random(int(m.sum())) < 0.5, np.float32(-20.0), np.float32(20.0))
    return orc.f32_to_bf16_bits(x)


def dev(torch, a: np.ndarray):
    """Device copy of a numpy array as a flat uint8 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1).copy()).cuda()


def host(t, dtype, shape=None):
    a = t.cpu().numpy().view(dtype)
    return a.reshape(shape) if shape is not None else a


def stream_ptr(torch):
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status(lib):
    st = C.c_int(0)
    capi.check(lib.pkv_device_status(C.byref(st)))
    return st.value


class PagedCase:
    """Sequences with shuffled block tables over one pool; the shape of benchmark configuration 1 by default."""

    def __init__(self, seed=1, nseq=8, len_lo=1024, len_hi=8192, num_pages=1024, k=2048, width=W, row_stride=None,
                 rows_per_page=RPP, with_keys=True, fill=True, append=1):
        g = rng(seed)
        self.width, self.rpp, self.k = width, rows_per_page, k
        self.row_stride = row_stride or width
        self.num_pages, self.nseq = num_pages, nseq
        while True:
            lens = g.integers(len_lo, len_hi + 1, size=nseq)
            need = [-(-(int(l) + append) // rows_per_page) for l in lens]
            if sum(need) <= num_pages:
                break
        self.lens = lens.astype(np.int32)
        self.pps = max(need) + 1
        perm = g.permutation(num_pages).astype(np.int32)
        self.tables = np.zeros((nseq, self.pps), np.int32)
        o = 0
        for s, nd in enumerate(need):
            self.tables[s, :nd] = perm[o:o + nd]
            o += nd
        self.pool = np.zeros((num_pages * rows_per_page, self.row_stride), np.uint16)
        if fill:
            self.pool[:, :] = normal_bf16(g, self.pool.shape)
        # the step: `append` new rows per sequence at row len
        self.T = nseq * append
        self.chunks = np.array([[s, int(self.lens[s]), append, s * append] for s in range(nseq)], np.int32)
        self.rows = normal_bf16(g, (self.T, width))
        self.keys = key_rows(g, self.T) if with_keys else None
        # one query per sequence at its last appended position: min(k, visible) distinct sorted positions, -1 padded
        self.q_chunk = np.arange(nseq, dtype=np.int32)
        self.q_slot = np.arange(nseq, dtype=np.int32)
        self.q_visible = (self.lens + append).astype(np.int32)
        self.idx = np.full((nseq, k), -1, np.int32)
        for s in range(nseq):
            vis = int(self.q_visible[s])
            m = min(k, vis)
            self.idx[s, :m] = np.sort(g.choice(vis, size=m, replace=False)).astype(np.int32)

    # ---- oracle results ----
    def oracle_append(self):
        pool = self.pool.copy()
        orc.store_rows_chunks(self.rows, pool, self.tables, self.rpp, self.row_stride, self.chunks)
        return pool

    def oracle_gather(self, pool):
        return orc.gather_rows(pool, self.tables, self.rpp, self.row_stride, self.width, self.idx, self.q_slot,
                               self.q_visible)


def make_step(case, d_tables, d_chunks, d_qchunk, d_qvis, T=None, Q=None, fp8_block=64):
    st = capi.PkvStep()
    st.width, st.row_stride, st.rows_per_page = case.width, case.row_stride, case.rpp
    st.max_pages_per_seq, st.num_pages, st.fp8_block = case.pps, case.num_pages, fp8_block
    st.max_slots = case.tables.shape[0]
    st.nchunks, st.T = case.chunks.shape[0], case.T if T is None else T
    st.Q, st.k = (case.idx.shape[0] if Q is None else Q), case.k
    st.tables, st.chunks = d_tables.data_ptr(), d_chunks.data_ptr()
    st.q_chunk, st.q_visible = d_qchunk.data_ptr(), d_qvis.data_ptr()
    return st


def make_layers(n):
    return (capi.PkvLayer * n)()
