"""Prefix-cache churn on the GPU (benchmark configuration 4, mode B, reduced): snapshots of unaligned prefixes stay
alive, live requests fork them copy-on-write and append, a quarter of the pages is freed from the LRU front, the pool
is compacted. After every phase the device pools of every layer equal a host mirror driven by the CPU oracle byte for
byte, and at the end every live sequence read back through its block table equals what was appended to it.
Copy-on-write, compaction and LRU freeing have no reference counterpart (parity unpinned); the appends, gathers and
allocator calls underneath are the pinned ones."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

pytestmark = pytest.mark.gpu
i32p = C.POINTER(C.c_int32)


def ptr(a):
    return a.ctypes.data_as(i32p)


class Store:
    """L layers of (bf16 row pool, MXFP4 key pool) on the device with a numpy mirror, one page pool, one block table."""

    def __init__(self, pkv, torch, num_pages, slots, pps, layers=3, seed=4):
        self.pkv, self.torch, self.N, self.L, self.slots, self.pps = pkv, torch, num_pages, layers, slots, pps
        self.pool = pkv.pkv_pool_create(num_pages, tl.RPP, slots, pps, 1)
        self.g = tl.rng(seed)
        self.h_rows = [np.zeros((num_pages * tl.RPP, tl.W), np.uint16) for _ in range(layers)]
        self.h_fp4 = [np.zeros(num_pages * tl.FP4_PAGE_BYTES, np.uint8) for _ in range(layers)]
        self.d_rows = [tl.dev(torch, a) for a in self.h_rows]
        self.d_fp4 = [tl.dev(torch, a) for a in self.h_fp4]
        self.content = {}  # handle -> list of per-layer arrays [len][W] of what the sequence holds
        self.length = {}

    def close(self):
        self.pkv.pkv_pool_destroy(self.pool)

    def tables(self):
        return np.ctypeslib.as_array(self.pkv.pkv_pool_tables(self.pool), shape=(self.slots, self.pps)).copy()

    def append(self, items):
        """items: [(handle, n)]: appends n fresh rows and keys per layer to each sequence in ONE launch over all layers
        (copy-on-write first where a touched page is shared)."""
        pkv, torch = self.pkv, self.torch
        src, dst = np.zeros(64, np.int32), np.zeros(64, np.int32)
        chunks, t0 = [], 0
        for h, n in items:
            s0 = self.length.get(h, 0)
            assert pkv.pkv_pool_alloc(self.pool, h, s0 + n) == 1
            m = pkv.pkv_pool_cow(self.pool, h, s0, n, ptr(src), ptr(dst), 64)
            assert m >= 0
            if m:
                self.copy_pages(src[:m].copy(), dst[:m].copy())
            chunks.append([pkv.pkv_pool_seq_slot(self.pool, h), s0, n, t0])
            t0 += n
        chunks = np.array(chunks, np.int32)
        T = t0
        tables = self.tables()
        d_tables, d_chunks = tl.dev(torch, tables), tl.dev(torch, chunks)
        step = capi.PkvStep()
        step.width = step.row_stride = tl.W
        step.rows_per_page, step.max_pages_per_seq, step.num_pages, step.fp8_block = tl.RPP, self.pps, self.N, 64
        step.nchunks, step.T, step.Q, step.k, step.max_slots = len(chunks), T, 0, 0, tables.shape[0]
        step.tables, step.chunks = d_tables.data_ptr(), d_chunks.data_ptr()
        layers = tl.make_layers(self.L)
        keep = []
        for l in range(self.L):
            rows, keys = tl.normal_bf16(self.g, (T, tl.W)), tl.key_rows(self.g, T)
            d_r, d_k = tl.dev(torch, rows), tl.dev(torch, keys)
            keep += [d_r, d_k]
            layers[l].rows, layers[l].row_pool = d_r.data_ptr(), self.d_rows[l].data_ptr()
            layers[l].keys, layers[l].key_pool_fp4 = d_k.data_ptr(), self.d_fp4[l].data_ptr()
            orc.store_rows_chunks(rows, self.h_rows[l], tables, tl.RPP, tl.W, chunks)
            orc.store_rows_fp4_chunks(keys, self.h_fp4[l], tables, tl.RPP, chunks)
            for (h, n), ch in zip(items, chunks):
                self.content.setdefault(h, [np.zeros((0, tl.W), np.uint16) for _ in range(self.L)])
                self.content[h][l] = np.concatenate([self.content[h][l], rows[ch[3]:ch[3] + n]])
        capi.check(pkv.pkv_step_run(C.byref(step), layers, self.L, capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4,
                                    tl.stream_ptr(torch)))
        torch.cuda.synchronize()
        for h, n in items:
            self.length[h] = self.length.get(h, 0) + n

    def copy_pages(self, src, dst):
        """The same page moves on every pool of every layer: device in one launch, mirror through the oracle."""
        descs = (capi.PkvPoolDesc * (2 * self.L))()
        for l in range(self.L):
            descs[2 * l].src_base = descs[2 * l].dst_base = self.d_rows[l].data_ptr()
            descs[2 * l].page_bytes = tl.PAGE_BYTES
            descs[2 * l + 1].src_base = descs[2 * l + 1].dst_base = self.d_fp4[l].data_ptr()
            descs[2 * l + 1].page_bytes = tl.FP4_PAGE_BYTES
            orc.copy_pages(self.h_rows[l], tl.PAGE_BYTES, src, dst)
            orc.copy_pages(self.h_fp4[l], tl.FP4_PAGE_BYTES, src, dst)
        d_s, d_d = tl.dev(self.torch, src), tl.dev(self.torch, dst)
        capi.check(self.pkv.pkv_copy_pages(descs, 2 * self.L, d_s.data_ptr(), d_d.data_ptr(), len(src), self.N, self.N,
                                           tl.stream_ptr(self.torch)))
        self.torch.cuda.synchronize()

    def fork(self, parent, ntokens):
        c = self.pkv.pkv_pool_fork(self.pool, parent, ntokens)
        assert c >= 0 and self.pkv.pkv_pool_assign_slot(self.pool, c) >= 0
        self.content[c] = [a[:ntokens].copy() for a in self.content[parent]]
        self.length[c] = ntokens
        return c

    def check_pools(self):
        for l in range(self.L):
            assert np.array_equal(tl.host(self.d_rows[l], np.uint16, self.h_rows[l].shape), self.h_rows[l]), f"rows {l}"
            assert np.array_equal(tl.host(self.d_fp4[l], np.uint8), self.h_fp4[l]), f"fp4 {l}"
        assert tl.device_status(self.pkv) == 0

    def check_readback(self, handles):
        """Every row of every live sequence, gathered through its block-table row on the device, equals what was
        appended to it (or inherited at the fork)."""
        pkv, torch = self.pkv, self.torch
        tables = self.tables()
        d_tables = tl.dev(torch, tables)
        for h in handles:
            n = self.length[h]
            slot = pkv.pkv_pool_seq_slot(self.pool, h)
            idx = np.arange(n, dtype=np.int32).reshape(1, n)
            vis = np.array([n], np.int32)
            d_idx, d_vis = tl.dev(torch, idx), tl.dev(torch, vis)
            for l in range(self.L):
                d_out = torch.empty(n * tl.ROW_BYTES, dtype=torch.uint8, device="cuda")
                capi.check(pkv.pkv_gather_rows(self.d_rows[l].data_ptr(), d_tables.data_ptr() + slot * self.pps * 4,
                                               tl.RPP, tl.W, tl.W, d_idx.data_ptr(), d_vis.data_ptr(), 1, n,
                                               d_out.data_ptr(), tl.stream_ptr(torch)))
                torch.cuda.synchronize()
                assert np.array_equal(tl.host(d_out, np.uint16, (n, tl.W)), self.content[h][l]), (h, l)


def test_fork_cow_evict_compact_on_device(pkv, cuda):
    g = tl.rng(404)
    N = 640
    st = Store(pkv, cuda, num_pages=N, slots=32, pps=48)
    try:
        # 12 "snapshots": sequences with unaligned lengths that stay alive and own their (partly filled) last page
        snaps = []
        for _ in range(12):
            h = pkv.pkv_pool_seq_open(st.pool)
            assert pkv.pkv_pool_assign_slot(st.pool, h) >= 0
            n = int(g.integers(70, 1500))
            st.append([(h, n)])
            toks = g.integers(2, 500, size=n).astype(np.int32)
            capi.check(pkv.pkv_pool_register(st.pool, h, ptr(toks), n, n))
            snaps.append(h)
        st.check_pools()
        # 6 live requests fork distinct snapshots at an unaligned point and append 150 rows each, in shared launches
        picks = g.choice(len(snaps), size=6, replace=False)
        live = [st.fork(snaps[j], int(g.integers(st.length[snaps[j]] // 2, st.length[snaps[j]]))) for j in picks]
        for rounds in (1, 64, 85):   # decode row, then chunks crossing pages
            st.append([(h, rounds) for h in live])
        st.check_pools()
        st.check_readback(live + snaps)   # parents are untouched by their children's writes
        # snapshots that were not forked finish: their named pages become evictable; free a quarter of the pool LRU-first
        for j, h in enumerate(snaps):
            if j not in picks:
                capi.check(pkv.pkv_pool_seq_close(st.pool, h))
        alive = live + [snaps[j] for j in picks]
        freed = np.zeros(N, np.int32)
        want = min(N // 4, pkv.pkv_pool_evictable_count(st.pool))
        assert pkv.pkv_pool_free_lru(st.pool, N // 4, ptr(freed), N) == want and want > 0
        # compact: the moves run on every layer's pools in one launch, then the tables name the new ids
        ms, md = np.zeros(N, np.int32), np.zeros(N, np.int32)
        m = pkv.pkv_pool_compact(st.pool, ptr(ms), ptr(md), N)
        assert m > 0
        st.copy_pages(ms[:m].copy(), md[:m].copy())
        st.check_pools()
        st.check_readback(alive)
        live_pages = N - pkv.pkv_pool_free_count(st.pool)
        tab = st.tables()
        for h in alive:
            n = pkv.pkv_pool_seq_pages(st.pool, h, None, 0)
            assert (tab[pkv.pkv_pool_seq_slot(st.pool, h), :n] < live_pages).all()
        # the compacted pool keeps working: more appends, read back again
        st.append([(h, 70) for h in live])
        st.check_pools()
        st.check_readback(alive)
    finally:
        st.close()


def test_migration_between_two_pools_on_one_device(pkv, cuda):
    """Migration between shards, with both shards on ONE device: two page pools with their own layer pools (different
    sizes, different base addresses), pkv_pool_migrate for the bookkeeping and pkv_copy_pages with src_base != dst_base
    for the payload — the call a destination GPU makes on a peer's mapped pool. The destination's pools must equal the
    oracle's orc_move_pages byte for byte, the migrated request read back through its NEW block table must equal what
    was written to it on the source, and the source keeps working. Migration has no reference counterpart (parity
    unpinned): this pins the stated rule."""
    g = tl.rng(511)
    a = Store(pkv, cuda, num_pages=96, slots=8, pps=40, layers=3, seed=5)
    b = Store(pkv, cuda, num_pages=160, slots=8, pps=40, layers=3, seed=6)
    try:
        # the destination is already in use (its free list is not 0, 1, 2, ...), one of its sequences was released again
        keepers = []
        for n in (300, 77, 450):
            h = pkv.pkv_pool_seq_open(b.pool)
            assert pkv.pkv_pool_assign_slot(b.pool, h) >= 0
            b.append([(h, n)])
            keepers.append(h)
        capi.check(pkv.pkv_pool_seq_close(b.pool, keepers.pop(1)))
        movers, stay = [], []
        for i, n in enumerate((1000, 64, 333, 129, 700)):
            h = pkv.pkv_pool_seq_open(a.pool)
            assert pkv.pkv_pool_assign_slot(a.pool, h) >= 0
            a.append([(h, n)])
            (movers if i % 2 == 0 else stay).append(h)
        a.check_pools()
        b.check_pools()
        arrived = []
        for h in movers:
            npages = pkv.pkv_pool_seq_pages(a.pool, h, None, 0)
            src, dst, out = np.zeros(npages, np.int32), np.zeros(npages, np.int32), C.c_int(-1)
            free_before = pkv.pkv_pool_free_count(a.pool)
            m = pkv.pkv_pool_migrate(a.pool, h, b.pool, C.byref(out), ptr(src), ptr(dst), npages)
            assert m == npages and pkv.pkv_pool_free_count(a.pool) == free_before + npages
            nh = out.value
            assert pkv.pkv_pool_assign_slot(b.pool, nh) >= 0
            descs = (capi.PkvPoolDesc * (2 * a.L))()
            for l in range(a.L):
                descs[2 * l].src_base, descs[2 * l].dst_base = a.d_rows[l].data_ptr(), b.d_rows[l].data_ptr()
                descs[2 * l].page_bytes = tl.PAGE_BYTES
                descs[2 * l + 1].src_base, descs[2 * l + 1].dst_base = a.d_fp4[l].data_ptr(), b.d_fp4[l].data_ptr()
                descs[2 * l + 1].page_bytes = tl.FP4_PAGE_BYTES
                orc.move_pages(a.h_rows[l], b.h_rows[l], tl.PAGE_BYTES, src, dst)
                orc.move_pages(a.h_fp4[l], b.h_fp4[l], tl.FP4_PAGE_BYTES, src, dst)
            d_s, d_d = tl.dev(cuda, src), tl.dev(cuda, dst)
            capi.check(pkv.pkv_copy_pages(descs, 2 * a.L, d_s.data_ptr(), d_d.data_ptr(), npages, a.N, b.N, tl.stream_ptr(cuda)))
            cuda.cuda.synchronize()
            b.content[nh], b.length[nh] = a.content.pop(h), a.length.pop(h)
            arrived.append(nh)
        a.check_pools()                       # the source pools are only read
        b.check_pools()                       # destination == oracle mirror, every byte of every layer
        b.check_readback(arrived + keepers)   # through the new owner's block table
        a.check_readback(stay)
        # both shards keep working: the migrated requests decode on, the source reuses the pages that left
        b.append([(h, 70) for h in arrived])
        h = pkv.pkv_pool_seq_open(a.pool)
        assert pkv.pkv_pool_assign_slot(a.pool, h) >= 0
        a.append([(h, 900)])
        b.check_pools()
        a.check_pools()
        b.check_readback(arrived)
        a.check_readback(stay + [h])
        # ids beyond either pool are reported by the kernel, not dereferenced
        bad_s, bad_d = tl.dev(cuda, np.array([a.N + 3], np.int32)), tl.dev(cuda, np.array([2], np.int32))
        capi.check(pkv.pkv_copy_pages(descs, 2 * a.L, bad_s.data_ptr(), bad_d.data_ptr(), 1, a.N, b.N, tl.stream_ptr(cuda)))
        assert pkv.pkv_stream_check(tl.stream_ptr(cuda)) == capi.PKV_ERR_DEVICE and b"page id out of range" in pkv.pkv_last_error()
        assert pkv.pkv_stream_check(tl.stream_ptr(cuda)) == capi.PKV_OK      # the record was cleared
        b.check_pools()
    finally:
        a.close()
        b.close()
