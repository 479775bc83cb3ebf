"""The from-scratch page pool against the reference's own engine, on the CPU.

oracle/_ref/libref_engine.so is the reference's unmodified src/engine/engine.cpp + sampler.cpp driven through a
recording StepModel (oracle/ref_engine_driver.cpp). Its trace — every set_block_tables() table, every chunk, state
save and finished request, and the allocator counters after each iterate() — is replayed into pkv_pool_* and the block
tables must match entry for entry (stale tails included), as must the free / cached page counts. This is the
reference's own test method (tools/sched_test/main.cpp drives iterate() on a fake model) turned into a differential.

Copy-on-write, LRU freeing and compaction have no reference counterpart (parity unpinned): their tests check the
stated rules and invariants.
"""
import ctypes as C
from collections import deque
from pathlib import Path

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import build_oracle
from unholy_b200 import capi

i32p = C.POINTER(C.c_int32)
u64p = C.POINTER(C.c_uint64)
u8p = C.POINTER(C.c_uint8)


def ptr(a):
    return a.ctypes.data_as(i32p)


@pytest.fixture(scope="module")
def refeng():
    libs = build_oracle.build_reference()
    if not libs["engine"]:
        pytest.skip("oracle/_ref/libref_engine.so not built (no reference checkout here)")
    h = C.CDLL(str(libs["engine"]))
    h.refeng_create.restype, h.refeng_create.argtypes = C.c_void_p, [C.c_int] * 6
    h.refeng_create_disk.restype, h.refeng_create_disk.argtypes = C.c_void_p, [C.c_int] * 6 + [C.c_char_p, C.c_int]
    h.refeng_io_release.argtypes = [C.c_void_p, C.c_int, C.c_int]
    h.refeng_abort.argtypes = [C.c_void_p, C.c_uint64]
    h.refeng_destroy.argtypes = [C.c_void_p]
    h.refeng_submit.restype, h.refeng_submit.argtypes = C.c_uint64, [C.c_void_p, i32p, C.c_int, C.c_int]
    h.refeng_submit_images.restype = C.c_uint64
    h.refeng_submit_images.argtypes = [C.c_void_p, i32p, C.c_int, C.c_int, i32p, i32p, u64p, C.c_int]
    h.refeng_iterate.restype, h.refeng_iterate.argtypes = C.c_int, [C.c_void_p]
    h.refeng_trace_len.restype, h.refeng_trace_len.argtypes = C.c_long, [C.c_void_p]
    h.refeng_trace_copy.argtypes = [C.c_void_p, C.c_void_p]
    h.refeng_num_tables.restype, h.refeng_num_tables.argtypes = C.c_int, [C.c_void_p]
    h.refeng_table_copy.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    h.refeng_token.restype, h.refeng_token.argtypes = C.c_int, [C.c_uint64, C.c_int]
    return h


class Replay:
    """Feeds the reference engine and the page pool the same requests; after every iterate() of the engine replays
    the new trace records into the pool and compares."""

    def __init__(self, pkv, refeng, num_pages, page_tokens, slots, pps, budget, snapshots=8192, disk=None):
        """disk: (directory, slots) turns the reference engine's snapshot disk tier on (gated I/O, see the driver)."""
        self.pkv, self.ref = pkv, refeng
        self.pt, self.slots, self.pps, self.budget, self.num_pages = page_tokens, slots, pps, budget, num_pages
        if disk:
            self.eng = refeng.refeng_create_disk(num_pages, page_tokens, slots, pps, budget, snapshots, str(disk[0]).encode(), disk[1])
        else:
            self.eng = refeng.refeng_create(num_pages, page_tokens, slots, pps, budget, snapshots)
        self.pool = pkv.pkv_pool_create(num_pages, page_tokens, slots, pps, 1)
        self.tokens, self.handle, self.computed = {}, {}, {}
        self.waiting, self.running = deque(), []
        self.saved = set()
        self.images = {}
        self.first_hit = {}
        self.aborts, self.aborted = [], set()
        self.cursor = 0
        self.tables_checked = 0
        self.max_cached = 0
        self.evicted_for_one_request = 0

    def close(self):
        self.ref.refeng_destroy(self.eng)
        self.pkv.pkv_pool_destroy(self.pool)

    def submit(self, prompt, max_tokens, images=None):
        """images: [(start, len, hash)] in position order, or None for a text prompt."""
        a = np.ascontiguousarray(prompt, np.int32)
        if images:
            st, ln = (np.array([im[j] for im in images], np.int32) for j in (0, 1))
            hs = np.array([im[2] for im in images], np.uint64)
            rid = int(self.ref.refeng_submit_images(self.eng, ptr(a), len(a), max_tokens, ptr(st), ptr(ln),
                                                    hs.ctypes.data_as(u64p), len(images)))
            self.images[rid] = (st, ln, hs)
        else:
            rid = int(self.ref.refeng_submit(self.eng, ptr(a), len(a), max_tokens))
        self.tokens[rid] = list(map(int, a))
        self.waiting.append(rid)
        return rid

    def abort(self, rid):
        """Engine::abort: the request ends at the start of the next iterate() (no step is ever in flight between two
        iterate() calls of this driver), before that call's disk completions and admissions."""
        self.ref.refeng_abort(self.eng, rid)
        self.aborts.append(rid)

    def keys(self, rid):
        """The sequence's positions as 64-bit page-name keys (text: the token id; image positions: hash and offset)."""
        t = np.asarray(self.tokens[rid], np.int32)
        k = np.zeros(len(t), np.uint64)
        st, ln, hs = self.images.get(rid, (None, None, None))
        capi.check(self.pkv.pkv_token_keys(ptr(t), len(t), ptr(st) if st is not None else None,
                                           ptr(ln) if st is not None else None,
                                           hs.ctypes.data_as(u64p) if st is not None else None,
                                           0 if st is None else len(st), k.ctypes.data_as(u64p)))
        return k

    def page_hash(self, rid, page_index):
        k = self.keys(rid)
        return int(self.pkv.pkv_page_hash_keys(k.ctypes.data_as(u64p), self.pt, page_index))

    def admit(self):
        pkv, pool = self.pkv, self.pool
        while self.waiting and len(self.running) < self.slots:
            rid = self.waiting[0]
            if rid not in self.handle:
                self.handle[rid] = pkv.pkv_pool_seq_open(pool)
            h = self.handle[rid]
            toks = self.keys(rid)
            limit = (len(toks) - 1) // self.pt
            ok = self.boundaries(rid, toks, limit)
            computed = pkv.pkv_pool_match_prefix_keys(pool, h, toks.ctypes.data_as(u64p), len(toks), ok.ctypes.data_as(u8p))
            first = min(len(toks) - computed, self.budget)
            npages = pkv.pkv_pool_seq_pages(pool, h, None, 0)
            need = -(-(computed + first) // self.pt) - npages + len(self.running)
            if need > pkv.pkv_pool_available(pool):
                pkv.pkv_pool_release(pool, h)
                self.on_admit_failed(rid)
                break
            assert pkv.pkv_pool_assign_slot(pool, h) >= 0
            self.computed[rid] = computed
            self.on_admitted(rid)
            self.first_hit.setdefault(rid, computed)
            self.running.append(rid)
            self.waiting.popleft()

    def iterate(self):
        did = self.ref.refeng_iterate(self.eng)
        n = self.ref.refeng_trace_len(self.eng)
        ev = np.empty(n, np.int64)
        self.ref.refeng_trace_copy(self.eng, ev.ctypes.data)
        for rid in self.aborts:                           # the engine's intake(): aborts come first
            if rid in self.waiting or rid in self.running:
                (self.waiting if rid in self.waiting else self.running).remove(rid)
                if rid in self.handle:
                    capi.check(self.pkv.pkv_pool_seq_close(self.pool, self.handle.pop(rid)))
                self.on_finished(rid)
                self.aborted.add(rid)
        self.aborts = []
        self.on_iterate_begin()
        self.admit()
        pkv, pool = self.pkv, self.pool
        i, pending_table = self.cursor, None
        while i < n:
            kind = int(ev[i])
            if kind == 2:
                pending_table = int(ev[i + 1])
                i += 2
            elif kind == 1:
                nch = int(ev[i + 1])
                chunks = ev[i + 2:i + 2 + 4 * nch].reshape(nch, 4)
                i += 2 + 4 * nch
                nsave = int(ev[i])
                save_ops = [(int(a), int(b)) for a, b in ev[i + 1:i + 1 + 2 * nsave].reshape(nsave, 2)]
                saves = [a for a, _ in save_ops]
                i += 1 + 2 * nsave
                nrest = int(ev[i])
                restore_ops = [(int(a), int(b)) for a, b in ev[i + 1:i + 1 + 2 * nrest].reshape(nrest, 2)]
                i += 1 + 2 * nrest
                self.on_step(chunks, save_ops, restore_ops)
                for seq, slot, s0, cn in chunks:
                    h = self.handle[int(seq)]
                    assert pkv.pkv_pool_seq_slot(pool, h) == slot, "slot assignment differs"
                    assert self.computed[int(seq)] == s0, "prefix-hit length differs"
                    assert pkv.pkv_pool_alloc(pool, h, int(s0 + cn)) == 1
                if pending_table is not None:
                    want = np.empty(self.slots * self.pps, np.int32)
                    self.ref.refeng_table_copy(self.eng, pending_table, want.ctypes.data)
                    got = np.ctypeslib.as_array(pkv.pkv_pool_tables(pool), shape=(self.slots * self.pps,))
                    assert np.array_equal(got, want), f"block tables differ at set_block_tables #{pending_table}"
                    self.tables_checked += 1
                    pending_table = None
                else:
                    assert not pkv.pkv_pool_dirty(pool), "the pool changed a table the engine did not upload"
                # completion, in plan order: register full pages, commit saves, sample
                for seq, slot, s0, cn in chunks:
                    rid, end = int(seq), int(s0 + cn)
                    self.computed[rid] = end
                    toks = self.keys(rid)
                    capi.check(pkv.pkv_pool_register_keys(pool, self.handle[rid], toks.ctypes.data_as(u64p), len(toks), end))
                    if slot in saves:
                        assert end % self.pt == 0
                        self.saved.add(self.page_hash(rid, end // self.pt - 1))
                    if end == len(self.tokens[rid]):
                        self.tokens[rid].append(int(self.ref.refeng_token(rid, end - 1)))
            elif kind == 3:
                rid = int(ev[i + 1])
                i += 2
                if rid in self.aborted:                   # (already taken out, where the engine does it)
                    continue
                capi.check(pkv.pkv_pool_seq_close(pool, self.handle.pop(rid)))
                self.running.remove(rid)
                self.on_finished(rid)
            elif kind == 4:
                running, waiting, free_pages, cached, preempt, snaps, free_snaps = (int(x) for x in ev[i + 1:i + 8])
                i += 8
                self.on_iterate_end()
                self.on_counters(snaps, free_snaps)
                assert preempt == 0, "scenario sized to avoid preemption"
                assert (running, waiting) == (len(self.running), len(self.waiting))
                assert free_pages == pkv.pkv_pool_available(pool)
                assert cached == pkv.pkv_pool_cached_count(pool)
                self.max_cached = max(self.max_cached, cached)
                if running == 1:
                    self.evicted_for_one_request = max(self.evicted_for_one_request, self.num_pages - free_pages)
            elif kind == 5:
                self.on_disk_counters(*(int(x) for x in ev[i + 1:i + 5]))
                i += 5
            else:
                raise AssertionError(f"unknown trace record {kind}")
        self.cursor = n
        return did

    def boundaries(self, rid, toks, limit):
        """Which page boundaries of the prompt can be resumed at: where some sequence saved its state ..."""
        ok = np.zeros(max(limit, 1), np.uint8)
        blocks = list(zip(*self.images[rid][:2])) if rid in self.images else []
        for i in range(limit):
            hh = int(self.pkv.pkv_page_hash_keys(toks.ctypes.data_as(u64p), self.pt, i))
            b = (i + 1) * self.pt   # ... and never inside a whole image block (engine.cpp:292-296)
            ok[i] = hh in self.saved and not any(st < b < st + ln for st, ln in blocks)
        return ok

    def on_admit_failed(self, rid):
        pass

    # Hooks for the snapshot-store differential (tests/test_snapshot_store.py); the page tests do not use them.
    def on_step(self, chunks, save_ops, restore_ops):
        pass

    def on_counters(self, snapshots, free_snapshots):
        pass

    def on_iterate_begin(self):     # the engine's poll_io, first thing in iterate()
        pass

    def on_finished(self, rid):     # the engine's release() of a request that ends
        pass

    def on_admitted(self, rid):     # the engine's start_load for a prefix that only the disk has
        pass

    def on_iterate_end(self):       # the engine's spill(), last thing in iterate()
        pass

    def on_disk_counters(self, disk_snapshots, snapshot_io, spills, disk_hits):
        pass

    def drain(self, limit=200000):
        for _ in range(limit):
            if not self.iterate() and not self.running and not self.waiting:
                return
        raise AssertionError("engine did not go idle")


def test_prefix_churn_matches_reference_engine(pkv, refeng):
    """Benchmark configuration 4, mode A (reference semantics), at 1/12 scale: prefixes written and released (cached),
    requests that extend a prefix (fork = match_prefix on shared full pages, no payload copy) and decode 512 tokens,
    then a filler request that forces LRU evictions of a quarter of the pool."""
    g = tl.rng(4)
    num_pages, pt = 2048, 64
    r = Replay(pkv, refeng, num_pages, pt, slots=8, pps=num_pages // 4 + 8, budget=2048)
    try:
        prefixes = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in g.integers(170, 5462, size=24)]
        for p in prefixes:  # one at a time: each finishes, its full pages stay cached and evictable tail-first
            r.submit(p, 1)
            r.drain()
        assert r.max_cached > 0
        picks = g.choice(len(prefixes), size=8, replace=False)
        for j in picks:  # eight live requests fork distinct prefixes and append 512 tokens each
            ext = g.integers(2, 500, size=100).astype(np.int32)
            r.submit(np.concatenate([prefixes[j], ext]), 512)
        r.drain()
        r.submit(g.integers(2, 500, size=num_pages // 4 * pt).astype(np.int32), 1)  # evicts >= 25 % from the LRU front
        r.drain()
        assert r.evicted_for_one_request >= num_pages // 4 - 2  # the filler really ran and held a quarter of the pool
        assert r.tables_checked > 100
        assert pkv.pkv_pool_available(r.pool) == num_pages  # no leak (tools/sched_test/main.cpp:1113-1116)
    finally:
        r.close()


def test_concurrent_admission_matches_reference_engine(pkv, refeng):
    """More requests than slots, shared and repeated prompts, small pages: admission order, headroom rule and
    duplicate-hash pages (a page whose name is already cached stays private)."""
    g = tl.rng(41)
    r = Replay(pkv, refeng, num_pages=192, page_tokens=16, slots=4, pps=64, budget=256)
    try:
        base = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in g.integers(40, 400, size=6)]
        for rounds in range(3):
            for j in g.permutation(len(base)):
                tail = g.integers(2, 500, size=int(g.integers(1, 40))).astype(np.int32)
                r.submit(np.concatenate([base[j], tail]) if rounds else base[j], int(g.integers(1, 48)))
            for _ in range(int(g.integers(1, 6))):
                r.iterate()
        r.drain()
        assert r.tables_checked > 20
        assert pkv.pkv_pool_available(r.pool) == 192
    finally:
        r.close()


def test_prefix_churn_full_size_matches_reference_engine(pkv, refeng):
    """Benchmark configuration 4, mode A, at its full size: a 24,576-page pool (1,572,864 tokens, page 64), 64 prefixes
    of 2k..64k tokens written one after the other (their sum exceeds the pool, so later ones evict earlier ones
    LRU-first), 8 requests that extend the 8 newest prefixes and decode 512 tokens, then a filler request of a quarter
    of the pool. Every uploaded block table, slot, prefix-hit length and page count must equal the reference engine's."""
    g = tl.rng(4)
    num_pages, pt = 24576, 64
    r = Replay(pkv, refeng, num_pages, pt, slots=16, pps=num_pages // 4 + 8, budget=2048)
    try:
        prefixes = [g.integers(2, 50000, size=int(n)).astype(np.int32) for n in g.integers(2048, 65537, size=64)]
        for p in prefixes:
            r.submit(p, 1)
            r.drain()
        for j in range(56, 64):
            r.submit(np.concatenate([prefixes[j], g.integers(2, 50000, size=100).astype(np.int32)]), 512)
        r.drain()
        r.submit(g.integers(2, 50000, size=num_pages // 4 * pt).astype(np.int32), 1)
        r.drain()
        assert r.evicted_for_one_request >= num_pages // 4 - 2
        assert r.tables_checked > 1000
        assert pkv.pkv_pool_available(r.pool) == num_pages
    finally:
        r.close()


def test_image_prompts_match_reference_engine(pkv, refeng):
    """Prompts that hold image blocks: every image's placeholder tokens are the same ids, so page names come from the
    image's hash and the offset in the block (engine.cpp:264-270) and a prefix is never resumed inside a block
    (:292-296). Same placeholder layout with the same image shares pages, with another image it does not; the block
    tables, prefix-hit lengths and cached-page counts must equal the reference engine's."""
    g = tl.rng(45)
    pt = 16
    r = Replay(pkv, refeng, num_pages=256, page_tokens=pt, slots=4, pps=64, budget=512)
    try:
        def prompt(img_hashes, tail):
            """text, then per image: 40 placeholder tokens (ids 7 7 ... 7) framed by ids 5 and 6, then text."""
            toks, images = list(range(100, 121)), []
            for hsh in img_hashes:
                toks.append(5)
                images.append((len(toks), 40, hsh))
                toks += [7] * 40 + [6] + list(range(200, 210))
            return np.array(toks + list(tail), np.int32), images

        tails = [g.integers(2, 500, size=int(n)).astype(np.int32) for n in (30, 75, 9, 120)]
        base, base_images = prompt((0xA1, 0xB2), tails[0])
        ends_in_block, eib_images = prompt((0xE5,), [])
        ends_in_block = ends_in_block[:64]     # the block covers 22..61: the prompt's last page boundary (48) lies inside it
        runs = [
            (base, base_images),                                                  # 0: cold
            (np.concatenate([base, tails[1]]), base_images),                      # 1: extends 0 with the same images
            (np.concatenate([base, tails[1]]), [(s_, n_, h_ ^ 0xFF) for s_, n_, h_ in base_images]),   # 2: other images
            (np.concatenate([base, tails[2]]), [base_images[0], (base_images[1][0], 40, 0xC3)]),       # 3: second differs
            (ends_in_block, eib_images),                                          # 4: cold; its state is saved before the block
            (np.concatenate([ends_in_block, tails[3]]), eib_images),              # 5: extends 4
        ]
        hits = []
        for p, images in runs:
            rid = r.submit(p, 20, images)
            r.drain()
            hits.append(r.first_hit[rid])
        last_boundary = (len(base) - 1) // pt * pt
        assert hits[0] == 0 and hits[1] == last_boundary        # resumes past both blocks, at the prompt's last boundary
        assert hits[2] == 0 and hits[3] == 0                    # same token ids, other images: other page names
        assert hits[4] == 0 and 0 < hits[5] <= eib_images[0][0]  # never resumed inside the block: at or before its start
        assert r.tables_checked > 10
        assert pkv.pkv_pool_available(r.pool) == 256
    finally:
        r.close()
