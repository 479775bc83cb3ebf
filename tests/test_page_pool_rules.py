"""Rules of the three page-pool operations the reference does not have (parity unpinned): copy-on-write, freeing
from the LRU front, hole-filling compaction — plus migration between two pools. CPU only; the rules are stated in
unholy_b200/csrc/page_pool.hpp and checked here as invariants."""
import ctypes as C

import numpy as np

import pkv_testlib as tl
from unholy_b200 import capi

i32p = C.POINTER(C.c_int32)


def ptr(a):
    return a.ctypes.data_as(i32p)


def pages_of(pkv, pool, h):
    n = pkv.pkv_pool_seq_pages(pool, h, None, 0)
    out = np.zeros(max(n, 1), np.int32)
    pkv.pkv_pool_seq_pages(pool, h, ptr(out), n)
    return out[:n].copy()


def lists(pkv, pool, num_pages):
    f = np.zeros(num_pages, np.int32)
    nf = pkv.pkv_pool_free_list(pool, ptr(f), num_pages)
    e = np.zeros(num_pages, np.int32)
    ne = pkv.pkv_pool_evictable_list(pool, ptr(e), num_pages)
    return f[:nf].copy(), e[:ne].copy()


def check_accounting(pkv, pool, num_pages, handles):
    """Every page is exactly one of: free, evictable (cached, refs 0), or referenced; refs equal the number of open
    sequences that hold the page."""
    free, evict = lists(pkv, pool, num_pages)
    refs = np.zeros(num_pages, int)
    for h in handles:
        for p in pages_of(pkv, pool, h):
            refs[p] += 1
    for p in range(num_pages):
        assert pkv.pkv_pool_page_refs(pool, p) == refs[p], p
    held = set(np.flatnonzero(refs))
    assert len(set(free)) == len(free) and len(set(evict)) == len(evict)
    assert not (set(free) & set(evict)) and not (set(free) & held) and not (set(evict) & held)
    assert len(free) + len(evict) + len(held) == num_pages
    assert pkv.pkv_pool_available(pool) == len(free) + len(evict)
    for p in evict:
        assert pkv.pkv_pool_page_hash(pool, int(p)) != 0


def test_initial_order_and_tail_first_release(pkv):
    pool = pkv.pkv_pool_create(16, 4, 4, 8, 1)
    h = pkv.pkv_pool_seq_open(pool)
    assert pkv.pkv_pool_assign_slot(pool, h) == 0          # slot 0 first (engine.cpp:95)
    assert pkv.pkv_pool_alloc(pool, h, 10) == 1            # 3 pages: 0, 1, 2 (engine.cpp:96)
    assert list(pages_of(pkv, pool, h)) == [0, 1, 2]
    assert pkv.pkv_pool_alloc(pool, h, 9) == 1 and len(pages_of(pkv, pool, h)) == 3
    assert pkv.pkv_pool_alloc(pool, h, 4 * 9) == 0         # wider than the block table: refused, nothing changes
    toks = np.arange(100, 110, dtype=np.int32)
    capi.check(pkv.pkv_pool_register(pool, h, ptr(toks), 10, 10))
    assert pkv.pkv_pool_cached_count(pool) == 2            # two full pages named, the partial third is not
    capi.check(pkv.pkv_pool_release(pool, h))
    free, evict = lists(pkv, pool, 16)
    assert list(evict) == [1, 0]                           # tail first (engine.cpp:208-217)
    assert free[-1] == 2                                   # the uncached page is reused first
    h2 = pkv.pkv_pool_seq_open(pool)
    assert pkv.pkv_pool_match_prefix(pool, h2, ptr(toks), 10, None) == 8
    assert list(pages_of(pkv, pool, h2)) == [0, 1]
    assert pkv.pkv_pool_evictable_count(pool) == 0
    assert pkv.pkv_page_hash(ptr(toks), 4, 1) == pkv.pkv_pool_page_hash(pool, 1)
    pkv.pkv_pool_destroy(pool)


def test_fork_cow_free_lru_compact(pkv):
    g = tl.rng(44)
    N, pt = 96, 8
    pool = pkv.pkv_pool_create(N, pt, 16, 24, 1)
    handles, toks = [], {}
    for _ in range(5):  # parents with unaligned lengths stay alive
        h = pkv.pkv_pool_seq_open(pool)
        n = int(g.integers(9, 90))
        t = g.integers(2, 500, size=n).astype(np.int32)
        assert pkv.pkv_pool_assign_slot(pool, h) >= 0 and pkv.pkv_pool_alloc(pool, h, n) == 1
        capi.check(pkv.pkv_pool_register(pool, h, ptr(t), n, n))
        handles.append(h)
        toks[h] = t
    parents = list(handles)
    src, dst = np.zeros(8, np.int32), np.zeros(8, np.int32)
    for p in parents[:3]:
        n = len(toks[p])
        c = pkv.pkv_pool_fork(pool, p, n)
        handles.append(c)
        assert list(pages_of(pkv, pool, c)) == list(pages_of(pkv, pool, p))
        for q in pages_of(pkv, pool, c):
            assert pkv.pkv_pool_page_refs(pool, int(q)) == 2
        assert pkv.pkv_pool_assign_slot(pool, c) >= 0
        before = pages_of(pkv, pool, c)
        # the child appends 10 rows at n: only a partial last page is shared-and-written -> at most one copy
        assert pkv.pkv_pool_alloc(pool, c, n + 10) == 1
        m = pkv.pkv_pool_cow(pool, c, n, 10, ptr(src), ptr(dst), 8)
        after = pages_of(pkv, pool, c)
        if n % pt == 0:
            assert m == 0
        else:
            assert m == 1 and src[0] == before[-1] and after[len(before) - 1] == dst[0] != src[0]
            assert pkv.pkv_pool_page_refs(pool, int(src[0])) == 1 and pkv.pkv_pool_page_refs(pool, int(dst[0])) == 1
        assert list(after[:len(before) - 1]) == list(before[:-1])           # untouched pages stay shared
        assert pkv.pkv_pool_cow(pool, c, n, 10, ptr(src), ptr(dst), 8) == 0  # idempotent
        tab = np.ctypeslib.as_array(pkv.pkv_pool_tables(pool), shape=(16, 24))
        assert list(tab[pkv.pkv_pool_seq_slot(pool, c), :len(after)]) == list(after)
    check_accounting(pkv, pool, N, handles)
    # parents 3, 4 finish: their named pages become evictable tail first; free the LRU front
    for p in parents[3:]:
        capi.check(pkv.pkv_pool_seq_close(pool, p))
        handles.remove(p)
    _, evict = lists(pkv, pool, N)
    want = list(evict[:3])
    freed = np.zeros(8, np.int32)
    assert pkv.pkv_pool_free_lru(pool, 3, ptr(freed), 8) == min(3, len(evict))
    assert list(freed[:len(want)]) == want                                  # oldest first, as take_page evicts
    for p in want:
        assert pkv.pkv_pool_page_hash(pool, int(p)) == 0
    check_accounting(pkv, pool, N, handles)
    # compaction
    free, evict = lists(pkv, pool, N)
    live = sorted(set(range(N)) - set(free))
    Wn = len(live)
    before = {h: pages_of(pkv, pool, h) for h in handles}
    hashes = {p: pkv.pkv_pool_page_hash(pool, p) for p in live}
    ms, md = np.zeros(N, np.int32), np.zeros(N, np.int32)
    m = pkv.pkv_pool_compact(pool, ptr(ms), ptr(md), N)
    moves = dict(zip(ms[:m].tolist(), md[:m].tolist()))
    assert sorted(moves) == [p for p in live if p >= Wn]                    # sources: live ids >= W, ascending
    assert sorted(moves.values()) == sorted(set(range(Wn)) - set(live))     # holes: free ids < W, ascending
    assert list(ms[:m]) == sorted(ms[:m]) and list(md[:m]) == sorted(md[:m])
    for h in handles:
        assert list(pages_of(pkv, pool, h)) == [moves.get(int(p), int(p)) for p in before[h]]
    for p in live:
        assert pkv.pkv_pool_page_hash(pool, moves.get(p, p)) == hashes[p]
    free2, evict2 = lists(pkv, pool, N)
    assert list(free2) == list(range(N - 1, Wn - 1, -1))                    # descending: page W is taken next
    assert list(evict2) == [moves.get(int(p), int(p)) for p in evict]       # LRU order kept
    assert pkv.pkv_pool_compact(pool, ptr(ms), ptr(md), N) == 0
    check_accounting(pkv, pool, N, handles)
    # a cached page still matches after it moved
    h = pkv.pkv_pool_seq_open(pool)
    t = toks[parents[0]]
    got = pkv.pkv_pool_match_prefix(pool, h, ptr(t), len(t), None)
    assert got == (len(t) - 1) // pt * pt
    pkv.pkv_pool_destroy(pool)


def test_cow_never_writes_a_page_the_prefix_cache_names(pkv):
    """A child forked in the middle of a page whose parent then finishes holds the only reference to a NAMED page.
    Writing it in place would leave modified rows under the old name; copy-on-write must move the child off it."""
    pt = 4
    pool = pkv.pkv_pool_create(8, pt, 4, 8, 1)
    parent = pkv.pkv_pool_seq_open(pool)
    toks = np.arange(100, 109, dtype=np.int32)                          # 9 tokens: pages 0, 1 full, page 2 partial
    assert pkv.pkv_pool_assign_slot(pool, parent) >= 0 and pkv.pkv_pool_alloc(pool, parent, 9) == 1
    capi.check(pkv.pkv_pool_register(pool, parent, ptr(toks), 9, 9))
    child = pkv.pkv_pool_fork(pool, parent, 6)                          # shares pages 0 and 1, page 1 only half used
    assert pkv.pkv_pool_assign_slot(pool, child) >= 0
    capi.check(pkv.pkv_pool_release(pool, parent))
    assert list(pages_of(pkv, pool, child)) == [0, 1] and pkv.pkv_pool_page_refs(pool, 1) == 1
    src, dst = np.zeros(4, np.int32), np.zeros(4, np.int32)
    assert pkv.pkv_pool_cow_pairs(pool, child, 6, 1) == 1
    assert pkv.pkv_pool_cow(pool, child, 6, 1, ptr(src), ptr(dst), 4) == 1
    fresh = int(dst[0])
    assert int(src[0]) == 1 and fresh not in (0, 1)
    assert list(pages_of(pkv, pool, child)) == [0, fresh]
    assert pkv.pkv_pool_page_refs(pool, 1) == 0 and pkv.pkv_pool_page_hash(pool, 1) != 0   # still named, now evictable
    _, evict = lists(pkv, pool, 8)
    assert 1 in evict
    other = pkv.pkv_pool_seq_open(pool)                                 # the parent's prompt again: hits both pages
    assert pkv.pkv_pool_match_prefix(pool, other, ptr(toks), 9, None) == 8
    assert list(pages_of(pkv, pool, other)) == [0, 1]                   # ... and page 1 is not the page the child writes
    assert fresh not in pages_of(pkv, pool, other)
    check_accounting(pkv, pool, 8, [parent, child, other])
    assert pkv.pkv_pool_cow(pool, child, 6, 1, ptr(src), ptr(dst), 4) == 0   # the fresh page is private: idempotent
    pkv.pkv_pool_destroy(pool)
    # Without a spare page the named page loses its name instead (no copy is possible, none is needed).
    pool = pkv.pkv_pool_create(2, pt, 4, 8, 1)
    parent = pkv.pkv_pool_seq_open(pool)
    toks = np.arange(100, 108, dtype=np.int32)
    assert pkv.pkv_pool_alloc(pool, parent, 8) == 1
    capi.check(pkv.pkv_pool_register(pool, parent, ptr(toks), 8, 8))
    child = pkv.pkv_pool_fork(pool, parent, 6)
    capi.check(pkv.pkv_pool_release(pool, parent))
    assert pkv.pkv_pool_available(pool) == 0 and pkv.pkv_pool_cached_count(pool) == 2
    assert pkv.pkv_pool_cow(pool, child, 6, 1, ptr(src), ptr(dst), 4) == 0
    assert pkv.pkv_pool_page_hash(pool, 1) == 0 and pkv.pkv_pool_cached_count(pool) == 1
    other = pkv.pkv_pool_seq_open(pool)
    assert pkv.pkv_pool_match_prefix(pool, other, ptr(np.append(toks, 1).astype(np.int32)), 9, None) == 4   # page 0 only
    check_accounting(pkv, pool, 2, [parent, child, other])
    pkv.pkv_pool_destroy(pool)


def test_short_output_arrays_change_nothing(pkv):
    """compact / cow / migrate with a cap below the pair count (or NULL outputs) return -2 and leave the pool as it
    was, so the call can be repeated with room; the pair count is available beforehand."""
    pt = 4
    pool = pkv.pkv_pool_create(8, pt, 4, 8, 0)
    a, b = pkv.pkv_pool_seq_open(pool), pkv.pkv_pool_seq_open(pool)
    for h in (a, b):
        assert pkv.pkv_pool_assign_slot(pool, h) >= 0 and pkv.pkv_pool_alloc(pool, h, 16) == 1
    capi.check(pkv.pkv_pool_release(pool, a))                           # pages 0..3 free, b holds 4..7
    before = list(pages_of(pkv, pool, b))
    tab = np.ctypeslib.as_array(pkv.pkv_pool_tables(pool), shape=(4, 8)).copy()
    ms, md = np.zeros(8, np.int32), np.zeros(8, np.int32)
    assert pkv.pkv_pool_compact_pairs(pool) == 4
    assert pkv.pkv_pool_compact(pool, ptr(ms), ptr(md), 1) == -2
    assert pkv.pkv_pool_compact(pool, None, None, 8) == -2
    assert list(pages_of(pkv, pool, b)) == before
    assert np.array_equal(np.ctypeslib.as_array(pkv.pkv_pool_tables(pool), shape=(4, 8)), tab)
    assert pkv.pkv_pool_compact(pool, ptr(ms), ptr(md), 8) == 4          # the retry emits every move
    assert list(ms[:4]) == before and list(md[:4]) == [0, 1, 2, 3]
    assert list(pages_of(pkv, pool, b)) == [0, 1, 2, 3]
    # cow
    c = pkv.pkv_pool_fork(pool, b, 16)
    assert pkv.pkv_pool_cow_pairs(pool, c, 0, 16) == 4
    assert pkv.pkv_pool_cow(pool, c, 0, 16, ptr(ms), ptr(md), 3) == -2
    assert list(pages_of(pkv, pool, c)) == [0, 1, 2, 3] and pkv.pkv_pool_page_refs(pool, 0) == 2
    assert pkv.pkv_pool_cow(pool, c, 0, 16, ptr(ms), ptr(md), 4) == 4
    # migrate
    dst = pkv.pkv_pool_create(8, pt, 4, 8, 0)
    out = C.c_int(-1)
    assert pkv.pkv_pool_migrate(pool, c, dst, C.byref(out), ptr(ms), ptr(md), 3) == -2
    assert pkv.pkv_pool_migrate(pool, c, dst, C.byref(out), None, None, 8) == -2
    assert len(pages_of(pkv, pool, c)) == 4 and pkv.pkv_pool_available(dst) == 8
    assert pkv.pkv_pool_migrate(pool, c, dst, C.byref(out), ptr(ms), ptr(md), 4) == 4
    pkv.pkv_pool_destroy(pool)
    pkv.pkv_pool_destroy(dst)


def test_image_positions_are_named_by_image_hash_and_offset(pkv):
    """token_key of src/engine/engine.cpp:264-270: inside an image block a position's key is mix64(hash + offset), so
    two prompts with the same placeholder tokens but different images do not share pages, and the same image does."""
    u64p = C.POINTER(C.c_uint64)
    pt = 4
    toks = np.array([5, 6, 9, 9, 9, 9, 9, 9, 7, 8, 3, 4, 2], np.int32)   # an image block of six placeholder tokens at 2
    starts, lens = np.array([2], np.int32), np.array([6], np.int32)

    def mix64(x):
        m = (1 << 64) - 1
        x = ((x ^ (x >> 30)) * 0xbf58476d1ce4e5b9) & m
        x = ((x ^ (x >> 27)) * 0x94d049bb133111eb) & m
        return x ^ (x >> 31)

    def keys_for(h):
        k = np.zeros(len(toks), np.uint64)
        capi.check(pkv.pkv_token_keys(ptr(toks), len(toks), ptr(starts), ptr(lens), np.array([h], np.uint64).ctypes.data_as(u64p), 1,
                                      k.ctypes.data_as(u64p)))
        return k

    ka, kb = keys_for(0x1234), keys_for(0x9999)
    assert list(ka[:2]) == [5, 6] and list(ka[8:]) == [7, 8, 3, 4, 2]
    assert [int(x) for x in ka[2:8]] == [mix64((0x1234 + i) & ((1 << 64) - 1)) for i in range(6)]
    text = np.zeros(len(toks), np.uint64)
    capi.check(pkv.pkv_token_keys(ptr(toks), len(toks), None, None, None, 0, text.ctypes.data_as(u64p)))
    assert [int(x) for x in text] == [int(t) for t in toks]
    assert pkv.pkv_page_hash_keys(text.ctypes.data_as(u64p), pt, 2) == pkv.pkv_page_hash(ptr(toks), pt, 2)
    pool = pkv.pkv_pool_create(16, pt, 4, 8, 1)
    h = pkv.pkv_pool_seq_open(pool)
    assert pkv.pkv_pool_alloc(pool, h, len(toks)) == 1
    capi.check(pkv.pkv_pool_register_keys(pool, h, ka.ctypes.data_as(u64p), len(toks), len(toks)))
    assert pkv.pkv_pool_page_hash(pool, 1) == pkv.pkv_page_hash_keys(ka.ctypes.data_as(u64p), pt, 1)
    same, other, plain = (pkv.pkv_pool_seq_open(pool) for _ in range(3))
    assert pkv.pkv_pool_match_prefix_keys(pool, same, ka.ctypes.data_as(u64p), len(toks), None) == 12
    assert pkv.pkv_pool_match_prefix_keys(pool, other, kb.ctypes.data_as(u64p), len(toks), None) == 0
    assert pkv.pkv_pool_match_prefix(pool, plain, ptr(toks), len(toks), None) == 0
    ok = np.array([1, 0, 1], np.uint8)                                  # "never resume inside a whole image block"
    capi.check(pkv.pkv_pool_release(pool, same))
    assert pkv.pkv_pool_match_prefix_keys(pool, same, ka.ctypes.data_as(u64p), len(toks), ok.ctypes.data_as(C.POINTER(C.c_uint8))) == 12
    pkv.pkv_pool_destroy(pool)


def test_migrate_between_pools(pkv):
    a = pkv.pkv_pool_create(32, 8, 4, 16, 1)
    b = pkv.pkv_pool_create(32, 8, 4, 16, 1)
    filler = pkv.pkv_pool_seq_open(b)
    assert pkv.pkv_pool_alloc(b, filler, 8 * 3) == 1          # dst already uses pages 0..2
    h = pkv.pkv_pool_seq_open(a)
    pkv.pkv_pool_assign_slot(a, h)
    assert pkv.pkv_pool_alloc(a, h, 8 * 5 + 3) == 1           # 6 pages: 0..5
    s, d, out = np.zeros(16, np.int32), np.zeros(16, np.int32), C.c_int(-1)
    m = pkv.pkv_pool_migrate(a, h, b, C.byref(out), ptr(s), ptr(d), 16)
    assert m == 6 and list(s[:6]) == [0, 1, 2, 3, 4, 5] and list(d[:6]) == [3, 4, 5, 6, 7, 8]
    assert pkv.pkv_pool_available(a) == 32 and pkv.pkv_pool_available(b) == 32 - 9
    assert list(pages_of(pkv, b, out.value)) == [3, 4, 5, 6, 7, 8]
    assert pkv.pkv_pool_assign_slot(b, out.value) == 0
    tab = np.ctypeslib.as_array(pkv.pkv_pool_tables(b), shape=(4, 16))
    assert list(tab[0, :6]) == [3, 4, 5, 6, 7, 8]
    big = pkv.pkv_pool_seq_open(a)
    assert pkv.pkv_pool_alloc(a, big, 8 * 16) == 1
    tiny = pkv.pkv_pool_create(4, 8, 4, 16, 1)
    assert pkv.pkv_pool_migrate(a, big, tiny, C.byref(out), ptr(s), ptr(d), 16) == -1   # does not fit: nothing changes
    assert len(pages_of(pkv, a, big)) == 16
    for p in (a, b, tiny):
        pkv.pkv_pool_destroy(p)


def test_cpp_class_api():
    """The pool through its C++ class, as a C++ engine would use it (tests/cpp/page_pool_test.cpp), compiled with g++."""
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    exe = root / "tests" / "cpp" / "page_pool_test.bin"
    cmd = ["g++", "-std=c++17", "-O1", "-I", str(root), str(root / "tests/cpp/page_pool_test.cpp"),
           str(root / "unholy_b200/csrc/page_pool.cpp"), "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and "all ok" in run.stdout, run.stdout + run.stderr
