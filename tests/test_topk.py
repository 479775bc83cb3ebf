"""Top-k index lists (the producer of the gather's input): the CPU oracle against an independent numpy statement of
the reference's contract, and the CUDA kernels against the oracle, bit for bit (src/kernels/indexer.hpp:74:
"ordered (score desc, index asc); -1 padded; -inf never selected"; the reference's own check compares the fast and the
reference index lists for equality: tools/kernel_test/indexer.hip:166-188)."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

NEG_INF = 0xFF80


def scores_case(g, T, n, ld, kind):
    s = np.full((T, ld), 0x1234, np.uint16)
    if kind == "normal":
        s[:, :n] = tl.normal_bf16(g, (T, n))
    elif kind == "ties":            # few distinct values: the threshold is always a tie
        s[:, :n] = orc.f32_to_bf16_bits(g.integers(-3, 4, size=(T, n)).astype(np.float32) * np.float32(0.5))
    elif kind == "masked":          # most keys invisible (-inf), as for early queries of a chunk
        s[:, :n] = tl.normal_bf16(g, (T, n))
        for t in range(T):
            s[t, int(g.integers(0, n)):n] = NEG_INF
        s[0, :n] = NEG_INF           # a row with nothing to select
    elif kind == "special":         # +-0, +-inf, NaN patterns of both signs, subnormals, all bit patterns
        s[:, :n] = g.integers(0, 65536, size=(T, n)).astype(np.uint16)
    return s


def numpy_topk(scores, n, k):
    T = scores.shape[0]
    out = np.full((T, k), -1, np.int32)
    for t in range(T):
        b = scores[t, :n].astype(np.uint32)
        key = np.where(b & 0x8000, ~b & 0xFFFF, b | 0x8000)
        valid = np.flatnonzero(key > 0x7F)
        order = valid[np.lexsort((valid, -key[valid].astype(np.int64)))]
        want = min(k, len(order))
        out[t, :want] = order[:want]
    return out


@pytest.mark.parametrize("kind", ["normal", "ties", "masked", "special"])
def test_oracle_topk_matches_contract(kind):
    g = tl.rng(70)
    for T, n, ld, k in ((5, 3000, 3008, 512), (3, 100, 100, 512), (2, 20000, 20000, 2048), (1, 1, 8, 4)):
        s = scores_case(g, T, n, ld, kind)
        assert np.array_equal(orc.topk_bf16(s, n, k), numpy_topk(s, n, k)), (kind, T, n, k)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["normal", "ties", "masked", "special"])
@pytest.mark.parametrize("T,n,ld,k", [(37, 5000, 5000, 512), (64, 131072, 131072, 2048), (3, 8192, 8200, 2048),
                                      (4, 8193, 8193, 100), (2, 300, 304, 2048), (1, 1, 8, 1), (5, 40000, 40000, 2051),
                                      (6, 1000, 1003, 64), (2, 524288, 524288, 2048), (1, 524289, 524289, 300),
                                      (1, 800000, 800000, 300), (16, 40000, 40000, 1000),
                                      (3, 7, 9, 2), (2, 65, 65, 129), (2, 655360, 655360, 2048),
                                      (300, 5000, 5003, 512), (200, 20000, 20000, 2048), (180, 40000, 40000, 1000),
                                      (400, 16384, 16384, 1024), (170, 32768, 32768, 1025)])
def test_topk_bf16_gpu(pkv, cuda, kind, T, n, ld, k):
    """Both paths of pkv_topk_bf16 (knob 7: 0 = one launch of thread-block clusters where the shape allows it — k <= 2048,
    n <= 655,360; CTAs of 1024 threads when the launch fits the SMs, of 512 or 256 threads when there are more rows —,
    1 = the four launches through the scratch) against the oracle."""
    g = tl.rng(71)
    s = scores_case(g, T, n, ld, kind)
    want = orc.topk_bf16(s, n, k, threads=8)
    d_s = tl.dev(cuda, s)
    words = pkv.pkv_topk_scratch_words(T, n, k)
    d_scratch = cuda.full((words * 4,), 0x5A, dtype=cuda.uint8, device="cuda")   # poison: nothing relies on zeroes
    try:
        for path in (0, 1):
            capi.check(pkv.pkv_tune(7, path))
            d_idx = cuda.full((T * k * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
            for _ in range(2):   # the second call reuses dirty scratch
                capi.check(pkv.pkv_topk_bf16(d_s.data_ptr(), T, n, ld, k, d_idx.data_ptr(), d_scratch.data_ptr(), words,
                                             tl.stream_ptr(cuda)))
                cuda.cuda.synchronize()
                assert np.array_equal(tl.host(d_idx, np.int32, (T, k)), want), path
    finally:
        capi.check(pkv.pkv_tune(7, 0))
    assert tl.device_status(pkv) == 0


@pytest.mark.gpu
def test_topk_feeds_the_gather(pkv, cuda):
    """Producer and consumer together: index lists from pkv_topk_bf16 drive pkv_gather_rows; the result equals the
    oracle's gather of the oracle's top-k."""
    g = tl.rng(72)
    rpp, pages, W, T, k = 64, 64, 576, 6, 512
    n = pages * rpp
    table = g.permutation(pages).astype(np.int32)
    pool = tl.normal_bf16(g, (n, W))
    s = scores_case(g, T, n, n, "masked")
    vis = np.full(T, n, np.int32)
    idx = orc.topk_bf16(s, n, k)
    want = orc.gather_rows(pool, table.reshape(1, -1), rpp, W, W, idx, np.zeros(T, np.int32), vis)
    d_s, d_pool, d_table, d_vis = tl.dev(cuda, s), tl.dev(cuda, pool), tl.dev(cuda, table), tl.dev(cuda, vis)
    words = pkv.pkv_topk_scratch_words(T, n, k)
    d_scratch = cuda.empty(words * 4, dtype=cuda.uint8, device="cuda")
    d_idx = cuda.empty(T * k * 4, dtype=cuda.uint8, device="cuda")
    d_out = cuda.full((T * k * W * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    st = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_topk_bf16(d_s.data_ptr(), T, n, n, k, d_idx.data_ptr(), d_scratch.data_ptr(), words, st))
    capi.check(pkv.pkv_gather_rows(d_pool.data_ptr(), d_table.data_ptr(), rpp, W, W, d_idx.data_ptr(), d_vis.data_ptr(), T, k,
                                   d_out.data_ptr(), st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


def test_topk_argument_errors(pkv):
    assert pkv.pkv_topk_scratch_words(64, 131072, 2048) == 64 * 16 * 512 + 64 * 8 + 64 * 16 * 2 + 64 * 2048 * 2
    assert pkv.pkv_topk_bf16(None, 0, 10, 10, 4, None, None, 0, None) == capi.PKV_OK
    assert pkv.pkv_topk_bf16(16, 1, 10, 10, 5000, 16, 16, 1 << 20, None) == capi.PKV_ERR_LIMIT
    assert pkv.pkv_topk_bf16(16, 1, 10, 4, 4, 16, 16, 1 << 20, None) == capi.PKV_ERR_ARG


@pytest.mark.gpu
def test_topk_scratch_is_optional(pkv, cuda):
    """As in the reference (src/kernels/indexer.hpp:91-92: scratch = nullptr, scratch_words = 0), a caller may pass no
    scratch or too little: the one-launch path needs none, the four-launch path falls back to the library's built-in
    array, and only a shape that fits neither is refused, before anything is launched."""
    g = tl.rng(12)
    T, n, k = 5, 20000, 300
    scores = tl.normal_bf16(g, (T, n))
    want = orc.topk_bf16(scores, n, k)
    d_s = tl.dev(cuda, scores)
    st = tl.stream_ptr(cuda)
    tiny = cuda.zeros(64, dtype=cuda.int32, device="cuda")
    try:
        for path in (0, 1):
            capi.check(pkv.pkv_tune(7, path))
            for scratch, words in ((None, 0), (tiny.data_ptr(), 64)):
                d_idx = cuda.full((T * k,), -7, dtype=cuda.int32, device="cuda")
                capi.check(pkv.pkv_topk_bf16(d_s.data_ptr(), T, n, n, k, d_idx.data_ptr(), scratch, words, st))
                cuda.cuda.synchronize()
                assert np.array_equal(tl.host(d_idx, np.int32, (T, k)), want), (path, words)
        capi.check(pkv.pkv_tune(7, 1))
        rc = pkv.pkv_topk_bf16(d_s.data_ptr(), 4096, 2, 2, 4096, tiny.data_ptr(), None, 0, st)   # 33 M words: nothing holds them
        assert rc == capi.PKV_ERR_LIMIT and b"scratch" in pkv.pkv_last_error()
    finally:
        capi.check(pkv.pkv_tune(7, 0))


def expand_case(g, n, k, pool):
    pos = g.integers(0, 4 * k * pool, size=n).astype(np.int32)
    pos[0], pos[-1] = 0, k * pool * 3 + pool - 2
    pools = np.full((n, k), -1, np.int32)
    for t in range(n):
        full = (int(pos[t]) + 1) // pool
        m = min(full, k)
        pools[t, :m] = g.choice(full, size=m, replace=False)
    return pools, pos


def test_oracle_idx_expand_matches_contract():
    g = tl.rng(73)
    for n, k, pool in ((9, 512, 4), (3, 5, 4), (4, 7, 1), (2, 3, 8)):
        pools, pos = expand_case(g, n, k, pool)
        got = orc.idx_expand(pools, pos, pool)
        assert got.shape == (n, k * pool + pool - 1)
        for t in range(n):
            p = int(pos[t])
            valid, tail = min((p + 1) // pool, k), (p + 1) % pool
            want = [int(pools[t, j // pool]) * pool + j % pool for j in range(valid * pool)] + list(range(p + 1 - tail, p + 1))
            assert list(got[t, :len(want)]) == want and (got[t, len(want):] == -1).all()
            assert len(want) == valid * pool + tail          # glm_sel_count (src/kernels/glm_fast.hpp:118-121)


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,pool", [(64, 512, 4), (3, 5, 4), (4, 7, 1), (1000, 16, 8)])
def test_idx_expand_gpu(pkv, cuda, n, k, pool):
    g = tl.rng(74)
    pools, pos = expand_case(g, n, k, pool)
    want = orc.idx_expand(pools, pos, pool)
    d_pools, d_pos = tl.dev(cuda, pools), tl.dev(cuda, pos)
    d_idx = cuda.full((want.size * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
    capi.check(pkv.pkv_idx_expand(d_pools.data_ptr(), d_pos.data_ptr(), d_idx.data_ptr(), n, k, pool, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_idx, np.int32, want.shape), want)


@pytest.mark.gpu
@pytest.mark.parametrize("many", [False, True])
def test_topk_batch_groups(pkv, cuda, many):
    """Several score blocks with their own row counts, key counts and k in one call (the decode chunks of a step):
    each group's lists equal the oracle's for that block. Knob 7 = 0 runs all groups in one launch of thread-block
    clusters (32 groups per launch: `many` has 40, one of them empty), 1 runs them one after the other through the
    scratch."""
    g = tl.rng(75)
    shapes = [(3, 9000, 512), (1, 300, 512), (5, 20000, 2048), (2, 64, 16)]
    if many:
        shapes = shapes + [(0, 100, 8)] + [(1 + i % 3, 500 + 37 * i, 64 + i) for i in range(35)]
    kinds = ("normal", "masked", "ties", "special")
    blocks = [scores_case(g, max(T, 1), n, n, kinds[i % 4]) for i, (T, n, k) in enumerate(shapes)]
    flat = np.concatenate([b.reshape(-1) for b in blocks])
    groups = (capi.PkvTopkGroup * len(shapes))()
    off = idx_off = 0
    for i, (T, n, k) in enumerate(shapes):
        groups[i].off, groups[i].rows, groups[i].n, groups[i].k, groups[i].idx_off = off, T, n, k, idx_off
        off += max(T, 1) * n
        idx_off += T * k
    words = pkv.pkv_topk_batch_scratch_words(groups, len(shapes))
    assert words == max(pkv.pkv_topk_scratch_words(T, n, k) for T, n, k in shapes)
    d_s = tl.dev(cuda, flat)
    d_scratch = cuda.full((words * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
    try:
        for path in (0, 1):
            capi.check(pkv.pkv_tune(7, path))
            d_idx = cuda.full((idx_off * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
            capi.check(pkv.pkv_topk_bf16_batch(d_s.data_ptr(), groups, len(shapes), d_idx.data_ptr(), d_scratch.data_ptr(),
                                               words, tl.stream_ptr(cuda)))
            cuda.cuda.synchronize()
            got = tl.host(d_idx, np.int32)
            o = 0
            for (T, n, k), b in zip(shapes, blocks):
                assert np.array_equal(got[o:o + T * k].reshape(T, k), orc.topk_bf16(b[:T], n, k)), (path, T, n, k)
                o += T * k
    finally:
        capi.check(pkv.pkv_tune(7, 0))
    assert tl.device_status(pkv) == 0
