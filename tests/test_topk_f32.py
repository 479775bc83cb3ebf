"""fp32 top-k index lists (topk_rows, src/kernels/ref.hpp:107, and glm_topk, src/kernels/glm_fast.hpp:86-93): the CPU
oracle against an independent numpy statement of the contract ("radix select ... keys above the threshold, plus
threshold ties by lowest index; -inf never selected; output sorted by (score desc, index asc)",
src/kernels/ref_attn.hip:143-145), the CUDA kernel against the oracle bit for bit, and the reference's own
cross-check of its two producers: on bf16-representable scores the fp32 and the bf16 selection give the same lists
(tools/kernel_test/indexer.hip:95-188)."""
import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi


def scores_case(g, T, n, ld, kind):
    s = np.full((T, ld), 123.0, np.float32)                  # the padding past n would win every selection
    if kind == "normal":
        s[:, :n] = g.standard_normal((T, n), dtype=np.float32)
    elif kind == "ties":                                     # few distinct values: the threshold is always a tie
        s[:, :n] = g.integers(-3, 4, size=(T, n)).astype(np.float32) * np.float32(0.5)
    elif kind == "masked":                                   # most keys invisible, as for early queries of a chunk
        s[:, :n] = g.standard_normal((T, n), dtype=np.float32)
        for t in range(T):
            s[t, int(g.integers(0, n)):n] = -np.inf
        s[0, :n] = -np.inf                                   # a row with nothing to select
    elif kind == "special":                                  # every bit pattern: +-0, +-inf, NaNs of both signs, subnormals
        s[:, :n] = g.integers(0, 2**32, size=(T, n), dtype=np.uint64).astype(np.uint32).view(np.float32)
    elif kind == "close":                                    # one exponent, keys differing only in the low mantissa bits
        s[:, :n] = (np.uint32(0x3F800000) + g.integers(0, 3000, size=(T, n)).astype(np.uint32)).view(np.float32)
    return s


def numpy_topk(scores, n, k):
    T = scores.shape[0]
    out = np.full((T, k), -1, np.int32)
    for t in range(T):
        u = scores[t, :n].view(np.uint32).astype(np.int64)
        key = np.where(u & 0x80000000, ~u & 0xFFFFFFFF, u | 0x80000000)
        valid = np.flatnonzero(key > 0x007FFFFF)
        order = valid[np.lexsort((valid, -key[valid]))]
        want = min(k, len(order))
        out[t, :want] = order[:want]
    return out


KINDS = ["normal", "ties", "masked", "special", "close"]


@pytest.mark.parametrize("kind", KINDS)
def test_oracle_topk_f32_matches_contract(kind):
    g = tl.rng(80)
    for T, n, ld, k in ((5, 3000, 3008, 512), (3, 100, 100, 512), (2, 20000, 20000, 1024), (1, 1, 8, 4)):
        s = scores_case(g, T, n, ld, kind)
        assert np.array_equal(orc.topk_f32(s, n, k), numpy_topk(s, n, k)), (kind, T, n, k)


def test_oracle_f32_and_bf16_producers_agree():
    """On bf16-representable scores both producers select the same lists (the reference checks one against the other)."""
    g = tl.rng(81)
    b = tl.normal_bf16(g, (7, 6000))
    b[:, 5000:] = 0xFF80
    f = (b.astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(orc.topk_f32(f, 6000, 512), orc.topk_bf16(b, 6000, 512))


@pytest.mark.gpu
@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("T,n,ld,k", [(37, 5000, 5000, 512), (64, 32768, 32768, 512), (3, 8192, 8200, 1024),
                                      (4, 8193, 8193, 100), (2, 300, 304, 1024), (1, 1, 8, 1), (2, 49152, 49152, 1000),
                                      (3, 49153, 49160, 1024), (2, 200000, 200000, 64), (5, 17, 17, 3),
                                      (2, 40960, 40960, 1024), (2, 40961, 40963, 1024), (200, 2000, 2001, 64),
                                      (64, 4096, 4096, 512), (3, 4095, 4100, 1024), (3, 4097, 4097, 1024),
                                      (3, 1025, 1025, 1000), (7, 2048, 2048, 1024), (5, 1024, 1024, 1024)])
def test_topk_f32_gpu(pkv, cuda, kind, T, n, ld, k):
    g = tl.rng(82)
    s = scores_case(g, T, n, ld, kind)
    want = orc.topk_f32(s, n, k, threads=8)
    d_s = tl.dev(cuda, s)
    d_idx = cuda.full((T * k * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
    for _ in range(2):
        capi.check(pkv.pkv_topk_f32(d_s.data_ptr(), T, n, ld, k, d_idx.data_ptr(), tl.stream_ptr(cuda)))
        cuda.cuda.synchronize()
        assert np.array_equal(tl.host(d_idx, np.int32, (T, k)), want)
    assert tl.device_status(pkv) == 0


@pytest.mark.gpu
def test_f32_and_bf16_kernels_agree(pkv, cuda):
    g = tl.rng(83)
    T, n, k = 16, 20000, 1024
    b = tl.normal_bf16(g, (T, n))
    b[3, 100:] = 0xFF80
    f = (b.astype(np.uint32) << 16).view(np.float32)
    d_b, d_f = tl.dev(cuda, b), tl.dev(cuda, f)
    words = pkv.pkv_topk_scratch_words(T, n, k)
    d_scratch = cuda.zeros((words * 4,), dtype=cuda.uint8, device="cuda")
    i_b = cuda.zeros((T, k), dtype=cuda.int32, device="cuda")
    i_f = cuda.zeros((T, k), dtype=cuda.int32, device="cuda")
    capi.check(pkv.pkv_topk_bf16(d_b.data_ptr(), T, n, n, k, i_b.data_ptr(), d_scratch.data_ptr(), words, tl.stream_ptr(cuda)))
    capi.check(pkv.pkv_topk_f32(d_f.data_ptr(), T, n, n, k, i_f.data_ptr(), tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert cuda.equal(i_b, i_f)


@pytest.mark.gpu
def test_topk_f32_feeds_expand_and_gather(pkv, cuda):
    """The GLM-style chain: pool scores -> pkv_topk_f32 -> pkv_idx_expand -> pkv_gather_rows equals the oracle's chain."""
    g = tl.rng(84)
    rpp, pages, W, T, kp, pool = 64, 32, 576, 5, 16, 4
    nrows = pages * rpp
    table = g.permutation(pages).astype(np.int32)
    kv = tl.normal_bf16(g, (nrows, W))                       # the physical pool; the table maps logical pages into it
    pos = g.integers(nrows // 2, nrows, size=T).astype(np.int32)
    npool = nrows // pool
    sc = g.standard_normal((T, npool), dtype=np.float32)
    for t in range(T):
        sc[t, (pos[t] + 1) // pool:] = -np.inf              # only complete pools are visible to the query
    pools = orc.topk_f32(sc, npool, kp)
    idx = orc.idx_expand(pools, pos, pool)
    w = idx.shape[1]
    vis = (pos + 1).astype(np.int32)
    want = orc.gather_rows(kv, table.reshape(1, -1), rpp, W, W, idx, np.zeros(T, np.int32), vis)
    d_sc, d_pos, d_kv, d_tab, d_vis = (tl.dev(cuda, a) for a in (sc, pos, kv, table, vis))
    d_pools = cuda.zeros((T, kp), dtype=cuda.int32, device="cuda")
    d_idx = cuda.zeros((T, w), dtype=cuda.int32, device="cuda")
    d_out = cuda.full((T * w * W * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    sp = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_topk_f32(d_sc.data_ptr(), T, npool, npool, kp, d_pools.data_ptr(), sp))
    capi.check(pkv.pkv_idx_expand(d_pools.data_ptr(), d_pos.data_ptr(), d_idx.data_ptr(), T, kp, pool, sp))
    capi.check(pkv.pkv_gather_rows(d_kv.data_ptr(), d_tab.data_ptr(), rpp, W, W, d_idx.data_ptr(), d_vis.data_ptr(), T, w,
                                   d_out.data_ptr(), sp))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_pools, np.int32, (T, kp)), pools)
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


def test_topk_f32_argument_errors(pkv):
    assert pkv.pkv_topk_f32(None, 0, 10, 10, 4, None, None) == 0            # nothing to do
    assert pkv.pkv_topk_f32(1, 1, 10, 10, 1025, 1, None) == capi.PKV_ERR_ARG  # the reference's limit: k <= 1024
    assert b"k > 1024" in pkv.pkv_last_error()
    assert pkv.pkv_topk_f32(None, 1, 10, 10, 4, None, None) == capi.PKV_ERR_ARG
    assert pkv.pkv_topk_f32(1, 1, 10, 9, 4, 1, None) == capi.PKV_ERR_ARG     # ld < n
