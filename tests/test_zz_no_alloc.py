"""pkv_topk_bf16_static: the top-k entry point that allocates nothing and brings its own scratch (an array compiled into
the library), for callers that can neither pass device scratch nor tolerate an allocation. Its index lists must be
identical to those of pkv_topk_bf16 (which takes caller scratch) on the same scores, and both must equal the CPU
oracle's — checked on two calls in a row, the second on different scores, so that whatever the first call left in the
shared scratch cannot leak into the second result. Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

pytestmark = pytest.mark.gpu


def test_static_scratch_topk_matches_caller_scratch_topk(pkv, cuda):
    T, n, k = 64, 131072, 2048                      # the decode shape: needs 788,992 of the 1,048,576 built-in words
    assert pkv.pkv_topk_scratch_words(T, n, k) <= pkv.pkv_topk_static_scratch_words()
    g = tl.rng(99)
    st = tl.stream_ptr(cuda)
    words = pkv.pkv_topk_scratch_words(T, n, k)
    d_scratch = cuda.empty(words * 4, dtype=cuda.uint8, device="cuda")
    for call in range(2):
        scores = tl.normal_bf16(g, (T, n))
        scores[call, : n // 2] = 0xFF80              # a row with half its keys invisible
        scores[5 + call, :] = 0x3F80                 # a row of ties: the lowest indices win
        d_s = tl.dev(cuda, scores)
        d_ref = cuda.full((T * k * 4,), 0x5A, dtype=cuda.uint8, device="cuda")
        d_got = cuda.full((T * k * 4,), 0xA5, dtype=cuda.uint8, device="cuda")
        capi.check(pkv.pkv_topk_bf16(d_s.data_ptr(), T, n, n, k, d_ref.data_ptr(), d_scratch.data_ptr(), words, st))
        capi.check(pkv.pkv_topk_bf16_static(d_s.data_ptr(), T, n, n, k, d_got.data_ptr(), st))
        cuda.cuda.synchronize()
        ref, got = tl.host(d_ref, np.int32, (T, k)), tl.host(d_got, np.int32, (T, k))
        assert np.array_equal(got, ref), f"call {call}"   # index lists are integers: identical, no tolerance
        assert np.array_equal(got, orc.topk_bf16(scores, n, k, threads=8)), f"call {call}: differs from the oracle"
        assert list(got[5 + call, :4]) == [0, 1, 2, 3]


def test_static_scratch_topk_refuses_oversized_shapes(pkv, cuda):
    d = cuda.zeros(1024, dtype=cuda.uint8, device="cuda")
    rc = pkv.pkv_topk_bf16_static(d.data_ptr(), 512, 131072, 131072, 2048, d.data_ptr(), tl.stream_ptr(cuda))
    assert rc == capi.PKV_ERR_LIMIT and b"built-in scratch" in pkv.pkv_last_error()
