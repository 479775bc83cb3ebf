"""The KV row chain fused with the append: pkv_store_rows_kv_chain = kv_chain (src/kernels/elem_fast.hpp:29; device
body src/kernels/elem_dev.hip.hpp:50-87: rmsnorm with weight, rope on the last 2 * npair values, fake_quant_fp8 block 64
of the others) + store_rows in one pass.

The reference's own result is not reproducible bit for bit on another GPU (its sum of squares runs over 256 threads and
a block reduction, its r is the hardware rsqrtf), so the bar here is the one a floating-point kernel gets, stated:
  * before the quantisation: every normalised value within ONE bf16 step of the oracle's fp32 restatement (sequential
    sum, correctly rounded 1 / sqrt), and more than 99 % of all values identical; a rotated value a*c - b*s (or
    a*s + b*c) inherits the steps of its two inputs, which cancellation can make many steps of a small result, so it is
    held to |difference| <= 2^-7 (|a| + |b|) plus one step of the result;
  * through the quantisation: bit-equal on equal inputs — the full chain's output equals the oracle's fake_quant_fp8
    applied to the kernel's own pre-quantisation values;
  * the append: every row lands where the block table says, bytes equal to rows_out."""
import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi


def bf16_steps(a, b):
    """Distance in bf16 steps between two arrays of bf16 bit patterns (+0 and -0 are the same value)."""
    a, b = a.astype(np.int32), b.astype(np.int32)
    same_sign = (a >> 15) == (b >> 15)
    return np.where(same_sign, np.abs(a - b), (a & 0x7FFF) + (b & 0x7FFF))


def make_case(seed, n, dim, npair, positions=4096):
    g = tl.rng(seed)
    x = tl.normal_bf16(g, (n, dim))
    x[0] *= 0                                           # an all-zero row: r = 1 / sqrt(eps)
    x[1, :64] = orc.f32_to_bf16_bits(np.full(64, 300.0, np.float32))   # outliers that set a block's scale
    w = orc.f32_to_bf16_bits((1.0 + 0.1 * g.standard_normal(dim)).astype(np.float32))
    pos = g.integers(0, positions, size=n).astype(np.int32)
    ang = g.uniform(0, 2 * np.pi, size=(positions, npair)).astype(np.float32)
    freqs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32).copy()
    return x, w, pos, freqs


def test_oracle_kv_chain_properties():
    """CPU: the restatement against numpy statements of its three parts."""
    x, w, pos, freqs = make_case(1, 9, 576, 32)
    got = x.copy()
    orc.kv_chain(got, w, 1e-6, pos, freqs, 32, quant=False)
    xf = (x.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    wf = (w.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    normed = wf * xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-6)
    gf = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.allclose(gf[:, :512], normed[:, :512], rtol=2 ** -7, atol=1e-30)      # bf16 rounding
    a, b = normed[:, 512::2], normed[:, 513::2]
    c, s = freqs[pos, :, 0].astype(np.float64), freqs[pos, :, 1].astype(np.float64)
    assert np.allclose(gf[:, 512::2], a * c - b * s, rtol=2 ** -6, atol=2 ** -6)
    assert np.allclose(gf[:, 513::2], a * s + b * c, rtol=2 ** -6, atol=2 ** -6)
    full = x.copy()
    orc.kv_chain(full, w, 1e-6, pos, freqs, 32, quant=True)
    want = got.copy()
    orc.fake_quant_fp8(want, 512, 64)
    assert np.array_equal(full, want) and np.array_equal(full[:, 512:], got[:, 512:])   # the rope part is not quantised


@pytest.mark.gpu
@pytest.mark.parametrize("n,dim,npair,stride", [(300, 576, 32, 576), (37, 576, 32, 640), (65, 512, 0, 512), (130, 1024, 64, 1024), (5, 128, 32, 128)])
def test_kv_chain_store(pkv, cuda, n, dim, npair, stride):
    x, w, pos, freqs = make_case(n + dim, n, dim, npair)
    rpp, row0 = 64, 29
    pages = -(-(row0 + n) // rpp) + 2
    g = tl.rng(7)
    table = g.permutation(pages).astype(np.int32)
    d_x, d_w, d_pos, d_f, d_t = (tl.dev(cuda, a) for a in (x, w, pos, freqs, table))
    st = tl.stream_ptr(cuda)
    results = {}
    for quant in (0, 1):
        d_out = cuda.full((n * dim * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
        d_pool = cuda.full((pages * rpp * stride * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
        capi.check(pkv.pkv_store_rows_kv_chain(d_x.data_ptr(), d_out.data_ptr(), d_w.data_ptr(), n, dim, 1e-6, d_pos.data_ptr(),
                                               d_f.data_ptr(), npair, quant, d_pool.data_ptr(), d_t.data_ptr(), rpp, stride, row0, st))
        cuda.cuda.synchronize()
        out = tl.host(d_out, np.uint16, (n, dim))
        pool = tl.host(d_pool, np.uint16, (pages * rpp, stride))
        want_pool = np.full((pages * rpp, stride), 0x5A5A, np.uint16)
        for r in range(n):
            lr = row0 + r
            want_pool[table[lr // rpp] * rpp + lr % rpp, :dim] = out[r]
        assert np.array_equal(pool, want_pool), "the appended rows are not rows_out at the block table's places"
        results[quant] = out
    # before the quantisation: within one bf16 step of the oracle, nearly always identical
    want = x.copy()
    orc.kv_chain(want, w, 1e-6, pos, freqs, npair, quant=False)
    steps = bf16_steps(results[0], want)
    off = dim - 2 * npair
    assert steps[:, :off].max() <= 1, f"largest difference {steps[:, :off].max()} bf16 steps"
    assert (steps == 0).mean() > 0.99
    if npair:
        f32 = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        normed = x.copy()
        orc.kv_chain(normed, w, 1e-6, pos, freqs, 0, quant=False)              # the rope's inputs
        a, b = np.abs(f32(normed[:, off::2])), np.abs(f32(normed[:, off + 1::2]))
        bound = np.repeat(2.0 ** -7 * (a + b), 2, axis=1) + 2.0 ** -7 * np.abs(f32(want[:, off:]))
        assert (np.abs(f32(results[0][:, off:]) - f32(want[:, off:])) <= bound).all()
    # through the quantisation: exact on the kernel's own pre-quantisation values
    through = results[0].copy()
    orc.fake_quant_fp8(through, dim - 2 * npair, 64)
    assert np.array_equal(results[1], through)
    # in place (rows_out == rows, no pool) gives the same rows: the reference's kv_chain call
    d_in = tl.dev(cuda, x)
    capi.check(pkv.pkv_store_rows_kv_chain(d_in.data_ptr(), d_in.data_ptr(), d_w.data_ptr(), n, dim, 1e-6, d_pos.data_ptr(), d_f.data_ptr(),
                                           npair, 1, None, None, 0, 0, 0, st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_in, np.uint16, (n, dim)), results[1])


def test_kv_chain_argument_errors(pkv):
    a = 4096
    assert pkv.pkv_store_rows_kv_chain(None, None, None, 0, 576, 1e-6, None, None, 32, 1, None, None, 0, 0, 0, None) == capi.PKV_OK
    assert pkv.pkv_store_rows_kv_chain(a, a, a, 1, 570, 1e-6, a, a, 32, 1, None, None, 0, 0, 0, None) == capi.PKV_ERR_ARG   # dim % 8
    assert pkv.pkv_store_rows_kv_chain(a, a, a, 1, 576, 1e-6, a, a, 30, 1, None, None, 0, 0, 0, None) == capi.PKV_ERR_ARG   # rope part
    assert pkv.pkv_store_rows_kv_chain(a, None, a, 1, 576, 1e-6, a, a, 32, 1, None, None, 0, 0, 0, None) == capi.PKV_ERR_ARG  # nowhere to write
