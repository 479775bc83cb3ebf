"""Pins of the CPU oracle (oracle/pkv_oracle.cpp), all on the CPU:

  1. against the reference's own scalar helpers (src/kernels/dev.hip.hpp compiled in place into
     oracle/_ref/libref_numeric.so) — exhaustive over every bf16 / e4m3 / e2m1 / e8m0 code and dense float sweeps;
  2. against golden vectors produced by the reference's pure-torch quantisers (tests/golden/quant_golden.npz,
     made by tests/golden/make_golden.py from tools/ref/oracle/kernel.py);
  3. the reference's own test property: fp4 store -> load == fake_quant_fp4 on a shuffled block table
     (tools/kernel_test/indexer.hip:66-69,82-95);
  4. paged addressing against a direct numpy statement of pool + (table[r / rpp] * rpp + r % rpp) * stride.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import build_oracle, oracle_lib as orc

GOLDEN = Path(__file__).resolve().parent / "golden" / "quant_golden.npz"


@pytest.fixture(scope="module")
def ref():
    libs = build_oracle.build_reference()
    if not libs["numeric"]:
        pytest.skip("oracle/_ref/libref_numeric.so not built (no reference checkout here)")
    h = C.CDLL(str(libs["numeric"]))
    h.ref_bf16_to_f32.restype, h.ref_bf16_to_f32.argtypes = C.c_float, [C.c_uint16]
    h.ref_e4m3_to_f32.restype, h.ref_e4m3_to_f32.argtypes = C.c_float, [C.c_uint8]
    h.ref_e8m0_to_f32.restype, h.ref_e8m0_to_f32.argtypes = C.c_float, [C.c_uint8]
    h.ref_e2m1_to_f32.restype, h.ref_e2m1_to_f32.argtypes = C.c_float, [C.c_uint32]
    for name in ("ref_f32_to_bf16_n", "ref_f32_to_e4m3_n", "ref_round_e2m1_n", "ref_pow2_ceil_e8m0_n"):
        getattr(h, name).restype, getattr(h, name).argtypes = None, [C.c_void_p, C.c_void_p, C.c_long]
    return h


def float_sweep():
    """Every bf16 bit pattern widened to fp32, the midpoints between neighbours, and random fp32 bit patterns."""
    g = tl.rng(7)
    b = (np.arange(65536, dtype=np.uint32) << 16)
    mids = b + 0x8000
    near = np.concatenate([b + 0x7FFF, b + 0x8001, b + 1])
    rand = g.integers(0, 1 << 32, size=1 << 20, dtype=np.uint64).astype(np.uint32)
    return np.concatenate([b, mids, near, rand]).view(np.float32)


def test_decoders_exhaustive(ref):
    o = orc.lib()
    for v in range(65536):
        a, b = o.orc_bf16_to_f32(v), ref.ref_bf16_to_f32(v)
        assert a == b or (a != a and b != b)
    for v in range(256):
        a, b = o.orc_e4m3_to_f32(v), ref.ref_e4m3_to_f32(v)
        assert (a == b and np.signbit(a) == np.signbit(b)) or (a != a and b != b), v
        a, b = o.orc_e8m0_to_f32(v), ref.ref_e8m0_to_f32(v)
        assert a == b or (a != a and b != b), v
    for v in range(16):
        a, b = o.orc_e2m1_to_f32(v), ref.ref_e2m1_to_f32(v)
        assert a == b and np.signbit(a) == np.signbit(b)


def _vec(fn_scalar, xs, restype):
    return np.array([fn_scalar(float(x)) for x in xs], dtype=restype)


def test_f32_to_bf16_sweep(ref):
    x = float_sweep()
    want = np.empty(x.size, np.uint16)
    ref.ref_f32_to_bf16_n(x.ctypes.data, want.ctypes.data, x.size)
    # the oracle through its array entry: fake-quant-free path = store of already-rounded rows; use the scalar export
    o = orc.lib()
    step = 97  # scalar ctypes calls are slow: every 97th element plus all NaN/inf/edge patterns
    sel = np.unique(np.concatenate([np.arange(0, x.size, step), np.flatnonzero(~np.isfinite(x))[:5000]]))
    got = _vec(o.orc_f32_to_bf16, x[sel], np.uint16)
    assert np.array_equal(got, want[sel])
    # and the numpy helper the tests use to build inputs agrees on finite values
    fin = np.isfinite(x) & (np.abs(x) < 3.3e38)
    assert np.array_equal(orc.f32_to_bf16_bits(x[fin]), want[fin])


def test_f32_to_e4m3_sweep(ref):
    g = tl.rng(8)
    # every e4m3 value, every midpoint between neighbours, +-1 ulp around both, plus random values in [-448, 448]
    o = orc.lib()
    vals = np.array(sorted({o.orc_e4m3_to_f32(c) for c in range(256) if (c & 0x7F) != 0x7F}), np.float32)
    mids = ((vals[:-1].astype(np.float64) + vals[1:].astype(np.float64)) / 2).astype(np.float32)
    base = np.concatenate([vals, mids])
    around = np.concatenate([base, np.nextafter(base, np.float32(1e9)), np.nextafter(base, np.float32(-1e9))])
    rand = (g.standard_normal(200000, dtype=np.float32) * np.float32(100)).clip(-448, 448)
    tiny = g.standard_normal(20000, dtype=np.float32) * np.float32(2 ** -8)
    x = np.concatenate([around, rand, tiny, np.array([0.0, -0.0], np.float32)]).astype(np.float32)
    x = x[np.abs(x) <= 448]
    want = np.empty(x.size, np.uint8)
    ref.ref_f32_to_e4m3_n(x.ctypes.data, want.ctypes.data, x.size)
    got = _vec(o.orc_f32_to_e4m3, x, np.uint8)
    assert np.array_equal(got, want)


def test_round_e2m1_and_pow2_sweep(ref):
    g = tl.rng(9)
    o = orc.lib()
    ties = np.array([0, .25, .5, .75, 1, 1.25, 1.5, 1.75, 2, 2.5, 3, 3.5, 4, 5, 6], np.float32)
    base = np.concatenate([ties, -ties, np.array([-0.0], np.float32)])
    x = np.concatenate([base, np.nextafter(base, np.float32(9)), np.nextafter(base, np.float32(-9)),
                        g.uniform(-6, 6, 50000).astype(np.float32)])
    want = np.empty(x.size, np.float32)
    ref.ref_round_e2m1_n(x.ctypes.data, want.ctypes.data, x.size)
    got = _vec(o.orc_round_e2m1, x, np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # bit compare: the sign of zero matters
    p = np.concatenate([np.ldexp(np.float32(1), np.arange(-126, 128)).astype(np.float32),
                        np.abs(g.standard_normal(50000, dtype=np.float32)) * np.float32(3) + np.float32(1e-30),
                        np.ldexp(g.uniform(1, 2, 5000), g.integers(-126, 127, 5000)).astype(np.float32)])
    wantp = np.empty(p.size, np.uint8)
    ref.ref_pow2_ceil_e8m0_n(p.ctypes.data, wantp.ctypes.data, p.size)
    assert np.array_equal(_vec(o.orc_pow2_ceil_e8m0, p, np.uint8), wantp)


def test_golden_quantisers():
    z = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in z.files})
    assert names == ["normal", "octaves", "outliers", "ties"]
    for name in names:
        x = z[f"{name}/x"]
        for block in (32, 64, 128):
            q, s = orc.act_quant_fp8(x.copy(), x.shape[1], block)
            assert np.array_equal(s, z[f"{name}/fp8_scales_b{block}"]), (name, block)
            wq = z[f"{name}/fp8_codes_b{block}"]
            # torch writes +0 for a value that rounds to zero from below; the reference kernel keeps the sign bit
            # (src/kernels/dev.hip.hpp:84). Compare modulo the sign of zero.
            same = (q == wq) | (((q | wq) & 0x7F) == 0)
            assert same.all(), (name, block, int((~same).sum()))
            f = x.copy()
            orc.fake_quant_fp8(f, x.shape[1], block)
            wf = z[f"{name}/fp8_fake_b{block}"]
            same = (f == wf) | (((f | wf) & 0x7FFF) == 0)
            assert same.all(), (name, block)
        f = x.copy()
        orc.fake_quant_fp4(f, x.shape[1], 32)
        wf = z[f"{name}/fp4_fake_b32"]
        same = (f == wf) | (((f | wf) & 0x7FFF) == 0)  # the reference's own test ignores the sign of zero (indexer.hip:92)
        assert same.all(), name


def test_fp4_store_load_equals_fake_quant():
    g = tl.rng(10)
    rpp, pages, n = 64, 79, 5000
    table = g.permutation(pages).astype(np.int32)
    rows = tl.key_rows(g, n)
    pool = np.full(pages * rpp * 68, 0x5A, np.uint8)
    orc.store_rows_fp4(rows, pool, table, rpp, 0)
    back = orc.load_rows_fp4(pool, table, rpp, 128, 0, n)
    fake = rows.copy()
    orc.fake_quant_fp4(fake, 128, 32)
    assert np.array_equal(back, fake)
    # layout: code row r of page p at p*4352 + r*64, scale row at p*4352 + 4096 + r*4 (src/kernels/indexer.hpp:20-28)
    r = 3 * rpp + 5
    p = int(table[3])
    q, _ = None, None
    blk = rows[r, :32]
    amax = max(float(np.abs(orc.bf16_bits_to_f32(blk)).max()), 6.0 * 2.0 ** -126)
    se = int(np.ceil(np.log2(np.float32(amax) * np.float32(1.0 / 6.0)))) + 127
    assert pool[p * 4352 + 4096 + 5 * 4] == se
    untouched = np.ones(pages * rpp, bool)
    untouched[[int(table[i // rpp]) * rpp + i % rpp for i in range(n)]] = False
    codes = pool.reshape(pages, 4352)[:, :4096].reshape(pages * rpp, 64)
    assert (codes[untouched] == 0x5A).all()


def test_paged_addressing_and_gather_masking():
    g = tl.rng(11)
    case = tl.PagedCase(seed=1)
    pool = case.oracle_append()
    # direct numpy statement of the addressing rule
    for s in range(case.nseq):
        r = int(case.lens[s])
        phys = int(case.tables[s, r // 64]) * 64 + r % 64
        assert np.array_equal(pool[phys, :576], case.rows[s])
    changed = np.flatnonzero((pool != case.pool).any(axis=1))
    assert len(changed) <= case.nseq
    out = case.oracle_gather(pool)
    for s in (0, 3, 7):
        for e in (0, 1, 1000, 2047):
            r = int(case.idx[s, e])
            if r < 0:
                assert not out[s, e].any()
            else:
                assert np.array_equal(out[s, e], pool[int(case.tables[s, r // 64]) * 64 + r % 64, :576])
    # masking by visibility: entries >= visible read as zeros
    vis = case.q_visible.copy()
    vis[0] = 10
    out2 = orc.gather_rows(pool, case.tables, 64, 576, 576, case.idx, case.q_slot, vis)
    assert not out2[0][case.idx[0] >= 10].any()
    assert np.array_equal(out2[1:], out[1:])
    # threads do not change the result
    out3 = orc.gather_rows(pool, case.tables, 64, 576, 576, case.idx, case.q_slot, case.q_visible, threads=4)
    assert np.array_equal(out3, out)
