"""Parity of the CUDA kernels with the CPU oracle, bit for bit, through the C ABI.

The shapes follow the reference's own kernel tests: shuffled block tables (tools/kernel_test/indexer.hip:66-69,
tools/kernel_test/attn.hip:70-121), key rows with per-row magnitudes over several octaves (indexer.hip:57-60), the
fp4 store -> load round trip equal to fake_quant_fp4 (indexer.hip:82-95), poison-filled outputs (indexer.hip:130)."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi

pytestmark = pytest.mark.gpu


def special_values(g, n, dim):
    """bf16 rows full of rounding edge cases: exact ties of both grids at several scales, zeros of both signs,
    subnormals, the largest finite values."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 7.0, 448.0, 480.0, 416.0,
                     0.001953125, 0.0009765625, 0.0029296875, 17.0, 19.0, 0.0], np.float32)
    x = g.choice(ties, size=(n, dim)).astype(np.float32)
    x *= np.ldexp(np.float32(1.0), g.integers(-20, 20, size=(n, 1))).astype(np.float32)
    x *= g.choice(np.array([-1.0, 1.0], np.float32), size=(n, dim))
    b = orc.f32_to_bf16_bits(x)
    b[0, :] = 0                      # all +0: amax floor
    b[1, :] = 0x8000                 # all -0
    b[2, :] = 0x0001                 # smallest subnormal
    b[3, :] = 0x7F7F                 # largest finite
    b[4, ::2] = 0xFF7F               # mixed signs of the largest
    b[5, :] = g.integers(0, 0x7F80, size=dim).astype(np.uint16)  # any positive finite pattern
    b[6, :] = (g.integers(0, 0x7F80, size=dim) | 0x8000).astype(np.uint16)
    return b


def shuffled_table(g, pages):
    return g.permutation(pages).astype(np.int32)


@pytest.mark.parametrize("width,stride,n,row0", [(576, 576, 300, 37), (576, 640, 129, 0), (512, 512, 64, 63),
                                                 (100, 104, 70, 5), (7, 9, 33, 1), (576, 576, 1, 200)])
def test_store_rows(pkv, cuda, width, stride, n, row0):
    g = tl.rng(11)
    rpp, pages = 64, 8
    table = shuffled_table(g, pages)
    rows = tl.normal_bf16(g, (n, width))
    pool0 = np.full((pages * rpp, stride), 0x5A5A, np.uint16)
    want = pool0.copy()
    orc.store_rows(rows, want, table, rpp, stride, row0)
    d_rows, d_pool, d_table = tl.dev(cuda, rows), tl.dev(cuda, pool0), tl.dev(cuda, table)
    capi.check(pkv.pkv_store_rows(d_rows.data_ptr(), n, width, d_pool.data_ptr(), d_table.data_ptr(), rpp, stride, row0,
                                  tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    got = tl.host(d_pool, np.uint16, want.shape)
    assert np.array_equal(got, want)
    assert tl.device_status(pkv) == 0


def test_store_rows_empty_and_bad_args(pkv, cuda):
    assert pkv.pkv_store_rows(None, 0, 576, None, None, 64, 576, 0, None) == capi.PKV_OK
    d = cuda.zeros(64, dtype=cuda.uint8, device="cuda")
    assert pkv.pkv_store_rows(d.data_ptr(), 1, 576, d.data_ptr(), d.data_ptr(), 64, 100, 0, None) == capi.PKV_ERR_ARG
    assert b"bad shape" in pkv.pkv_last_error()
    assert pkv.pkv_act_quant_fp8(d.data_ptr(), 128, d.data_ptr(), d.data_ptr(), 1, 128, 48, None) == capi.PKV_ERR_ARG


@pytest.mark.parametrize("kind", ["normal", "special"])
def test_store_rows_fp4_and_round_trip(pkv, cuda, kind):
    g = tl.rng(12)
    rpp, pages, n, row0 = 64, 12, 700, 19
    table = shuffled_table(g, pages)
    rows = tl.key_rows(g, n) if kind == "normal" else special_values(g, n, 128)
    pool0 = np.full(pages * rpp * 68, 0x5A, np.uint8)
    want = pool0.copy()
    orc.store_rows_fp4(rows, want, table, rpp, row0)
    d_rows, d_pool, d_table = tl.dev(cuda, rows), tl.dev(cuda, pool0), tl.dev(cuda, table)
    st = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_store_rows_fp4(d_rows.data_ptr(), n, d_pool.data_ptr(), d_table.data_ptr(), rpp, row0, st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_pool, np.uint8), want)
    # round trip: decoded rows == fake_quant_fp4 of the inputs (tools/kernel_test/indexer.hip:82-95), on the GPU ...
    d_back = cuda.empty(n * 128 * 2, dtype=cuda.uint8, device="cuda")
    capi.check(pkv.pkv_load_rows_fp4(d_pool.data_ptr(), d_table.data_ptr(), rpp, row0, n, d_back.data_ptr(), st))
    capi.check(pkv.pkv_fake_quant_fp4(d_rows.data_ptr(), 128, n, 128, 32, st))
    cuda.cuda.synchronize()
    back, fake = tl.host(d_back, np.uint16, (n, 128)), tl.host(d_rows, np.uint16, (n, 128))
    assert np.array_equal(back, fake)
    # ... and both equal the oracle's
    want_back = orc.load_rows_fp4(want, table, rpp, 128, row0, n)
    want_fake = rows.copy()
    orc.fake_quant_fp4(want_fake, 128, 32)
    assert np.array_equal(back, want_back)
    assert np.array_equal(fake, want_fake)


@pytest.mark.parametrize("block", [32, 64, 128])
@pytest.mark.parametrize("kind", ["normal", "outliers", "special"])
def test_act_quant_fp8(pkv, cuda, block, kind):
    g = tl.rng(13 + block)
    rows, cols, ldx = 257, 512, 520
    x = np.zeros((rows, ldx), np.uint16)
    x[:, :cols] = {"normal": lambda: tl.normal_bf16(g, (rows, cols)), "outliers": lambda: tl.outlier_rows(g, rows, cols),
                   "special": lambda: special_values(g, rows, cols)}[kind]()
    x[:, cols:] = 0x1234
    wq, ws = orc.act_quant_fp8(x, cols, block)
    d_x = tl.dev(cuda, x)
    d_q = cuda.full((rows * cols,), 0x5A, dtype=cuda.uint8, device="cuda")
    d_s = cuda.full((rows * (cols // block),), 0x5A, dtype=cuda.uint8, device="cuda")
    st = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_act_quant_fp8(d_x.data_ptr(), ldx, d_q.data_ptr(), d_s.data_ptr(), rows, cols, block, st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_q, np.uint8, wq.shape), wq)
    assert np.array_equal(tl.host(d_s, np.uint8, ws.shape), ws)
    wf = x.copy()
    orc.fake_quant_fp8(wf, cols, block)
    capi.check(pkv.pkv_fake_quant_fp8(d_x.data_ptr(), ldx, rows, cols, block, st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_x, np.uint16, wf.shape), wf)


def test_fake_quant_unaligned(pkv, cuda):
    """ldx not a multiple of 8 and a base pointer off the 16-byte grid take the scalar load path."""
    g = tl.rng(14)
    rows, cols, ldx = 33, 64, 67
    x = tl.normal_bf16(g, (rows, ldx))
    for fn, ofn, block in ((pkv.pkv_fake_quant_fp8, orc.fake_quant_fp8, 64), (pkv.pkv_fake_quant_fp4, orc.fake_quant_fp4, 32)):
        want = x.copy()
        ofn(want, cols, block)
        buf = cuda.zeros(x.nbytes + 16, dtype=cuda.uint8, device="cuda")
        buf[2:2 + x.nbytes] = tl.dev(cuda, x)
        capi.check(fn(buf.data_ptr() + 2, ldx, rows, cols, block, tl.stream_ptr(cuda)))
        cuda.cuda.synchronize()
        assert np.array_equal(tl.host(buf[2:2 + x.nbytes].contiguous(), np.uint16, x.shape), want)


@pytest.mark.parametrize("width,block,rpp", [(512, 64, 256), (128, 64, 64), (128, 128, 64), (128, 32, 64)])
def test_store_rows_fp8(pkv, cuda, width, block, rpp):
    g = tl.rng(15)
    pages, n, s0 = 6, 3 * rpp + 17, rpp - 5
    table = shuffled_table(g, pages)
    rows = tl.outlier_rows(g, n, width)
    codes0 = np.full((pages * rpp, width), 0x5A, np.uint8)
    scales0 = np.full((pages * rpp, width // block), 0x5A, np.uint8)
    wc, ws = codes0.copy(), scales0.copy()
    orc.store_rows_fp8(rows, block, wc, ws, table, rpp, s0)
    d_rows, d_c, d_s, d_t = tl.dev(cuda, rows), tl.dev(cuda, codes0), tl.dev(cuda, scales0), tl.dev(cuda, table)
    capi.check(pkv.pkv_store_rows_fp8(d_rows.data_ptr(), n, width, block, d_c.data_ptr(), d_s.data_ptr(), d_t.data_ptr(),
                                      rpp, s0, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_c, np.uint8, wc.shape), wc)
    assert np.array_equal(tl.host(d_s, np.uint8, ws.shape), ws)


@pytest.mark.parametrize("nbytes,off", [(1 << 20, 0), (12345, 0), (4096, 3), (16, 0), (1, 0)])
def test_copy(pkv, cuda, nbytes, off):
    g = tl.rng(16)
    src = g.integers(0, 256, size=nbytes + 32, dtype=np.uint8)
    d_src = tl.dev(cuda, src)
    d_dst = cuda.full((nbytes + 32,), 0x5A, dtype=cuda.uint8, device="cuda")
    capi.check(pkv.pkv_copy(d_dst.data_ptr() + off, d_src.data_ptr() + off, nbytes, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    got = tl.host(d_dst, np.uint8)
    assert np.array_equal(got[off:off + nbytes], src[off:off + nbytes])
    assert (got[:off] == 0x5A).all() and (got[off + nbytes:] == 0x5A).all()


def test_gather_rows_single_table(pkv, cuda):
    """One sequence, one block-table row: the shape of one reference attention call (tools/kernel_test/attn.hip:70-121)."""
    g = tl.rng(17)
    rpp, pages, width, T, k = 64, 40, 576, 5, 512
    nrows = pages * rpp
    table = shuffled_table(g, pages)
    pool = tl.normal_bf16(g, (nrows, width))
    visible = np.array([nrows, nrows - 100, 600, 1, 0], np.int32)
    idx = np.full((T, k), -1, np.int32)
    for t in range(T):
        m = min(k - 7 * t, max(int(visible[t]), 1))
        idx[t, :m] = g.choice(nrows, size=m, replace=False)  # unsorted, some beyond `visible`: masked
    want = orc.gather_rows(pool, table.reshape(1, -1), rpp, width, width, idx, np.zeros(T, np.int32), visible)
    d_pool, d_table, d_idx, d_vis = tl.dev(cuda, pool), tl.dev(cuda, table), tl.dev(cuda, idx), tl.dev(cuda, visible)
    d_out = cuda.full((T * k * width * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    capi.check(pkv.pkv_gather_rows(d_pool.data_ptr(), d_table.data_ptr(), rpp, width, width, d_idx.data_ptr(),
                                   d_vis.data_ptr(), T, k, d_out.data_ptr(), tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


# The bulk variant has two kernels (a single-warp pipeline and a warp-specialised one, chosen by launch shape): the tests
# force each in turn through pkv_tune knob 8, encoded here as two extra bits on the variant flag.
BULK_SINGLE_WARP = capi.PKV_VARIANT_BULK | (1 << 20)
BULK_SPECIALISED = capi.PKV_VARIANT_BULK | (1 << 21)
VARIANTS = pytest.mark.parametrize("variant", [0, BULK_SINGLE_WARP, BULK_SPECIALISED], ids=["vec", "bulk-single-warp", "bulk-specialised"])


def launch_step(pkv, step, layers, L, flags, stream):
    pipe = 0 if flags & (1 << 20) else 1 if flags & (1 << 21) else -1
    capi.check(pkv.pkv_tune(8, pipe))
    try:
        capi.check(pkv.pkv_step_run(C.byref(step), layers, L, flags & ~(3 << 20), stream))
    finally:
        capi.check(pkv.pkv_tune(8, -1))


def run_step(pkv, cuda, case, L, flags, fp8_block=64, poison=True):
    """Runs pkv_step_run over L layers that share the case's tables but own their pools, rows, keys and index lists
    (layer l's inputs are the case's rotated by l). Returns per-layer device results as numpy arrays."""
    d_tables, d_chunks = tl.dev(cuda, case.tables), tl.dev(cuda, case.chunks)
    d_qchunk, d_qvis = tl.dev(cuda, case.q_chunk), tl.dev(cuda, case.q_visible)
    step = tl.make_step(case, d_tables, d_chunks, d_qchunk, d_qvis, fp8_block=fp8_block)
    layers = tl.make_layers(L)
    keep, per_layer = [d_tables, d_chunks, d_qchunk, d_qvis], []
    nrows = case.num_pages * case.rpp
    for l in range(L):
        inp = {
            "pool": np.roll(case.pool, l, axis=0), "rows": np.roll(case.rows, l, axis=1),
            "keys": np.roll(case.keys, l, axis=1), "idx": case.idx,
        }
        d = {k: tl.dev(cuda, v) for k, v in inp.items()}
        d["fp4"] = cuda.full((case.num_pages * case.rpp * 68,), 0x5A, dtype=cuda.uint8, device="cuda")
        d["codes"] = cuda.full((nrows * 128,), 0x5A, dtype=cuda.uint8, device="cuda")
        d["scales"] = cuda.full((nrows * (128 // fp8_block),), 0x5A, dtype=cuda.uint8, device="cuda")
        d["out"] = cuda.full((case.idx.shape[0] * case.k * case.width * 2,), 0x5A if poison else 0, dtype=cuda.uint8, device="cuda")
        y = layers[l]
        y.rows, y.row_pool, y.keys = d["rows"].data_ptr(), d["pool"].data_ptr(), d["keys"].data_ptr()
        y.key_pool_fp4, y.key_fp8_codes, y.key_fp8_scales = d["fp4"].data_ptr(), d["codes"].data_ptr(), d["scales"].data_ptr()
        y.idx, y.gathered = d["idx"].data_ptr(), d["out"].data_ptr()
        keep.append(d)
        per_layer.append((inp, d))
    launch_step(pkv, step, layers, L, flags, tl.stream_ptr(cuda))
    cuda.cuda.synchronize()
    assert tl.device_status(pkv) == 0
    return per_layer


def check_step(case, per_layer, flags, fp8_block=64):
    nrows = case.num_pages * case.rpp
    for inp, d in per_layer:
        pool = inp["pool"].copy()
        if flags & capi.PKV_DO_ROWS:
            orc.store_rows_chunks(inp["rows"], pool, case.tables, case.rpp, case.row_stride, case.chunks)
        assert np.array_equal(tl.host(d["pool"], np.uint16, pool.shape), pool), "row pool"
        if flags & capi.PKV_DO_KEYS_FP4:
            fp4 = np.full(case.num_pages * case.rpp * 68, 0x5A, np.uint8)
            orc.store_rows_fp4_chunks(inp["keys"], fp4, case.tables, case.rpp, case.chunks)
            assert np.array_equal(tl.host(d["fp4"], np.uint8), fp4), "fp4 key pool"
        if flags & capi.PKV_DO_KEYS_FP8:
            codes = np.full((nrows, 128), 0x5A, np.uint8)
            scales = np.full((nrows, 128 // fp8_block), 0x5A, np.uint8)
            orc.store_rows_fp8_chunks(inp["keys"], fp8_block, codes, scales, case.tables, case.rpp, case.chunks)
            assert np.array_equal(tl.host(d["codes"], np.uint8, codes.shape), codes), "fp8 codes"
            assert np.array_equal(tl.host(d["scales"], np.uint8, scales.shape), scales), "fp8 scales"
        if flags & capi.PKV_DO_GATHER:
            want = orc.gather_rows(pool, case.tables, case.rpp, case.row_stride, case.width, inp["idx"], case.q_slot,
                                   case.q_visible)
            got = tl.host(d["out"], np.uint16, want.shape)
            assert np.array_equal(got, want), "gathered rows"


ALL = capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4 | capi.PKV_DO_KEYS_FP8 | capi.PKV_DO_GATHER


@VARIANTS
def test_step_config1(pkv, cuda, variant):
    """Benchmark configuration 1: 8 sequences of 1024..8192 rows over a 1024-page pool, one appended row each, then a
    2048-entry gather per sequence (-1 padded), all in one launch; every byte against the oracle."""
    case = tl.PagedCase(seed=1)
    check_step(case, run_step(pkv, cuda, case, 1, ALL | variant), ALL)


@VARIANTS
def test_step_layers_and_prefill_chunks(pkv, cuda, variant):
    """Several layers in one launch, chunks of different lengths (decode rows and prefill chunks that cross pages),
    a row stride wider than the row, index lists that include the rows being appended."""
    case = tl.PagedCase(seed=2, nseq=5, len_lo=300, len_hi=900, num_pages=96, k=160, row_stride=640, append=1)
    g = tl.rng(22)
    ns = [1, 37, 128, 211, 1]  # the chunk sizes of tools/batch_test/main.hip:124-192
    t0 = np.concatenate([[0], np.cumsum(ns)[:-1]])
    case.chunks = np.array([[s, int(case.lens[s]) - ns[s] + 1, ns[s], int(t0[s])] for s in range(5)], np.int32)
    case.T = int(sum(ns))
    case.rows, case.keys = tl.normal_bf16(g, (case.T, case.width)), tl.key_rows(g, case.T)
    for fp8_block in (32, 128):
        check_step(case, run_step(pkv, cuda, case, 3, ALL | variant, fp8_block), ALL, fp8_block)


@VARIANTS
def test_gather_only_and_append_only(pkv, cuda, variant):
    case = tl.PagedCase(seed=3, nseq=4, len_lo=64, len_hi=700, num_pages=64, k=96)
    check_step(case, run_step(pkv, cuda, case, 2, capi.PKV_DO_GATHER | variant), capi.PKV_DO_GATHER)
    check_step(case, run_step(pkv, cuda, case, 2, capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4 | variant),
               capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4)


@VARIANTS
def test_gather_ragged_k(pkv, cuda, variant):
    """k that is not a multiple of the tile, fully masked queries, a query with nothing visible."""
    case = tl.PagedCase(seed=4, nseq=3, len_lo=10, len_hi=90, num_pages=16, k=77)
    case.q_visible[1] = 0
    case.idx[2, :] = -1
    check_step(case, run_step(pkv, cuda, case, 1, capi.PKV_DO_GATHER | variant), capi.PKV_DO_GATHER)


def test_bad_page_id_is_reported_not_dereferenced(pkv, cuda):
    """A block-table entry outside the pool is skipped and recorded in the status word; the launch completes."""
    case = tl.PagedCase(seed=5, nseq=2, len_lo=64, len_hi=128, num_pages=8, k=32)
    case.tables[1, 0] = 1 << 20
    d_tables, d_chunks = tl.dev(cuda, case.tables), tl.dev(cuda, case.chunks)
    d_qchunk, d_qvis = tl.dev(cuda, case.q_chunk), tl.dev(cuda, case.q_visible)
    step = tl.make_step(case, d_tables, d_chunks, d_qchunk, d_qvis)
    layers = tl.make_layers(1)
    d_pool, d_idx = tl.dev(cuda, case.pool), tl.dev(cuda, case.idx)
    d_out = cuda.zeros(2 * 32 * 576 * 2, dtype=cuda.uint8, device="cuda")
    layers[0].row_pool, layers[0].idx, layers[0].gathered = d_pool.data_ptr(), d_idx.data_ptr(), d_out.data_ptr()
    capi.check(pkv.pkv_step_run(C.byref(step), layers, 1, capi.PKV_DO_GATHER, tl.stream_ptr(cuda)))
    status = tl.device_status(pkv)
    assert status & 0xFF == 1
    assert tl.device_status(pkv) == 0  # reading clears it


def test_bounded_wait_gives_up_and_the_library_keeps_working(pkv, cuda):
    """The only device-side waits are mbarrier waits with a poll limit. Made to run out WITHOUT anything going wrong on
    the GPU: the test hook (pkv_tune knob 10) makes CTA 0 of the warp-specialised kernel expect 16 bytes more than its
    first tile brings, and knob 9 shortens the limit to a few milliseconds. The kernel must return, the status word
    must say "bounded wait gave up" (kind 3), pkv_stream_check must return PKV_ERR_DEVICE, and the next launch must
    produce exact results again."""
    case = tl.PagedCase(seed=8, nseq=4, len_lo=200, len_hi=900, num_pages=128, k=256)
    flags = capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4 | capi.PKV_DO_GATHER
    try:
        capi.check(pkv.pkv_tune(9, 4000))     # polls of at most a microsecond each
        capi.check(pkv.pkv_tune(10, 0))       # CTA 0, its first tile
        run = lambda: run_step(pkv, cuda, case, 1, flags | BULK_SPECIALISED)
        with pytest.raises(AssertionError):   # run_step asserts a clean status word
            run()
    finally:
        capi.check(pkv.pkv_tune(10, -1))
        capi.check(pkv.pkv_tune(9, 0))
    assert tl.device_status(pkv) == 0         # ... which run_step's own status read has cleared
    # the same again in the steady-state loop of a CTA with several tiles, read through the stream-ordered check
    case = tl.PagedCase(seed=9, nseq=4, len_lo=2100, len_hi=4000, num_pages=512, k=2048)
    d_tables, d_chunks = tl.dev(cuda, case.tables), tl.dev(cuda, case.chunks)
    d_qchunk, d_qvis = tl.dev(cuda, case.q_chunk), tl.dev(cuda, case.q_visible)
    step = tl.make_step(case, d_tables, d_chunks, d_qchunk, d_qvis)
    layers = tl.make_layers(1)
    d_pool, d_idx = tl.dev(cuda, case.pool), tl.dev(cuda, case.idx)
    d_out = cuda.zeros(case.idx.shape[0] * case.k * case.width * 2, dtype=cuda.uint8, device="cuda")
    layers[0].row_pool, layers[0].idx, layers[0].gathered = d_pool.data_ptr(), d_idx.data_ptr(), d_out.data_ptr()
    try:
        capi.check(pkv.pkv_tune(9, 4000))
        capi.check(pkv.pkv_tune(10, 2))       # CTA 0's third tile
        capi.check(pkv.pkv_tune(1, 2))        # two CTAs per SM: 1024 tiles over 296 CTAs
        launch_step(pkv, step, layers, 1, capi.PKV_DO_GATHER | BULK_SPECIALISED, tl.stream_ptr(cuda))
        assert pkv.pkv_stream_check(tl.stream_ptr(cuda)) == capi.PKV_ERR_DEVICE
        assert b"bounded wait gave up" in pkv.pkv_last_error()
    finally:
        capi.check(pkv.pkv_tune(10, -1))
        capi.check(pkv.pkv_tune(9, 0))
        capi.check(pkv.pkv_tune(1, 0))
    assert pkv.pkv_stream_check(tl.stream_ptr(cuda)) == capi.PKV_OK
    check_step(case, run_step(pkv, cuda, case, 1, flags | BULK_SPECIALISED), flags)   # the context is intact


def test_copy_pages(pkv, cuda):
    g = tl.rng(18)
    pages, n = 64, 20
    pools = [g.integers(0, 65536, size=(pages, tl.PAGE_BYTES // 2), dtype=np.uint16),
             g.integers(0, 256, size=(pages, tl.FP4_PAGE_BYTES), dtype=np.uint8)]
    perm = g.permutation(pages).astype(np.int32)
    src, dst = perm[:n].copy(), perm[n:2 * n].copy()
    want = [p.copy() for p in pools]
    orc.copy_pages(want[0], tl.PAGE_BYTES, src, dst)
    orc.copy_pages(want[1], tl.FP4_PAGE_BYTES, src, dst)
    d_pools = [tl.dev(cuda, p) for p in pools]
    descs = (capi.PkvPoolDesc * 2)()
    for i, (d, pb) in enumerate(zip(d_pools, (tl.PAGE_BYTES, tl.FP4_PAGE_BYTES))):
        descs[i].src_base = descs[i].dst_base = d.data_ptr()
        descs[i].page_bytes = pb
    d_src, d_dst = tl.dev(cuda, src), tl.dev(cuda, dst)
    capi.check(pkv.pkv_copy_pages(descs, 2, d_src.data_ptr(), d_dst.data_ptr(), n, pages, pages, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_pools[0], np.uint16, want[0].shape), want[0])
    assert np.array_equal(tl.host(d_pools[1], np.uint8, want[1].shape), want[1])
    assert tl.device_status(pkv) == 0


def test_repeat_is_stable(pkv, cuda):
    """The reference's REPEAT=n race check (tools/kernel_test/indexer.hip:122-140): the same launch, poisoned outputs,
    identical bytes every time."""
    case = tl.PagedCase(seed=6, nseq=4, len_lo=500, len_hi=3000, num_pages=256, k=512)
    first = None
    for variant in (0, BULK_SINGLE_WARP, BULK_SPECIALISED):
        for _ in range(3):
            per_layer = run_step(pkv, cuda, case, 2, ALL | variant)
            sig = [tl.host(d[k], np.uint8).tobytes() for _, d in per_layer for k in ("pool", "fp4", "codes", "scales", "out")]
            if first is None:
                first = sig
            assert sig == first


@VARIANTS
def test_config3_chunked_prefill(pkv, cuda, variant):
    """Benchmark configuration 3, reduced: one sequence grows in chunks (the first short, then 4096 rows each) over
    freshly allocated non-contiguous pages; every chunk appends bf16 rows with 1 % outliers at +-20 and quantises its
    128-wide keys to BOTH fp8 e4m3 (two-array layout, block 64) and MXFP4; 8 query rows at the chunk's last 8 positions
    gather 2048 positions skewed toward recent tokens (cur - 1 - Geometric(1e-4), distinct, sorted; -1 padded while
    fewer exist). Pools persist across chunks on the device and in the oracle mirror; everything is compared after
    every chunk."""
    g = tl.rng(3)
    L, k, rpp, W = 2, 2048, tl.RPP, tl.W
    chunk_sizes = [1000, 4096, 4096, 4096]
    total = sum(chunk_sizes)
    pages = -(-total // rpp) + 7
    pps = pages
    perm = g.permutation(pages).astype(np.int32)
    tables = np.zeros((1, pps), np.int32)
    nrows = pages * rpp
    h_pool = [np.zeros((nrows, W), np.uint16) for _ in range(L)]
    h_fp4 = [np.zeros(pages * tl.FP4_PAGE_BYTES, np.uint8) for _ in range(L)]
    h_codes = [np.zeros((nrows, 128), np.uint8) for _ in range(L)]
    h_scales = [np.zeros((nrows, 2), np.uint8) for _ in range(L)]
    d_pool, d_fp4 = [tl.dev(cuda, a) for a in h_pool], [tl.dev(cuda, a) for a in h_fp4]
    d_codes, d_scales = [tl.dev(cuda, a) for a in h_codes], [tl.dev(cuda, a) for a in h_scales]
    s0 = 0
    for n in chunk_sizes:
        end = s0 + n
        have = -(-end // rpp)
        tables[0, :have] = perm[:have]                       # pages for the chunk are taken as it arrives
        chunks = np.array([[0, s0, n, 0]], np.int32)
        qpos = np.arange(end - 8, end, dtype=np.int32)
        q_visible = qpos + 1
        idx = np.full((8, k), -1, np.int32)
        for i, p in enumerate(qpos):
            want = min(k, int(p) + 1)
            chosen = set()
            while len(chosen) < want:
                cand = int(p) - (g.geometric(1e-4, size=2 * k) - 1)
                chosen.update(int(c) for c in cand[cand >= 0][: want - len(chosen)])
            idx[i, :want] = np.sort(np.fromiter(chosen, np.int32))
        d_tables, d_chunks = tl.dev(cuda, tables), tl.dev(cuda, chunks)
        d_qc, d_qv = tl.dev(cuda, np.zeros(8, np.int32)), tl.dev(cuda, q_visible)
        step = capi.PkvStep()
        step.width = step.row_stride = W
        step.rows_per_page, step.max_pages_per_seq, step.num_pages, step.fp8_block = rpp, pps, pages, 64
        step.nchunks, step.T, step.Q, step.k, step.max_slots = 1, n, 8, k, tables.shape[0]
        step.tables, step.chunks, step.q_chunk, step.q_visible = (d_tables.data_ptr(), d_chunks.data_ptr(),
                                                                  d_qc.data_ptr(), d_qv.data_ptr())
        layers = tl.make_layers(L)
        keep, outs, wants = [], [], []
        for l in range(L):
            rows, keys = tl.outlier_rows(g, n, W), tl.key_rows(g, n)
            d_r, d_k, d_i = tl.dev(cuda, rows), tl.dev(cuda, keys), tl.dev(cuda, idx)
            d_o = cuda.full((8 * k * W * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
            keep += [d_r, d_k, d_i]
            outs.append(d_o)
            y = layers[l]
            y.rows, y.row_pool, y.keys, y.key_pool_fp4 = d_r.data_ptr(), d_pool[l].data_ptr(), d_k.data_ptr(), d_fp4[l].data_ptr()
            y.key_fp8_codes, y.key_fp8_scales, y.idx, y.gathered = (d_codes[l].data_ptr(), d_scales[l].data_ptr(),
                                                                    d_i.data_ptr(), d_o.data_ptr())
            orc.store_rows_chunks(rows, h_pool[l], tables, rpp, W, chunks)
            orc.store_rows_fp4_chunks(keys, h_fp4[l], tables, rpp, chunks)
            orc.store_rows_fp8_chunks(keys, 64, h_codes[l], h_scales[l], tables, rpp, chunks)
            wants.append(orc.gather_rows(h_pool[l], tables, rpp, W, W, idx, np.zeros(8, np.int32), q_visible))
        launch_step(pkv, step, layers, L, ALL | variant, tl.stream_ptr(cuda))
        cuda.cuda.synchronize()
        assert tl.device_status(pkv) == 0
        for l in range(L):
            assert np.array_equal(tl.host(d_pool[l], np.uint16, h_pool[l].shape), h_pool[l]), ("rows", s0, l)
            assert np.array_equal(tl.host(d_fp4[l], np.uint8), h_fp4[l]), ("fp4", s0, l)
            assert np.array_equal(tl.host(d_codes[l], np.uint8, h_codes[l].shape), h_codes[l]), ("fp8 codes", s0, l)
            assert np.array_equal(tl.host(d_scales[l], np.uint8, h_scales[l].shape), h_scales[l]), ("fp8 scales", s0, l)
            assert np.array_equal(tl.host(outs[l], np.uint16, wants[l].shape), wants[l]), ("gather", s0, l)
        s0 = end


def test_full_size_decode_step_properties(pkv, cuda):
    """Benchmark configuration 2 at its full per-layer size (64 sequences x 131,072 rows, 131,072 pages of 73,728 B:
    a 9.7 GB row pool and a 0.57 GB MXFP4 key pool, block tables shuffled), one layer, checked through properties
    that do not need a CPU copy of the pool: every gathered row equals the pool row its block-table entry names (all
    64 x 2048 entries, torch indexing on the device as the checker), the appended rows landed in the last row of each
    sequence's last page, the stored MXFP4 keys decode to fake_quant_fp4 of the inputs (the reference's own round-trip
    property, tools/kernel_test/indexer.hip:82-95), and running the step again changes nothing."""
    torch = cuda
    free, _ = torch.cuda.mem_get_info()
    if free < 16 << 30:
        pytest.skip("needs 16 GB of free device memory")
    nseq, ctx, k, W, rpp = 64, 131072, 2048, tl.W, tl.RPP
    pps, pages = ctx // rpp, nseq * (ctx // rpp)
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    pool = torch.empty(pages * rpp * W, dtype=torch.bfloat16, device="cuda")
    pool.normal_(generator=g)
    fp4 = torch.zeros(pages * tl.FP4_PAGE_BYTES, dtype=torch.uint8, device="cuda")
    tables = torch.randperm(pages, generator=g, device="cuda").to(torch.int32).view(nseq, pps).contiguous()
    chunks = torch.tensor([[s, ctx - 1, 1, s] for s in range(nseq)], dtype=torch.int32, device="cuda")
    q_chunk = torch.arange(nseq, dtype=torch.int32, device="cuda")
    q_vis = torch.full((nseq,), ctx, dtype=torch.int32, device="cuda")
    rows = torch.randn(nseq, W, generator=g, device="cuda").to(torch.bfloat16)
    keys = (torch.randn(nseq, 128, generator=g, device="cuda") * 4).to(torch.bfloat16)
    idx = torch.rand(nseq, ctx, generator=g, device="cuda").topk(k, dim=1).indices.sort(dim=1).values.to(torch.int32)
    idx[:, -1] = ctx - 1                                   # every query also selects the row appended in this step
    idx[0, :7] = -1                                        # and a few masked entries
    out = torch.full((nseq, k, W), float("nan"), dtype=torch.bfloat16, device="cuda")
    step = capi.PkvStep()
    step.width = step.row_stride = W
    step.rows_per_page, step.max_pages_per_seq, step.num_pages, step.fp8_block = rpp, pps, pages, 64
    step.nchunks = step.T = step.Q = step.max_slots = nseq
    step.k = k
    step.tables, step.chunks, step.q_chunk, step.q_visible = (tables.data_ptr(), chunks.data_ptr(), q_chunk.data_ptr(),
                                                               q_vis.data_ptr())
    layers = tl.make_layers(1)
    y = layers[0]
    y.rows, y.row_pool, y.keys, y.key_pool_fp4 = rows.data_ptr(), pool.data_ptr(), keys.data_ptr(), fp4.data_ptr()
    y.idx, y.gathered = idx.data_ptr(), out.data_ptr()
    flags = capi.PKV_DO_ROWS | capi.PKV_DO_KEYS_FP4 | capi.PKV_DO_GATHER | capi.PKV_VARIANT_BULK
    results = []
    for _ in range(2):
        capi.check(pkv.pkv_step_run(C.byref(step), layers, 1, flags, tl.stream_ptr(cuda)))
        torch.cuda.synchronize()
        results.append(out.view(torch.int16).clone())
    assert tl.device_status(pkv) == 0
    assert torch.equal(results[0], results[1])                                  # idempotent
    pool2 = pool.view(-1, W)
    last = tables[:, pps - 1].long() * rpp + rpp - 1
    assert torch.equal(pool2[last].view(torch.int16), rows.view(torch.int16))   # appended rows landed
    pos = idx.long().clamp(min=0)
    phys = torch.gather(tables.long(), 1, pos // rpp) * rpp + pos % rpp
    want = pool2[phys.view(-1)].view(nseq, k, W).clone()
    want[idx < 0] = 0
    assert torch.equal(results[1], want.view(torch.int16))                      # every gathered row
    # MXFP4 keys: decode the appended key row of each sequence and compare with fake_quant_fp4 of the input
    back = torch.empty(nseq, 128, dtype=torch.bfloat16, device="cuda")
    for s in range(nseq):
        capi.check(pkv.pkv_load_rows_fp4(fp4.data_ptr(), tables[s].data_ptr(), rpp, ctx - 1, 1, back[s].data_ptr(),
                                         tl.stream_ptr(cuda)))
    fake = keys.clone()
    capi.check(pkv.pkv_fake_quant_fp4(fake.data_ptr(), 128, nseq, 128, 32, tl.stream_ptr(cuda)))
    torch.cuda.synchronize()
    assert torch.equal(back.view(torch.int16), fake.view(torch.int16))


@pytest.mark.parametrize("width,block,rpp,k", [(512, 64, 256, 2051), (128, 32, 64, 100), (256, 128, 64, 64), (384, 64, 64, 77),
                                            (2048, 128, 32, 33), (64, 32, 64, 1000)])
def test_gather_rows_fp8_dequant(pkv, cuda, width, block, rpp, k):
    """fp8 rows stored by pkv_store_rows_fp8, gathered and dequantised: equals the oracle's bf16(e4m3 * 2^scale) per
    entry, zero rows for masked entries; also equals fake_quant_fp8 of the original rows (store then gather-dequant is
    the reference's fake quantisation: src/kernels/glm_fast.hip:203-218 vs src/kernels/ref_elem.hip:18-41)."""
    g = tl.rng(19)
    pages, T = 5, 3
    n = pages * rpp - 3
    table = shuffled_table(g, pages)
    rows = tl.outlier_rows(g, n, width)
    codes = np.zeros((pages * rpp, width), np.uint8)
    scales = np.zeros((pages * rpp, width // block), np.uint8)
    orc.store_rows_fp8(rows, block, codes, scales, table, rpp, 0)
    vis = np.array([n, n // 2, 1], np.int32)
    idx = np.full((T, k), -1, np.int32)
    for t in range(T):
        m = min(k - 5, n)
        idx[t, :m] = g.choice(n, size=m, replace=m > n)
    want = orc.gather_rows_fp8(codes, scales, table, rpp, block, idx, vis)
    fake = rows.copy()
    orc.fake_quant_fp8(fake, width, block)
    sel = idx[0] >= 0
    assert np.array_equal(want[0][sel], fake[idx[0][sel]])
    d_rows, d_t, d_idx, d_vis = tl.dev(cuda, rows), tl.dev(cuda, table), tl.dev(cuda, idx), tl.dev(cuda, vis)
    d_c = cuda.zeros(codes.size, dtype=cuda.uint8, device="cuda")
    d_s = cuda.zeros(scales.size, dtype=cuda.uint8, device="cuda")
    d_out = cuda.full((want.size * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    st = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_store_rows_fp8(d_rows.data_ptr(), n, width, block, d_c.data_ptr(), d_s.data_ptr(), d_t.data_ptr(), rpp, 0, st))
    capi.check(pkv.pkv_gather_rows_fp8(d_c.data_ptr(), d_s.data_ptr(), d_t.data_ptr(), rpp, width, block, d_idx.data_ptr(),
                                       d_vis.data_ptr(), T, k, d_out.data_ptr(), st))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


def test_gather_rows_fp8_every_code_and_scale(pkv, cuda):
    """Every e4m3 bit pattern (zeros, subnormals, both NaN codes) under scales from 2^-127 to 2^127 and the NaN scale:
    results in bf16's subnormal range, overflow to infinity and NaN all equal the oracle's scalar arithmetic (scale
    byte 0 decodes to +0 and 255 to +inf, as the reference's e8m0_to_f32 does: src/kernels/dev.hip.hpp:96)."""
    g = tl.rng(29)
    width, block, rpp, pages, T, k = 512, 64, 256, 4, 2, 700
    n = pages * rpp
    table = shuffled_table(g, pages)
    codes = g.integers(0, 256, size=(n, width), dtype=np.uint8)
    codes[:256, :] = np.arange(256, dtype=np.uint8)[:, None]          # rows of one code each
    codes[256:300, :] &= 0x7E                                           # rows without any NaN code (the paired decode)
    mixed = g.integers(8, 0x7F, size=(60, width), dtype=np.uint8) | (g.integers(0, 2, size=(60, width), dtype=np.uint8) << 7)
    mixed[g.random((60, width)) < 0.2] &= 0x80                          # normal codes with +-0 sprinkled in, no subnormal:
    codes[300:360, :] = mixed                                           # the integer decode with masked zero lanes
    codes[360:364, :] = 0                                               # rows never written
    scales = g.choice(np.array([0, 1, 5, 100, 119, 120, 126, 127, 128, 140, 200, 246, 247, 254, 255], np.uint8),
                      size=(n, width // block))
    vis = np.array([n, n], np.int32)
    idx = np.stack([g.permutation(n)[:k], g.permutation(n)[:k]]).astype(np.int32)
    idx[0, :364] = np.arange(364)                                      # logical rows; the table scatters them
    phys_codes, phys_scales = np.zeros_like(codes), np.zeros_like(scales)
    for r in range(n):                                                 # logical row r lives at table[r // rpp] * rpp + r % rpp
        p = int(table[r // rpp]) * rpp + r % rpp
        phys_codes[p], phys_scales[p] = codes[r], scales[r]
    want = orc.gather_rows_fp8(phys_codes, phys_scales, table, rpp, block, idx, vis)
    d_c, d_s, d_t, d_idx, d_vis = (tl.dev(cuda, a) for a in (phys_codes, phys_scales, table, idx, vis))
    d_out = cuda.full((want.size * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    capi.check(pkv.pkv_gather_rows_fp8(d_c.data_ptr(), d_s.data_ptr(), d_t.data_ptr(), rpp, width, block, d_idx.data_ptr(),
                                       d_vis.data_ptr(), T, k, d_out.data_ptr(), tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    got = tl.host(d_out, np.uint16, want.shape)
    def is_nan(a):
        return ((a & 0x7F80) == 0x7F80) & ((a & 0x7F) != 0)
    # NaN results (a NaN code, or 0 x inf under the scale byte 255) must be NaN; their payload is the processor's
    bad = np.argwhere((got != want) & ~(is_nan(got) & is_nan(want)))
    examples = [(int(codes[idx[t, e], c]), int(scales[idx[t, e], c // block]), hex(int(got[t, e, c])), hex(int(want[t, e, c])))
                for t, e, c in bad[:12]]
    assert len(bad) == 0, f"{len(bad)} values differ; (code, scale, got, want): {examples}"


def test_step_gather_fp8_all_sequences_in_one_launch(pkv, cuda):
    """pkv_step_gather_fp8: every sequence of a step gathers from its own block table in one launch; per query row the
    result equals the single-sequence oracle gather with that sequence's table (GLM geometry: 256 rows per page, 512
    codes + 8 scales per row, 2051 entries)."""
    g = tl.rng(31)
    width, block, rpp, k = 512, 64, 256, 2051
    case = tl.PagedCase(seed=31, nseq=6, len_lo=300, len_hi=5000, num_pages=160, k=k, width=width, rows_per_page=rpp,
                        with_keys=False, fill=False)
    nrows = case.num_pages * rpp
    codes = g.integers(0, 256, size=(nrows, width), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3A
    scales = g.integers(118, 136, size=(nrows, width // block), dtype=np.uint8)
    idx = case.idx.copy()
    idx[2, 5] = int(case.q_visible[2]) + 3                     # past the visible rows: a zero row
    want = np.stack([orc.gather_rows_fp8(codes, scales, case.tables[s], rpp, block, idx[s:s + 1], case.q_visible[s:s + 1])[0]
                     for s in range(case.nseq)])
    d = {n: tl.dev(cuda, a) for n, a in dict(codes=codes, scales=scales, tables=case.tables, chunks=case.chunks,
                                              q_chunk=case.q_chunk, q_vis=case.q_visible, idx=idx).items()}
    d_out = cuda.full((want.size * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    step = tl.make_step(case, d["tables"], d["chunks"], d["q_chunk"], d["q_vis"])
    capi.check(pkv.pkv_step_gather_fp8(C.byref(step), d["codes"].data_ptr(), d["scales"].data_ptr(), width, block,
                                       d["idx"].data_ptr(), d_out.data_ptr(), tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert tl.device_status(pkv) == 0
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


def test_step_gather_fp8_from_pool_lists(pkv, cuda):
    """pkv_step_gather_fp8_pools: the selected pools and the positions go in, the expansion happens during address
    resolution; equals the oracle's idx_expand followed by its fp8 gather, per sequence."""
    g = tl.rng(32)
    width, block, rpp, kp, pool = 512, 64, 256, 37, 4
    k = kp * pool + pool - 1
    case = tl.PagedCase(seed=32, nseq=5, len_lo=40, len_hi=4000, num_pages=120, k=k, width=width, rows_per_page=rpp,
                        with_keys=False, fill=False)
    nrows = case.num_pages * rpp
    codes = g.integers(0, 256, size=(nrows, width), dtype=np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3A
    scales = g.integers(118, 136, size=(nrows, width // block), dtype=np.uint8)
    pos = (case.q_visible - 1).astype(np.int32)                    # each query sits at its sequence's last row
    pos[0] = 2                                                     # fewer rows than one pool: only the tail entries
    pools = np.full((case.nseq, kp), -1, np.int32)
    for s in range(case.nseq):
        full = (int(pos[s]) + 1) // pool
        m = min(full, kp)
        pools[s, :m] = g.choice(full, size=m, replace=False)
    vis = (pos + 1).astype(np.int32)
    idx = orc.idx_expand(pools, pos, pool)
    assert idx.shape == (case.nseq, k)
    want = np.stack([orc.gather_rows_fp8(codes, scales, case.tables[s], rpp, block, idx[s:s + 1], vis[s:s + 1])[0]
                     for s in range(case.nseq)])
    d = {n: tl.dev(cuda, a) for n, a in dict(codes=codes, scales=scales, tables=case.tables, chunks=case.chunks,
                                              q_chunk=case.q_chunk, q_vis=vis, pools=pools, pos=pos).items()}
    d_out = cuda.full((want.size * 2,), 0x5A, dtype=cuda.uint8, device="cuda")
    step = tl.make_step(case, d["tables"], d["chunks"], d["q_chunk"], d["q_vis"])
    capi.check(pkv.pkv_step_gather_fp8_pools(C.byref(step), d["codes"].data_ptr(), d["scales"].data_ptr(), width, block,
                                             d["pools"].data_ptr(), d["pos"].data_ptr(), kp, pool, d_out.data_ptr(),
                                             tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert tl.device_status(pkv) == 0
    assert np.array_equal(tl.host(d_out, np.uint16, want.shape), want)


@pytest.mark.parametrize("width,quant_cols,block,stride", [(576, 512, 64, 576), (576, 512, 64, 640), (512, 512, 128, 512),
                                                           (128, 64, 32, 128)])
def test_store_rows_fake_fp8_one_pass(pkv, cuda, width, quant_cols, block, stride):
    """pkv_store_rows_fake_fp8 equals the reference's pair fake_quant_fp8 (first quant_cols columns) then store_rows
    (src/model/forward_ref.hip:739-741); the caller's rows stay as they were."""
    g = tl.rng(33)
    rpp, pages, row0 = 64, 7, 37
    n = pages * rpp - row0 - 5
    table = shuffled_table(g, pages)
    rows = tl.outlier_rows(g, n, width)
    pool = tl.normal_bf16(g, (pages * rpp, stride))
    want = pool.copy()
    fake = rows.copy()
    orc.fake_quant_fp8(fake, quant_cols, block)
    orc.store_rows(fake, want, table, rpp, stride, row0)
    d_rows, d_pool, d_t = tl.dev(cuda, rows), tl.dev(cuda, pool), tl.dev(cuda, table)
    capi.check(pkv.pkv_store_rows_fake_fp8(d_rows.data_ptr(), n, width, quant_cols, block, d_pool.data_ptr(), d_t.data_ptr(),
                                           rpp, stride, row0, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d_pool, np.uint16, want.shape), want)
    assert np.array_equal(tl.host(d_rows, np.uint16, rows.shape), rows)


def test_copy_between_device_and_pinned_host(pkv, cuda):
    """The snapshot save / restore primitive: the reference's state_copies moves slot state between device memory and
    pinned host staging with copy_kernel, i.e. with ordinary loads and stores issued by SMs
    (src/engine/resident.hip:545-557, src/kernels/ref.hpp:87-90). Same here: device -> pinned host -> device."""
    torch = cuda
    g = tl.rng(20)
    n = (7 << 20) + 4096
    src = g.integers(0, 256, size=n, dtype=np.uint8)
    d_src = tl.dev(cuda, src)
    h_snap = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_snap.fill_(0x5A)
    d_back = torch.full((n,), 0xA5, dtype=torch.uint8, device="cuda")
    st = tl.stream_ptr(cuda)
    capi.check(pkv.pkv_copy(h_snap.data_ptr(), d_src.data_ptr(), n, st))       # save
    capi.check(pkv.pkv_copy(d_back.data_ptr(), h_snap.data_ptr(), n, st))      # restore (stream-ordered after the save)
    torch.cuda.synchronize()
    assert np.array_equal(h_snap.numpy(), src)
    assert np.array_equal(d_back.cpu().numpy(), src)
