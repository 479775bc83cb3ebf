"""hadamard128 (src/kernels/ref.hpp:63, src/kernels/ref_elem.hip:111-135) and its fusion into the key append
(PKV_KEYS_HADAMARD: the reference's hadamard128 + store_rows_fp4 pair, src/model/forward_ref.hip:736-738). The oracle is
checked against an independent numpy statement of the butterflies (same operands per result, fp32) and, loosely,
against the Sylvester matrix; the CUDA paths against the oracle bit for bit."""
import ctypes as C

import numpy as np
import pytest

import pkv_testlib as tl
from oracle import oracle_lib as orc
from unholy_b200 import capi


def numpy_hadamard128(bits):
    b = (bits.astype(np.uint32) << 16).view(np.float32).reshape(-1, 128).copy()
    h = 1
    while h < 128:
        v = b.reshape(-1, 128 // (2 * h), 2, h)
        lo, hi = v[:, :, 0, :].copy(), v[:, :, 1, :].copy()
        v[:, :, 0, :] = lo + hi
        v[:, :, 1, :] = lo - hi
        h *= 2
    return orc.f32_to_bf16_bits((b * np.float32(0.08838834764831845)).astype(np.float32)).reshape(bits.shape)


def test_oracle_hadamard_matches_butterflies_and_matrix():
    g = tl.rng(95)
    x = tl.normal_bf16(g, (37, 128))
    x[0] = 0
    x[1, 5] = 0x7F80                                   # +inf spreads as inf / NaN the same way in both
    got = orc.hadamard128(x.copy())
    assert np.array_equal(got[2:], numpy_hadamard128(x)[2:])
    assert np.array_equal(got[0], np.zeros(128, np.uint16))
    H = np.array([[1.0]])
    while H.shape[0] < 128:
        H = np.block([[H, H], [H, -H]])
    xf = (x[2:].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    want = xf @ H.T / np.sqrt(128.0)
    gf = (got[2:].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.allclose(gf, want, rtol=1e-2, atol=1e-2)   # bf16 output: 8 bits of mantissa


@pytest.mark.gpu
@pytest.mark.parametrize("nseg", [1, 2, 3, 1000, 4097])
def test_hadamard128_gpu(pkv, cuda, nseg):
    g = tl.rng(96)
    x = tl.normal_bf16(g, (nseg, 128))
    want = orc.hadamard128(x.copy())
    d = tl.dev(cuda, x)
    capi.check(pkv.pkv_hadamard128(d.data_ptr(), nseg, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert np.array_equal(tl.host(d, np.uint16, x.shape), want)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [0, capi.PKV_VARIANT_BULK])
@pytest.mark.parametrize("append", [1, 37])
def test_step_keys_rotated_in_the_append(pkv, cuda, variant, append):
    """pkv_step_run with PKV_KEYS_HADAMARD: MXFP4 and fp8 key rows equal the oracle's hadamard128 followed by its key
    stores; the caller's key rows are left as they were."""
    case = tl.PagedCase(seed=97, nseq=5, len_lo=100, len_hi=3000, num_pages=400, k=64, append=append)
    rotated = orc.hadamard128(case.keys.copy())
    fp4_want = np.zeros(case.num_pages * case.rpp * 68, np.uint8)
    orc.store_rows_fp4_chunks(rotated, fp4_want, case.tables, case.rpp, case.chunks)
    codes_want = np.zeros((case.num_pages * case.rpp, 128), np.uint8)
    scales_want = np.zeros((case.num_pages * case.rpp, 2), np.uint8)
    orc.store_rows_fp8_chunks(rotated, 64, codes_want, scales_want, case.tables, case.rpp, case.chunks)
    d = {n: tl.dev(cuda, a) for n, a in dict(tables=case.tables, chunks=case.chunks, q_chunk=case.q_chunk,
                                              q_vis=case.q_visible, keys=case.keys).items()}
    d["fp4"] = cuda.zeros(fp4_want.size, dtype=cuda.uint8, device="cuda")
    d["codes"] = cuda.zeros(codes_want.size, dtype=cuda.uint8, device="cuda")
    d["scales"] = cuda.zeros(scales_want.size, dtype=cuda.uint8, device="cuda")
    step = tl.make_step(case, d["tables"], d["chunks"], d["q_chunk"], d["q_vis"], Q=0)
    layers = tl.make_layers(1)
    y = layers[0]
    y.keys, y.key_pool_fp4 = d["keys"].data_ptr(), d["fp4"].data_ptr()
    y.key_fp8_codes, y.key_fp8_scales = d["codes"].data_ptr(), d["scales"].data_ptr()
    flags = capi.PKV_DO_KEYS_FP4 | capi.PKV_DO_KEYS_FP8 | capi.PKV_KEYS_HADAMARD | variant
    capi.check(pkv.pkv_step_run(C.byref(step), layers, 1, flags, tl.stream_ptr(cuda)))
    cuda.cuda.synchronize()
    assert tl.device_status(pkv) == 0
    assert np.array_equal(tl.host(d["fp4"], np.uint8), fp4_want)
    assert np.array_equal(tl.host(d["codes"], np.uint8, codes_want.shape), codes_want)
    assert np.array_equal(tl.host(d["scales"], np.uint8, scales_want.shape), scales_want)
    assert np.array_equal(tl.host(d["keys"], np.uint16, case.keys.shape), case.keys)
