"""Checks the C oracle against the reference's own SIMD kernels compiled from the reference tree
(oracle/_ref, built by oracle/Makefile).  Skipped where that library has not been built; the
committed fixtures in tests/golden/ cover the same functions everywhere."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def ref(oracle):
    R = oracle.ref()
    if R is None:
        pytest.skip("oracle/_ref/libvsag_ref_simd.so not built (no reference tree on this machine)")
    return R


def _p(a):
    return C.c_void_p(a.ctypes.data)


@pytest.mark.parametrize("dim", [3, 17, 96, 128, 255, 960])
def test_sq8_distance_matches_reference(oracle, ref, dim):
    rng = np.random.default_rng(dim)
    x = rng.normal(size=(2000, dim)).astype(np.float32)
    lower, diff = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x[:64], lower, diff)
    q = rng.normal(size=(8, dim)).astype(np.float32)
    for qi in q:
        for c in codes:
            want_l2 = ref.ref_SQ8ComputeL2Sqr(_p(qi), _p(c), _p(lower), _p(diff), dim)
            want_ip = ref.ref_SQ8ComputeIP(_p(qi), _p(c), _p(lower), _p(diff), dim)
            assert oracle.sq8_l2sqr(qi, c, lower, diff) == pytest.approx(want_l2, rel=1e-5)
            # an inner product cancels: bound the error by the size of the terms, not of the sum
            assert oracle.sq8_ip(qi, c, lower, diff) == pytest.approx(want_ip, rel=1e-5, abs=1e-7 * dim)


def test_ivf_scan_same_result_with_reference_kernel(oracle, ref):
    """The restated scan loop driven by the reference's compiled SQ8ComputeL2Sqr returns the same
    neighbours as with the oracle's scalar kernel (distances to 1e-5)."""
    from conftest import assert_topk_equal, mixture

    dim, nlist = 96, 32
    x = mixture(11, 6000, dim, 32, 0.15)
    q = mixture(12, 50, dim, 32, 0.15)
    centroids = x[:nlist].copy()
    labels, _ = oracle.kmeans_assign(x, centroids)
    off, order = oracle.build_lists(labels, nlist)
    lower, diff = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x, lower, diff)[order]
    probes, _ = oracle.route(q, centroids, 8)
    a = oracle.ivf_sq8_search(codes, off, order, lower, diff, q, probes, 10)
    fn = C.cast(ref.ref_SQ8ComputeL2Sqr, C.c_void_p)
    b = oracle.ivf_sq8_search(codes, off, order, lower, diff, q, probes, 10, fn=fn)
    assert_topk_equal(a[0], a[1], b[0], b[1], rtol=1e-5)


def test_fp32_and_bf16_match_reference(oracle, ref):
    rng = np.random.default_rng(0)
    for dim in (5, 128, 768):
        a = rng.normal(size=dim).astype(np.float32)
        b = rng.normal(size=dim).astype(np.float32)
        assert oracle.fp32_l2sqr(a, b) == pytest.approx(ref.ref_FP32ComputeL2Sqr(_p(a), _p(b), dim), rel=1e-5)
        assert oracle.fp32_ip(a, b) == pytest.approx(ref.ref_FP32ComputeIP(_p(a), _p(b), dim), rel=1e-5, abs=1e-5)
        ab, bb = oracle.float_to_bf16(a), oracle.float_to_bf16(b)
        want = ref.ref_BF16ComputeIP(_p(ab), _p(bb), dim)
        got = float(oracle.lib().orc_bf16_ip(_p(ab), _p(bb), C.c_uint64(dim)))
        assert got == pytest.approx(want, rel=1e-5, abs=1e-5)
    vals = rng.normal(size=1000).astype(np.float32)
    want = np.array([ref.ref_FloatToBF16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(oracle.float_to_bf16(vals), want)


def test_fp16_matches_reference(oracle, ref):
    """generic::FloatToFP16 / FP16ToFloat bit for bit, FP16ComputeIP / L2Sqr (dispatched and generic) on encoded
    vectors: every code the encoder writes is a normal half, so the vector paths' IEEE widening agrees with the
    generic bit formula and only the summation order differs."""
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-3, 500),
                           [0.0, -0.0, 1.0, 65504.0, 1e5, -1e5, 1e-8, 6e-5]]).astype(np.float32)
    ref.ref_FloatToFP16.restype = C.c_uint16
    ref.ref_FloatToFP16.argtypes = [C.c_float]
    ref.ref_FP16ToFloat.restype = C.c_float
    ref.ref_FP16ToFloat.argtypes = [C.c_uint16]
    want = np.array([ref.ref_FloatToFP16(float(v)) for v in vals], np.uint16)
    got = oracle.float_to_half(vals, "fp16")
    assert np.array_equal(got, want)
    back = np.array([ref.ref_FP16ToFloat(int(v)) for v in got], np.float32)
    assert np.array_equal(oracle.half_to_float(got, "fp16"), back)
    lib = oracle.lib()
    lib.orc_half_ip.restype = C.c_float
    lib.orc_half_l2sqr.restype = C.c_float
    for fn in (ref.ref_FP16ComputeIP, ref.ref_FP16ComputeL2Sqr, ref.ref_generic_FP16ComputeL2Sqr):
        fn.restype = C.c_float
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
    for dim in (1, 7, 16, 96, 100, 768):
        a = oracle.float_to_half(rng.normal(0, 1, dim).astype(np.float32), "fp16")
        b = oracle.float_to_half(rng.normal(0, 1, dim).astype(np.float32), "fp16")
        ip = lib.orc_half_ip(_p(a), _p(b), C.c_uint64(dim), C.c_int(1))
        l2 = lib.orc_half_l2sqr(_p(a), _p(b), C.c_uint64(dim), C.c_int(1))
        assert l2 == ref.ref_generic_FP16ComputeL2Sqr(a.ctypes.data, b.ctypes.data, dim)      # same order: same bits
        assert ip == pytest.approx(ref.ref_FP16ComputeIP(a.ctypes.data, b.ctypes.data, dim), rel=1e-5, abs=1e-5)
        assert l2 == pytest.approx(ref.ref_FP16ComputeL2Sqr(a.ctypes.data, b.ctypes.data, dim), rel=1e-5)


def test_sq8_uniform_codes_ip_matches_reference(oracle, ref):
    """SQ8UniformComputeCodesIP as the reference dispatches it (AVX-512 here): an exact integer, whatever the order."""
    rng = np.random.default_rng(4)
    ref.ref_SQ8UniformComputeCodesIP.restype = C.c_float
    ref.ref_SQ8UniformComputeCodesIP.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
    lib = oracle.lib()
    lib.orc_sq8u_codes_ip.restype = C.c_float
    for dim in (1, 7, 64, 96, 100, 960):
        a = rng.integers(0, 256, dim, dtype=np.uint8)
        b = rng.integers(0, 256, dim, dtype=np.uint8)
        want = ref.ref_SQ8UniformComputeCodesIP(a.ctypes.data, b.ctypes.data, dim)
        assert lib.orc_sq8u_codes_ip(_p(a), _p(b), C.c_uint64(dim)) == want == float(a.astype(np.int64) @ b.astype(np.int64))
