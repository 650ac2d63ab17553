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
