"""Pins the CPU oracle: the reference's known-answer test, libstdc++'s generator, and the outputs of
the reference's own SIMD kernels recorded in tests/golden/ref_simd_golden.npz."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

from conftest import mixture

GOLDEN = Path(__file__).resolve().parent / "golden" / "ref_simd_golden.npz"


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_sq8_known_answer(oracle):
    # src/quantization/scalar_quantization/scalar_quantizer_test.cpp:101-116
    lower, diff = oracle.sq8_train(np.array([[0.0, 0.0], [1.0, 1.0]], np.float32))
    codes = oracle.sq8_encode(np.array([[np.nan, 0.5]], np.float32), lower, diff)
    decoded = oracle.sq8_decode(codes, lower, diff)
    assert codes[0, 0] == 0
    assert codes[0, 1] == int(255.0 * 0.5)
    assert np.isfinite(decoded[0, 0]) and abs(decoded[0, 0]) <= 1e-6
    assert abs(decoded[0, 1] - 127.0 / 255.0) <= 1e-6


def test_generator_matches_libstdcxx(oracle):
    # First eight draws of std::mt19937(47) through std::uniform_real_distribution<float>(0.1, 0.9)
    # (the reference's fixture generator, tests/fixtures/data/vector_generator.h:55-70), printed by
    # a g++ 13 program.
    want = np.array([0.19079077, 0.78140599, 0.87958646, 0.82773650, 0.68298769, 0.75874496,
                     0.38117424, 0.39765069], np.float32)
    got = oracle.gen_uniform(47, 8, 0.1, 0.9)
    assert np.array_equal(got, want)
    total = oracle.gen_uniform(48, 1_000_000).astype(np.float64).sum()
    assert abs(total - 499726.322004) < 1e-3


def test_float_to_bf16_bit_exact(oracle, golden):
    assert np.array_equal(oracle.float_to_bf16(golden["bf16_in"]), golden["bf16_out"])


@pytest.mark.parametrize("dim", [1, 7, 16, 33, 96, 100, 128, 960])
def test_kernels_match_reference_simd(oracle, golden, dim):
    g = lambda k: golden[f"d{dim}_{k}"]  # noqa: E731
    q, x, lower, diff, codes = g("q"), g("x"), g("lower"), g("diff"), g("codes")
    qb, xb, bits, centroid = g("qb"), g("xb"), g("bits"), g("centroid")  # keep the buffers alive
    inv_sqrt_d = np.float32(1.0) / np.sqrt(np.float32(dim))
    L = oracle.lib()
    import ctypes as C

    p = lambda a: C.c_void_p(a.ctypes.data)  # noqa: E731
    for i in range(int(golden["cases"])):
        for name, val in (
            ("sq8_l2", oracle.sq8_l2sqr(q[i], codes[i], lower, diff)),
            ("sq8_ip", oracle.sq8_ip(q[i], codes[i], lower, diff)),
            ("fp32_l2", oracle.fp32_l2sqr(q[i], x[i])),
            ("fp32_ip", oracle.fp32_ip(q[i], x[i])),
            ("bf16_ip", float(L.orc_bf16_ip(p(qb[i]), p(xb[i]), C.c_uint64(dim)))),
            ("bf16_l2", float(L.orc_bf16_l2sqr(p(qb[i]), p(xb[i]), C.c_uint64(dim)))),
            ("rabitq_ip", float(L.orc_rabitq_float_binary_ip(p(q[i]), p(bits[i]), dim, inv_sqrt_d))),
        ):
            # dispatched (AVX-512 on the generating host) and scalar reference variants differ from
            # each other by summation order only; the oracle must sit within that band.
            for variant in (name, name + "_generic"):
                key = f"d{dim}_{variant}"
                if key in golden:
                    scale = max(1.0, float(dim) ** 0.5)
                    assert val == pytest.approx(float(golden[key][i]), rel=2e-6 * scale, abs=2e-6 * scale), variant
        out = np.empty(dim, np.float32)
        norm = float(L.orc_normalize_with_centroid(p(x[i]), p(centroid), p(out), C.c_uint64(dim)))
        assert norm == pytest.approx(float(g("norm")[i]), rel=1e-6)
        np.testing.assert_allclose(out, g("normed")[i], rtol=2e-6, atol=1e-7)


def test_rabitq_binary_ip_generic_is_bit_exact(oracle, golden):
    """The scalar reference loop (src/simd/generic.cpp:447-471) has one defined order; the oracle
    follows it exactly."""
    import ctypes as C

    L = oracle.lib()
    for dim in (7, 96, 960):
        inv_sqrt_d = np.float32(1.0) / np.sqrt(np.float32(dim))
        q, bits = golden[f"d{dim}_q"], golden[f"d{dim}_bits"]
        for i in range(int(golden["cases"])):
            got = np.float32(L.orc_rabitq_float_binary_ip(C.c_void_p(q[i].ctypes.data),
                                                          C.c_void_p(bits[i].ctypes.data), dim, inv_sqrt_d))
            assert got == golden[f"d{dim}_rabitq_ip_generic"][i]


def test_sq8_trainer_order_statistics(oracle):
    rng = np.random.default_rng(5)
    x = rng.normal(size=(5000, 6)).astype(np.float32)
    lower, diff = oracle.sq8_train(x, mode=3)
    m = max(1, int((5000 - 1) * 0.001))
    s = np.sort(x, axis=0)
    assert np.array_equal(lower, s[m - 1])
    assert np.array_equal(diff, s[5000 - m] - s[m - 1])
    lower_c, diff_c = oracle.sq8_train(x, mode=1)
    assert np.array_equal(lower_c, s[0]) and np.array_equal(diff_c, s[-1] - s[0])
    # more rows than the 100000-row sample: the stride rule picks row (j * (2147483647 % n)) % n
    n = 150_001
    y = rng.normal(size=(n, 2)).astype(np.float32)
    step = 2147483647 % n
    rows = (np.arange(100000, dtype=np.int64) * step) % n
    s = np.sort(y[rows], axis=0)
    lower, diff = oracle.sq8_train(y, mode=3)
    assert np.array_equal(lower, s[98]) and np.array_equal(diff, s[100000 - 99] - s[98])


def test_trainer_matches_reference_heap_walk(oracle):
    """The reference keeps two bounded heaps (scalar_quantization_trainer.cpp:89-121); replay that
    walk literally, with duplicates, and compare with the oracle's order statistics."""
    import heapq

    rng = np.random.default_rng(9)
    x = rng.integers(-5, 5, size=(3000, 3)).astype(np.float32)
    m = max(1, int((3000 - 1) * 0.001))
    lower, diff = oracle.sq8_train(x, mode=3)
    for d in range(3):
        hmax = [np.finfo(np.float32).min]   # min-heap of the largest values
        hmin = [-np.finfo(np.float32).max]  # max-heap (negated) of the smallest values
        for v in x[:, d]:
            if v > hmax[0] or len(hmax) < m:
                heapq.heappush(hmax, v)
            if len(hmax) > m:
                heapq.heappop(hmax)
            if v < -hmin[0] or len(hmin) < m:
                heapq.heappush(hmin, -v)
            if len(hmin) > m:
                heapq.heappop(hmin)
        assert lower[d] == -hmin[0]
        assert diff[d] == np.float32(hmax[0]) - np.float32(-hmin[0])


def test_heap_semantics_ties_keep_earlier(oracle):
    # FlatBucketSearcher inserts only on a strict improvement (flat_bucket_searcher.cpp:88-91): of
    # two equal distances at the cut-off the one scanned first stays.
    codes = np.zeros((4, 2), np.uint8)
    lower = np.zeros(2, np.float32)
    diff = np.ones(2, np.float32)
    q = np.zeros((1, 2), np.float32)
    off = np.array([0, 4], np.int64)
    ids, dists = oracle.ivf_sq8_search(codes, off, np.array([10, 11, 12, 13]), lower, diff, q,
                                       np.array([[0]], np.int32), k=2)
    assert sorted(ids[0].tolist()) == [10, 11]
    assert np.all(dists == 0)


def test_kmeans_histogram_like_reference(oracle):
    # src/impl/cluster/kmeans_cluster_test.cpp:39-104: well separated blobs are recovered exactly.
    rng = np.random.default_rng(3)
    k, per, dim = 8, 250, 3
    centres = np.arange(k)[:, None] * 10.0 + np.zeros((1, dim))
    x = (np.repeat(centres, per, axis=0) + rng.normal(0, 0.1, (k * per, dim))).astype(np.float32)
    perm = rng.permutation(k * per)
    x = np.ascontiguousarray(x[perm])
    init = np.ascontiguousarray(x[[int(np.nonzero(perm // per == j)[0][0]) for j in range(k)]])
    centroids, labels, err, _ = oracle.kmeans_run(x, init, 5)
    assert sorted(np.bincount(labels, minlength=k).tolist()) == [per] * k
    assert err < 0.2


def test_empty_and_ragged_lists(oracle):
    rng = np.random.default_rng(1)
    dim, nlist = 5, 6
    x = rng.normal(size=(40, dim)).astype(np.float32)
    labels = rng.integers(0, nlist - 2, 40).astype(np.int32)  # lists 4 and 5 stay empty
    off, order = oracle.build_lists(labels, nlist)
    lower, diff = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x, lower, diff)[order]
    q = x[:3]
    probes = np.array([[4, 5, -1], [0, 4, 1], [3, 2, 1]], np.int32)
    ids, dists = oracle.ivf_sq8_search(codes, off, order, lower, diff, q, probes, k=50)
    assert np.all(ids[0] == -1) and np.all(np.isinf(dists[0]))
    n1 = int((off[1] - off[0]) + (off[2] - off[1]))
    assert np.sum(ids[1] >= 0) == n1
    assert np.all(np.diff(dists[1][: n1]) >= 0)


@pytest.mark.parametrize("n", [1, 7, 1000, 100_000, 2**31 + 5, 2**32])
def test_restated_draws_match_cxx_library(oracle, n):
    """k-means++ draws through std::uniform_int_distribution<uint64_t> and
    std::uniform_real_distribution<double> over std::mt19937 (kmeans_cluster.cpp:388-417); the C
    restatement of those two must give the library's own values."""
    want = oracle.std_draws(47, n, 3000, restated=False)
    got = oracle.std_draws(47, n, 3000, restated=True)
    assert np.array_equal(got[0], want[0])
    assert np.array_equal(got[1], want[1])


def test_kmeans_pp_seeding_properties(oracle):
    x = mixture(5, 4000, 16, 8, 0.05)
    centroids, picked = oracle.kmeans_pp_init(x, 8, seed=47)
    assert np.array_equal(centroids, x[picked])
    assert picked[0] == oracle.std_draws(47, 4000, 1, restated=False)[0][0]
    # eight well-separated clusters: the squared-distance weighting reaches all of them
    truth = np.argmin(((x[picked][:, None, :] - x[None, :, :]) ** 2).sum(-1), axis=0)
    assert len(np.unique(truth)) == 8
    # every row identical: total weight 0 after the first pick, later picks are uniform draws
    flat = np.ones((50, 4), np.float32)
    c2, p2 = oracle.kmeans_pp_init(flat, 5, seed=3)
    assert np.all(c2 == 1.0) and np.all((p2 >= 0) & (p2 < 50))
