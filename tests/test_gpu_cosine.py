"""GPU parity for metric_type "cosine": rows, queries and centroids are normalised the way the
reference's Normalize does, then the inner-product path runs; the oracle is fed normalised inputs."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def test_bruteforce_cosine_fp32_and_bf16(engine, oracle):
    n, dim, nq, k = 7000, 72, 120, 15
    base = mixture(71, n, dim, 32, 0.3) + 0.5
    q = mixture(72, nq, dim, 32, 0.3) + 0.5
    base[17] = 0.0                                   # a zero row is divided by 1, not by 0
    ids = np.arange(n, dtype=np.int64) + 3
    unit_base, unit_q = oracle.normalize_rows(base), oracle.normalize_rows(q)
    assert np.all(unit_base[17] == 0.0)
    ix = engine.BfHandle(dim, engine.METRIC_COSINE, engine.QUANT_FP32)
    ix.add(base[:3000], ids[:3000])
    ix.add(base[3000:], ids[3000:])
    want_i, want_d = oracle.bf_search_fp32(unit_base, unit_q, k, 1)
    got_i, got_d = ix.search(q, k)
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_i, got_d, np.where(want_i >= 0, want_i + 3, -1), want_d, rtol=0, atol=0)
    assert np.all(got_d > -1e-5) and np.all(got_d < 2.0 + 1e-5)   # 1 - cos
    hx = engine.BfHandle(dim, engine.METRIC_COSINE, engine.QUANT_BF16)
    hx.add(base, ids)
    want16 = oracle.bf_search_bf16(oracle.float_to_bf16(unit_base), unit_q, k, metric=1)
    got16 = hx.search(q, k)
    assert np.array_equal(got16[1], want16[1])
    with pytest.raises(engine.VsagB200Error, match="cosine"):
        hx.add_bf16(oracle.float_to_bf16(base[:4]), ids[:4])


@pytest.mark.parametrize("quant", ["sq8", "fp32"])
def test_ivf_cosine_matches_oracle(engine, oracle, quant):
    n, dim, nlist, nprobe, nq, k = 12_000, 40, 24, 8, 200, 10
    x = mixture(73, n, dim, nlist, 0.2) + 0.3
    q = mixture(74, nq, dim, nlist, 0.2) + 0.3
    ux, uq = oracle.normalize_rows(x), oracle.normalize_rows(q)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    ucent = oracle.normalize_rows(centroids)                    # ivf_nearest_partition.cpp:81-85
    labels = np.argmax(ux @ ucent.T, axis=1).astype(np.int32)   # any fixed assignment will do here
    off, order = oracle.build_lists(labels, nlist)
    ids = np.arange(n, dtype=np.int64) * 2 + 1
    ix = engine.IvfHandle(dim, engine.METRIC_COSINE, nlist, engine.QUANT_SQ8 if quant == "sq8" else engine.QUANT_FP32)
    ix.set_centroids(ucent)
    if quant == "sq8":
        lower, diff = oracle.sq8_train(ux)
        ix.set_sq8_model(lower, diff)
    ix.add(x, ids, labels=labels)                               # raw rows in: the index normalises them
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(inner, order)
    probes, _ = oracle.route(uq, ucent, nprobe, 1)
    if quant == "sq8":
        want_codes = oracle.sq8_encode(ux, lower, diff)[order]
        assert np.array_equal(codes, want_codes)
        want = oracle.ivf_sq8_search(want_codes, off, ids[order], lower, diff, uq, probes, k, 1)
    else:
        assert np.array_equal(codes.view(np.float32).reshape(-1, dim), ux[order])
        want = oracle.ivf_fp32_search(ux[order], off, ids[order], uq, probes, k, 1)
    got = ix.search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    gp, gd = ix.route(q, nprobe)                                 # queries are normalised for routing too
    wp, wd = oracle.route(uq, ucent, nprobe, 1)
    assert np.array_equal(gd, wd)


def test_ivf_cosine_training_normalises_centroids_and_model(engine, oracle):
    n, dim, nlist = 8000, 24, 16
    x = mixture(75, n, dim, nlist, 0.2) + 0.4
    ix = engine.IvfHandle(dim, engine.METRIC_COSINE, nlist, engine.QUANT_SQ8)
    ix.train(x, iters=3)
    cents = ix.get_centroids()
    np.testing.assert_allclose(np.linalg.norm(cents, axis=1), 1.0, rtol=1e-6)
    want_c, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    # training is bit-exact (labels, and centroid sums in ascending row order), and so is the normalisation
    assert np.array_equal(cents, oracle.normalize_rows(want_c))
    lower, diff = ix.get_sq8_model()
    want_l, want_d = oracle.sq8_train(oracle.normalize_rows(x))
    assert np.array_equal(lower, want_l) and np.array_equal(diff, want_d)


def test_factory_accepts_cosine(oracle):
    from vsag_b200.index import Index

    n, dim, nq, k = 3000, 32, 50, 10
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, nq * dim).reshape(nq, dim)
    ids = np.arange(n, dtype=np.int64)
    ub, uq = oracle.normalize_rows(base), oracle.normalize_rows(queries)
    truth, truth_d = oracle.bf_search_fp32(ub, uq, k, 1)
    for name, extra, search in (("brute_force", {}, "{}"),
                                ("ivf", {"buckets_count": 10}, json.dumps({"ivf": {"scan_buckets_count": 10}}))):
        params = json.dumps({"dtype": "float32", "metric_type": "cosine", "dim": dim, "index_param": extra})
        index = Index(name, params)
        index.build(base, ids, n, dim)
        for i in range(nq):
            got_i, got_d = index.knn_search(queries[i], k, search)
            assert np.array_equal(got_d, truth_d[i])
            assert_topk_equal(got_i[None], got_d[None], truth[i][None], truth_d[i][None], rtol=0, atol=0)
