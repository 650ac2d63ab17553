"""IVF with use_residual and sq8 buckets (src/datacell/bucket_datacell.h:526-651): lists hold the codes of
x - centroid, the quantizer is trained on residuals, and a distance is the quantizer's distance between the raw
query and the residual code, minus the row's bias (L2), minus the query-centroid term.  Model, codes and returned
distances are compared with the oracle's restatement bit for bit."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("metric", [0, 1, 2])
@pytest.mark.parametrize("dim,k", [(7, 1), (96, 10), (100, 40)])
def test_residual_codes_and_search_equal_the_oracle(engine, oracle, metric, dim, k):
    n, nlist, nprobe = 12_000, 40, 9
    x = mixture(dim + metric, n, dim, nlist, 0.15)
    q = mixture(77, 300, dim, nlist, 0.15)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    stored, q_used, om = x, q, metric
    if metric == 2:                                             # cosine: normalised rows, queries and centroids, then IP
        centroids = oracle.normalize_rows(centroids)
        stored, q_used, om = oracle.normalize_rows(x), oracle.normalize_rows(q), 1
    if om == 0:
        labels, _ = oracle.kmeans_assign(stored, centroids)
    else:
        labels = oracle.route(stored, centroids, 1, 1)[0][:, 0].astype(np.int32)
    residuals = oracle.residual_rows(stored, labels, centroids)
    lower, diff = oracle.sq8_train(residuals)
    off, order = oracle.build_lists(labels, nlist)
    want_codes, want_bias = oracle.sq8_residual_encode(stored[order], labels[order], centroids, lower, diff, om)

    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_use_residual(True)
    ix.set_centroids(centroids)
    ix.set_sq8_model(lower, diff)
    ids = np.arange(n, dtype=np.int64) * 5 + 11
    half = n // 2
    ix.add(x[:half], ids[:half], labels=labels[:half])
    ix.add(x[half:], ids[half:], labels=labels[half:])
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(sizes, np.diff(off)) and np.array_equal(inner, order)
    assert np.array_equal(codes, want_codes)
    probes, _ = oracle.route(q_used, centroids, nprobe, om)
    probes[3, 2:] = -1
    want = oracle.ivf_sq8_residual_search(want_codes, want_bias, off, ids[order], lower, diff, centroids, q_used, probes, k, om)
    got = ix.search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


@pytest.mark.parametrize("metric", [0, 1])
def test_engine_trains_the_quantizer_on_residuals(engine, oracle, metric):
    n, dim, nlist = 20_000, 24, 16
    x = mixture(9, n, dim, nlist, 0.2)
    init = x[:nlist].copy()
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_use_residual(True)
    ix.train(x, iters=4, init=init)
    centroids = ix.get_centroids()
    if metric == 0:
        labels, _ = oracle.kmeans_assign(x, centroids)
    else:
        labels = oracle.route(x, centroids, 1, 1)[0][:, 0].astype(np.int32)
    lower, diff = oracle.sq8_train(oracle.residual_rows(x, labels, centroids))
    got_lower, got_diff = ix.get_sq8_model()
    assert np.array_equal(got_lower, lower) and np.array_equal(got_diff, diff)


def test_factory_index_with_residual_codes_recalls_better_than_plain_sq8(oracle, tmp_path):
    from vsag_b200.index import Index

    n, dim, nq, k = 6000, 48, 100, 10
    # tight clusters far apart: the range of a residual is a fraction of the range of a coordinate
    both = mixture(31, n + nq, dim, 24, 0.02, lo=0.0, hi=50.0)
    base, queries = both[:n].copy(), both[n:].copy()
    ids = np.arange(n, dtype=np.int64)
    search = json.dumps({"ivf": {"scan_buckets_count": 24}})
    exact_i, _ = oracle.bf_search_fp32(base, queries, k)

    def recall(index):
        got_i, _ = index.knn_search_batch(queries, k, search)
        return np.mean([len(set(a.tolist()) & set(b.tolist())) / k for a, b in zip(got_i, exact_i)])

    made = {}
    for residual in (False, True):
        made[residual] = Index("ivf", json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                                                  "index_param": {"buckets_count": 24, "base_quantization_type": "sq8",
                                                                  "use_residual": residual}}))
        made[residual].build(base, ids, n, dim)
    # lists that hold one cluster quantize residuals of a tiny range, lists that hold two do not: better than
    # plain sq8 (whose step is 50 / 255 everywhere), not perfect
    assert recall(made[True]) > recall(made[False]) + 0.1
    path = tmp_path / "r.idx"
    made[True].serialize_file(str(path))
    again = Index("ivf", json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                                     "index_param": {"buckets_count": 24, "base_quantization_type": "sq8",
                                                     "use_residual": True}}))
    again.deserialize_file(str(path))
    a = made[True].knn_search_batch(queries, k, search)
    b = again.knn_search_batch(queries, k, search)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
