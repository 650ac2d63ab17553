"""Functional tests through vsag::Factory::CreateIndex / Build / KnnSearch, in the style of the
reference's tests/test_ivf.cpp and tests/test_brute_force.cpp: fixture vectors from
std::mt19937(47) + uniform(0.1, 0.9) (tests/fixtures/data/vector_generator.h:55-70), exhaustive
ground truth (tests/fixtures/data/ground_truth.cpp:27-63), recall floors of the reference
(tests/test_ivf.cpp:94-102: sq8 0.84; tests/test_brute_force.cpp:215-221: fp32 0.99, bf16 0.92)."""
from __future__ import annotations

import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def fixture_vectors(oracle, count, dim, seed=47):
    return oracle.gen_uniform(seed, count * dim, 0.1, 0.9).reshape(count, dim)


def params(dim, metric="l2", **index_param):
    return json.dumps({"dtype": "float32", "metric_type": metric, "dim": dim, "index_param": index_param})


def recall(found, truth):
    return np.mean([len(set(a.tolist()) & set(b.tolist())) / len(b) for a, b in zip(found, truth)])


@pytest.mark.parametrize("dim", [32, 128])
def test_ivf_sq8_recall_like_reference(oracle, dim):
    from vsag_b200.index import Index

    n, nq, k = 3000, 200, 10
    base = fixture_vectors(oracle, n, dim)
    queries = fixture_vectors(oracle, nq, dim, seed=48)
    ids = np.arange(n, dtype=np.int64) + 10_000
    index = Index("ivf", params(dim, buckets_count=30, base_quantization_type="sq8"))
    index.build(base, ids, n, dim)
    assert index.get_num_elements() == n
    truth, _ = oracle.bf_search_fp32(base, queries, k)
    search = json.dumps({"ivf": {"scan_buckets_count": 30}})  # all buckets: recall is the codec's
    found = np.stack([index.knn_search(q, k, search)[0] for q in queries])
    assert recall(found - 10_000, truth) > 0.84 * 0.98
    # 12 of 30 buckets on uniform data (no cluster structure at all) still finds most neighbours
    search = json.dumps({"ivf": {"scan_buckets_count": 12}})
    found = np.stack([index.knn_search(q, k, search)[0] for q in queries[:50]])
    assert recall(found - 10_000, truth[:50]) > 0.6


def test_ivf_batch_equals_serial(oracle):
    # tests/test_ivf.cpp:3283-3341: a batch call returns exactly the rows of the single calls
    from vsag_b200.index import Index

    dim, n, nq, k = 64, 4000, 64, 7
    base = fixture_vectors(oracle, n, dim)
    queries = fixture_vectors(oracle, nq, dim, seed=49)
    index = Index("ivf", params(dim, buckets_count=20, base_quantization_type="sq8"))
    index.build(base, np.arange(n, dtype=np.int64), n, dim)
    search = json.dumps({"ivf": {"scan_buckets_count": 5}})
    batch_ids, batch_d = index.knn_search_batch(queries, k, search)
    for i, q in enumerate(queries):
        ids, dists = index.knn_search(q, k, search)
        assert np.array_equal(ids, batch_ids[i][: len(ids)]) and np.array_equal(dists, batch_d[i][: len(ids)])


def test_ivf_rabitq_with_reorder(oracle):
    from vsag_b200.index import Index

    dim, n, nq, k = 128, 3000, 100, 10
    base = fixture_vectors(oracle, n, dim)
    queries = fixture_vectors(oracle, nq, dim, seed=50)
    index = Index("ivf", params(dim, buckets_count=10, base_quantization_type="rabitq", use_reorder=True))
    index.build(base, np.arange(n, dtype=np.int64), n, dim)
    truth, truth_d = oracle.bf_search_fp32(base, queries, k)
    search = json.dumps({"ivf": {"scan_buckets_count": 10, "factor": 8.0}})
    ids, dists = index.knn_search_batch(queries, k, search)
    assert recall(ids, truth) > 0.7  # 1-bit codes on uniform data: 80 of 3000 candidates reranked
    # reranked distances are exact fp32 distances of the returned rows
    want = np.array([[oracle.fp32_l2sqr(queries[i], base[j]) for j in ids[i]] for i in range(5)], np.float32)
    np.testing.assert_allclose(dists[:5], want, rtol=1e-5)


@pytest.mark.parametrize("quant,floor", [("fp32", 0.99), ("bf16", 0.92)])
def test_brute_force_recall_like_reference(oracle, quant, floor):
    from vsag_b200.index import Index

    dim, n, nq, k = 128, 3000, 100, 10
    base = fixture_vectors(oracle, n, dim)
    queries = fixture_vectors(oracle, nq, dim, seed=48)
    index = Index("brute_force", params(dim, base_quantization_type=quant))
    index.build(base, np.arange(n, dtype=np.int64), n, dim)
    truth, truth_d = oracle.bf_search_fp32(base, queries, k)
    found = np.stack([index.knn_search(q, k, "{}")[0] for q in queries])
    assert recall(found, truth) >= floor
    if quant == "fp32":
        ids, dists = index.knn_search(queries[0], k)
        assert np.array_equal(ids, truth[0]) and np.array_equal(dists, truth_d[0])


def test_index_state_errors(oracle):
    from vsag_b200.index import Index, VsagError

    dim = 16
    base = fixture_vectors(oracle, 600, dim)
    ids = np.arange(600, dtype=np.int64)
    index = Index("ivf", params(dim, buckets_count=8, base_quantization_type="sq8"))
    search = json.dumps({"ivf": {"scan_buckets_count": 4}})
    got_ids, _ = index.knn_search(base[0], 5, search)  # empty index -> empty result, not an error
    assert len(got_ids) == 0
    index.build(base, ids, 600, dim)
    with pytest.raises(VsagError) as e:
        index.build(base, ids, 600, dim)
    assert e.value.code == -5  # BUILD_TWICE
    with pytest.raises(VsagError) as e:
        index.add(np.zeros((3, dim + 1), np.float32), np.arange(3, dtype=np.int64), 3, dim + 1)
    assert e.value.code == -9  # DIMENSION_NOT_EQUAL
    with pytest.raises(VsagError, match="scan_buckets_count"):
        index.knn_search(base[0], 5, json.dumps({"ivf": {}}))
    with pytest.raises(VsagError, match="ivf"):
        index.knn_search(base[0], 5, "{}")
    with pytest.raises(VsagError):
        index.knn_search(base[0], 0, search)
    index.add(base[:10] + 0.01, np.arange(600, 610, dtype=np.int64), 10, dim)  # Add after Build
    assert index.get_num_elements() == 610
    small = Index("ivf", params(dim, buckets_count=50, base_quantization_type="sq8"))
    with pytest.raises(VsagError, match="k cannot be larger than count"):
        small.build(base[:20], ids[:20], 20, dim)


def test_routing_only_mode(oracle):
    # "IVF Search Disable Bucket Scan" (tests/test_ivf.cpp:2200-2309)
    from vsag_b200.index import Index

    dim, n = 32, 2000
    base = fixture_vectors(oracle, n, dim)
    index = Index("ivf", params(dim, buckets_count=16, base_quantization_type="sq8"))
    index.build(base, np.arange(n, dtype=np.int64), n, dim)
    search = json.dumps({"ivf": {"scan_buckets_count": 5, "disable_bucket_scan": True}})
    ids, dists = index.knn_search(base[3], 5, search)
    assert len(ids) == 5 and len(set(ids.tolist())) == 5 and np.all((ids >= 0) & (ids < 16))
    assert np.all(np.diff(dists) >= 0)
