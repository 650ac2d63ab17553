"""RangeSearch through the factory API (include/vsag/index.h:380-397): the answer is the k-nearest
answer cut at the radius, as in the reference's range mode (bruteforce.cpp:388-545,
flat_bucket_searcher.cpp:105-137); checked against the oracle's exact search, like the reference's
TestRangeSearch (tests/test_index.cpp) checks radius and limit."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


def params(dim, metric="l2", **index_param):
    return json.dumps({"dtype": "float32", "metric_type": metric, "dim": dim, "index_param": index_param})


@pytest.mark.parametrize("name,index_param,search", [
    ("brute_force", dict(base_quantization_type="fp32"), {}),
    ("ivf", dict(buckets_count=12, base_quantization_type="fp32"), {"ivf": {"scan_buckets_count": 12}}),
])
def test_range_is_knn_cut_at_the_radius(oracle, name, index_param, search):
    from vsag_b200.index import Index, VsagError

    n, dim = 3000, 32
    base = mixture(21, n, dim, 12, 0.1)
    queries = mixture(22, 20, dim, 12, 0.1)
    ids = np.arange(n, dtype=np.int64) + 50
    index = Index(name, params(dim, **index_param))
    index.build(base, ids, n, dim)
    sp = json.dumps(search)
    truth_i, truth_d = oracle.bf_search_fp32(base, queries, 600)
    for qi in range(len(queries)):
        d = truth_d[qi]
        for want_count in (0, 1, 7, 100, 300):
            # a radius strictly between two neighbouring distances
            radius = float(d[0]) * 0.5 if want_count == 0 else float((d[want_count - 1] + d[want_count]) / 2)
            got_i, got_d = index.range_search(queries[qi], radius, -1, sp)
            assert len(got_i) == want_count
            assert np.array_equal(got_d, d[:want_count])
            assert set(got_i.tolist()) == set((truth_i[qi][:want_count] + 50).tolist())
            lim_i, lim_d = index.range_search(queries[qi], radius, 5, sp)       # the nearest five of them
            assert np.array_equal(lim_d, d[:min(5, want_count)])
    # more in-radius vectors than one search can return (512): fetched in pages, still every one of them
    far_i, far_d = oracle.bf_search_fp32(base, queries[:2], 1400)
    for qi, count in ((0, 599), (1, 1300)):
        wide = float((far_d[qi][count - 1] + far_d[qi][count]) / 2)
        got_i, got_d = index.range_search(queries[qi], wide, -1, sp)
        assert len(got_i) == count and len(set(got_i.tolist())) == count
        assert np.array_equal(got_d, far_d[qi][:count])
        assert set(got_i.tolist()) == set((far_i[qi][:count] + 50).tolist())
    wide = float(truth_d[0][599])
    got_i, got_d = index.range_search(queries[0], wide, 40, sp)
    assert np.array_equal(got_d, truth_d[0][:40])
    for bad in (dict(radius=-1.0, k=5), dict(radius=float("nan"), k=5), dict(radius=1.0, k=0)):
        with pytest.raises(VsagError) as e:
            index.range_search(queries[0], bad["radius"], bad["k"], sp)
        assert e.value.code == -3
    assert len(Index(name, params(dim, **index_param)).range_search(queries[0], 1.0, 5, sp)[0]) == 0   # empty index


def test_range_search_skips_removed_vectors(oracle):
    from vsag_b200.index import Index

    n, dim = 1000, 16
    base = mixture(23, n, dim, 6, 0.1)
    ids = np.arange(n, dtype=np.int64)
    index = Index("brute_force", params(dim))
    index.build(base, ids, n, dim)
    _, d = oracle.bf_search_fp32(base, base[:1], 20)
    radius = float(d[0][9] + d[0][10]) / 2
    before, _ = index.range_search(base[0], radius, -1)
    assert len(before) == 10 and before[0] == 0
    index.remove(before[:3])
    after, _ = index.range_search(base[0], radius, -1)
    assert after.tolist() == before[3:].tolist()


@pytest.mark.parametrize("name,index_param,search", [
    ("brute_force", dict(base_quantization_type="fp32"), {}),
    ("ivf", dict(buckets_count=8, base_quantization_type="fp32"), {"ivf": {"scan_buckets_count": 8}}),
])
def test_with_filter_functions_keep_valid_ids_only(oracle, name, index_param, search):
    """vsag_index_knn_search_with_filter / _range_search_with_filter: the callback says which ids are
    valid (VsagFilterWrapper::CheckValid, src/vsag_c_api.cpp:337-343)."""
    from vsag_b200.index import Index

    n, dim, k = 2000, 24, 10
    base = mixture(24, n, dim, 8, 0.1)
    queries = mixture(25, 10, dim, 8, 0.1)
    ids = np.arange(n, dtype=np.int64) * 3
    index = Index(name, params(dim, **index_param))
    index.build(base, ids, n, dim)
    sp = json.dumps(search)
    valid = lambda i: i % 2 == 0            # noqa: E731
    keep = np.array([valid(int(i)) for i in ids])
    truth_i, truth_d = oracle.bf_search_fp32(base[keep], queries, 40)
    kept_ids = ids[keep]
    for qi in range(len(queries)):
        got_i, got_d = index.knn_search_with_filter(queries[qi], k, sp, valid)
        assert np.array_equal(got_d, truth_d[qi][:k])
        assert set(got_i.tolist()) == set(kept_ids[truth_i[qi][:k]].tolist())
        radius = float(truth_d[qi][24] + truth_d[qi][25]) / 2
        rng_i, rng_d = index.range_search_with_filter(queries[qi], radius, 30, sp, valid)
        assert np.array_equal(rng_d, truth_d[qi][:25])
        assert set(rng_i.tolist()) == set(kept_ids[truth_i[qi][:25]].tolist())
        few_i, few_d = index.range_search_with_filter(queries[qi], radius, 4, sp, valid)
        assert np.array_equal(few_d, truth_d[qi][:4])


@pytest.mark.parametrize("name,index_param,search", [
    ("brute_force", dict(base_quantization_type="fp32"), {}),
    ("ivf", dict(buckets_count=12, base_quantization_type="fp32"), {"ivf": {"scan_buckets_count": 12}}),
])
def test_k_beyond_one_search_is_fetched_in_pages(oracle, name, index_param, search):
    """The engine returns at most a few hundred neighbours per search; a larger k is served in pages of 512
    (the found vectors join the deny bitmap of the next page), as the reference serves any k."""
    from vsag_b200.index import Index

    n, dim, k = 3000, 32, 1300
    base = mixture(21, n, dim, 12, 0.1)
    queries = mixture(22, 3, dim, 12, 0.1)
    ids = np.arange(n, dtype=np.int64) + 50
    index = Index(name, params(dim, **index_param))
    index.build(base, ids, n, dim)
    sp = json.dumps(search)
    want_i, want_d = oracle.bf_search_fp32(base, queries, k)
    got_i, got_d = index.knn_search_batch(queries, k, sp)
    assert np.array_equal(got_d, want_d)
    for q in range(len(queries)):
        assert len(set(got_i[q].tolist())) == k
        assert set(got_i[q].tolist()) == set((want_i[q] + 50).tolist())
    one_i, one_d = index.knn_search(queries[0], n + 10, sp)          # more than the index holds: all of it, once
    assert len(one_i) == n and len(set(one_i.tolist())) == n
    assert np.array_equal(one_d, oracle.bf_search_fp32(base, queries[:1], n)[1][0])
