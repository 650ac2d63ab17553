"""Index::SearchWithRequest with SearchRequest::bucket_ids_, section by section after the reference's
own test of that field (tests/test_ivf.cpp:3046-3281): explicit bucket lists bypass routing, an empty
outer vector means default routing, and the lists are validated as IVF::SearchWithRequest does
(src/algorithm/ivf/ivf.cpp:2075-2112)."""
from __future__ import annotations

import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

DIM, N, NLIST, K = 32, 3000, 12, 10
SEARCH = json.dumps({"ivf": {"scan_buckets_count": NLIST}})


@pytest.fixture(scope="module")
def built(oracle):
    from vsag_b200.index import Index

    base = oracle.gen_uniform(47, N * DIM, 0.1, 0.9).reshape(N, DIM)
    queries = oracle.gen_uniform(48, 8 * DIM, 0.1, 0.9).reshape(8, DIM)
    index = Index("ivf", json.dumps({"dtype": "float32", "metric_type": "l2", "dim": DIM,
                                     "index_param": {"buckets_count": NLIST, "base_quantization_type": "sq8"}}))
    index.build(base, np.arange(N, dtype=np.int64), N, DIM)
    return index, base, queries


def test_all_buckets_listed_equals_scanning_all_buckets(built):
    index, _, queries = built
    all_buckets = list(range(NLIST))
    want = index.knn_search_batch(queries[:1], K, SEARCH)
    got = index.search_with_request(queries[:1], K, SEARCH, [all_buckets])
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    # the order of the listed buckets does not matter to the result
    got = index.search_with_request(queries[:1], K, SEARCH, [all_buckets[::-1]])
    assert np.array_equal(got[1], want[1])


def test_empty_outer_vector_is_default_routing(built):
    index, _, queries = built
    search = json.dumps({"ivf": {"scan_buckets_count": 3}})
    want = index.knn_search_batch(queries, K, search)
    got = index.search_with_request(queries, K, search, [])
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_single_buckets_merge_into_the_full_result(built):
    index, _, queries = built
    full = index.search_with_request(queries[:1], K, SEARCH, [list(range(NLIST))])
    pairs = []
    for b in range(NLIST):
        ids, dists = index.search_with_request(queries[:1], K, SEARCH, [[b]])
        pairs += [(d, i) for d, i in zip(dists[0].tolist(), ids[0].tolist()) if i >= 0]
    assert len({i for _, i in pairs}) == len(pairs)          # a vector lives in one bucket only
    pairs.sort()
    assert [i for _, i in pairs[:K]] == full[0][0].tolist()
    assert np.array_equal(np.array([d for d, _ in pairs[:K]], np.float32), full[1][0])


def test_batch_uses_each_querys_own_list(built):
    index, _, queries = built
    lists = [[0, 1], [2], list(range(NLIST)), [5, 3, 4]]
    batch = index.search_with_request(queries[:4], K, SEARCH, lists)
    for i, buckets in enumerate(lists):
        single = index.search_with_request(queries[i:i + 1], K, SEARCH, [buckets])
        assert np.array_equal(batch[0][i], single[0][0]) and np.array_equal(batch[1][i], single[1][0])


@pytest.mark.parametrize("lists,fragment", [
    ([[NLIST + 100]], "out of range"),
    ([[-1]], "out of range"),
    ([[]], "must not be empty"),
    ([[0, 0]], "duplicate bucket_id"),
])
def test_invalid_lists_are_rejected(built, lists, fragment):
    from vsag_b200.index import VsagError

    index, _, queries = built
    with pytest.raises(VsagError) as err:
        index.search_with_request(queries[:1], K, SEARCH, lists)
    assert err.value.code == -3 and fragment in str(err.value)


def test_list_count_must_match_query_count(built):
    from vsag_b200.index import VsagError

    index, _, queries = built
    with pytest.raises(VsagError, match="must match the number of query vectors"):
        index.search_with_request(queries[:2], K, SEARCH, [[0]])


def test_bucket_lists_do_not_mix_with_routing_only_mode(built):
    from vsag_b200.index import VsagError

    index, _, queries = built
    search = json.dumps({"ivf": {"scan_buckets_count": 3, "disable_bucket_scan": True}})
    with pytest.raises(VsagError, match="incompatible with disable_bucket_scan"):
        index.search_with_request(queries[:1], K, search, [[0]])


def test_brute_force_rejects_bucket_lists(oracle):
    from vsag_b200.index import Index, VsagError

    base = oracle.gen_uniform(47, 500 * DIM, 0.1, 0.9).reshape(500, DIM)
    index = Index("brute_force", json.dumps({"dtype": "float32", "metric_type": "l2", "dim": DIM}))
    index.build(base, np.arange(500, dtype=np.int64), 500, DIM)
    want = index.knn_search_batch(base[:3], K, "{}")
    got = index.search_with_request(base[:3], K, "{}")
    assert np.array_equal(got[0], want[0])
    with pytest.raises(VsagError, match="only supported by the ivf index"):
        index.search_with_request(base[:1], K, "{}", [[0]])


def test_enable_reorder_false_answers_like_an_index_without_reorder(oracle):
    """`enable_reorder` (src/algorithm/index_search_parameter.h:46-48): with it off, an index built with
    use_reorder scans for k candidates and returns their quantized distances, which is what the same index
    built without reorder returns (IVF::SearchWithRequest, src/algorithm/ivf/ivf.cpp:2312-2321)."""
    from vsag_b200.index import Index

    base = oracle.gen_uniform(47, N * DIM, 0.1, 0.9).reshape(N, DIM)
    queries = oracle.gen_uniform(48, 8 * DIM, 0.1, 0.9).reshape(8, DIM)
    made = {}
    for reorder in (False, True):
        made[reorder] = Index("ivf", json.dumps({
            "dtype": "float32", "metric_type": "l2", "dim": DIM,
            "index_param": {"buckets_count": NLIST, "base_quantization_type": "sq8", "use_reorder": reorder}}))
        made[reorder].build(base, np.arange(N, dtype=np.int64), N, DIM)
    plain = made[False].knn_search_batch(queries, K, SEARCH)
    off = made[True].knn_search_batch(queries, K, json.dumps({"ivf": {"scan_buckets_count": NLIST, "enable_reorder": False}}))
    on = made[True].knn_search_batch(queries, K, json.dumps({"ivf": {"scan_buckets_count": NLIST, "factor": 3.0}}))
    assert np.array_equal(off[0], plain[0]) and np.array_equal(off[1], plain[1])
    # with reorder the distances are exact fp32 ones and differ from the quantized ones
    exact = ((base[on[0]] - queries[:, None, :]) ** 2).sum(-1)      # of the ids it returned
    np.testing.assert_allclose(on[1], exact, rtol=1e-5)
    assert not np.array_equal(on[1], plain[1])
    # keys the reference's parser does not know are ignored, as IVFSearchParameters::FromJson does
    odd = made[False].knn_search_batch(queries, K, json.dumps({"ivf": {"scan_buckets_count": NLIST, "no_such_key": 1,
                                                                       "parallelism": 4}}))
    assert np.array_equal(odd[0], plain[0])


def test_timeout_stops_the_scan_and_is_reported(engine, oracle):
    """`timeout_ms` (src/algorithm/index_search_parameter.h:35-38): the reference checks its timer between
    buckets, stops scanning and reports is_timeout (src/algorithm/ivf/ivf.cpp:1747-1751).  A budget that has
    passed before the scan starts returns nothing and says so; a generous one changes nothing."""
    n, dim, nlist = 20_000, 32, 64
    from conftest import mixture

    x = mixture(5, n, dim, nlist, 0.15)
    q = mixture(6, 50, dim, nlist, 0.15)
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    ix.train(x, iters=3, init=x[:nlist].copy())
    ix.add(x, np.arange(n, dtype=np.int64))
    want_i, want_d = ix.search(q, 10, 8)
    got_i, got_d, late = ix.search_ex(q, 10, 8, timeout_ms=60_000)
    assert not late and np.array_equal(got_i, want_i) and np.array_equal(got_d, want_d)
    got_i, got_d, late = ix.search_ex(q, 10, 8, timeout_ms=0)
    assert late
    assert np.all(got_i == -1) and np.all(np.isinf(got_d))
    # and the next search is whole again
    got_i, got_d, late = ix.search_ex(q, 10, 8)
    assert not late and np.array_equal(got_i, want_i)
