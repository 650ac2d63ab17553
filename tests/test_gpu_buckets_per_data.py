"""IVF with buckets_per_data > 1: every vector is stored in its b nearest lists (IVF::Add,
src/algorithm/ivf/ivf.cpp:607, :659-676), a search looks for b times as many postings and folds the duplicates
of a vector into its smallest distance (:1722-1727, :1799-1825).  Checked against the oracle's scan over the
same postings followed by that fold."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def fold(ids, dists, k):
    """The reference's de-duplication: smallest distance per id, then the k best."""
    out_i = np.full((len(ids), k), -1, np.int64)
    out_d = np.full((len(ids), k), np.inf, np.float32)
    for q in range(len(ids)):
        best = {}
        for i, d in zip(ids[q].tolist(), dists[q].tolist()):
            if i >= 0 and (i not in best or d < best[i]):
                best[i] = d
        ranked = sorted(best.items(), key=lambda t: (t[1], t[0]))[:k]
        for j, (i, d) in enumerate(ranked):
            out_i[q, j], out_d[q, j] = i, d
    return out_i, out_d


@pytest.mark.parametrize("quant,b", [("sq8", 2), ("fp32", 3)])
def test_postings_and_folded_search_equal_the_oracle(engine, oracle, quant, b):
    n, dim, nlist, k, nprobe = 9000, 32, 30, 10, 8
    x = mixture(3, n, dim, nlist, 0.2)
    q = mixture(4, 200, dim, nlist, 0.2)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    lists, _ = oracle.route(x, centroids, b)                    # a vector's b nearest lists, nearest first
    # postings in the reference's order: vector by vector, list by list; inner id of a posting = its vector
    post_list = lists.reshape(-1)
    post_vec = np.repeat(np.arange(n, dtype=np.int64), b)
    off, order = oracle.build_lists(post_list.astype(np.int32), nlist)
    ids = np.arange(n, dtype=np.int64) * 3 + 7
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8 if quant == "sq8" else engine.QUANT_FP32)
    ix.set_buckets_per_data(b)
    ix.set_centroids(centroids)
    if quant == "sq8":
        lower, diff = oracle.sq8_train(x)
        ix.set_sq8_model(lower, diff)
    half = n // 2
    ix.add(x[:half], ids[:half])                                # the engine routes each vector to its b lists itself
    ix.add(x[half:], ids[half:])
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(sizes, np.diff(off))
    assert np.array_equal(inner, post_vec[order])
    probes, _ = oracle.route(q, centroids, nprobe)
    labels_of_posting = ids[post_vec[order]]
    if quant == "sq8":
        want_codes = oracle.sq8_encode(x[post_vec[order]], lower, diff)
        assert np.array_equal(codes, want_codes)
        raw = oracle.ivf_sq8_search(want_codes, off, labels_of_posting, lower, diff, q, probes, k * b)
    else:
        raw = oracle.ivf_fp32_search(x[post_vec[order]], off, labels_of_posting, q, probes, k * b)
    want = fold(raw[0], raw[1], k)
    got = ix.search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    for row in got[0]:
        live = row[row >= 0]
        assert len(set(live.tolist())) == len(live)            # no vector twice
    # and more lists per vector find more of the true neighbours with the same number of probes
    single = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_FP32)
    single.set_centroids(centroids)
    single.add(x, ids)
    if quant == "fp32":
        exact_i, _ = oracle.bf_search_fp32(x, q, k)
        few = 2
        r_multi = np.mean([len(set(a.tolist()) & set((e * 3 + 7).tolist())) / k for a, e in zip(ix.search(q, k, few)[0], exact_i)])
        r_single = np.mean([len(set(a.tolist()) & set((e * 3 + 7).tolist())) / k for a, e in zip(single.search(q, k, few)[0], exact_i)])
        assert r_multi >= r_single


def test_factory_parameter_and_limits(oracle):
    from vsag_b200.index import Index, VsagError

    n, dim, k = 3000, 24, 10
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, 50 * dim).reshape(50, dim)
    ids = np.arange(n, dtype=np.int64)

    def make(b):
        return Index("ivf", json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                                        "index_param": {"buckets_count": 16, "base_quantization_type": "sq8",
                                                        "buckets_per_data": b}}))
    index = make(2)
    index.build(base, ids, n, dim)
    got_i, got_d = index.knn_search_batch(queries, k, json.dumps({"ivf": {"scan_buckets_count": 16}}))
    plain = make(1)
    plain.build(base, ids, n, dim)
    want_i, want_d = plain.knn_search_batch(queries, k, json.dumps({"ivf": {"scan_buckets_count": 16}}))
    # every list scanned: the folded answer of the doubled index is the plain index's answer
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_i, got_d, want_i, want_d, rtol=0, atol=0)
    with pytest.raises(VsagError):
        make(0)
    with pytest.raises(VsagError):
        make(17)
