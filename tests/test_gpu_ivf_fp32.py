"""GPU parity: IVF with fp32 buckets (the reference's default base_quantization_type) against the
CPU oracle.  Distances are the reference's own FMA chains, so they are compared bit for bit."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def build(engine, oracle, n, dim, nlist, metric, seed):
    x = mixture(seed, n, dim, max(nlist, 2), 0.15)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    labels, _ = oracle.kmeans_assign(x, centroids)
    off, order = oracle.build_lists(labels, nlist)
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_FP32)
    ix.set_centroids(centroids)
    ids = np.arange(n, dtype=np.int64) * 5 + 11
    half = n // 2
    ix.add(x[:half], ids[:half], labels=labels[:half])
    ix.add(x[half:], ids[half:], labels=labels[half:])
    return dict(x=x, centroids=centroids, labels=labels, off=off, order=order, ids=ids, ix=ix)


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("dim,k", [(7, 1), (96, 10), (100, 50)])
def test_scan_is_bit_exact(engine, oracle, metric, dim, k):
    nlist, nprobe = 40, 9
    m = build(engine, oracle, 15_000, dim, nlist, metric, seed=dim)
    sizes, codes, inner = m["ix"].get_lists()
    assert np.array_equal(sizes, np.diff(m["off"])) and np.array_equal(inner, m["order"])
    assert np.array_equal(codes.view(np.float32).reshape(-1, dim), m["x"][m["order"]])
    q = mixture(77, 300, dim, nlist, 0.15)
    probes, _ = oracle.route(q, m["centroids"], nprobe, metric)
    probes[3, 2:] = -1
    want = oracle.ivf_fp32_search(m["x"][m["order"]], m["off"], m["ids"][m["order"]], q, probes, k, metric)
    got = m["ix"].search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    # routed by the engine itself: same lists except at centroid ties, same answer
    free = oracle.route(q, m["centroids"], nprobe, metric)[0]
    want2 = oracle.ivf_fp32_search(m["x"][m["order"]], m["off"], m["ids"][m["order"]], q, free, k, metric)
    got2 = m["ix"].search(q, k, nprobe)
    assert np.array_equal(got2[1], want2[1])


def test_default_factory_index_is_exact_with_all_buckets(oracle):
    from vsag_b200.index import Index

    n, dim, nq, k = 4000, 48, 100, 10
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, nq * dim).reshape(nq, dim)
    ids = np.arange(n, dtype=np.int64) + 1
    params = json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                         "index_param": {"buckets_count": 20}})      # base_quantization_type defaults to fp32
    index = Index("ivf", params)
    index.build(base, ids, n, dim)
    want_i, want_d = oracle.bf_search_fp32(base, queries, k, 0)
    search = json.dumps({"ivf": {"scan_buckets_count": 20}})
    for i in range(nq):
        got_i, got_d = index.knn_search(queries[i], k, search)
        assert np.array_equal(got_d, want_d[i])
        assert_topk_equal(got_i[None], got_d[None], want_i[i][None] + 1, want_d[i][None], rtol=0, atol=0)
