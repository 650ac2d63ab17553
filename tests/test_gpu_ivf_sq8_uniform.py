"""GPU parity: IVF with sq8_uniform buckets (SQ8UniformQuantizer,
src/quantization/scalar_quantization/sq8_uniform_quantizer.cpp:76-186) against the CPU oracle: the trained
bound and range, the code records (codes, uint64 norm or fp32 sum) byte for byte, and the distances --
exact integer inner products of the byte codes combined in the reference's operation order -- bit for bit."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def build(engine, oracle, n, dim, nlist, metric, seed):
    x = mixture(seed, n, dim, max(nlist, 2), 0.15)
    x[1, 0] = 50.0                                   # far outside the bulk: stretches the single range
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    if metric == 2:
        centroids = oracle.normalize_rows(centroids)
    labels, _ = oracle.kmeans_assign(x, centroids)
    off, order = oracle.build_lists(labels, nlist)
    model = oracle.sq8u_train(x, metric)
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8_UNIFORM)
    ix.set_centroids(centroids)
    ix.set_sq8_uniform_model(model[0], model[1])
    ids = np.arange(n, dtype=np.int64) * 5 + 11
    half = n // 2
    ix.add(x[:half], ids[:half], labels=labels[:half])
    ix.add(x[half:], ids[half:], labels=labels[half:])
    return dict(x=x, centroids=centroids, labels=labels, off=off, order=order, ids=ids, ix=ix, model=model)


@pytest.mark.parametrize("metric", [0, 1, 2])
@pytest.mark.parametrize("dim,k", [(7, 1), (96, 10), (100, 50)])
def test_records_and_scan_are_bit_exact(engine, oracle, metric, dim, k):
    nlist, nprobe = 40, 9
    m = build(engine, oracle, 12_000, dim, nlist, metric, seed=dim + metric)
    sizes, codes, inner = m["ix"].get_lists()
    assert np.array_equal(sizes, np.diff(m["off"])) and np.array_equal(inner, m["order"])
    want_codes = oracle.sq8u_encode(m["x"][m["order"]], m["model"], metric)
    assert codes.shape == want_codes.shape and np.array_equal(codes, want_codes)
    q = mixture(77, 300, dim, nlist, 0.15)
    q[0] = 1e3                                       # a query beyond the trained range: clamped like a row
    route_metric = 1 if metric == 2 else metric
    q_route = oracle.normalize_rows(q) if metric == 2 else q
    probes, _ = oracle.route(q_route, m["centroids"], nprobe, route_metric)
    probes[3, 2:] = -1
    want = oracle.ivf_sq8u_search(want_codes, m["off"], m["ids"][m["order"]], dim, m["model"], q, probes, k, metric)
    got = m["ix"].search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


@pytest.mark.parametrize("metric", [0, 2])
def test_engine_training_gives_the_oracle_model(engine, oracle, metric):
    n, dim, nlist = 130_000, 16, 8                   # more rows than the 100000-row sample
    x = mixture(5, n, dim, nlist, 0.2)
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8_UNIFORM)
    ix.train(x, iters=1, init=x[:nlist].copy())
    assert np.array_equal(ix.get_sq8_uniform_model(), oracle.sq8u_train(x, metric))


def test_factory_index_with_sq8_uniform_buckets(oracle, tmp_path):
    from vsag_b200.index import Index

    n, dim, nq, k = 4000, 48, 100, 10
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, nq * dim).reshape(nq, dim)
    ids = np.arange(n, dtype=np.int64) + 1
    params = json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                         "index_param": {"buckets_count": 20, "base_quantization_type": "sq8_uniform"}})
    index = Index("ivf", params)
    index.build(base, ids, n, dim)
    search = json.dumps({"ivf": {"scan_buckets_count": 20}})
    got_i, got_d = index.knn_search_batch(queries, k, search)
    model = oracle.sq8u_train(base, 0)
    codes = oracle.sq8u_encode(base, model, 0)
    want = oracle.ivf_sq8u_search(codes, np.array([0, n], np.int64), ids, dim, model, queries,
                                  np.zeros((nq, 1), np.int32), k, 0)
    assert np.array_equal(got_d, want[1])
    assert_topk_equal(got_i, got_d, want[0], want[1], rtol=0, atol=0)
    exact_i, _ = oracle.bf_search_fp32(base, queries, k)
    recall = np.mean([len(set(a.tolist()) & set((b + 1).tolist())) / k for a, b in zip(got_i, exact_i)])
    assert recall > 0.9
    # saved and reloaded: the same answer
    path = tmp_path / "u.idx"
    index.serialize_file(str(path))
    again = Index("ivf", params)
    again.deserialize_file(str(path))
    re_i, re_d = again.knn_search_batch(queries, k, search)
    assert np.array_equal(re_i, got_i) and np.array_equal(re_d, got_d)
