"""GPU parity: IVF with half-precision buckets (base_quantization_type "bf16" / "fp16",
src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123) against the CPU oracle: codes are
byte-equal, distances are the reference's fp32 chains over the widened codes of row and query, bit for bit."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def build(engine, oracle, n, dim, nlist, metric, fmt, seed):
    x = mixture(seed, n, dim, max(nlist, 2), 0.15)
    if metric != 2:
        x[0, :] = 0.0                               # fp16 has no zero: 0.0f encodes as 2^-14
    x[1, 0] = 1e6                                   # beyond the fp16 range: the exponent is clamped
    x[2, 0] = 1e-9
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    if metric == 2:
        centroids = oracle.normalize_rows(centroids)
    labels, _ = oracle.kmeans_assign(x, centroids)
    off, order = oracle.build_lists(labels, nlist)
    quant = engine.QUANT_BF16 if fmt == "bf16" else engine.QUANT_FP16
    ix = engine.IvfHandle(dim, metric, nlist, quant)
    ix.set_centroids(centroids)
    ids = np.arange(n, dtype=np.int64) * 5 + 11
    half = n // 2
    ix.add(x[:half], ids[:half], labels=labels[:half])
    ix.add(x[half:], ids[half:], labels=labels[half:])
    stored = oracle.normalize_rows(x) if metric == 2 else x
    return dict(x=x, stored=stored, centroids=centroids, labels=labels, off=off, order=order, ids=ids, ix=ix)


@pytest.mark.parametrize("fmt", ["bf16", "fp16"])
@pytest.mark.parametrize("metric", [0, 1, 2])
@pytest.mark.parametrize("dim,k", [(7, 1), (96, 10), (100, 50)])
def test_codes_and_scan_are_bit_exact(engine, oracle, fmt, metric, dim, k):
    nlist, nprobe = 40, 9
    m = build(engine, oracle, 12_000, dim, nlist, metric, fmt, seed=dim + metric)
    sizes, codes, inner = m["ix"].get_lists()
    assert np.array_equal(sizes, np.diff(m["off"])) and np.array_equal(inner, m["order"])
    want_codes = oracle.float_to_half(m["stored"][m["order"]], fmt)
    assert np.array_equal(codes.view(np.uint16).reshape(-1, dim), want_codes)
    q = mixture(77, 300, dim, nlist, 0.15)
    route_metric = 1 if metric == 2 else metric
    q_route = oracle.normalize_rows(q) if metric == 2 else q
    probes, _ = oracle.route(q_route, m["centroids"], nprobe, route_metric)
    probes[3, 2:] = -1
    want = oracle.ivf_half_search(want_codes, m["off"], m["ids"][m["order"]], q, probes, k, metric, fmt)
    got = m["ix"].search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


@pytest.mark.parametrize("fmt", ["bf16", "fp16"])
def test_factory_index_with_half_precision_buckets(oracle, fmt):
    from vsag_b200.index import Index

    n, dim, nq, k = 4000, 48, 100, 10
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, nq * dim).reshape(nq, dim)
    ids = np.arange(n, dtype=np.int64) + 1
    params = json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim,
                         "index_param": {"buckets_count": 20, "base_quantization_type": fmt}})
    index = Index("ivf", params)
    index.build(base, ids, n, dim)
    got_i, got_d = index.knn_search_batch(queries, k, json.dumps({"ivf": {"scan_buckets_count": 20}}))
    # all buckets scanned: the answer is the exhaustive search over the encoded rows
    codes = oracle.float_to_half(base, fmt)
    off = np.array([0, n], np.int64)
    want = oracle.ivf_half_search(codes, off, ids, queries, np.zeros((nq, 1), np.int32), k, 0, fmt)
    assert np.array_equal(got_d, want[1])
    assert_topk_equal(got_i, got_d, want[0], want[1], rtol=0, atol=0)
    exact_i, _ = oracle.bf_search_fp32(base, queries, k)
    recall = np.mean([len(set(a.tolist()) & set((b + 1).tolist())) / k for a, b in zip(got_i, exact_i)])
    assert recall > 0.95
