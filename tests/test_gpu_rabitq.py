"""GPU parity: 1-bit RaBitQ encoder, query transform, IVF scan and fp32 rerank against the oracle."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dim", [7, 64, 100, 960])
def test_encode_and_query_bit_exact(engine, oracle, dim):
    n = 1500 if dim < 960 else 600
    x = mixture(dim, n, dim, 16, 0.05, lo=0.0, hi=1.0, clip=True)
    rot = oracle.random_rotation(dim, seed=dim)
    centroid = oracle.rabitq_train(x, rot)
    want = oracle.rabitq_encode(x, rot, centroid)
    got = engine.rabitq_encode(x, rot, centroid)
    assert got.shape == (n, engine.rabitq_code_size(dim))
    assert np.array_equal(got, want)
    q = mixture(dim + 1, 40, dim, 16, 0.05, lo=0.0, hi=1.0, clip=True)
    assert np.array_equal(engine.rabitq_process_query(q, rot, centroid),
                          oracle.rabitq_process_query(q, rot, centroid))


@pytest.mark.parametrize("n,dim", [(20_000, 48), (1003, 7), (5, 100), (70_001, 960)])
def test_train_centroid_bit_equal_to_oracle(engine, oracle, n, dim):
    x = mixture(3, n, dim, 16, 0.05, lo=0.0, hi=1.0, clip=True)
    rot = oracle.random_rotation(dim, seed=1)
    # the reference keeps a running fp32 sum over the rows in their order (rabitq_quantizer.cpp:229-243);
    # the engine adds in that order too, so the trained centroid is the reference's bit for bit
    assert np.array_equal(engine.rabitq_train(x, rot), oracle.rabitq_train(x, rot))


def test_engine_trained_index_reproduces_oracle_codes(engine, oracle):
    """An index trained by the engine itself (not given a centroid) holds the codes the oracle encodes
    with its own trained centroid: training and encoding are both bit-exact."""
    dim, n, nlist = 64, 6000, 12
    x = mixture(9, n, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    rot = oracle.random_rotation(dim, seed=9)
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_RABITQ)
    ix.set_rabitq_rotation(rot)
    ix.train(x, iters=3)
    centroid = oracle.rabitq_train(x, rot)
    assert np.array_equal(ix.get_rabitq_centroid(), centroid)
    ix.add(x, np.arange(n, dtype=np.int64))
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(codes, oracle.rabitq_encode(x, rot, centroid)[inner])


def build_rabitq(engine, oracle, n, dim, nlist, use_reorder, seed):
    x = mixture(seed, n, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    rot = oracle.random_rotation(dim, seed=seed)
    centroid = oracle.rabitq_train(x, rot)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    labels, _ = oracle.kmeans_assign(x, centroids)
    off, order = oracle.build_lists(labels, nlist)
    codes = oracle.rabitq_encode(x, rot, centroid)[order]
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_RABITQ, use_reorder=use_reorder)
    ix.set_centroids(centroids)
    ix.set_rabitq_rotation(rot)
    ix.set_rabitq_centroid(centroid)
    ix.add(x, np.arange(n, dtype=np.int64))
    return dict(x=x, rot=rot, centroid=centroid, centroids=centroids, off=off, order=order, codes=codes, ix=ix)


@pytest.mark.parametrize("dim,k", [(64, 10), (100, 50), (960, 100)])
def test_scan_matches_oracle(engine, oracle, dim, k):
    n, nlist, nprobe = (6000, 24, 6) if dim < 960 else (3000, 12, 4)
    m = build_rabitq(engine, oracle, n, dim, nlist, False, seed=dim)
    sizes, codes, inner = m["ix"].get_lists()
    assert np.array_equal(codes, m["codes"]) and np.array_equal(inner, m["order"])
    q = mixture(77, 60, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    probes, _ = oracle.route(q, m["centroids"], nprobe)
    qcodes = oracle.rabitq_process_query(q, m["rot"], m["centroid"])
    want = oracle.ivf_rabitq_search(m["codes"], m["off"], m["order"], dim, qcodes, probes, k)
    got = m["ix"].search(q, k, nprobe, bucket_ids=probes)
    # same operation order as the oracle: estimates are bit-equal, ids may differ at ties only
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


def test_rerank_matches_oracle(engine, oracle):
    dim, n, nlist, nprobe, k, factor = 128, 8000, 16, 6, 10, 4.0
    m = build_rabitq(engine, oracle, n, dim, nlist, True, seed=5)
    q = mixture(78, 80, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    probes, _ = oracle.route(q, m["centroids"], nprobe)
    qcodes = oracle.rabitq_process_query(q, m["rot"], m["centroid"])
    cand, _ = oracle.ivf_rabitq_search(m["codes"], m["off"], m["order"], dim, qcodes, probes, int(factor * k))
    want = oracle.rerank_fp32(m["x"], q, cand, k)
    got = m["ix"].search(q, k, nprobe, factor=factor, bucket_ids=probes)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=1e-5, atol=1e-6)
    # the rerank exists to raise recall against exact search over the 1-bit estimate alone
    exact, _ = oracle.bf_search_fp32(m["x"], q, k)

    def recall(ids):
        return np.mean([len(set(a) & set(b)) / k for a, b in zip(ids.tolist(), exact.tolist())])

    assert recall(got[0]) > recall(cand[:, :k])
