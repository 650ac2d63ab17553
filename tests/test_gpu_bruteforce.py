"""GPU parity: exact BruteForce kNN (fp32 L2/IP and bf16 IP) against the CPU oracle."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("n,dim,k", [(5000, 128, 10), (777, 7, 1), (3000, 100, 100), (40, 16, 64)])
def test_fp32_matches_oracle(engine, oracle, metric, n, dim, k):
    # base and queries drawn like the reference's fixtures: mt19937 + uniform_real_distribution
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    q = oracle.gen_uniform(48, 64 * dim).reshape(64, dim)
    ids = np.arange(n, dtype=np.int64) + 1000
    ix = engine.BfHandle(dim, metric, engine.QUANT_FP32)
    ix.add(base[: n // 2], ids[: n // 2])
    ix.add(base[n // 2:], ids[n // 2:])
    want_i, want_d = oracle.bf_search_fp32(base, q, k, metric)
    want_i = np.where(want_i >= 0, want_i + 1000, -1)
    got_i, got_d = ix.search(q, k)
    # re-scored distances follow the oracle's FMA order exactly
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_i, got_d, want_i, want_d, rtol=0, atol=0)
    one = ix.search(q[3:4], k)  # the reference's one-query call
    assert np.array_equal(one[0][0], got_i[3]) and np.array_equal(one[1][0], got_d[3])


def test_bf16_ip_matches_oracle(engine, oracle):
    n, dim, k = 6000, 96, 20
    rng = np.random.default_rng(6)
    base = rng.normal(size=(n, dim)).astype(np.float32)
    base /= np.linalg.norm(base, axis=1, keepdims=True)
    q = rng.normal(size=(50, dim)).astype(np.float32)
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    ids = np.arange(n, dtype=np.int64)
    base_bf16 = oracle.float_to_bf16(base)
    want = oracle.bf_search_bf16(base_bf16, q, k, metric=1)
    a = engine.BfHandle(dim, engine.METRIC_IP, engine.QUANT_BF16)
    a.add(base, ids)                      # fp32 rows rounded by the engine
    got = a.search(q, k)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-2, atol=1e-2)
    assert np.array_equal(got[1], want[1])  # in fact the same FMA chain
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    b = engine.BfHandle(dim, engine.METRIC_IP, engine.QUANT_BF16)
    b.add_bf16(base_bf16, ids)            # rows that are already bf16
    got2 = b.search(q, k)
    assert np.array_equal(got2[0], got[0]) and np.array_equal(got2[1], got[1])


def test_edge_cases(engine):
    ix = engine.BfHandle(4, engine.METRIC_L2)
    q = np.zeros((2, 4), np.float32)
    ids, dists = ix.search(q, 3)
    assert np.all(ids == -1) and np.all(np.isinf(dists))
    ix.add(np.eye(4, dtype=np.float32)[:2], np.array([5, 6], np.int64))
    ids, dists = ix.search(q, 3)
    assert sorted(ids[0][:2].tolist()) == [5, 6] and ids[0][2] == -1 and np.isinf(dists[0][2])
    assert np.all(dists[:, :2] == 1.0)
    with pytest.raises(engine.VsagB200Error):
        ix.search(q, 0)
    with pytest.raises(engine.VsagB200Error, match="bf16"):
        ix.add_bf16(np.zeros((1, 4), np.uint16), np.zeros(1, np.int64))


def test_row_sharded_search_equals_unsharded(engine, oracle):
    import torch

    n, dim, k, nq, world = 9000, 32, 10, 100, 2
    base = mixture(1, n, dim, 16, 0.3)
    q = mixture(2, nq, dim, 16, 0.3)
    ids = np.arange(n, dtype=np.int64)
    full = engine.BfHandle(dim, engine.METRIC_L2)
    full.add(base, ids)
    want = full.search(q, k)
    keys = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    labels = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    parts = []
    for r in range(world):
        lo, hi = r * n // world, (r + 1) * n // world
        s = engine.BfHandle(dim, engine.METRIC_L2)
        s.add(base[lo:hi], ids[lo:hi])
        s.search_partial(q, k, keys[r], labels[r])
        parts.append(s)
    got = engine.merge_partials(keys, labels, world, nq, k)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


@pytest.mark.parametrize("metric,quant,n,dim,nq,k", [
    (0, "fp32", 100_000, 128, 2000, 10),
    (1, "fp32", 120_077, 100, 2000, 40),
    (1, "bf16", 150_001, 96, 2000, 100),
    (0, "bf16", 100_000, 128, 1800, 10),
    # bases beyond 64 MB of tiled operand with several query tiles: the interleaved tile schedule
    (0, "fp32", 300_000, 128, 2000, 10),
    (1, "bf16", 700_001, 64, 1000, 20),
])
def test_tensor_core_candidates_equal_simt_path(engine, oracle, metric, quant, n, dim, nq, k):
    """Large searches nominate candidates with the tcgen05 kernel; after the exact re-scoring the
    results must be the ones the fixed-order SIMT path gives, and match the oracle."""
    base = mixture(11, n, dim, 64, 0.25)
    q = mixture(12, nq, dim, 64, 0.25)
    ids = np.arange(n, dtype=np.int64) * 3 + 1
    ix = engine.BfHandle(dim, metric, engine.QUANT_FP32 if quant == "fp32" else engine.QUANT_BF16)
    ix.add(base[:70_000], ids[:70_000])
    ix.add(base[70_000:], ids[70_000:])
    try:
        engine.set_tensor_cores(True)
        before = engine.kernel_launches()
        got_i, got_d = ix.search(q, k)
        tc_launches = engine.kernel_launches() - before
        engine.set_tensor_cores(False)
        before = engine.kernel_launches()
        want_i, want_d = ix.search(q, k)
        simt_launches = engine.kernel_launches() - before
    finally:
        engine.set_tensor_cores(True)
    assert tc_launches > 0 and simt_launches > 0
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_i, got_d, want_i, want_d, rtol=0, atol=0)
    sub = slice(0, 32)
    if quant == "fp32":
        o_i, o_d = oracle.bf_search_fp32(base, q[sub], k, metric)
    else:
        o_i, o_d = oracle.bf_search_bf16(oracle.float_to_bf16(base), q[sub], k, metric=metric)
    o_i = np.where(o_i >= 0, o_i * 3 + 1, -1)
    assert np.array_equal(got_d[sub], o_d)
    assert_topk_equal(got_i[sub], got_d[sub], o_i, o_d, rtol=0, atol=0)
