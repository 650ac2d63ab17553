"""GPU parity: an index filled from already-encoded lists (the bucket datacell and label table a
serialised index carries, src/datacell/bucket_datacell.h:891-904, ivf.cpp:990-1000) answers exactly
like the index that encoded them, and like the CPU oracle run over the same lists."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def sq8_model(oracle, n, dim, nlist, seed):
    x = mixture(seed, n, dim, max(nlist, 2), 0.15)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    labels, _ = oracle.kmeans_assign(x, centroids)
    lower, diff = oracle.sq8_train(x)
    off, order = oracle.build_lists(labels, nlist)
    codes = oracle.sq8_encode(x, lower, diff)[order]
    ids = np.arange(n, dtype=np.int64) * 3 + 7
    return dict(x=x, centroids=centroids, lower=lower, diff=diff, off=off, order=order, codes=codes, ids=ids)


def empty_sq8(engine, m, dim, nlist, metric):
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_centroids(m["centroids"])
    ix.set_sq8_model(m["lower"], m["diff"])
    return ix


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("dim", [7, 96, 100])
def test_sq8_lists_from_the_oracle(engine, oracle, metric, dim):
    """Lists encoded by the oracle, never seen as vectors by the engine."""
    n, nlist, nprobe, k = 12_000, 32, 8, 10
    m = sq8_model(oracle, n, dim, nlist, seed=dim)
    ix = empty_sq8(engine, m, dim, nlist, metric)
    ix.set_lists(np.diff(m["off"]), m["codes"], m["order"].astype(np.int64), m["ids"])
    assert ix.num_elements() == n
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(sizes, np.diff(m["off"])) and np.array_equal(codes, m["codes"])
    assert np.array_equal(inner, m["order"])
    q = mixture(91, 200, dim, nlist, 0.15)
    probes, _ = oracle.route(q, m["centroids"], nprobe, metric)
    want = oracle.ivf_sq8_search(m["codes"], m["off"], m["ids"][m["order"]], m["lower"], m["diff"], q, probes, k,
                                 metric)
    got = ix.search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])      # re-scored in the reference's operation order: bit-equal
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    # the loaded index behaves like a built one afterwards: removing and adding both work
    assert ix.remove(m["ids"][:5]) == 5
    ix.add(m["x"][:100], np.arange(100, dtype=np.int64) + 10**9)
    assert ix.num_elements() == n - 5 + 100


def test_roundtrip_equals_the_source_index(engine, oracle):
    """get_lists -> set_lists, host and device buffers: identical answers, bit for bit."""
    import torch

    n, dim, nlist, nprobe, k = 30_000, 64, 48, 12, 20
    m = sq8_model(oracle, n, dim, nlist, seed=3)
    src = empty_sq8(engine, m, dim, nlist, 0)
    src.add(m["x"][: n // 2], m["ids"][: n // 2])
    src.add(m["x"][n // 2:], m["ids"][n // 2:])
    sizes, codes, inner = src.get_lists()
    q = mixture(92, 500, dim, nlist, 0.15)
    want = src.search(q, k, nprobe)
    for device_side in (False, True):
        dst = empty_sq8(engine, m, dim, nlist, 0)
        if device_side:
            dst.set_lists(sizes, torch.from_numpy(codes).cuda(), torch.from_numpy(inner).cuda(),
                          torch.from_numpy(m["ids"]).cuda())
        else:
            dst.set_lists(sizes, codes, inner, m["ids"])
        got = dst.search(q, k, nprobe)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
        dst.close()


def test_shards_keep_their_own_lists(engine, oracle):
    import torch

    n, dim, nlist, nprobe, k, world = 20_000, 32, 40, 10, 10, 2
    m = sq8_model(oracle, n, dim, nlist, seed=4)
    whole = empty_sq8(engine, m, dim, nlist, 0)
    sizes = np.diff(m["off"])
    whole.set_lists(sizes, m["codes"], m["order"].astype(np.int64), m["ids"])
    q = mixture(93, 300, dim, nlist, 0.15)
    want = whole.search(q, k, nprobe)
    keys = torch.empty((world, len(q), k), dtype=torch.int64, device="cuda")
    labels = torch.empty((world, len(q), k), dtype=torch.int64, device="cuda")
    for rank in range(world):
        shard = empty_sq8(engine, m, dim, nlist, 0)
        shard.set_shard(rank, world)
        shard.set_lists(sizes, m["codes"], m["order"].astype(np.int64), m["ids"])
        got_sizes, _, _ = shard.get_lists()
        keep = np.arange(nlist) % world == rank
        assert np.array_equal(got_sizes[keep], sizes[keep]) and not got_sizes[~keep].any()
        shard.search_partial(q, k, nprobe, 1.0, keys[rank], labels[rank])
        shard.close()
    got = engine.merge_partials(keys, labels, world, len(q), k)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)


def test_fp32_and_rabitq_with_reorder(engine, oracle):
    n, dim, nlist, nprobe, k = 8000, 128, 16, 6, 10
    x = mixture(5, n, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    ids = np.arange(n, dtype=np.int64) + 100
    q = mixture(94, 80, dim, nlist, 0.05, lo=0.0, hi=1.0, clip=True)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 3)
    rot = oracle.random_rotation(dim, seed=5)
    centroid = oracle.rabitq_train(x, rot)

    def make(quant, reorder):
        ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, quant, use_reorder=reorder)
        ix.set_centroids(centroids)
        if quant == engine.QUANT_RABITQ:
            ix.set_rabitq_rotation(rot)
            ix.set_rabitq_centroid(centroid)
        return ix

    for quant, reorder in ((engine.QUANT_FP32, False), (engine.QUANT_RABITQ, True)):
        src = make(quant, reorder)
        src.add(x, ids)
        want = src.search(q, k, nprobe, factor=4.0)
        sizes, codes, inner = src.get_lists()
        dst = make(quant, reorder)
        if reorder:
            with pytest.raises(engine.VsagB200Error):
                dst.set_lists(sizes, codes, inner, ids)          # the rerank needs the fp32 rows
        dst.set_lists(sizes, codes, inner, ids, rows=x if reorder else None)
        got = dst.search(q, k, nprobe, factor=4.0)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_rejects_bad_input(engine, oracle):
    n, dim, nlist = 2000, 16, 8
    m = sq8_model(oracle, n, dim, nlist, seed=6)
    sizes = np.diff(m["off"])
    inner = m["order"].astype(np.int64)
    untrained = engine.IvfHandle(dim, 0, nlist, engine.QUANT_SQ8)
    with pytest.raises(engine.VsagB200Error):
        untrained.set_lists(sizes, m["codes"], inner, m["ids"])
    ix = empty_sq8(engine, m, dim, nlist, 0)
    bad = inner.copy()
    bad[17] = n                      # an inner id nothing is labelled with
    with pytest.raises(engine.VsagB200Error):
        ix.set_lists(sizes, m["codes"], bad, m["ids"])
    ix.set_lists(sizes, m["codes"], inner, m["ids"])
    with pytest.raises(engine.VsagB200Error):                      # only an empty index can be filled
        ix.set_lists(sizes, m["codes"], inner, m["ids"])
