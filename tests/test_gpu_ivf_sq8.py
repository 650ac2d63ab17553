"""GPU parity: IVF-SQ8 build layout, routing, list scan with fused top-k, sharding and merge,
against the CPU oracle, through the C ABI."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def build_pair(engine, oracle, n, dim, nlist, metric=0, seed=0, iters=3):
    """Oracle model (centroids, bounds, lists) and an engine index fed with the same model."""
    x = mixture(seed, n, dim, max(nlist, 2), 0.15)
    centroids, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), iters)
    labels, _ = oracle.kmeans_assign(x, centroids)
    lower, diff = oracle.sq8_train(x)
    off, order = oracle.build_lists(labels, nlist)
    codes = oracle.sq8_encode(x, lower, diff)[order]
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_centroids(centroids)
    ix.set_sq8_model(lower, diff)
    ids = np.arange(n, dtype=np.int64) * 3 + 7  # labels differ from inner ids
    return dict(x=x, centroids=centroids, labels=labels, lower=lower, diff=diff, off=off, order=order,
                codes=codes, ids=ids, ix=ix)


@pytest.mark.parametrize("dim", [1, 7, 96, 100])
def test_build_layout_matches_oracle(engine, oracle, dim):
    m = build_pair(engine, oracle, 8000, dim, 24, seed=dim)
    m["ix"].add(m["x"], m["ids"])  # the engine assigns rows itself
    sizes, codes, inner = m["ix"].get_lists()
    assert np.array_equal(sizes, np.diff(m["off"]))
    assert np.array_equal(inner, m["order"])
    assert np.array_equal(codes, m["codes"])
    assert m["ix"].num_elements() == 8000


def test_trained_model_matches_oracle(engine, oracle):
    n, dim, nlist = 20_000, 32, 40
    x = mixture(4, n, dim, nlist, 0.15)
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    ix.train(x, iters=4)
    want_c, _, _, _ = oracle.kmeans_run(x, x[:nlist].copy(), 4)
    # labels and centroid sums (ascending row order) are bit-exact on both sides, so the model is
    assert np.array_equal(ix.get_centroids(), want_c)
    lower, diff = ix.get_sq8_model()
    want_lower, want_diff = oracle.sq8_train(x)
    assert np.array_equal(lower, want_lower) and np.array_equal(diff, want_diff)


def test_incremental_add_equals_single_add(engine, oracle):
    m = build_pair(engine, oracle, 9000, 16, 20, seed=3)
    ix = m["ix"]
    ix.add(m["x"][:4000], m["ids"][:4000])
    ix.add(m["x"][4000:4001], m["ids"][4000:4001])
    ix.add(m["x"][4001:], m["ids"][4001:])
    sizes, codes, inner = ix.get_lists()
    assert np.array_equal(sizes, np.diff(m["off"]))
    assert np.array_equal(inner, m["order"])
    assert np.array_equal(codes, m["codes"])


@pytest.mark.parametrize("metric", [0, 1])
def test_routing_matches_exact_oracle(engine, oracle, metric):
    m = build_pair(engine, oracle, 6000, 48, 200, metric=metric, seed=8)
    q = mixture(80, 300, 48, 200, 0.15)
    for nprobe in (1, 16, 200):
        want_ids, want_d = oracle.route(q, m["centroids"], nprobe, metric)
        got_ids, got_d = m["ix"].route(q, nprobe)
        np.testing.assert_allclose(got_d, want_d, rtol=1e-6, atol=1e-6)
        assert_topk_equal(got_ids, got_d, want_ids, want_d, rtol=1e-6)


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("dim,k", [(96, 10), (7, 1), (100, 100), (1, 5)])
def test_scan_matches_oracle_with_same_buckets(engine, oracle, metric, dim, k):
    nlist = 30
    m = build_pair(engine, oracle, 12_000, dim, nlist, metric=metric, seed=dim + k)
    m["ix"].add(m["x"], m["ids"], labels=m["labels"])
    q = mixture(99, 257, dim, nlist, 0.15)
    probes, _ = oracle.route(q, m["centroids"], 9, metric)
    probes[5, 3:] = -1          # a query with fewer buckets
    probes[6, :] = -1           # and one with none
    want = oracle.ivf_sq8_search(m["codes"], m["off"], m["ids"][m["order"]], m["lower"], m["diff"], q,
                                 probes, k, metric)
    got = m["ix"].search(q, k, 9, bucket_ids=probes)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=1e-5, atol=1e-5)
    # survivors are re-scored in the reference's operation order: distances are bit-equal
    assert np.array_equal(got[1], want[1])
    assert np.all(got[0][6] == -1) and np.all(np.isinf(got[1][6]))
    assert np.all(got[1][:, 1:] >= got[1][:, :-1])  # ascending, +inf padding last


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("dim,k,nlist,nq", [(96, 10, 12, 3000), (100, 100, 8, 700), (7, 3, 5, 500), (128, 10, 40, 2000),
                                            (33, 26, 3, 257)])
def test_tensor_core_scan_equals_simt_scan_and_oracle(engine, oracle, metric, dim, k, nlist, nq):
    """The SQ8 scan as integer MMAs (32-query work items, 128-row tiles, three signed-byte weight terms)
    nominates the survivors the SIMT scan nominates: ids and distances equal the SIMT path's and the
    oracle's.  Lists here are probed by hundreds of queries each (several work items per list) and run
    from a few rows to over a thousand (several tiles, ragged last tile)."""
    n = 9000
    m = build_pair(engine, oracle, n, dim, nlist, metric=metric, seed=dim + nlist)
    m["ix"].add(m["x"], m["ids"], labels=m["labels"])
    q = mixture(300 + dim, nq, dim, nlist, 0.15)
    nprobe = min(nlist, 6)
    probes, _ = oracle.route(q, m["centroids"], nprobe, metric)
    want = oracle.ivf_sq8_search(m["codes"], m["off"], m["ids"][m["order"]], m["lower"], m["diff"], q, probes, k, metric)
    try:
        for pruning in (True, False):
            m["ix"].set_list_pruning(pruning)
            engine.set_tensor_cores(True)
            before = engine.kernel_launches()
            tc = m["ix"].search(q, k, nprobe, bucket_ids=probes)
            tc_launches = engine.kernel_launches() - before
            engine.set_tensor_cores(False)
            simt = m["ix"].search(q, k, nprobe, bucket_ids=probes)
            engine.set_tensor_cores(True)
            assert np.array_equal(tc[1], simt[1]), f"pruning={pruning}"
            assert_topk_equal(tc[0], tc[1], simt[0], simt[1], rtol=0, atol=0)
            assert np.array_equal(tc[1], want[1])
            assert_topk_equal(tc[0], tc[1], want[0], want[1], rtol=0, atol=0)
            assert tc_launches > 0
    finally:
        engine.set_tensor_cores(True)


def test_tensor_core_scan_with_filters_and_removed_rows(engine, oracle):
    """Id filters act on the candidates the tensor-core scan offers exactly as on the SIMT scan's."""
    dim, nlist, k, n = 64, 10, 10, 6000
    m = build_pair(engine, oracle, n, dim, nlist, seed=77)
    m["ix"].add(m["x"], m["ids"], labels=m["labels"])
    q = mixture(78, 400, dim, nlist, 0.15)
    gone = m["ids"][::3]
    assert m["ix"].remove(gone) == gone.size
    deny = np.zeros((n + 31) // 32, np.uint32)
    denied = np.arange(1, n, 7)
    np.bitwise_or.at(deny, denied // 32, (1 << (denied % 32)).astype(np.uint32))
    try:
        engine.set_tensor_cores(True)
        tc = m["ix"].search_filtered(q, k, 5, deny_inner_bits=deny)
        engine.set_tensor_cores(False)
        simt = m["ix"].search_filtered(q, k, 5, deny_inner_bits=deny)
    finally:
        engine.set_tensor_cores(True)
    assert np.array_equal(tc[1], simt[1])
    assert_topk_equal(tc[0], tc[1], simt[0], simt[1], rtol=0, atol=0)
    banned = set(gone.tolist()) | set(m["ids"][denied].tolist())
    assert not (set(tc[0].ravel().tolist()) & banned)


def test_ragged_lists(engine, oracle):
    """List lengths 0, 1, 31, 32, 33, 127, 128, 129, 300 (the reference scans 32 codes at a time,
    the engine 128 rows per pass)."""
    dim = 24
    lens = [0, 1, 31, 32, 33, 127, 128, 129, 300, 0]
    nlist = len(lens)
    labels = np.concatenate([np.full(c, l, np.int32) for l, c in enumerate(lens)])
    rng = np.random.default_rng(0)
    rng.shuffle(labels)
    n = labels.size
    x = mixture(5, n, dim, 8, 0.2)
    lower, diff = oracle.sq8_train(x)
    off, order = oracle.build_lists(labels, nlist)
    codes = oracle.sq8_encode(x, lower, diff)[order]
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    ix.set_centroids(mixture(6, nlist, dim, 8, 0.2))
    ix.set_sq8_model(lower, diff)
    ids = np.arange(n, dtype=np.int64)
    ix.add(x, ids, labels=labels)
    sizes, got_codes, inner = ix.get_lists()
    assert sizes.tolist() == lens and np.array_equal(got_codes, codes) and np.array_equal(inner, order)
    q = mixture(7, 40, dim, 8, 0.2)
    probes = np.tile(np.arange(nlist, dtype=np.int32), (40, 1))
    for k in (1, 10, 400):
        want = oracle.ivf_sq8_search(codes, off, order, lower, diff, q, probes, k)
        got = ix.search(q, k, nlist, bucket_ids=probes)
        assert_topk_equal(got[0], got[1], want[0], want[1], rtol=1e-5, atol=1e-5)


def test_end_to_end_search_matches_oracle_pipeline(engine, oracle):
    dim, nlist, k, nprobe = 96, 64, 10, 8
    m = build_pair(engine, oracle, 30_000, dim, nlist, seed=21)
    m["ix"].add(m["x"], m["ids"])
    q = mixture(22, 500, dim, nlist, 0.15)
    probes, _ = oracle.route(q, m["centroids"], nprobe)
    want = oracle.ivf_sq8_search(m["codes"], m["off"], m["ids"][m["order"]], m["lower"], m["diff"], q,
                                 probes, k)
    got = m["ix"].search(q, k, nprobe)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=1e-5, atol=1e-5)
    # single-query calls give the rows of the batched call (the reference's batch branch loops
    # over queries, ivf.cpp:2137-2210)
    for i in (0, 17, 499):
        one = m["ix"].search(q[i:i + 1], k, nprobe)
        assert np.array_equal(one[0][0], got[0][i]) and np.array_equal(one[1][0], got[1][i])
    assert m["ix"].last_scan_bytes() == int(dim) * int(np.sum(np.diff(m["off"])[probes[499]]))


def test_device_resident_queries_and_outputs(engine, oracle):
    import torch

    m = build_pair(engine, oracle, 10_000, 32, 16, seed=31)
    m["ix"].add(torch.from_numpy(m["x"]).cuda(), torch.from_numpy(m["ids"]).cuda())
    q = mixture(32, 64, 32, 16, 0.15)
    host = m["ix"].search(q, 5, 4)
    dev = m["ix"].search(torch.from_numpy(q).cuda(), 5, 4)
    assert dev[0].is_cuda and np.array_equal(dev[0].cpu().numpy(), host[0])
    assert np.array_equal(dev[1].cpu().numpy(), host[1])


def test_search_edge_cases(engine, oracle):
    dim, nlist = 8, 4
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    q = np.zeros((3, dim), np.float32)
    with pytest.raises(engine.VsagB200Error, match="not trained"):
        ix.search(q, 5, 2)
    x = mixture(1, 50, dim, 4, 0.2)
    ix.train(x, iters=2)
    ids, dists = ix.search(q, 5, 2)           # trained but empty
    assert np.all(ids == -1) and np.all(np.isinf(dists))
    ix.add(x[:3], np.array([100, 200, 300], np.int64))
    ids, dists = ix.search(q, 5, 99)          # nprobe clamps to nlist, k exceeds the population
    assert sorted(ids[0][:3].tolist()) == [100, 200, 300] and np.all(ids[:, 3:] == -1)
    with pytest.raises(engine.VsagB200Error):
        ix.search(q, 0, 2)
    with pytest.raises(engine.VsagB200Error):
        ix.search(q, 5, 0)
    empty = ix.search(np.zeros((0, dim), np.float32), 5, 2)
    assert empty[0].shape == (0, 5)
    with pytest.raises(engine.VsagB200Error, match="precede"):
        ix.set_shard(0, 2)


def test_list_sharded_search_equals_unsharded(engine, oracle):
    """Two shards on one GPU (lists dealt round-robin), partial results merged the way the ranks
    merge them after the all-gather."""
    import torch

    dim, nlist, k, nprobe, nq = 32, 48, 10, 12, 200
    m = build_pair(engine, oracle, 20_000, dim, nlist, seed=41)
    m["ix"].add(m["x"], m["ids"])
    q = mixture(42, nq, dim, nlist, 0.15)
    want = m["ix"].search(q, k, nprobe)
    world = 3
    keys = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    labels = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    shards = []
    for r in range(world):
        s = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
        s.set_shard(r, world)
        s.set_centroids(m["centroids"])
        s.set_sq8_model(m["lower"], m["diff"])
        s.add(m["x"], m["ids"])
        sizes, _, _ = s.get_lists()
        assert np.all(sizes[np.arange(nlist) % world != r] == 0)
        s.search_partial(q, k, nprobe, 2.0, keys[r], labels[r])
        shards.append(s)
    got = engine.merge_partials(keys, labels, world, nq, k)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    # the same with the probe lists handed in (the ranks route disjoint slices of the batch and
    # share them), on either side of the bus, and merged twice through the kept workspace
    probes, _ = m["ix"].route(q, nprobe)
    probes_dev = torch.empty((nq, nprobe), dtype=torch.int32, device="cuda")
    m["ix"].route(torch.from_numpy(q).cuda(), nprobe, out=probes_dev)
    assert np.array_equal(probes_dev.cpu().numpy(), probes)
    for r in range(world):
        shards[r].search_partial(q, k, nprobe, 2.0, keys[r], labels[r],
                                 bucket_ids=probes if r == 0 else probes_dev)
    for _ in range(2):
        again = engine.merge_partials(keys, labels, world, nq, k)
        assert np.array_equal(again[0], got[0]) and np.array_equal(again[1], got[1])


def test_bound_exchange_between_shards(engine, oracle):
    """Three shards on one GPU take turns: a first pass collects the bounds each shard finds after
    its nearest lists, a second pass hands every shard the minimum over all of them through the
    exchange callback.  Results equal the unsharded search either way."""
    import torch

    from vsag_b200 import _capi, parallel

    dim, nlist, k, nprobe, nq, world = 32, 48, 10, 12, 200, 3
    m = build_pair(engine, oracle, 20_000, dim, nlist, seed=43)
    m["ix"].add(m["x"], m["ids"])
    q = mixture(44, nq, dim, nlist, 0.15)
    want = m["ix"].search(q, k, nprobe)
    shards = []
    for r in range(world):
        s = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
        s.set_shard(r, world)
        s.set_centroids(m["centroids"])
        s.set_sq8_model(m["lower"], m["diff"])
        s.add(m["x"], m["ids"])
        shards.append(s)
    keys = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    labels = torch.empty((world, nq, k), dtype=torch.int64, device="cuda")
    local_bounds = []

    def record(ptr, n, _stream, _arg):
        b = torch.as_tensor(parallel._DevicePointer(ptr, n), device="cuda")
        local_bounds.append(b.clone())
        return 0

    cb = _capi.EXCHANGE_FN(record)
    for r in range(world):
        shards[r].search_partial(q, k, nprobe, 2.0, keys[r], labels[r], exchange=cb)
    plain = engine.merge_partials(keys, labels, world, nq, k)
    assert_topk_equal(plain[0], plain[1], want[0], want[1], rtol=0, atol=0)
    assert len(local_bounds) == world and all(b.shape == (nq,) for b in local_bounds)
    tightest = torch.stack(local_bounds).min(dim=0).values
    assert torch.isfinite(tightest).all()

    def reduce_min(ptr, n, _stream, _arg):
        b = torch.as_tensor(parallel._DevicePointer(ptr, n), device="cuda")
        torch.minimum(b, tightest, out=b)
        return 0

    cb2 = _capi.EXCHANGE_FN(reduce_min)
    for r in range(world):
        shards[r].search_partial(q, k, nprobe, 2.0, keys[r], labels[r], exchange=cb2)
    got = engine.merge_partials(keys, labels, world, nq, k)
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    # the bounds that come back are the ones the second phase prunes with: with a bound of zero
    # only what each shard found in its nearest list is left, which is worse somewhere
    zero = _capi.EXCHANGE_FN(lambda ptr, n, _s, _a: int(
        torch.as_tensor(parallel._DevicePointer(ptr, n), device="cuda").zero_().numel() != n))
    for r in range(world):
        shards[r].search_partial(q, k, nprobe, 2.0, keys[r], labels[r], exchange=zero)
    pruned = engine.merge_partials(keys, labels, world, nq, k)
    assert np.all(pruned[1] >= want[1]) and np.any(pruned[1] > want[1])
    # a failing callback is reported, not swallowed
    bad = _capi.EXCHANGE_FN(lambda *_: 7)
    with pytest.raises(engine.VsagB200Error, match="exchange"):
        shards[0].search_partial(q, k, nprobe, 2.0, keys[0], labels[0], exchange=bad)
    shards[0].search_partial(q, k, nprobe, 2.0, keys[0], labels[0])   # the handle is still usable


@pytest.mark.parametrize("metric", [0, 1])
def test_tensor_core_routing_equals_simt_and_oracle(engine, oracle, metric):
    """Batches of 256+ queries over 1024+ lists nominate their probe lists with the tcgen05 kernel;
    after the exact re-scoring the lists and distances are those of the SIMT path and the oracle."""
    dim, nlist, nq, nprobe = 96, 2048, 700, 40
    cents = mixture(51, nlist, dim, 64, 0.3)
    q = mixture(52, nq, dim, 64, 0.3)
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_centroids(cents)
    try:
        engine.set_tensor_cores(True)
        before = engine.kernel_launches()
        got_ids, got_d = ix.route(q, nprobe)
        tc_launches = engine.kernel_launches() - before
        engine.set_tensor_cores(False)
        before = engine.kernel_launches()
        simt_ids, simt_d = ix.route(q, nprobe)
        simt_launches = engine.kernel_launches() - before
    finally:
        engine.set_tensor_cores(True)
    assert tc_launches != simt_launches
    assert np.array_equal(got_d, simt_d)
    assert_topk_equal(got_ids, got_d, simt_ids, simt_d, rtol=0, atol=0)
    want_ids, want_d = oracle.route(q, cents, nprobe, metric)
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_ids, got_d, want_ids, want_d, rtol=0, atol=0)


@pytest.mark.parametrize("metric,nlist,nprobe,dup", [(0, 4096, 64, False), (1, 4096, 20, False), (0, 8192, 130, False),
                                                     (0, 4096, 64, True)])
def test_threshold_routing_equals_oracle(engine, oracle, metric, nlist, nprobe, dup):
    """From 4096 lists on, routing keeps no score matrix: a threshold per query from a sample of the
    centroids, one tensor-core pass that keeps what scores below it, exact re-scoring of the best.  The
    probe lists and distances are the oracle's bit for bit -- also when many centroids coincide, which
    piles candidates at one score (a query whose candidate lists overflow is answered inside the pick
    kernel from exact distances to every centroid)."""
    dim, nq = 96, 600
    cents = mixture(71 + nlist, nlist, dim, 200, 0.3)
    if dup:
        cents[1000:3000] = cents[999]          # 2001 coincident centroids: ties, lowest id first
    q = mixture(72, nq, dim, 200, 0.3)
    if dup:
        q[:50] = cents[999] + 0.01 * q[:50]    # queries whose nearest centroids are the coincident ones
    ix = engine.IvfHandle(dim, metric, nlist, engine.QUANT_SQ8)
    ix.set_centroids(cents)
    got_ids, got_d = ix.route(q, nprobe)
    want_ids, want_d = oracle.route(q, cents, nprobe, metric)
    assert np.array_equal(got_d, want_d)
    assert_topk_equal(got_ids, got_d, want_ids, want_d, rtol=0, atol=0)
    if dup:
        assert np.array_equal(got_ids[:50], want_ids[:50])   # ties broken by list id on both sides


@pytest.mark.parametrize("metric", [0, 1])
def test_list_pruning_changes_nothing_but_the_bytes_read(engine, oracle, metric):
    """A (query, list) pair is dropped when the list's ball around its centroid lies beyond the
    query's current bound; the answer must be the one of the full scan (and of the oracle), with
    fewer code bytes read on clustered data."""
    # enough (list, query tile) items that most start after the first bounds exist
    dim, nlist, k, nprobe, nq = 32, 256, 10, 24, 4000
    m = build_pair(engine, oracle, 60_000, dim, nlist, metric=metric, seed=61)
    m["ix"].add(m["x"][:22_000], m["ids"][:22_000], labels=m["labels"][:22_000])
    m["ix"].add(m["x"][22_000:], m["ids"][22_000:], labels=m["labels"][22_000:])   # radii follow incremental adds
    q = mixture(62, nq, dim, nlist, 0.15)
    pruned = m["ix"].search(q, k, nprobe)
    logical, touched = m["ix"].last_scan_bytes(), m["ix"].last_scanned_bytes()
    m["ix"].set_list_pruning(False)
    full = m["ix"].search(q, k, nprobe)
    assert m["ix"].last_scanned_bytes() == m["ix"].last_scan_bytes() == logical
    m["ix"].set_list_pruning(True)
    assert np.array_equal(pruned[0], full[0]) and np.array_equal(pruned[1], full[1])
    assert 0 < touched < logical
    sub = slice(0, 400)
    probes, _ = oracle.route(q[sub], m["centroids"], nprobe, metric)
    want = oracle.ivf_sq8_search(m["codes"], m["off"], m["ids"][m["order"]], m["lower"], m["diff"], q[sub], probes,
                                 k, metric)
    assert np.array_equal(pruned[1][sub], want[1])
    assert_topk_equal(pruned[0][sub], pruned[1][sub], want[0], want[1], rtol=1e-5, atol=1e-5)
    with pytest.raises(engine.VsagB200Error):
        m["ix"].set_centroids(m["centroids"])   # would invalidate lists and radii
