"""Multi-rank plumbing on CPU: two gloo ranks exchange per-shard partial results in the layout the
merge kernel expects ([world][nq][k], keys with the distance in the high word).  The merge itself is a
GPU kernel (tests/test_gpu_ivf_sq8.py); here a numpy restatement of it checks that what arrives after
the exchange merges to the global top-k."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def ordered(d: np.ndarray) -> np.ndarray:
    b = d.astype(np.float32).view(np.uint32)
    return np.where(b & 0x80000000, ~b, b | 0x80000000).astype(np.uint32)


def make_keys(dists, payload):
    return (ordered(dists).astype(np.uint64) << np.uint64(32)) | payload.astype(np.uint64)


def numpy_merge(keys_all, labels_all, k):
    """What vb200_merge_partials computes: per query the k smallest keys over all parts."""
    world, nq, kk = keys_all.shape
    flat_k = keys_all.transpose(1, 0, 2).reshape(nq, world * kk)
    flat_l = labels_all.transpose(1, 0, 2).reshape(nq, world * kk)
    order = np.argsort(flat_k, axis=1, kind="stable")[:, :k]
    return np.take_along_axis(flat_l, order, axis=1), np.take_along_axis(flat_k, order, axis=1)


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vsag_b200 import parallel

    nq, k, n = 37, 5, 400
    rng = np.random.default_rng(123)             # same data on every rank
    d = rng.random((nq, n)).astype(np.float32)
    labels = np.arange(n, dtype=np.int64) * 10
    lists = rng.integers(0, 16, n)               # row -> inverted list
    mine = np.array([parallel.owner_of_list(l, world) == rank for l in lists])
    # this rank's partial top-k over the rows whose list it owns
    local = np.where(mine[None, :], d, np.inf)
    idx = np.argsort(local, axis=1, kind="stable")[:, :k]
    ld = np.take_along_axis(local, idx, axis=1)
    keys = make_keys(ld, idx.astype(np.uint32))
    keys[~np.isfinite(ld)] = np.uint64(0xFFFFFFFFFFFFFFFF)
    lab = np.where(np.isfinite(ld), labels[idx], -1)
    keys_local = torch.from_numpy(keys.view(np.int64).copy())
    labels_local = torch.from_numpy(lab.copy())
    keys_all = torch.empty((world, nq, k), dtype=torch.int64)
    labels_all = torch.empty((world, nq, k), dtype=torch.int64)
    parallel.exchange_partials(keys_local, labels_local, keys_all, labels_all, dist)
    got_labels, _ = numpy_merge(keys_all.numpy().view(np.uint64), labels_all.numpy(), k)
    want = labels[np.argsort(d, axis=1, kind="stable")[:, :k]]
    ok = bool(np.array_equal(got_labels, want))
    # every rank sees the same gathered buffer, rank r's block at index r
    same_block = bool(np.array_equal(keys_all[rank].numpy(), keys_local.numpy()))
    # query-sharded routing: every rank ranks the centroids for its slice only (here 37 queries
    # over 2 ranks: 19 + 18, the gathered buffer padded to 2 x 19), all ranks end with all rows
    cents = rng.random((16, 8)).astype(np.float32)
    q = rng.random((nq, 8)).astype(np.float32)

    class FakeIndex:
        calls = []

        def route(self, queries, nprobe, out=None):
            qq = queries.numpy()
            self.calls.append(qq.shape[0])
            dd = ((qq[:, None, :] - cents[None, :, :]) ** 2).sum(-1)
            out.copy_(torch.from_numpy(np.argsort(dd, axis=1, kind="stable")[:, :nprobe].astype(np.int32)))
            return out

    fake = FakeIndex()
    sharded = parallel.ShardedIvfSearch(fake, nq, k, world, torch.device("cpu"), dist, rank)
    probes = sharded._route(torch.from_numpy(q), 4).numpy()
    full = np.argsort(((q[:, None, :] - cents[None, :, :]) ** 2).sum(-1), axis=1, kind="stable")[:, :4]
    lo, hi, per = parallel.query_slice(nq, rank, world)
    routed = bool(np.array_equal(probes, full)) and fake.calls == [hi - lo] and probes.shape == (nq, 4)
    ok = ok and routed
    Path(out_dir, f"rank{rank}.txt").write_text(f"{ok} {same_block}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_exchange_and_merge(tmp_path):
    world, port = 2, 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "True True"


def test_shard_rules():
    from vsag_b200 import parallel

    assert [parallel.owner_of_list(l, 4) for l in range(6)] == [0, 1, 2, 3, 0, 1]
    ranges = [parallel.row_range(10, r, 3) for r in range(3)]
    assert ranges == [(0, 3), (3, 6), (6, 10)]
    assert [parallel.query_slice(37, r, 2) for r in range(2)] == [(0, 19, 19), (19, 37, 19)]
    assert [parallel.query_slice(2, r, 4) for r in range(4)] == [(0, 1, 1), (1, 2, 1), (2, 2, 1), (2, 2, 1)]
    assert parallel.query_slice(10, 0, 1) == (0, 10, 10)
