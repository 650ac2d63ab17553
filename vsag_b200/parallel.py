"""One process per GPU: list-sharded IVF / row-sharded BruteForce search with one exchange step.

Every rank holds a shard (IVF: lists l with l % world == rank; BruteForce: a contiguous row range),
computes its partial top-k on its own GPU, and the per-shard results -- sortable 64-bit keys with the
distance in the high word, plus the user labels -- are exchanged with one all-gather and merged
locally by vb200_merge_partials.  torch.distributed is only the transport: NCCL over NVLink on GPUs,
gloo in the CPU tests of the plumbing.
"""
from __future__ import annotations

import numpy as np

KEY_INF = np.uint64(0xFFFFFFFFFFFFFFFF)


def owner_of_list(list_id: int, world: int) -> int:
    """Rank that stores inverted list `list_id` (the rule vb200_ivf_set_shard applies)."""
    return int(list_id) % int(world)


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range of `rank` for a row-sharded BruteForce index."""
    return rank * n // world, (rank + 1) * n // world


def exchange_partials(keys_local, labels_local, keys_all, labels_all, dist, group=None):
    """All-gathers the [nq, k] partial results of every rank into [world, nq, k] buffers.

    Tensors live wherever the backend wants them (CUDA for NCCL, CPU for gloo); int64 carries the
    uint64 key bits unchanged."""
    dist.all_gather_into_tensor(keys_all.view(-1), keys_local.view(-1), group=group)
    dist.all_gather_into_tensor(labels_all.view(-1), labels_local.view(-1), group=group)
    return keys_all, labels_all


class ShardedIvfSearch:
    """Search step of a list-sharded IVF index on this rank's GPU."""

    def __init__(self, index, nq: int, k: int, world: int, device, dist):
        import torch

        self.index, self.nq, self.k, self.world, self.dist = index, nq, k, world, dist
        self.keys_local = torch.empty((nq, k), dtype=torch.int64, device=device)
        self.labels_local = torch.empty((nq, k), dtype=torch.int64, device=device)
        self.keys_all = torch.empty((world, nq, k), dtype=torch.int64, device=device)
        self.labels_all = torch.empty((world, nq, k), dtype=torch.int64, device=device)

    def search(self, queries, nprobe: int, factor: float, out_ids, out_dists):
        from . import _capi

        self.index.search_partial(queries, self.k, nprobe, factor, self.keys_local, self.labels_local)
        exchange_partials(self.keys_local, self.labels_local, self.keys_all, self.labels_all, self.dist)
        _capi.check(_capi.load().vb200_merge_partials(
            _capi.ptr(self.keys_all), _capi.ptr(self.labels_all), self.world, self.nq, self.k,
            _capi.ptr(out_ids), _capi.ptr(out_dists)))
        return out_ids, out_dists
