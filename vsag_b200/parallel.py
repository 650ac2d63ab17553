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


def query_slice(nq: int, rank: int, world: int) -> tuple[int, int, int]:
    """(first, last, per): the rows of a batch of nq queries that `rank` routes, and the common
    slice length `per` = ceil(nq / world) the gathered buffers are padded to."""
    per = (nq + world - 1) // world
    lo = min(nq, rank * per)
    return lo, min(nq, lo + per), per


class _DevicePointer:
    """Presents a raw device pointer to torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False),
                                         "version": 2}


def make_bounds_exchange(dist, device, group=None, seen=None):
    """The callback vb200_ivf_search_partial runs between its two scan phases: an all-reduce with
    MIN over the per-query bounds, so every shard prunes with the tightest bound any shard found.

    torch orders the collective with its current stream, which must be the stream the library
    launches on (both are the default stream unless vb200_set_stream changed it).  `seen`, when
    given, collects the batch sizes the callback was called with (tests)."""
    import torch

    from . import _capi

    views = {}   # (pointer, length) -> tensor over the library's bounds buffer, which is stable between steps

    def exchange(ptr, nq, _stream, _arg):
        try:
            bounds = views.get((ptr, nq))
            if bounds is None:
                bounds = torch.as_tensor(_DevicePointer(ptr, nq), device=device)
                views.clear()
                views[(ptr, nq)] = bounds
            dist.all_reduce(bounds, op=dist.ReduceOp.MIN, group=group)
            if seen is not None:
                seen.append(int(nq))
            return 0
        except Exception:  # an exception must not unwind through the C frames
            import traceback

            traceback.print_exc()
            return 1

    return _capi.EXCHANGE_FN(exchange)


class Comm:
    """A communicator of the library's own (vb200_comm_init: NCCL opened by the shared library), one rank
    per GPU.  The id rank 0 draws travels to the others through an existing torch.distributed group, which
    is used for nothing else; the CUDA device must be selected before."""

    def __init__(self, dist, rank: int, world: int, device):
        import ctypes as C

        import torch

        from . import _capi

        lib = _capi.load()
        ident = np.zeros(128, np.uint8)
        if rank == 0:
            _capi.check(lib.vb200_comm_unique_id(_capi.ptr(ident)))
        on_gpu = getattr(device, "type", str(device)) == "cuda"
        carrier = torch.from_numpy(ident).to(device) if on_gpu else torch.from_numpy(ident)
        dist.broadcast(carrier, src=0)
        ident = carrier.cpu().numpy().copy()
        handle = C.c_void_p()
        _capi.check(lib.vb200_comm_init(C.byref(handle), _capi.ptr(ident), rank, world))
        self.handle, self.rank, self.world, self._lib = handle, rank, world, lib

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._lib.vb200_comm_destroy(self.handle)
            self.handle = None

    __del__ = close


class ShardedIvfSearch:
    """Search step of a list-sharded IVF index on this rank's GPU.

    Routing is query-sharded (every rank holds all centroids and ranks a 1/world slice of the
    batch), the probe lists are all-gathered, every rank scans the lists it owns for the whole
    batch -- first each query's nearest list on the rank, then, after an all-reduce (MIN) of the
    per-query bounds, the others -- and the partial top-k are all-gathered and merged."""

    def __init__(self, index, nq: int, k: int, world: int, device, dist, rank: int = 0, comm=None):
        import torch

        self.index, self.nq, self.k, self.world, self.dist, self.rank = index, nq, k, world, dist, rank
        self.comm = comm   # a Comm: the whole step then runs inside the library (vb200_ivf_search_sharded)
        self.keys_local = torch.empty((nq, k), dtype=torch.int64, device=device)
        self.labels_local = torch.empty((nq, k), dtype=torch.int64, device=device)
        self.keys_all = torch.empty((world, nq, k), dtype=torch.int64, device=device)
        self.labels_all = torch.empty((world, nq, k), dtype=torch.int64, device=device)
        self.device = device
        self._probes_local = None
        self._probes_all = None
        on_gpu = getattr(device, "type", str(device)) == "cuda"
        self._exchange = make_bounds_exchange(dist, device) if world > 1 and on_gpu else None

    def _route(self, queries, nprobe: int):
        import torch

        lo, hi, per = query_slice(self.nq, self.rank, self.world)
        if self._probes_local is None or self._probes_local.shape != (per, nprobe):
            self._probes_local = torch.zeros((per, nprobe), dtype=torch.int32, device=self.device)
            self._probes_all = torch.empty((self.world * per, nprobe), dtype=torch.int32, device=self.device)
        if hi > lo:
            self.index.route(queries[lo:hi], nprobe, out=self._probes_local[: hi - lo])
        self.dist.all_gather_into_tensor(self._probes_all.view(-1), self._probes_local.view(-1))
        return self._probes_all[: self.nq]

    def search(self, queries, nprobe: int, factor: float, out_ids, out_dists):
        from . import _capi

        if self.comm is not None:
            return self.index.search_sharded(self.comm, queries, self.k, nprobe, factor, out=(out_ids, out_dists))

        probes = self._route(queries, nprobe) if self.world > 1 else None
        self.index.search_partial(queries, self.k, nprobe, factor, self.keys_local, self.labels_local,
                                  bucket_ids=probes, exchange=self._exchange)
        exchange_partials(self.keys_local, self.labels_local, self.keys_all, self.labels_all, self.dist)
        _capi.check(_capi.load().vb200_merge_partials(
            _capi.ptr(self.keys_all), _capi.ptr(self.labels_all), self.world, self.nq, self.k,
            _capi.ptr(out_ids), _capi.ptr(out_dists)))
        return out_ids, out_dists
