"""Thin Python handles over the C ABI (include/vsag_b200.h).

Every function takes numpy arrays (host) or torch tensors (host or CUDA) and forwards plain
pointers; all arithmetic happens in libvsag_b200.so on the GPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi
from ._capi import VsagB200Error, check, ptr

METRIC_L2, METRIC_IP, METRIC_COSINE = 0, 1, 2
QUANT_FP32, QUANT_SQ8, QUANT_RABITQ, QUANT_BF16, QUANT_FP16, QUANT_SQ8_UNIFORM = 0, 1, 2, 3, 4, 5
SQ_TRAIN_CLASSIC, SQ_TRAIN_TRUNC_BOUND = 1, 3

METRICS = {"l2": METRIC_L2, "ip": METRIC_IP, "cosine": METRIC_COSINE}


def _is_torch(x) -> bool:
    return hasattr(x, "data_ptr")


def _rows(x) -> int:
    return int(x.shape[0])


def _empty_like_side(ref, shape, dtype):
    """Output buffer on the same side (host numpy / torch device) as `ref`."""
    if _is_torch(ref) and ref.is_cuda:
        import torch

        tdt = {np.float32: torch.float32, np.int64: torch.int64, np.int32: torch.int32,
               np.uint8: torch.uint8}[dtype]
        return torch.empty(shape, dtype=tdt, device=ref.device)
    return np.empty(shape, dtype=dtype)


def device_count() -> int:
    n = _capi.load().vb200_device_count()
    if n < 0:
        check(n)
    return n


def kernel_launches() -> int:
    return int(_capi.load().vb200_kernel_launches())


def set_tensor_cores(enable: bool) -> None:
    """Tensor-core candidate kernels (default) or the fixed-order SIMT kernels."""
    check(_capi.load().vb200_set_tensor_cores(int(bool(enable))))


def set_stream(stream_handle: int | None) -> None:
    check(_capi.load().vb200_set_stream(C.c_void_p(stream_handle or 0)))


# ------------------------------------------------------------------------------------------------
# quantizers and k-means
# ------------------------------------------------------------------------------------------------
def sq8_train(data, mode: int = SQ_TRAIN_TRUNC_BOUND):
    n, d = data.shape
    lower = np.empty(d, np.float32)
    diff = np.empty(d, np.float32)
    check(_capi.load().vb200_sq8_train(ptr(data, np.float32), n, d, mode, ptr(lower), ptr(diff)))
    return lower, diff


def sq8_encode(data, lower, diff):
    n, d = data.shape
    codes = _empty_like_side(data, (n, d), np.uint8)
    check(_capi.load().vb200_sq8_encode(ptr(data, np.float32), n, d, ptr(lower, np.float32),
                                        ptr(diff, np.float32), ptr(codes)))
    return codes


def kmeans_assign(data, centroids, want_err: bool = False):
    n, d = data.shape
    k = _rows(centroids)
    labels = _empty_like_side(data, (n,), np.int32)
    err = C.c_double(0.0)
    check(_capi.load().vb200_kmeans_assign(ptr(data, np.float32), n, d, ptr(centroids, np.float32), k,
                                           ptr(labels), C.byref(err) if want_err else None))
    return (labels, err.value) if want_err else labels


def kmeans_update(data, labels, k: int, it: int = 0):
    n, d = data.shape
    centroids = np.empty((k, d), np.float32)
    counts = np.empty(k, np.int32)
    check(_capi.load().vb200_kmeans_update(ptr(data, np.float32), n, d, ptr(labels, np.int32), k, it,
                                           ptr(centroids), ptr(counts)))
    return centroids, counts


def kmeans_init(data, k: int, seed: int = 47, want_rows: bool = False):
    """k-means++ seeding: k rows of `data` as initial centroids (and their row numbers)."""
    n, d = data.shape
    centroids = _empty_like_side(data, (k, d), np.float32)
    rows = _empty_like_side(data, (k,), np.int64)
    check(_capi.load().vb200_kmeans_init(ptr(data, np.float32), n, d, k, seed, ptr(centroids), ptr(rows)))
    return (centroids, rows) if want_rows else centroids


def kmeans_train(data, init_centroids: np.ndarray, iters: int):
    n, d = data.shape
    if _is_torch(init_centroids):
        centroids = init_centroids.detach().clone().contiguous()
    else:
        centroids = np.ascontiguousarray(init_centroids, dtype=np.float32).copy()
    k = centroids.shape[0]
    labels = _empty_like_side(data, (n,), np.int32)
    err = C.c_double(0.0)
    check(_capi.load().vb200_kmeans_train(ptr(data, np.float32), n, d, k, iters, ptr(centroids),
                                          ptr(labels), C.byref(err)))
    return centroids, labels, err.value


def rabitq_code_size(dim: int) -> int:
    return int(_capi.load().vb200_rabitq_code_size(dim))


def rabitq_train(data, rotation):
    n, d = data.shape
    centroid = np.empty(d, np.float32)
    check(_capi.load().vb200_rabitq_train(ptr(data, np.float32), n, d, ptr(rotation, np.float32),
                                          ptr(centroid)))
    return centroid


def rabitq_encode(data, rotation, centroid):
    n, d = data.shape
    codes = np.empty((n, rabitq_code_size(d)), np.uint8)
    check(_capi.load().vb200_rabitq_encode(ptr(data, np.float32), n, d, ptr(rotation, np.float32),
                                           ptr(centroid, np.float32), ptr(codes)))
    return codes


def rabitq_process_query(queries, rotation, centroid):
    n, d = queries.shape
    out = np.empty((n, d + 1), np.float32)
    check(_capi.load().vb200_rabitq_process_query(ptr(queries, np.float32), n, d,
                                                  ptr(rotation, np.float32), ptr(centroid, np.float32),
                                                  ptr(out)))
    return out


def merge_partials(keys_dev, labels_dev, parts: int, nq: int, k: int, out=None):
    if out is None:
        ids = np.empty((nq, k), np.int64)
        dists = np.empty((nq, k), np.float32)
    else:
        ids, dists = out
    check(_capi.load().vb200_merge_partials(ptr(keys_dev), ptr(labels_dev), parts, nq, k, ptr(ids),
                                            ptr(dists)))
    return ids, dists


# ------------------------------------------------------------------------------------------------
# index handles
# ------------------------------------------------------------------------------------------------
class IvfHandle:
    """Owns a vb200_ivf_t."""

    def __init__(self, dim: int, metric: int, nlist: int, quant: int, use_reorder: bool = False):
        self._lib = _capi.load()
        h = C.c_void_p()
        check(self._lib.vb200_ivf_create(dim, metric, nlist, quant, int(use_reorder), C.byref(h)))
        self._h = h
        self.dim, self.metric, self.nlist, self.quant, self.use_reorder = dim, metric, nlist, quant, use_reorder
        self.n_added = 0     # vectors ever added (removed ones included): the range of inner ids

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.vb200_ivf_destroy(self._h)
            self._h = None

    __del__ = close

    @property
    def code_size(self) -> int:
        if self.quant == QUANT_SQ8:
            return self.dim
        if self.quant in (QUANT_BF16, QUANT_FP16):
            return self.dim * 2
        if self.quant == QUANT_SQ8_UNIFORM:
            align = 8 if self.metric == METRIC_L2 else 4
            return (self.dim + align - 1) // align * align + align
        return self.dim * 4 if self.quant == QUANT_FP32 else rabitq_code_size(self.dim)

    def set_use_residual(self, on: bool = True) -> None:
        check(self._lib.vb200_ivf_set_use_residual(self._h, int(bool(on))))

    def set_buckets_per_data(self, b: int) -> None:
        check(self._lib.vb200_ivf_set_buckets_per_data(self._h, int(b)))

    def set_sq8_uniform_model(self, lower: float, diff: float) -> None:
        check(self._lib.vb200_ivf_set_sq8_uniform_model(self._h, float(lower), float(diff)))

    def get_sq8_uniform_model(self):
        lower, diff = C.c_float(0), C.c_float(0)
        check(self._lib.vb200_ivf_get_sq8_uniform_model(self._h, C.byref(lower), C.byref(diff)))
        return np.array([lower.value, diff.value], np.float32)

    def set_shard(self, rank: int, world: int) -> None:
        check(self._lib.vb200_ivf_set_shard(self._h, rank, world))

    def train(self, data, iters: int = 25, init=None) -> None:
        check(self._lib.vb200_ivf_train(self._h, ptr(data, np.float32), _rows(data), iters,
                                        ptr(init, np.float32)))

    def set_centroids(self, centroids) -> None:
        check(self._lib.vb200_ivf_set_centroids(self._h, ptr(centroids, np.float32)))

    def get_centroids(self) -> np.ndarray:
        out = np.empty((self.nlist, self.dim), np.float32)
        check(self._lib.vb200_ivf_get_centroids(self._h, ptr(out)))
        return out

    def set_sq8_model(self, lower, diff) -> None:
        check(self._lib.vb200_ivf_set_sq8_model(self._h, ptr(lower, np.float32), ptr(diff, np.float32)))

    def get_sq8_model(self):
        lower = np.empty(self.dim, np.float32)
        diff = np.empty(self.dim, np.float32)
        check(self._lib.vb200_ivf_get_sq8_model(self._h, ptr(lower), ptr(diff)))
        return lower, diff

    def set_rabitq_rotation(self, rotation) -> None:
        check(self._lib.vb200_ivf_set_rabitq_rotation(self._h, ptr(rotation, np.float32)))

    def set_rabitq_centroid(self, centroid) -> None:
        check(self._lib.vb200_ivf_set_rabitq_centroid(self._h, ptr(centroid, np.float32)))

    def get_rabitq_centroid(self) -> np.ndarray:
        out = np.empty(self.dim, np.float32)
        check(self._lib.vb200_ivf_get_rabitq_centroid(self._h, ptr(out)))
        return out

    def add(self, data, ids, labels=None) -> None:
        check(self._lib.vb200_ivf_add(self._h, ptr(data, np.float32), _rows(data), ptr(ids, np.int64),
                                      ptr(labels, np.int32)))
        self.n_added += _rows(data)

    def num_elements(self) -> int:
        return int(self._lib.vb200_ivf_num_elements(self._h))

    def memory_usage(self) -> int:
        return int(self._lib.vb200_ivf_memory_usage(self._h))

    def get_lists(self):
        sizes = np.empty(self.nlist, np.int64)
        check(self._lib.vb200_ivf_get_lists(self._h, ptr(sizes), None, None))
        total = int(sizes.sum())
        codes = np.empty((total, self.code_size), np.uint8)
        inner = np.empty(total, np.int64)
        check(self._lib.vb200_ivf_get_lists(self._h, None, ptr(codes), ptr(inner)))
        return sizes, codes, inner

    def set_lists(self, sizes, codes, inner_ids, labels, rows=None) -> None:
        """Fills an empty, trained index from lists that are already encoded (what `get_lists` returns,
        or the bucket datacell and label table of a serialised index); `rows` are the fp32 vectors by
        inner id, needed when reorder is on."""
        sizes = np.ascontiguousarray(sizes, np.int64)
        if sizes.shape != (self.nlist,):
            raise ValueError("sizes must have one entry per list")
        n_total = _rows(labels) if hasattr(labels, "shape") else len(labels)
        if not hasattr(labels, "shape"):
            labels = np.asarray(labels, np.int64)
        check(self._lib.vb200_ivf_set_lists(self._h, ptr(sizes), ptr(codes, np.uint8), ptr(inner_ids, np.int64),
                                            ptr(labels, np.int64), n_total,
                                            ptr(rows, np.float32) if rows is not None else None))
        self.n_added = n_total

    def get_rows(self) -> np.ndarray:
        """The fp32 rows kept for the rerank, by inner id (reorder only)."""
        out = np.empty((self.n_added, self.dim), np.float32)
        check(self._lib.vb200_ivf_get_rows(self._h, ptr(out)))
        return out

    def route(self, queries, nprobe: int, out=None):
        """(bucket ids, centroid distances) as numpy arrays, or with `out` (an int32 [nq, nprobe]
        buffer on either side) only the ids, written there."""
        nq = _rows(queries)
        if out is not None:
            check(self._lib.vb200_ivf_route(self._h, ptr(queries, np.float32), nq, nprobe, ptr(out), None))
            return out
        ids = np.empty((nq, nprobe), np.int32)
        dists = np.empty((nq, nprobe), np.float32)
        check(self._lib.vb200_ivf_route(self._h, ptr(queries, np.float32), nq, nprobe, ptr(ids), ptr(dists)))
        return ids, dists

    def search(self, queries, k: int, nprobe: int, factor: float = 2.0, bucket_ids=None, out=None):
        nq = _rows(queries)
        if out is None:
            ids = _empty_like_side(queries, (nq, k), np.int64)
            dists = _empty_like_side(queries, (nq, k), np.float32)
        else:
            ids, dists = out
        check(self._lib.vb200_ivf_search(self._h, ptr(queries, np.float32), nq, k, nprobe, factor,
                                         ptr(bucket_ids, np.int32), ptr(ids), ptr(dists)))
        return ids, dists

    def remove(self, labels) -> int:
        """Marks the vectors with these labels as removed; returns how many were newly marked."""
        labels = np.ascontiguousarray(labels, np.int64)
        n = C.c_uint64(0)
        check(self._lib.vb200_ivf_remove(self._h, ptr(labels, np.int64), labels.size, C.byref(n)))
        return int(n.value)

    def search_filtered(self, queries, k: int, nprobe: int, factor: float = 2.0, bucket_ids=None,
                        invalid_label_bits=None, deny_inner_bits=None):
        """invalid_label_bits: uint64 words, bit (label & 0xFFFFFFFF) set = filtered out;
        deny_inner_bits: uint32 words over insertion order."""
        nq = _rows(queries)
        ids = _empty_like_side(queries, (nq, k), np.int64)
        dists = _empty_like_side(queries, (nq, k), np.float32)
        f = _capi.Filter()
        if invalid_label_bits is not None:
            invalid_label_bits = np.ascontiguousarray(invalid_label_bits, np.uint64)
            f.invalid_label_bits, f.n_label_bits = invalid_label_bits.ctypes.data, invalid_label_bits.size * 64
        if deny_inner_bits is not None:
            deny_inner_bits = np.ascontiguousarray(deny_inner_bits, np.uint32)
            f.deny_inner_bits, f.n_inner_bits = deny_inner_bits.ctypes.data, deny_inner_bits.size * 32
        check(self._lib.vb200_ivf_search_filtered(self._h, ptr(queries, np.float32), nq, k, nprobe, factor,
                                                  ptr(bucket_ids, np.int32), C.byref(f), ptr(ids), ptr(dists)))
        return ids, dists

    def search_ex(self, queries, k: int, nprobe: int, factor: float = 2.0, bucket_ids=None, enable_reorder: bool = True,
                  timeout_ms=None):
        """vb200_ivf_search_ex: the search with IndexSearchParameter's per-call options; returns
        (ids, dists, timed_out)."""
        nq = _rows(queries)
        ids = _empty_like_side(queries, (nq, k), np.int64)
        dists = _empty_like_side(queries, (nq, k), np.float32)

        class Options(C.Structure):
            _fields_ = [("enable_reorder", C.c_int), ("has_timeout", C.c_int), ("timeout_ms", C.c_double)]

        opt = Options(int(bool(enable_reorder)), int(timeout_ms is not None), float(timeout_ms or 0.0))
        timed_out = C.c_int(0)
        check(self._lib.vb200_ivf_search_ex(self._h, ptr(queries, np.float32), nq, k, nprobe, factor,
                                            ptr(bucket_ids, np.int32), None, C.cast(C.byref(opt), C.c_void_p), ptr(ids),
                                            ptr(dists), C.byref(timed_out)))
        return ids, dists, bool(timed_out.value)

    def search_partial(self, queries, k: int, nprobe: int, factor: float, keys_dev, labels_dev,
                       bucket_ids=None, exchange=None) -> None:
        """exchange: an _capi.EXCHANGE_FN instance (kept alive by the caller) that reduces the
        per-query bounds over the shards, or None."""
        cb = C.cast(exchange, C.c_void_p) if exchange is not None else None
        check(self._lib.vb200_ivf_search_partial(self._h, ptr(queries, np.float32), _rows(queries), k,
                                                 nprobe, factor, ptr(bucket_ids, np.int32), cb, None,
                                                 ptr(keys_dev), ptr(labels_dev)))

    def search_sharded(self, comm, queries, k: int, nprobe: int, factor: float = 2.0, out=None):
        """The whole step of a list-sharded search (vb200_ivf_search_sharded); `comm` is a parallel.Comm.
        Every rank calls it with the same batch and gets the full result."""
        nq = _rows(queries)
        if out is None:
            ids = _empty_like_side(queries, (nq, k), np.int64)
            dists = _empty_like_side(queries, (nq, k), np.float32)
        else:
            ids, dists = out
        check(self._lib.vb200_ivf_search_sharded(self._h, comm.handle, ptr(queries, np.float32), nq, k, nprobe, factor,
                                                 ptr(ids), ptr(dists)))
        return ids, dists

    def last_scanned_bytes(self) -> int:
        """Bytes of codes the last search read after list pruning (<= last_scan_bytes)."""
        return int(self._lib.vb200_ivf_last_scanned_bytes(self._h))

    def set_list_pruning(self, enable: bool) -> None:
        check(self._lib.vb200_ivf_set_list_pruning(self._h, int(bool(enable))))

    def last_scan_bytes(self) -> int:
        return int(self._lib.vb200_ivf_last_scan_bytes(self._h))

    def last_scan_ms(self) -> float:
        ms = C.c_float(0.0)
        check(self._lib.vb200_ivf_last_scan_ms(self._h, C.byref(ms)))
        return float(ms.value)


class BfHandle:
    """Owns a vb200_bf_t."""

    def __init__(self, dim: int, metric: int, quant: int = QUANT_FP32):
        self._lib = _capi.load()
        h = C.c_void_p()
        check(self._lib.vb200_bf_create(dim, metric, quant, C.byref(h)))
        self._h = h
        self.dim, self.metric, self.quant = dim, metric, quant
        self.n_added = 0     # vectors ever added (removed ones included)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.vb200_bf_destroy(self._h)
            self._h = None

    __del__ = close

    def add(self, data, ids) -> None:
        check(self._lib.vb200_bf_add(self._h, ptr(data, np.float32), _rows(data), ptr(ids, np.int64)))
        self.n_added += _rows(data)

    def add_bf16(self, data, ids) -> None:
        check(self._lib.vb200_bf_add_bf16(self._h, ptr(data, np.uint16), _rows(data), ptr(ids, np.int64)))
        self.n_added += _rows(data)

    def get_rows(self) -> np.ndarray:
        """The rows as stored: fp32, or bf16 bit patterns (uint16) for a bf16 index."""
        out = np.empty((self.n_added, self.dim), np.float32 if self.quant == QUANT_FP32 else np.uint16)
        check(self._lib.vb200_bf_get_rows(self._h, ptr(out)))
        return out

    def set_rows(self, rows, ids) -> None:
        """Puts rows from `get_rows` back into an empty index, bit for bit."""
        check(self._lib.vb200_bf_set_rows(self._h, ptr(rows, np.float32 if self.quant == QUANT_FP32 else np.uint16),
                                          _rows(rows), ptr(ids, np.int64)))
        self.n_added = _rows(rows)

    def num_elements(self) -> int:
        return int(self._lib.vb200_bf_num_elements(self._h))

    def search(self, queries, k: int, out=None):
        nq = _rows(queries)
        if out is None:
            ids = _empty_like_side(queries, (nq, k), np.int64)
            dists = _empty_like_side(queries, (nq, k), np.float32)
        else:
            ids, dists = out
        check(self._lib.vb200_bf_search(self._h, ptr(queries, np.float32), nq, k, ptr(ids), ptr(dists)))
        return ids, dists

    def remove(self, labels) -> int:
        labels = np.ascontiguousarray(labels, np.int64)
        n = C.c_uint64(0)
        check(self._lib.vb200_bf_remove(self._h, ptr(labels, np.int64), labels.size, C.byref(n)))
        return int(n.value)

    def search_filtered(self, queries, k: int, invalid_label_bits=None, deny_inner_bits=None):
        nq = _rows(queries)
        ids = _empty_like_side(queries, (nq, k), np.int64)
        dists = _empty_like_side(queries, (nq, k), np.float32)
        f = _capi.Filter()
        if invalid_label_bits is not None:
            invalid_label_bits = np.ascontiguousarray(invalid_label_bits, np.uint64)
            f.invalid_label_bits, f.n_label_bits = invalid_label_bits.ctypes.data, invalid_label_bits.size * 64
        if deny_inner_bits is not None:
            deny_inner_bits = np.ascontiguousarray(deny_inner_bits, np.uint32)
            f.deny_inner_bits, f.n_inner_bits = deny_inner_bits.ctypes.data, deny_inner_bits.size * 32
        check(self._lib.vb200_bf_search_filtered(self._h, ptr(queries, np.float32), nq, k, C.byref(f), ptr(ids),
                                                 ptr(dists)))
        return ids, dists

    def search_partial(self, queries, k: int, keys_dev, labels_dev) -> None:
        check(self._lib.vb200_bf_search_partial(self._h, ptr(queries, np.float32), _rows(queries), k,
                                                ptr(keys_dev), ptr(labels_dev)))

    def search_sharded(self, comm, queries, k: int, out=None):
        """The whole step of a row-sharded search (vb200_bf_search_sharded); `comm` is a parallel.Comm."""
        nq = _rows(queries)
        if out is None:
            ids = _empty_like_side(queries, (nq, k), np.int64)
            dists = _empty_like_side(queries, (nq, k), np.float32)
        else:
            ids, dists = out
        check(self._lib.vb200_bf_search_sharded(self._h, comm.handle, ptr(queries, np.float32), nq, k, ptr(ids),
                                                ptr(dists)))
        return ids, dists


def release_workspaces() -> None:
    """Frees the device workspace vb200_kmeans_train keeps between calls."""
    check(_capi.load().vb200_release_workspaces())


__all__ = [name for name in globals() if not name.startswith("_")]
