"""Python face of the Factory / Index mirror, shaped like the reference's pyvsag.Index
(python_bindings/index_binding.cpp:629-900): Index(name, parameters_json), build, add, knn_search.
It calls the vsag_index_* C functions exported by libvsag_b200.so (the names of the reference's
include/vsag/vsag_c_api.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi


class _Error(C.Structure):
    _fields_ = [("code", C.c_int), ("message", C.c_char * 1024)]


class _SearchResult(C.Structure):
    _fields_ = [("dists", C.POINTER(C.c_float)), ("ids", C.POINTER(C.c_int64)), ("count", C.c_int64),
                ("other_result", C.c_void_p)]


class VsagError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


_bound = False


def _lib():
    global _bound
    lib = _capi.load()
    if not _bound:
        lib.vsag_index_factory.restype = C.c_void_p
        lib.vsag_index_factory.argtypes = [C.c_char_p, C.c_char_p]
        lib.vsag_index_factory_error.restype = C.c_char_p
        lib.vsag_index_destroy.restype = _Error
        lib.vsag_index_destroy.argtypes = [C.c_void_p]
        for name in ("vsag_index_build", "vsag_index_add", "vsag_index_train"):
            fn = getattr(lib, name)
            fn.restype = _Error
            fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64]
        lib.vsag_index_knn_search.restype = _Error
        lib.vsag_index_knn_search.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int64, C.c_char_p,
                                              C.POINTER(_SearchResult)]
        lib.vsag_index_knn_search_batch.restype = _Error
        lib.vsag_index_knn_search_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int64,
                                                    C.c_char_p, C.c_void_p, C.c_void_p]
        lib.vsag_index_search_with_request.restype = _Error
        lib.vsag_index_search_with_request.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int64,
                                                       C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.vsag_index_knn_search_filtered.restype = _Error
        lib.vsag_index_knn_search_filtered.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int64, C.c_char_p,
                                                       C.c_void_p, C.c_uint64, C.c_int64, C.POINTER(_SearchResult)]
        lib.vsag_index_remove.restype = _Error
        lib.vsag_index_remove.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32)]
        lib.vsag_index_knn_search_with_filter.restype = _Error
        lib.vsag_index_knn_search_with_filter.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int64, C.c_char_p,
                                                          _FILTER_FUNC, C.POINTER(_SearchResult)]
        lib.vsag_index_range_search_with_filter.restype = _Error
        lib.vsag_index_range_search_with_filter.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_float, C.c_int64,
                                                            C.c_char_p, _FILTER_FUNC, C.POINTER(_SearchResult)]
        lib.vsag_index_range_search.restype = _Error
        lib.vsag_index_range_search.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_float, C.c_int64, C.c_char_p,
                                                C.POINTER(_SearchResult)]
        for fn in (lib.vsag_serialize_file, lib.vsag_deserialize_file):
            fn.restype = _Error
            fn.argtypes = [C.c_void_p, C.c_char_p]
        lib.vsag_index_get_num_elements.restype = C.c_int64
        lib.vsag_index_get_num_elements.argtypes = [C.c_void_p]
        _bound = True
    return lib


_FILTER_FUNC = C.CFUNCTYPE(C.c_bool, C.c_int64)   # FilterFunc_t: True = the id may be returned


def _check(err: _Error) -> None:
    if err.code != 0:
        raise VsagError(err.code, err.message.decode("utf-8", "replace"))


class Index:
    """vsag.Index(name, parameters): "ivf" or "brute_force" with the reference's JSON parameters."""

    def __init__(self, name: str, parameters: str):
        lib = _lib()
        self._h = lib.vsag_index_factory(name.encode(), parameters.encode())
        if not self._h:
            msg = lib.vsag_index_factory_error().decode("utf-8", "replace")
            raise VsagError(-3 if "unsupported" not in msg else -7, msg)

    def __del__(self):
        if getattr(self, "_h", None):
            _lib().vsag_index_destroy(self._h)
            self._h = None

    @staticmethod
    def _rows(vectors, ids, num_elements, dim):
        vectors = np.ascontiguousarray(vectors, np.float32).reshape(num_elements, dim)
        ids = np.ascontiguousarray(ids, np.int64)
        return vectors, ids

    def build(self, vectors, ids, num_elements: int, dim: int) -> None:
        vectors, ids = self._rows(vectors, ids, num_elements, dim)
        _check(_lib().vsag_index_build(self._h, vectors.ctypes.data, ids.ctypes.data, dim, num_elements))

    def add(self, vectors, ids, num_elements: int, dim: int) -> None:
        vectors, ids = self._rows(vectors, ids, num_elements, dim)
        _check(_lib().vsag_index_add(self._h, vectors.ctypes.data, ids.ctypes.data, dim, num_elements))

    def train(self, vectors, num_elements: int, dim: int) -> None:
        vectors = np.ascontiguousarray(vectors, np.float32).reshape(num_elements, dim)
        _check(_lib().vsag_index_train(self._h, vectors.ctypes.data, None, dim, num_elements))

    def knn_search(self, vector, k: int, parameters: str = "{}"):
        """One query -> (ids, dists) of the entries found (at most k), ascending by distance."""
        vector = np.ascontiguousarray(vector, np.float32).reshape(-1)
        ids = np.empty(max(k, 1), np.int64)
        dists = np.empty(max(k, 1), np.float32)
        res = _SearchResult(dists.ctypes.data_as(C.POINTER(C.c_float)), ids.ctypes.data_as(C.POINTER(C.c_int64)), 0, None)
        _check(_lib().vsag_index_knn_search(self._h, vector.ctypes.data, vector.size, k, parameters.encode(),
                                            C.byref(res)))
        return ids[: res.count].copy(), dists[: res.count].copy()

    def knn_search_filtered(self, vector, k: int, parameters: str = "{}", invalid_ids=None, deny_modulus: int = 0):
        """knn_search with a pre-filter: `invalid_ids` become the bitset of filtered-out ids;
        `deny_modulus` > 0 filters every id divisible by it through the callback overload."""
        vector = np.ascontiguousarray(vector, np.float32).reshape(-1)
        ids = np.empty(max(k, 1), np.int64)
        dists = np.empty(max(k, 1), np.float32)
        res = _SearchResult(dists.ctypes.data_as(C.POINTER(C.c_float)), ids.ctypes.data_as(C.POINTER(C.c_int64)), 0, None)
        words = None
        if invalid_ids is not None and len(invalid_ids) > 0:
            invalid_ids = np.asarray(invalid_ids, np.int64) & 0xFFFFFFFF
            words = np.zeros(int(invalid_ids.max()) // 64 + 1, np.uint64)
            np.bitwise_or.at(words, invalid_ids // 64, np.uint64(1) << (invalid_ids % 64).astype(np.uint64))
        _check(_lib().vsag_index_knn_search_filtered(
            self._h, vector.ctypes.data, vector.size, k, parameters.encode(),
            None if words is None else words.ctypes.data, 0 if words is None else words.size, deny_modulus,
            C.byref(res)))
        return ids[: res.count].copy(), dists[: res.count].copy()

    def remove(self, ids) -> int:
        """Index::Remove with MARK_REMOVE: how many of the ids were found and newly marked."""
        ids = np.ascontiguousarray(ids, np.int64)
        removed = C.c_uint32(0)
        _check(_lib().vsag_index_remove(self._h, ids.ctypes.data, ids.size, C.byref(removed)))
        return int(removed.value)

    def range_search(self, vector, radius: float, k: int, parameters: str = "{}"):
        """vsag_index_range_search: the nearest k of the vectors within `radius`, ascending; k < 0 asks
        for all of them."""
        vector = np.ascontiguousarray(vector, np.float32).reshape(-1)
        room = k if k > 0 else max(1, self.get_num_elements())
        ids = np.empty(room, np.int64)
        dists = np.empty(room, np.float32)
        res = _SearchResult(dists.ctypes.data_as(C.POINTER(C.c_float)), ids.ctypes.data_as(C.POINTER(C.c_int64)), 0, None)
        _check(_lib().vsag_index_range_search(self._h, vector.ctypes.data, vector.size, radius, k, parameters.encode(),
                                              C.byref(res)))
        return ids[: res.count].copy(), dists[: res.count].copy()

    def knn_search_with_filter(self, vector, k: int, parameters: str, valid):
        """vsag_index_knn_search_with_filter: `valid(id)` says which ids may be returned."""
        vector = np.ascontiguousarray(vector, np.float32).reshape(-1)
        ids = np.empty(max(k, 1), np.int64)
        dists = np.empty(max(k, 1), np.float32)
        res = _SearchResult(dists.ctypes.data_as(C.POINTER(C.c_float)), ids.ctypes.data_as(C.POINTER(C.c_int64)), 0, None)
        cb = _FILTER_FUNC(lambda i: bool(valid(i)))
        _check(_lib().vsag_index_knn_search_with_filter(self._h, vector.ctypes.data, vector.size, k,
                                                        parameters.encode(), cb, C.byref(res)))
        return ids[: res.count].copy(), dists[: res.count].copy()

    def range_search_with_filter(self, vector, radius: float, k: int, parameters: str, valid):
        """vsag_index_range_search_with_filter: the nearest k valid vectors within `radius`."""
        vector = np.ascontiguousarray(vector, np.float32).reshape(-1)
        ids = np.empty(max(k, 1), np.int64)
        dists = np.empty(max(k, 1), np.float32)
        res = _SearchResult(dists.ctypes.data_as(C.POINTER(C.c_float)), ids.ctypes.data_as(C.POINTER(C.c_int64)), 0, None)
        cb = _FILTER_FUNC(lambda i: bool(valid(i)))
        _check(_lib().vsag_index_range_search_with_filter(self._h, vector.ctypes.data, vector.size, radius, k,
                                                          parameters.encode(), cb, C.byref(res)))
        return ids[: res.count].copy(), dists[: res.count].copy()

    def serialize_file(self, path: str) -> None:
        """vsag_serialize_file: the whole index (model, lists, labels, removed ids) to one file."""
        _check(_lib().vsag_serialize_file(self._h, str(path).encode()))

    def deserialize_file(self, path: str) -> None:
        """vsag_deserialize_file into an empty index created with the same parameters."""
        _check(_lib().vsag_deserialize_file(self._h, str(path).encode()))

    def knn_search_batch(self, vectors, k: int, parameters: str = "{}"):
        """nq queries -> ids[nq, k], dists[nq, k] padded with -1 / +inf."""
        vectors = np.ascontiguousarray(vectors, np.float32)
        nq, dim = vectors.shape
        ids = np.empty((nq, k), np.int64)
        dists = np.empty((nq, k), np.float32)
        _check(_lib().vsag_index_knn_search_batch(self._h, vectors.ctypes.data, dim, nq, k, parameters.encode(),
                                                  ids.ctypes.data, dists.ctypes.data))
        return ids, dists

    def search_with_request(self, vectors, k: int, parameters: str = "{}", bucket_ids=None):
        """Index::SearchWithRequest for nq queries: `bucket_ids` is a list with, per query, the list of
        buckets to scan instead of routing (SearchRequest::bucket_ids_); None or [] = default routing."""
        vectors = np.ascontiguousarray(vectors, np.float32)
        nq, dim = vectors.shape
        ids = np.empty((nq, k), np.int64)
        dists = np.empty((nq, k), np.float32)
        flat = counts = None
        if bucket_ids:
            counts = np.array([len(b) for b in bucket_ids], np.uint64)
            flat = np.array([x for b in bucket_ids for x in b], np.int64)
            if counts.size != nq:
                # the library checks this too; it needs one count per query to read the lists at all
                raise VsagError(-3, f"bucket_ids_ size must match the number of query vectors; got {counts.size} "
                                    f"bucket lists for {nq} queries")
        _check(_lib().vsag_index_search_with_request(
            self._h, vectors.ctypes.data, dim, nq, k, parameters.encode(),
            flat.ctypes.data if flat is not None and flat.size else None,
            counts.ctypes.data if counts is not None else None, ids.ctypes.data, dists.ctypes.data))
        return ids, dists

    def get_num_elements(self) -> int:
        return int(_lib().vsag_index_get_num_elements(self._h))
