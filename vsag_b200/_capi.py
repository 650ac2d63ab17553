"""ctypes binding of libvsag_b200.so (the C ABI declared in include/vsag_b200.h).

The library is the product; this module only loads it and marshals numpy arrays / torch tensors
into plain pointers.  There is no fallback: if the shared library is missing the import of any
compute entry point raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent / "libvsag_b200.so"

c_void_p, c_int, c_u32, c_u64, c_i64, c_float = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64, C.c_int64, C.c_float
class Filter(C.Structure):
    """vb200_filter: label bitset and / or inner-id bitmap, host or device pointers."""

    _fields_ = [("invalid_label_bits", C.c_void_p), ("n_label_bits", C.c_uint64),
                ("deny_inner_bits", C.c_void_p), ("n_inner_bits", C.c_uint64)]


# vb200_exchange_fn: int (*)(float* bounds_dev, uint64_t nq, void* cuda_stream, void* arg)
EXCHANGE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p)

# name -> (restype, argtypes); the single source for the "every declared symbol is exported" test.
SIGNATURES = {
    "vb200_last_error": (c_int, [C.c_char_p, C.c_size_t]),
    "vb200_release_workspaces": (c_int, []),
    "vb200_set_stream": (c_int, [c_void_p]),
    "vb200_kernel_launches": (c_u64, []),
    "vb200_device_count": (c_int, []),
    "vb200_set_tensor_cores": (c_int, [c_int]),
    "vb200_debug_set_wait_limit": (c_int, [c_int]),
    "vb200_sq8_train": (c_int, [c_void_p, c_u64, c_u32, c_int, c_void_p, c_void_p]),
    "vb200_sq8_encode": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_void_p, c_void_p]),
    "vb200_kmeans_assign": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_u32, c_void_p, c_void_p]),
    "vb200_kmeans_update": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_u32, c_u32, c_void_p, c_void_p]),
    "vb200_kmeans_init": (c_int, [c_void_p, c_u64, c_u32, c_u32, c_u32, c_void_p, c_void_p]),
    "vb200_kmeans_train": (c_int, [c_void_p, c_u64, c_u32, c_u32, c_int, c_void_p, c_void_p, c_void_p]),
    "vb200_kmeans_assign_noalloc": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_u32, c_void_p]),
    "vb200_rabitq_code_size": (c_u64, [c_u32]),
    "vb200_rabitq_train": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_void_p]),
    "vb200_rabitq_encode": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_void_p, c_void_p]),
    "vb200_rabitq_process_query": (c_int, [c_void_p, c_u64, c_u32, c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_create": (c_int, [c_u32, c_int, c_u32, c_int, c_int, C.POINTER(c_void_p)]),
    "vb200_ivf_destroy": (c_int, [c_void_p]),
    "vb200_ivf_set_shard": (c_int, [c_void_p, c_u32, c_u32]),
    "vb200_ivf_train": (c_int, [c_void_p, c_void_p, c_u64, c_int, c_void_p]),
    "vb200_ivf_set_centroids": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_get_centroids": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_set_sq8_model": (c_int, [c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_get_sq8_model": (c_int, [c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_set_rabitq_rotation": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_set_rabitq_centroid": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_get_rabitq_centroid": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_add": (c_int, [c_void_p, c_void_p, c_u64, c_void_p, c_void_p]),
    "vb200_ivf_num_elements": (c_i64, [c_void_p]),
    "vb200_ivf_memory_usage": (c_i64, [c_void_p]),
    "vb200_ivf_get_lists": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_set_lists": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_ivf_get_rows": (c_int, [c_void_p, c_void_p]),
    "vb200_ivf_search": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_u32, c_float, c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_search_filtered": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_u32, c_float, c_void_p, c_void_p,
                                          c_void_p, c_void_p]),
    "vb200_ivf_remove": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_ivf_route": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_void_p]),
    "vb200_ivf_search_partial": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_u32, c_float, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p]),
    "vb200_ivf_last_scan_bytes": (c_i64, [c_void_p]),
    "vb200_ivf_last_scanned_bytes": (c_i64, [c_void_p]),
    "vb200_ivf_set_list_pruning": (c_int, [c_void_p, c_int]),
    "vb200_ivf_last_scan_ms": (c_int, [c_void_p, C.POINTER(c_float)]),
    "vb200_merge_partials": (c_int, [c_void_p, c_void_p, c_u32, c_u64, c_u32, c_void_p, c_void_p]),
    "vb200_bf_create": (c_int, [c_u32, c_int, c_int, C.POINTER(c_void_p)]),
    "vb200_bf_destroy": (c_int, [c_void_p]),
    "vb200_bf_add": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_bf_add_bf16": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_bf_get_rows": (c_int, [c_void_p, c_void_p]),
    "vb200_bf_set_rows": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_bf_num_elements": (c_i64, [c_void_p]),
    "vb200_bf_search": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_void_p]),
    "vb200_bf_search_filtered": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_void_p, c_void_p]),
    "vb200_bf_remove": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "vb200_bf_search_partial": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_void_p]),
    "vb200_ivf_search_ex": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_u32, c_float, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, C.POINTER(c_int)]),
    "vb200_ivf_set_use_residual": (c_int, [c_void_p, c_int]),
    "vb200_ivf_set_buckets_per_data": (c_int, [c_void_p, c_u32]),
    "vb200_ivf_set_sq8_uniform_model": (c_int, [c_void_p, c_float, c_float]),
    "vb200_ivf_get_sq8_uniform_model": (c_int, [c_void_p, C.POINTER(c_float), C.POINTER(c_float)]),
    "vb200_comm_unique_id": (c_int, [c_void_p]),
    "vb200_comm_init": (c_int, [C.POINTER(c_void_p), c_void_p, c_int, c_int]),
    "vb200_comm_destroy": (c_int, [c_void_p]),
    "vb200_comm_rank": (c_int, [c_void_p]),
    "vb200_comm_world": (c_int, [c_void_p]),
    "vb200_ivf_search_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u32, c_u32, C.c_float, c_void_p,
                                         c_void_p]),
    "vb200_bf_search_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_u64, c_u32, c_void_p, c_void_p]),
}

_lib = None


class VsagB200Error(RuntimeError):
    """An entry point returned a negative VB200_* code."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(
                f"{_LIB_PATH} is missing: build it with `python -m vsag_b200.build` "
                "(the engine has no Python or CPU fallback)")
        lib = C.CDLL(os.fspath(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> tuple[int, str]:
    buf = C.create_string_buffer(1024)
    code = load().vb200_last_error(buf, 1024)
    return code, buf.value.decode("utf-8", "replace")


def check(status: int) -> None:
    if status != 0:
        _, msg = last_error()
        raise VsagB200Error(status, msg)


def ptr(x, dtype=None):
    """Address of a C-contiguous numpy array or torch tensor (host or device); None -> NULL."""
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        if dtype is not None and x.dtype != np.dtype(dtype):
            raise TypeError(f"expected dtype {np.dtype(dtype)}, got {x.dtype}")
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):  # torch.Tensor
        if not x.is_contiguous():
            raise ValueError("tensor must be contiguous")
        if dtype is not None:
            import torch

            want = {np.dtype("float32"): torch.float32, np.dtype("int64"): torch.int64,
                    np.dtype("int32"): torch.int32, np.dtype("uint8"): torch.uint8,
                    np.dtype("uint16"): (torch.bfloat16, torch.uint16, torch.int16),
                    np.dtype("uint64"): (torch.int64, torch.uint64),
                    np.dtype("float64"): torch.float64}[np.dtype(dtype)]
            ok = x.dtype in want if isinstance(want, tuple) else x.dtype == want
            if not ok:
                raise TypeError(f"expected tensor dtype {want}, got {x.dtype}")
        return C.c_void_p(x.data_ptr())
    raise TypeError(f"unsupported buffer type {type(x)}")
