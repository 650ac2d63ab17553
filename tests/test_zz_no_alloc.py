"""The allocation-free k-means assignment entry point against the regular one.

vb200_kmeans_assign_noalloc is for callers that cannot touch the CUDA allocator (fixed device-memory
budget, or no tolerance for the device-wide synchronisation of cudaMalloc/cudaFree): it keeps its
only scratch, the centroid norms, in a fixed array inside the library.  This file is collected last
so a failure here cannot hide the result of any other test.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


def _assign_noalloc(lib, x_dev, c_dev, labels_dev):
    n, dim = x_dev.shape
    return lib.vb200_kmeans_assign_noalloc(C.c_void_p(x_dev.data_ptr()), n, dim, C.c_void_p(c_dev.data_ptr()),
                                           c_dev.shape[0], C.c_void_p(labels_dev.data_ptr()))


def test_noalloc_assignment_matches_regular_entry_point(engine, oracle):
    import torch

    from vsag_b200 import _capi

    lib = _capi.load()
    dim = 64
    x = mixture(11, 20_000, dim, 300, 0.1)
    x_dev = torch.from_numpy(x).cuda()
    labels_dev = torch.empty(x.shape[0], dtype=torch.int32, device="cuda")
    # two calls in a row with different centroid counts: the second must not be disturbed by what
    # the first left in the shared scratch array (labels are integers: exact equality), and both must
    # give the labels of the regular entry point and of the CPU oracle
    for k in (300, 17):
        centroids = x[:k].copy()
        want = engine.kmeans_assign(x, centroids)
        want_oracle, _ = oracle.kmeans_assign(x, centroids)
        c_dev = torch.from_numpy(centroids).cuda()
        labels_dev.fill_(-7)
        assert _assign_noalloc(lib, x_dev, c_dev, labels_dev) == 0, _capi.last_error()
        got = labels_dev.cpu().numpy()
        assert np.array_equal(got, want)
        assert np.array_equal(got, want_oracle)


def test_noalloc_call_leaves_device_memory_as_it_found_it(engine):
    """What the entry point exists for: free device memory (cudaMemGetInfo, as torch reports it) is the
    same before and after a call -- nothing was taken from the allocator, nothing given back."""
    import torch

    from vsag_b200 import _capi

    lib = _capi.load()
    x = mixture(12, 4096, 32, 64, 0.1)
    x_dev = torch.from_numpy(x).cuda()
    c_dev = x_dev[:64].clone()
    labels_dev = torch.empty(x.shape[0], dtype=torch.int32, device="cuda")
    # the first call on a device looks up the scratch array's address (module load happens here at the latest)
    assert _assign_noalloc(lib, x_dev, c_dev, labels_dev) == 0, _capi.last_error()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert _assign_noalloc(lib, x_dev, c_dev, labels_dev) == 0, _capi.last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_noalloc_rejects_what_it_cannot_serve(engine):
    import torch

    from vsag_b200 import _capi

    lib = _capi.load()
    x_dev = torch.zeros((8, 4), dtype=torch.float32, device="cuda")
    labels_dev = torch.empty(8, dtype=torch.int32, device="cuda")
    too_many = torch.zeros((65537, 4), dtype=torch.float32, device="cuda")
    assert _assign_noalloc(lib, x_dev, too_many, labels_dev) == -3
    assert "65536" in _capi.last_error()[1]
    # host pointers would need staging buffers, which this entry point never creates
    host_centroids = np.zeros((2, 4), np.float32)
    rc = lib.vb200_kmeans_assign_noalloc(C.c_void_p(x_dev.data_ptr()), 8, 4,
                                         C.c_void_p(host_centroids.ctypes.data), 2,
                                         C.c_void_p(labels_dev.data_ptr()))
    assert rc == -3 and "device pointers" in _capi.last_error()[1]
