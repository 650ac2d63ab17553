"""A bounded wait of the tensor-core kernels that runs out: the call fails with VB200_INTERNAL_ERROR,
nothing hangs, and the next call on the same context works.

Every wait inside those kernels (on a bulk copy, on an accumulator) polls a limited number of times.
vb200_debug_set_wait_limit lowers that number to zero, so the kernels give
up at their first wait, raise their error flag, pause until what they had in flight has landed, free
their tensor memory and return.  Nothing here faults the GPU: the kernels leave by their ordinary
exit path.  Collected late so that a failure cannot hide the result of another test.
"""
from __future__ import annotations

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


def test_scan_wait_runs_out_then_recovers(engine, oracle):
    from vsag_b200 import _capi

    dim, nlist, n, k = 64, 8, 4000, 5
    x = mixture(401, n, dim, nlist, 0.15)
    ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    ix.train(x, iters=2)
    ix.add(x, np.arange(n, dtype=np.int64))
    q = mixture(402, 64, dim, nlist, 0.15)
    want = ix.search(q, k, 4)
    lib = _capi.load()
    assert lib.vb200_debug_set_wait_limit(0) == 0
    try:
        with pytest.raises(_capi.VsagB200Error) as err:
            ix.search(q, k, 4)
        assert err.value.code == -2 and "bounded wait" in str(err.value)
    finally:
        assert lib.vb200_debug_set_wait_limit(-1) == 0
    again = ix.search(q, k, 4)
    assert np.array_equal(again[0], want[0]) and np.array_equal(again[1], want[1])


def test_candidate_kernel_wait_runs_out_then_recovers(engine, oracle):
    from vsag_b200 import _capi

    dim, k = 64, 128
    x = mixture(403, 5000, dim, k, 0.2)
    c = x[:k].copy()
    want = engine.kmeans_assign(x, c)          # k >= 64 and 128+ rows: the tensor-core candidate kernel
    lib = _capi.load()
    assert lib.vb200_debug_set_wait_limit(0) == 0
    try:
        with pytest.raises(_capi.VsagB200Error) as err:
            engine.kmeans_assign(x, c)
        assert err.value.code == -2 and "bounded wait" in str(err.value)
    finally:
        assert lib.vb200_debug_set_wait_limit(-1) == 0
    assert np.array_equal(engine.kmeans_assign(x, c), want)
    assert np.array_equal(want, oracle.kmeans_assign(x, c)[0])
