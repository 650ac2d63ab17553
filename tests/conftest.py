"""Shared fixtures.  Tests marked `gpu` need a CUDA device and call the engine through its C ABI;
everything else runs on CPU (oracle, host logic, symbol checks)."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle

    pyoracle.lib()
    return pyoracle


@pytest.fixture(scope="session")
def engine():
    """The C-ABI binding; building is a prerequisite, never a fallback."""
    from vsag_b200 import engine as eng

    from vsag_b200 import _capi

    _capi.load()
    return eng


def mixture(seed: int, n: int, dim: int, centres: int, sigma: float, lo: float = -1.0, hi: float = 1.0,
            clip: bool = False) -> np.ndarray:
    """Gaussian-mixture rows shaped like the benchmark configs (seeded, synthetic)."""
    rng = np.random.default_rng(seed)
    c = rng.uniform(lo, hi, (centres, dim)).astype(np.float32)
    which = rng.integers(0, centres, n)
    x = c[which] + rng.normal(0.0, sigma, (n, dim)).astype(np.float32)
    if clip:
        x = np.clip(x, lo, hi)
    return np.ascontiguousarray(x, np.float32)


def assert_topk_equal(ids_a, dists_a, ids_b, dists_b, rtol=1e-5, atol=1e-6):
    """Distances agree within tolerance; ids agree except inside groups of (near-)tied distances."""
    ids_a, ids_b = np.asarray(ids_a), np.asarray(ids_b)
    dists_a, dists_b = np.asarray(dists_a, np.float64), np.asarray(dists_b, np.float64)
    assert ids_a.shape == ids_b.shape and dists_a.shape == dists_b.shape
    fin = np.isfinite(dists_b)
    assert np.array_equal(np.isfinite(dists_a), fin), "padding differs"
    np.testing.assert_allclose(dists_a[fin], dists_b[fin], rtol=rtol, atol=atol)
    assert np.array_equal(ids_a[~fin], ids_b[~fin])
    mismatch = (ids_a != ids_b) & fin
    for q, j in zip(*np.nonzero(mismatch)):
        d = dists_b[q, j]
        tol = atol + rtol * abs(d)
        # the differing id must sit in a run of tied distances, or be tied with the cut-off
        tied_b = np.abs(dists_b[q] - d) <= 2 * tol
        tied_a = np.abs(dists_a[q] - d) <= 2 * tol
        in_b = ids_a[q, j] in set(ids_b[q][tied_b].tolist())
        at_edge = tied_b[-1] or tied_a[-1]
        assert in_b or at_edge, f"query {q} rank {j}: id {ids_a[q, j]} vs {ids_b[q, j]} is not a tie (d={d})"
