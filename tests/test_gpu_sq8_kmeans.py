"""GPU parity: SQ8 trainer/encoder and k-means against the CPU oracle, through the C ABI."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,dim", [(1, 3), (999, 7), (5000, 96), (150_001, 16)])
@pytest.mark.parametrize("mode", [1, 3])
def test_sq8_train_bit_exact(engine, oracle, n, dim, mode):
    x = mixture(n + dim, n, dim, 16, 0.3)
    want_lower, want_diff = oracle.sq8_train(x, mode)
    lower, diff = engine.sq8_train(x, mode)
    assert np.array_equal(lower, want_lower)
    assert np.array_equal(diff, want_diff)


def test_sq8_train_device_input(engine, oracle):
    import torch

    x = mixture(3, 120_000, 8, 16, 0.3)
    want = oracle.sq8_train(x, 3)
    got = engine.sq8_train(torch.from_numpy(x).cuda(), 3)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_sq8_known_answer_on_gpu(engine):
    # src/quantization/scalar_quantization/scalar_quantizer_test.cpp:101-116
    lower, diff = engine.sq8_train(np.array([[0.0, 0.0], [1.0, 1.0]], np.float32))
    codes = engine.sq8_encode(np.array([[np.nan, 0.5]], np.float32), lower, diff)
    assert codes.tolist() == [[0, 127]]


@pytest.mark.parametrize("dim", [1, 7, 96, 100])
def test_sq8_encode_bit_exact(engine, oracle, dim):
    rng = np.random.default_rng(dim)
    x = mixture(dim, 20_000, dim, 32, 0.2)
    lower, diff = oracle.sq8_train(x)
    # out-of-range values, exact bounds, NaN, infinities and a degenerate dimension
    x[0, :] = lower
    x[1, :] = lower + diff
    x[2, :] = 1e9
    x[3, :] = -1e9
    x[4, 0] = np.nan
    x[5, 0] = np.inf
    x[6, 0] = -np.inf
    x[7:2000] += rng.normal(0, 2.0, x[7:2000].shape).astype(np.float32)
    if dim > 1:
        diff = diff.copy()
        diff[dim - 1] = 0.0
    want = oracle.sq8_encode(x, lower, diff)
    got = engine.sq8_encode(x, lower, diff)
    assert got.dtype == np.uint8 and np.array_equal(got, want)


def test_sq8_encode_empty(engine):
    out = engine.sq8_encode(np.zeros((0, 4), np.float32), np.zeros(4, np.float32), np.ones(4, np.float32))
    assert out.shape == (0, 4)


@pytest.mark.parametrize("n,dim,k", [(4000, 7, 1), (4000, 7, 37), (6000, 96, 300), (3000, 128, 129), (2000, 130, 64)])
def test_kmeans_assign_bit_exact(engine, oracle, n, dim, k):
    x = mixture(n + k, n, dim, max(k, 2), 0.1)
    centroids = x[:k].copy()
    want, want_err = oracle.kmeans_assign(x, centroids)
    got, err = engine.kmeans_assign(x, centroids, want_err=True)
    assert np.array_equal(got, want)
    assert err == pytest.approx(want_err, rel=1e-9, abs=1e-9)


def test_kmeans_assign_ties_take_lowest_index(engine, oracle):
    x = mixture(5, 500, 8, 4, 0.1)
    centroids = np.repeat(x[:3], 4, axis=0)  # every centroid appears four times
    want, _ = oracle.kmeans_assign(x, centroids)
    got = engine.kmeans_assign(x, centroids)
    assert np.array_equal(got, want)
    assert np.all(got % 4 == 0)


@pytest.mark.parametrize("case", ["duplicates", "one_ulp_apart", "far_from_origin", "mixed"])
def test_tensor_core_assignment_with_crowded_candidates(engine, oracle, case):
    """The tensor-core path (64+ centroids) nominates four candidates per list and decides among them
    exactly.  Here more than four centroids sit within the nomination error of a row's best -- copies of
    one centroid, centroids one float apart, data so far from the origin that every score gap is below
    the error margin -- so a list can fill up with near-winners.  Such rows are detected and decided over
    all centroids: labels still equal the oracle's, lowest index on ties (kmeans_cluster.cpp:284)."""
    dim, k, n = 32, 160, 3000
    x = mixture(31, n, dim, 40, 0.1)
    c = x[:k].copy()
    if case in ("duplicates", "mixed"):
        c[20:29] = c[20]                       # nine copies of one centroid
        c[100:112] = c[7]                      # twelve of another, spread over the column groups
    if case in ("one_ulp_apart", "mixed"):
        for j in range(40, 48):                # eight centroids one float apart in one coordinate
            c[j] = c[40]
            c[j, 3] = np.nextafter(c[40, 3], np.float32(10.0), dtype=np.float32) if j % 2 else c[40, 3]
            c[j, 5] = np.float32(c[40, 5]) + np.float32(j - 40) * np.spacing(np.float32(c[40, 5]))
    if case == "far_from_origin":
        x = x + np.float32(1000.0)
        c = c + np.float32(1000.0)
    want, _ = oracle.kmeans_assign(x, c)
    got = engine.kmeans_assign(x, c)
    assert np.array_equal(got, want)
    try:
        engine.set_tensor_cores(False)
        assert np.array_equal(engine.kmeans_assign(x, c), want)
    finally:
        engine.set_tensor_cores(True)


def test_kmeans_update_matches_oracle(engine, oracle):
    n, dim, k = 20_000, 24, 50
    x = mixture(1, n, dim, 40, 0.1)
    labels, _ = oracle.kmeans_assign(x, x[:k].copy())
    labels[labels == 7] = 8  # force an empty cluster
    labels[0] = -1           # ignored rows
    want_c, want_counts = oracle.kmeans_update(x, labels, k, it=3)
    got_c, got_counts = engine.kmeans_update(x, labels, k, it=3)
    assert np.array_equal(got_counts, want_counts) and got_counts[7] == 0
    # every cluster is summed in ascending row order on both sides (the reference itself merges partial
    # blocks in thread-completion order and is reproducible only to rounding): centroids are bit-equal
    assert np.array_equal(got_c, want_c)
    row = (7 * 2654435761 + 3) % n
    assert np.array_equal(got_c[7], x[row])


def test_kmeans_train_follows_oracle(engine, oracle):
    n, dim, k, iters = 30_000, 32, 64, 6
    x = mixture(2, n, dim, k, 0.1)
    init = x[:k].copy()
    want_c, want_l, want_err, _ = oracle.kmeans_run(x, init, iters)
    got_c, got_l, got_err = engine.kmeans_train(x, init, iters)
    # assignments are bit-exact given equal centroids, and centroids are bit-exact given equal assignments
    # (clusters are summed in ascending row order on both sides), so the whole run is: no tolerance
    assert np.array_equal(got_l, want_l)
    assert np.array_equal(got_c, want_c)
    assert got_err == pytest.approx(want_err, rel=1e-6)
    # and twice the same run gives twice the same bits
    again_c, again_l, _ = engine.kmeans_train(x, init, iters)
    assert np.array_equal(again_c, got_c) and np.array_equal(again_l, got_l)
    # size-independent properties: assigning against the returned centroids is a fixed point of
    # the label step, and every label is in range
    again = engine.kmeans_assign(x, want_c)
    assert np.array_equal(again, oracle.kmeans_assign(x, want_c)[0])
    assert got_l.min() >= 0 and got_l.max() < k


def test_kmeans_argument_errors(engine):
    x = np.zeros((4, 3), np.float32)
    with pytest.raises(engine.VsagB200Error, match="k cannot be larger than count"):
        engine.kmeans_train(x, np.zeros((5, 3), np.float32), 1)


@pytest.mark.parametrize("n,dim,k,seed", [(20_000, 32, 64, 47), (5_000, 100, 200, 1), (1025, 7, 33, 9)])
def test_kmeans_pp_seeding_matches_oracle(engine, oracle, n, dim, k, seed):
    x = mixture(seed, n, dim, 16, 0.2)
    want_c, want_rows = oracle.kmeans_pp_init(x, k, seed)
    got_c, got_rows = engine.kmeans_init(x, k, seed, want_rows=True)
    # the running sums are added in another order on the device: a pick can differ only where
    # the draw falls within rounding of a boundary, which these seeds do not hit
    assert np.array_equal(got_rows, want_rows)
    assert np.array_equal(got_c, want_c)
    import torch

    dev_c = engine.kmeans_init(torch.from_numpy(x).cuda(), k, seed)
    assert np.array_equal(dev_c.cpu().numpy(), want_c)


def test_kmeans_pp_seeding_with_coinciding_rows(engine, oracle):
    x = np.repeat(np.arange(3, dtype=np.float32)[:, None], 4, axis=1)[np.arange(300) % 3]
    want_c, want_rows = oracle.kmeans_pp_init(x, 10, 5)
    got_c, got_rows = engine.kmeans_init(x, 10, 5, want_rows=True)
    assert np.array_equal(got_rows, want_rows) and np.array_equal(got_c, want_c)
    with pytest.raises(engine.VsagB200Error):
        engine.kmeans_init(x[:5], 6)
