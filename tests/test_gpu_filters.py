"""GPU parity for removed vectors (MARK_REMOVE) and id filters: the filtered search must equal the
oracle's search over an index from which the same rows were taken out."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_topk_equal, mixture

pytestmark = pytest.mark.gpu


def without_rows(off, order, deny_inner):
    """CSR lists with the denied inner ids taken out (order = inner id per position)."""
    keep = ~deny_inner[order]
    kept_before = np.r_[0, np.cumsum(keep)]
    new_off = kept_before[off].astype(off.dtype)
    return new_off, keep


def bits(mask, word):
    n = (mask.size + word - 1) // word * word
    padded = np.zeros(n, np.uint8)
    padded[: mask.size] = mask
    packed = np.packbits(padded, bitorder="little")
    return packed.view(np.uint32 if word == 32 else np.uint64)


@pytest.mark.parametrize("quant", ["sq8", "fp32"])
def test_ivf_remove_and_filters(engine, oracle, quant):
    from test_gpu_ivf_sq8 import build_pair

    n, dim, nlist, nprobe, nq, k = 20_000, 24, 32, 10, 300, 10
    rng = np.random.default_rng(5)
    if quant == "sq8":
        m = build_pair(engine, oracle, n, dim, nlist, seed=81)
        ix = m["ix"]
    else:
        m = build_pair(engine, oracle, n, dim, nlist, seed=81)
        ix = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_FP32)
        ix.set_centroids(m["centroids"])
    ids = np.arange(n, dtype=np.int64) * 3 + 7          # labels, all below 2^32
    ix.add(m["x"], ids, labels=m["labels"])
    q = mixture(82, nq, dim, nlist, 0.15)
    probes, _ = oracle.route(q, m["centroids"], nprobe, 0)
    off, order = m["off"], m["order"]

    def oracle_search(deny_inner):
        new_off, keep = without_rows(off, order, deny_inner)
        kept = order[keep]
        if quant == "sq8":
            return oracle.ivf_sq8_search(m["codes"][keep], new_off, ids[kept], m["lower"], m["diff"], q, probes, k, 0)
        return oracle.ivf_fp32_search(m["x"][kept], new_off, ids[kept], q, probes, k, 0)

    # 1. tombstones: remove the nearest neighbour of every query plus random others (some twice, some unknown)
    first = ix.search(q, k, nprobe, bucket_ids=probes)[0][:, 0]
    gone_labels = np.unique(np.r_[first[first >= 0], ids[rng.choice(n, 500, replace=False)]])
    assert ix.remove(np.r_[gone_labels, gone_labels[:10], [10**12]]) == gone_labels.size
    assert ix.remove(gone_labels[:5]) == 0 and ix.num_elements() == n - gone_labels.size
    deny = np.isin(ids, gone_labels)
    want = oracle_search(deny)
    got = ix.search(q, k, nprobe, bucket_ids=probes)
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    assert not np.isin(got[0], gone_labels).any()

    # 2. the caller's label bitset on top: every label with (label % 5 == 0) is filtered out
    label_mask = np.zeros(int(ids.max()) + 1, bool)
    label_mask[ids[ids % 5 == 0]] = True
    deny2 = deny | (ids % 5 == 0)
    want = oracle_search(deny2)
    got = ix.search_filtered(q, k, nprobe, bucket_ids=probes, invalid_label_bits=bits(label_mask, 64))
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)

    # 3. an inner-id bitmap (what a host callback becomes), shorter than the index, plus both at once
    inner_mask = rng.random(n // 2) < 0.6
    deny3 = deny.copy()
    deny3[: n // 2] |= inner_mask
    want = oracle_search(deny3)
    got = ix.search_filtered(q, k, nprobe, bucket_ids=probes, deny_inner_bits=bits(inner_mask, 32))
    assert np.array_equal(got[1], want[1])
    assert_topk_equal(got[0], got[1], want[0], want[1], rtol=0, atol=0)
    want = oracle_search(deny3 | deny2)
    got = ix.search_filtered(q, k, nprobe, bucket_ids=probes, deny_inner_bits=bits(inner_mask, 32),
                             invalid_label_bits=bits(label_mask, 64))
    assert np.array_equal(got[1], want[1])

    # 4. everything filtered: padded result
    all_bits = bits(np.ones(n, bool), 32)
    got = ix.search_filtered(q[:5], k, nprobe, deny_inner_bits=all_bits)
    assert np.all(got[0] == -1) and np.all(np.isinf(got[1]))
    # rows added after a removal are searchable and can be removed too
    ix.add(m["x"][:100] + 0.001, np.arange(100, dtype=np.int64) + 10**9, labels=m["labels"][:100])
    assert ix.remove([10**9 + 3]) == 1


@pytest.mark.parametrize("metric,quant,n,nq", [(0, "fp32", 6000, 100), (1, "fp32", 6000, 100),
                                                (1, "bf16", 120_000, 4000), (0, "fp32", 100_000, 4000)])
def test_bruteforce_remove_and_filters(engine, oracle, metric, quant, n, nq):
    """Small cases take the SIMT path, the large ones the tensor-core path; filtered rows get an
    infinite score bias and can never be nominated."""
    dim, k = 64, 10
    rng = np.random.default_rng(9)
    base = mixture(91, n, dim, 32, 0.3)
    q = mixture(92, nq, dim, 32, 0.3)
    ids = np.arange(n, dtype=np.int64) * 2 + 5
    ix = engine.BfHandle(dim, metric, engine.QUANT_FP32 if quant == "fp32" else engine.QUANT_BF16)
    ix.add(base, ids)
    sub = slice(0, 64)

    def oracle_search(deny):
        kept = np.flatnonzero(~deny)
        if quant == "fp32":
            wi, wd = oracle.bf_search_fp32(base[kept], q[sub], k, metric)
        else:
            wi, wd = oracle.bf_search_bf16(oracle.float_to_bf16(base[kept]), q[sub], k, metric=metric)
        return np.where(wi >= 0, ids[kept][np.maximum(wi, 0)], -1), wd

    first = ix.search(q, k)[0][:, 0]
    gone = np.unique(np.r_[first, ids[rng.choice(n, n // 10, replace=False)]])
    assert ix.remove(gone) == gone.size and ix.num_elements() == n - gone.size
    deny = np.isin(ids, gone)
    want = oracle_search(deny)
    got = ix.search(q, k)
    assert np.array_equal(got[1][sub], want[1])
    assert_topk_equal(got[0][sub], got[1][sub], want[0], want[1], rtol=0, atol=0)
    assert not np.isin(got[0], gone).any()
    label_mask = np.zeros(int(ids.max()) + 1, bool)
    label_mask[ids[ids % 3 == 0]] = True
    inner_mask = rng.random(n) < 0.5
    deny2 = deny | (ids % 3 == 0) | inner_mask
    want = oracle_search(deny2)
    got = ix.search_filtered(q, k, invalid_label_bits=bits(label_mask, 64), deny_inner_bits=bits(inner_mask, 32))
    assert np.array_equal(got[1][sub], want[1])
    assert_topk_equal(got[0][sub], got[1][sub], want[0], want[1], rtol=0, atol=0)
    # fewer valid rows than k: the rest is padding, not filtered rows
    keep_only = np.ones(n, bool)
    keep_only[[1, 2, 3]] = False
    got = ix.search_filtered(q[:4], k, deny_inner_bits=bits(keep_only, 32))
    valid = (~deny[[1, 2, 3]]).sum()
    assert np.all((got[0] >= 0).sum(axis=1) == valid) and np.all(np.isin(got[0][got[0] >= 0], ids[[1, 2, 3]]))


@pytest.mark.parametrize("name", ["ivf", "brute_force"])
def test_factory_index_remove_and_prefilters(oracle, name):
    """Through the vsag::Index mirror: Remove, the bitset pre-filter and the callback pre-filter."""
    import json

    from vsag_b200.index import Index

    n, dim, k = 3000, 32, 8
    base = oracle.gen_uniform(47, n * dim).reshape(n, dim)
    queries = oracle.gen_uniform(48, 20 * dim).reshape(20, dim)
    ids = np.arange(n, dtype=np.int64) + 100
    extra = {"buckets_count": 12} if name == "ivf" else {}
    index = Index(name, json.dumps({"dtype": "float32", "metric_type": "l2", "dim": dim, "index_param": extra}))
    index.build(base, ids, n, dim)
    search = json.dumps({"ivf": {"scan_buckets_count": 12}}) if name == "ivf" else "{}"

    def exact(deny):
        kept = np.flatnonzero(~deny)
        wi, wd = oracle.bf_search_fp32(base[kept], queries, k, 0)
        return ids[kept][wi], wd

    none = np.zeros(n, bool)
    for i, q in enumerate(queries):
        got = index.knn_search(q, k, search)
        assert np.array_equal(got[1], exact(none)[1][i])
    top = np.unique(exact(none)[0][:, :2])
    assert index.remove(np.r_[top, [5]]) == top.size            # id 5 does not exist
    assert index.get_num_elements() == n - top.size
    deny = np.isin(ids, top)
    want = exact(deny)
    for i, q in enumerate(queries):
        got = index.knn_search(q, k, search)
        assert np.array_equal(got[1], want[1][i]) and not np.isin(got[0], top).any()
    invalid = ids[::3]
    want = exact(deny | np.isin(ids, invalid))
    for i, q in enumerate(queries):
        got = index.knn_search_filtered(q, k, search, invalid_ids=invalid)
        assert np.array_equal(got[1], want[1][i])
        assert_topk_equal(got[0][None], got[1][None], want[0][i][None], want[1][i][None], rtol=0, atol=0)
    want = exact(deny | (ids % 7 == 0))
    for i, q in enumerate(queries):
        got = index.knn_search_filtered(q, k, search, deny_modulus=7)
        assert np.array_equal(got[1], want[1][i])
