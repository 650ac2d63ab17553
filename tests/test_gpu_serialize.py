"""Serialize / Deserialize through the factory API (include/vsag/index.h:903-940,
include/vsag/vsag_c_api.h:319-330), in the style of the reference's serialize-then-search checks
(tests/test_index.cpp TestSerializeFile): the reloaded index answers exactly like the original."""
from __future__ import annotations

import json

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


def params(dim, metric="l2", **index_param):
    return json.dumps({"dtype": "float32", "metric_type": metric, "dim": dim, "index_param": index_param})


CASES = [
    ("ivf", "l2", dict(buckets_count=24, base_quantization_type="sq8"), {"ivf": {"scan_buckets_count": 6}}),
    ("ivf", "ip", dict(buckets_count=24, base_quantization_type="sq8"), {"ivf": {"scan_buckets_count": 6}}),
    ("ivf", "cosine", dict(buckets_count=24, base_quantization_type="fp32"), {"ivf": {"scan_buckets_count": 6}}),
    ("ivf", "l2", dict(buckets_count=24, base_quantization_type="bf16"), {"ivf": {"scan_buckets_count": 6}}),
    ("ivf", "l2", dict(buckets_count=24, base_quantization_type="sq8_uniform", buckets_per_data=2),
     {"ivf": {"scan_buckets_count": 6}}),
    ("ivf", "cosine", dict(buckets_count=24, base_quantization_type="fp16", use_reorder=True),
     {"ivf": {"scan_buckets_count": 6, "factor": 3.0}}),
    ("ivf", "l2", dict(buckets_count=16, base_quantization_type="rabitq", use_reorder=True),
     {"ivf": {"scan_buckets_count": 6, "factor": 4.0}}),
    ("brute_force", "l2", dict(base_quantization_type="fp32"), {}),
    ("brute_force", "cosine", dict(base_quantization_type="bf16"), {}),
]


@pytest.mark.parametrize("name,metric,index_param,search", CASES)
def test_reloaded_index_answers_like_the_original(tmp_path, name, metric, index_param, search):
    from vsag_b200.index import Index

    n, dim, nq, k = 6000, 64, 120, 10
    base = mixture(11, n, dim, 24, 0.1, lo=0.0, hi=1.0, clip=True)
    queries = mixture(12, nq, dim, 24, 0.1, lo=0.0, hi=1.0, clip=True)
    ids = np.arange(n, dtype=np.int64) * 2 + 5
    p = params(dim, metric, **index_param)
    src = Index(name, p)
    src.build(base[:5000], ids[:5000], 5000, dim)
    src.add(base[5000:], ids[5000:], n - 5000, dim)
    assert src.remove(ids[100:140]) == 40
    want = src.knn_search_batch(queries, k, json.dumps(search))
    path = tmp_path / "index.bin"
    src.serialize_file(path)

    dst = Index(name, p)
    dst.deserialize_file(path)
    assert dst.get_num_elements() == n - 40
    got = dst.knn_search_batch(queries, k, json.dumps(search))
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert not np.isin(got[0], ids[100:140]).any()
    # it keeps working as an index: new vectors can be added and found
    extra = base[:3] + 0.5
    dst.add(extra, np.array([900_011, 900_012, 900_013], np.int64), 3, dim)
    assert dst.get_num_elements() == n - 40 + 3
    if metric == "l2":
        found, _ = dst.knn_search(extra[1], 1, json.dumps(search if name == "brute_force" else
                                                           {"ivf": {"scan_buckets_count": index_param["buckets_count"],
                                                                    "factor": 4.0}}))
        assert found[0] == 900_012


def test_stream_errors(tmp_path):
    from vsag_b200.index import Index, VsagError

    dim = 16
    base = mixture(13, 800, dim, 8, 0.1)
    ids = np.arange(800, dtype=np.int64)
    p = params(dim, buckets_count=8, base_quantization_type="sq8")
    index = Index("ivf", p)
    index.build(base, ids, 800, dim)
    path = tmp_path / "ivf.bin"
    index.serialize_file(path)

    with pytest.raises(VsagError) as e:           # the target must be empty
        index.deserialize_file(path)
    assert e.value.code == -6                     # INDEX_NOT_EMPTY
    with pytest.raises(VsagError) as e:
        Index("ivf", p).deserialize_file(tmp_path / "absent.bin")
    assert e.value.code == -13                    # MISSING_FILE
    with pytest.raises(VsagError) as e:           # other creation parameters
        Index("ivf", params(dim, buckets_count=9, base_quantization_type="sq8")).deserialize_file(path)
    assert e.value.code == -3                     # INVALID_ARGUMENT
    with pytest.raises(VsagError) as e:           # another kind of index
        Index("brute_force", params(dim)).deserialize_file(path)
    assert e.value.code == -3
    blob = path.read_bytes()
    short = tmp_path / "short.bin"
    short.write_bytes(blob[: len(blob) // 2])
    with pytest.raises(VsagError) as e:
        Index("ivf", p).deserialize_file(short)
    assert e.value.code == -12                    # READ_ERROR
    junk = tmp_path / "junk.bin"
    junk.write_bytes(b"not an index at all" * 10)
    with pytest.raises(VsagError) as e:
        Index("ivf", p).deserialize_file(junk)
    assert e.value.code == -14                    # INVALID_BINARY

    # an index that was never built round-trips too
    empty = tmp_path / "empty.bin"
    Index("ivf", p).serialize_file(empty)
    fresh = Index("ivf", p)
    fresh.deserialize_file(empty)
    assert fresh.get_num_elements() == 0
    fresh.build(base, ids, 800, dim)
    assert fresh.get_num_elements() == 800


def test_bruteforce_rows_roundtrip(engine, oracle):
    n, dim, k = 3000, 48, 10
    x = mixture(14, n, dim, 10, 0.2)
    q = mixture(15, 50, dim, 10, 0.2)
    ids = np.arange(n, dtype=np.int64) + 9
    for metric, quant in ((engine.METRIC_COSINE, engine.QUANT_FP32), (engine.METRIC_IP, engine.QUANT_BF16)):
        src = engine.BfHandle(dim, metric, quant)
        src.add(x, ids)
        rows = src.get_rows()
        if quant == engine.QUANT_BF16:
            assert np.array_equal(rows, oracle.float_to_bf16(x))
        dst = engine.BfHandle(dim, metric, quant)
        dst.set_rows(rows, ids)
        assert np.array_equal(dst.get_rows(), rows)
        want, got = src.search(q, k), dst.search(q, k)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
        with pytest.raises(engine.VsagB200Error):
            dst.set_rows(rows, ids)                # only into an empty index
