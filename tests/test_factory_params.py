"""Factory parameter handling (no GPU needed): the creation JSON is validated before any device is
touched, with the reference's rules -- required dtype / metric_type / dim
(src/index_common_param.cpp:117-174), unknown index names and keys rejected
(tests/test_ivf.cpp:1045-1167)."""
from __future__ import annotations

import json

import pytest


def make(name, **over):
    from vsag_b200.index import Index

    params = {"dtype": "float32", "metric_type": "l2", "dim": 16,
              "index_param": {"buckets_count": 4, "base_quantization_type": "sq8"}}
    params.update(over)
    return Index(name, json.dumps(params))


def expect_invalid(match, name="ivf", **over):
    from vsag_b200.index import VsagError

    with pytest.raises(VsagError, match=match) as info:
        make(name, **over)
    return info.value


def test_unknown_index_name():
    e = expect_invalid("unsupported", name="hnsw_on_gpu")
    assert e.code == -7


def test_required_top_level_keys():
    from vsag_b200.index import Index, VsagError

    for missing in ("dtype", "metric_type", "dim"):
        params = {"dtype": "float32", "metric_type": "l2", "dim": 16}
        del params[missing]
        with pytest.raises(VsagError, match=missing):
            Index("ivf", json.dumps(params))
    with pytest.raises(VsagError):
        Index("ivf", "{not json")


def test_bad_values():
    expect_invalid("float32", dtype="int8")
    expect_invalid("metric_type", metric_type="manhattan")
    expect_invalid("dim", dim=0)
    expect_invalid("dim", dim=1.5)
    expect_invalid("integer", index_param={"buckets_count": "many", "base_quantization_type": "sq8"})
    expect_invalid("buckets_count", index_param={"buckets_count": 0, "base_quantization_type": "sq8"})
    expect_invalid("not served", index_param={"base_quantization_type": "pq"})
    expect_invalid("buckets_per_data", index_param={"base_quantization_type": "sq8", "buckets_per_data": 0})
    expect_invalid("buckets_per_data", index_param={"base_quantization_type": "sq8", "buckets_per_data": 17})
    expect_invalid("use_residual", index_param={"base_quantization_type": "fp32", "use_residual": True})
    expect_invalid("train_sample_count", index_param={"base_quantization_type": "sq8", "train_sample_count": 10})


def test_unknown_keys_are_rejected():
    expect_invalid("unknown parameter", index_param={"base_quantization_type": "sq8", "bucket_count": 7})
    expect_invalid("unknown parameter", name="brute_force", index_param={"max_degree": 16})
    expect_invalid("not served", name="brute_force", index_param={"base_quantization_type": "sq8"})


def test_names_are_case_insensitive_and_valid_params_reach_the_device():
    """With valid parameters the only thing that can fail on a machine without a GPU is the device."""
    from vsag_b200 import engine
    from vsag_b200.index import VsagError

    try:
        have_gpu = engine.device_count() > 0
    except Exception:
        have_gpu = False
    for name in ("IVF", "Brute_Force"):
        over = {} if name == "IVF" else {"index_param": {"base_quantization_type": "fp32"}}
        if have_gpu:
            assert make(name, **over).get_num_elements() == 0
        else:
            with pytest.raises(VsagError, match="CUDA"):
                make(name, **over)
