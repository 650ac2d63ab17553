"""The C-ABI library builds, loads, and exports exactly what include/vsag_b200.h declares.
No compute call is made here (no GPU needed)."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols() -> list[str]:
    text = (ROOT / "include" / "vsag_b200.h").read_text()
    return re.findall(r"^VB200_API\s+[A-Za-z0-9_]+\s+(vb200_[a-z0-9_]+)\s*\(", text, flags=re.M)


def test_library_is_built_and_loads():
    from vsag_b200 import _capi

    assert _capi.lib_path().exists(), "run `python -m vsag_b200.build` first"
    _capi.load()


def test_every_declared_symbol_is_exported():
    from vsag_b200 import _capi

    names = declared_symbols()
    assert len(names) >= 38
    lib = C.CDLL(str(_capi.lib_path()))
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/vsag_b200.h but not exported: {missing}"
    assert sorted(names) == sorted(_capi.SIGNATURES), "python binding table is out of sync with the header"


def test_no_cpu_fallback_without_a_device(engine):
    """On a machine without a GPU the engine must refuse loudly instead of computing on the CPU."""
    from vsag_b200 import _capi

    lib = _capi.load()
    if lib.vb200_device_count() > 0:
        pytest.skip("a CUDA device is present")
    h = C.c_void_p()
    assert lib.vb200_ivf_create(8, 0, 4, 1, 0, C.byref(h)) == -2
    code, msg = _capi.last_error()
    assert code == -2 and "CUDA" in msg
    assert lib.vb200_bf_create(8, 0, 0, C.byref(h)) == -2
    with pytest.raises(engine.VsagB200Error):
        engine.IvfHandle(8, engine.METRIC_L2, 4, engine.QUANT_SQ8)


def test_argument_validation_needs_no_device(engine):
    from vsag_b200 import _capi

    lib = _capi.load()
    h = C.c_void_p()
    assert lib.vb200_ivf_create(0, 0, 4, 1, 0, C.byref(h)) == -3      # dim must be positive
    assert lib.vb200_ivf_create(8, 7, 4, 1, 0, C.byref(h)) == -3      # unknown metric
    assert lib.vb200_ivf_create(8, 0, 4, 9, 0, C.byref(h)) == -3      # no such bucket codec
    assert lib.vb200_bf_create(8, 0, 1, C.byref(h)) == -3             # sq8 is not a brute-force codec here
    assert lib.vb200_kmeans_train(None, 10, 4, 2, 1, None, None, None) == -3
    code, msg = _capi.last_error()
    assert code == -3 and msg
    assert engine.rabitq_code_size(960) == 128
    assert engine.rabitq_code_size(7) == 12


def test_reference_named_c_functions_are_exported():
    """The functions a program written against include/vsag/vsag_c_api.h links to for this path."""
    from vsag_b200 import _capi

    lib = C.CDLL(str(_capi.lib_path()))
    names = ["vsag_index_factory", "vsag_index_destroy", "vsag_index_build", "vsag_index_add", "vsag_index_train",
             "vsag_index_knn_search", "vsag_index_knn_search_with_filter", "vsag_index_range_search",
             "vsag_index_range_search_with_filter", "vsag_serialize_file", "vsag_deserialize_file"]
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"not exported: {missing}"


def test_factory_rejects_bad_parameters_without_a_device():
    """Parameter checks run before any device work: unknown index names and keys fail the same way
    with or without a GPU (Factory::CreateIndex, src/factory/index_registry.cpp)."""
    from vsag_b200.index import Index, VsagError

    with pytest.raises(VsagError):
        Index("hnsw_like_nothing", '{"dtype": "float32", "metric_type": "l2", "dim": 8}')
    with pytest.raises(VsagError):
        Index("ivf", '{"dtype": "float32", "metric_type": "l2", "dim": 8, "index_param": {"no_such_key": 1}}')
    with pytest.raises(VsagError):
        Index("ivf", "this is not json")
