"""The host layer mirrors VSAG's public API from scratch (vsag_b200/host/vsag_host.h).  This compile-only test
holds the mirror against the reference's own headers: tests/api_mirror_check.cpp instantiates one piece of user
code against both and static_asserts error codes, search modes and request fields.  It needs the reference's
include directory and is skipped where that is absent."""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REFERENCE_INCLUDE = Path("/root/reference/include")


def test_user_code_compiles_against_reference_headers_and_mirror():
    if not (REFERENCE_INCLUDE / "vsag" / "index.h").exists():
        pytest.skip("the reference's headers are not on this machine")
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    res = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", f"-I{REFERENCE_INCLUDE}", f"-I{ROOT / 'vsag_b200' / 'host'}",
                          str(ROOT / "tests" / "api_mirror_check.cpp")], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-4000:]
