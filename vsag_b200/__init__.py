"""vsag_b200: B200 (sm_100a) engine for VSAG's IVF / BruteForce hot path.

`vsag_b200.engine` binds the C ABI (include/vsag_b200.h); `vsag_b200.index` mirrors the
reference's Factory / Index / Dataset surface on top of it.
"""
from . import engine  # noqa: F401
from ._capi import VsagB200Error, lib_path, load  # noqa: F401

__all__ = ["engine", "VsagB200Error", "lib_path", "load"]
