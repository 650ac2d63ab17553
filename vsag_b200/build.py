"""Builds libvsag_b200.so (sm_100a) in-tree with nvcc.

Usage: python -m vsag_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR.parent / "build" / "obj"
LIB_PATH = PKG_DIR / "libvsag_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the engine cannot be built")
    return nvcc


HOST = PKG_DIR / "host"


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")) + list(HOST.glob("*.cpp")))


def _headers_mtime() -> float:
    hdrs = (list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(HOST.glob("*.h"))
            + list((PKG_DIR.parent / "include").glob("*.h")))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _extra_flags() -> list[str]:
    """VB200_NVCC_FLAGS adds compiler flags: -DVB200_TCS_PROFILE for the scan kernel's cycle counters,
    -DVB200_TC_DIAG for the candidate kernel's timing switches (VB200_TC_DIAG=1/2/4/8 at run time skips the
    selection, the MMAs, the list appends, the final sorts: wrong results, for finding the slowest stage)."""
    return os.environ.get("VB200_NVCC_FLAGS", "").split()


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if not force and obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *_extra_flags(), "-x", "cu", "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJ_DIR / (src.stem + ".ptxas.log")
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every csrc file for sm_100a and links the shared library."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest_obj:
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
