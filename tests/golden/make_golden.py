"""Generates tests/golden/ref_simd_golden.npz by running the reference's own SIMD kernels.

Run in a container that has the reference tree: `make -C oracle` compiles the reference's
src/simd/*.cpp unchanged into oracle/_ref/libvsag_ref_simd.so, and this script records its outputs
on seeded inputs.  The fixture travels to machines without the reference; tests/test_oracle_golden.py
checks the C oracle against it.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import pyoracle as O  # noqa: E402

DIMS = [1, 7, 16, 33, 96, 100, 128, 960]
CASES = 6


def _p(a):
    return C.c_void_p(a.ctypes.data)


def main() -> None:
    O.build()
    R = O.ref()
    if R is None:
        raise SystemExit("oracle/_ref/libvsag_ref_simd.so is missing: the reference tree is needed")
    rng = np.random.default_rng(20240607)
    out = {"dims": np.array(DIMS, np.int64), "cases": np.int64(CASES),
           "avx512": np.int64(R.ref_supports_avx512())}
    for d in DIMS:
        q = rng.uniform(-1, 1, (CASES, d)).astype(np.float32)
        x = rng.uniform(-1, 1, (CASES, d)).astype(np.float32)
        lower = rng.uniform(-1.2, -0.8, d).astype(np.float32)
        diff = rng.uniform(1.6, 2.4, d).astype(np.float32)
        codes = rng.integers(0, 256, (CASES, d), dtype=np.uint8)
        bits = rng.integers(0, 256, (CASES, (d + 7) // 8), dtype=np.uint8)
        centroid = rng.uniform(-0.1, 0.1, d).astype(np.float32)
        inv_sqrt_d = np.float32(1.0) / np.sqrt(np.float32(d))
        qb = O.float_to_bf16(q)
        xb = O.float_to_bf16(x)
        res = {k: np.zeros(CASES, np.float32) for k in (
            "sq8_l2", "sq8_ip", "sq8_l2_generic", "sq8_ip_generic", "fp32_l2", "fp32_ip",
            "fp32_l2_generic", "fp32_ip_generic", "bf16_ip", "bf16_l2", "bf16_ip_generic",
            "rabitq_ip", "rabitq_ip_generic", "norm", "norm_generic")}
        normed = np.zeros((CASES, d), np.float32)
        normed_generic = np.zeros((CASES, d), np.float32)
        for i in range(CASES):
            a = (_p(q[i]), _p(codes[i]), _p(lower), _p(diff), d)
            res["sq8_l2"][i] = R.ref_SQ8ComputeL2Sqr(*a)
            res["sq8_ip"][i] = R.ref_SQ8ComputeIP(*a)
            res["sq8_l2_generic"][i] = R.ref_generic_SQ8ComputeL2Sqr(*a)
            res["sq8_ip_generic"][i] = R.ref_generic_SQ8ComputeIP(*a)
            b = (_p(q[i]), _p(x[i]), d)
            res["fp32_l2"][i] = R.ref_FP32ComputeL2Sqr(*b)
            res["fp32_ip"][i] = R.ref_FP32ComputeIP(*b)
            res["fp32_l2_generic"][i] = R.ref_generic_FP32ComputeL2Sqr(*b)
            res["fp32_ip_generic"][i] = R.ref_generic_FP32ComputeIP(*b)
            h = (_p(qb[i]), _p(xb[i]), d)
            res["bf16_ip"][i] = R.ref_BF16ComputeIP(*h)
            res["bf16_l2"][i] = R.ref_BF16ComputeL2Sqr(*h)
            res["bf16_ip_generic"][i] = R.ref_generic_BF16ComputeIP(*h)
            res["rabitq_ip"][i] = R.ref_RaBitQFloatBinaryIP(_p(q[i]), _p(bits[i]), d, inv_sqrt_d)
            res["rabitq_ip_generic"][i] = R.ref_generic_RaBitQFloatBinaryIP(_p(q[i]), _p(bits[i]), d, inv_sqrt_d)
            res["norm"][i] = R.ref_NormalizeWithCentroid(_p(x[i]), _p(centroid), _p(normed[i]), d)
            res["norm_generic"][i] = R.ref_generic_NormalizeWithCentroid(_p(x[i]), _p(centroid),
                                                                        _p(normed_generic[i]), d)
        pre = f"d{d}_"
        for name, arr in (("q", q), ("x", x), ("lower", lower), ("diff", diff), ("codes", codes),
                          ("bits", bits), ("centroid", centroid), ("qb", qb), ("xb", xb),
                          ("normed", normed), ("normed_generic", normed_generic)):
            out[pre + name] = arr
        for name, arr in res.items():
            out[pre + name] = arr
    # FloatToBF16 on values that exercise the round-half-up rule
    vals = np.concatenate([rng.uniform(-4, 4, 200).astype(np.float32),
                           np.array([0.0, -0.0, 1.0, 1.00390625, 1.005859375, 3.0e38, 1e-40], np.float32)])
    out["bf16_in"] = vals
    out["bf16_out"] = np.array([R.ref_FloatToBF16(float(v)) for v in vals], np.uint16)
    path = Path(__file__).resolve().parent / "ref_simd_golden.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
