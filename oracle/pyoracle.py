"""ctypes binding of the CPU oracle (oracle/vsag_oracle.c) and of the reference's own SIMD kernels
(oracle/_ref/libvsag_ref_simd.so).  TEST INFRASTRUCTURE: imported by tests/, by the smoke check and
by the benchmark's CPU-baseline leg only -- never by the vsag_b200 package.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "liboracle.so"
REF_SO = HERE / "_ref" / "libvsag_ref_simd.so"

_p = C.c_void_p
_u64, _i64, _u32, _i32, _f32 = C.c_uint64, C.c_int64, C.c_uint32, C.c_int, C.c_float


def build(quiet: bool = True) -> None:
    """Runs oracle/Makefile (the C restatement always; the reference SIMD library when the
    reference tree is present on this machine)."""
    res = subprocess.run(["make", "-C", os.fspath(HERE)], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"oracle build failed:\n{res.stdout}\n{res.stderr}")
    if not quiet:
        print(res.stdout)


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not ORACLE_SO.exists():
            build()
        L = C.CDLL(os.fspath(ORACLE_SO))
        L.orc_fp32_l2sqr.restype = _f32
        L.orc_fp32_ip.restype = _f32
        L.orc_sq8_l2sqr.restype = _f32
        L.orc_sq8_ip.restype = _f32
        L.orc_bf16_ip.restype = _f32
        L.orc_bf16_l2sqr.restype = _f32
        L.orc_float_to_bf16.restype = C.c_uint16
        L.orc_float_to_bf16.argtypes = [_f32]
        L.orc_bf16_to_float.restype = _f32
        L.orc_bf16_to_float.argtypes = [C.c_uint16]
        L.orc_kmeans_assign.restype = C.c_double
        L.orc_kmeans_run.restype = C.c_double
        L.orc_rabitq_code_size.restype = _u64
        L.orc_rabitq_code_size.argtypes = [_u64]
        L.orc_normalize_with_centroid.restype = _f32
        L.orc_rabitq_float_binary_ip.restype = _f32
        L.orc_rabitq_float_binary_ip.argtypes = [_p, _p, _u64, _f32]
        L.orc_rabitq_dist.restype = _f32
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def ref():
    """The reference's compiled SIMD kernels, or None when oracle/_ref has not been built."""
    global _ref
    if _ref is None:
        if not REF_SO.exists():
            return None
        R = C.CDLL(os.fspath(REF_SO))
        for name in ("ref_SQ8ComputeL2Sqr", "ref_SQ8ComputeIP", "ref_generic_SQ8ComputeL2Sqr",
                     "ref_generic_SQ8ComputeIP"):
            getattr(R, name).restype = _f32
            getattr(R, name).argtypes = [_p, _p, _p, _p, _u64]
        for name in ("ref_FP32ComputeL2Sqr", "ref_FP32ComputeIP", "ref_generic_FP32ComputeL2Sqr",
                     "ref_generic_FP32ComputeIP", "ref_BF16ComputeIP", "ref_BF16ComputeL2Sqr",
                     "ref_generic_BF16ComputeIP"):
            getattr(R, name).restype = _f32
            getattr(R, name).argtypes = [_p, _p, _u64]
        for name in ("ref_RaBitQFloatBinaryIP", "ref_generic_RaBitQFloatBinaryIP"):
            getattr(R, name).restype = _f32
            getattr(R, name).argtypes = [_p, _p, _u64, _f32]
        for name in ("ref_NormalizeWithCentroid", "ref_generic_NormalizeWithCentroid"):
            getattr(R, name).restype = _f32
            getattr(R, name).argtypes = [_p, _p, _p, _u64]
        R.ref_FloatToBF16.restype = C.c_uint16
        R.ref_FloatToBF16.argtypes = [_f32]
        R.ref_BF16ToFloat.restype = _f32
        R.ref_BF16ToFloat.argtypes = [C.c_uint16]
        R.ref_supports_avx512.restype = C.c_int
        _ref = R
    return _ref


def _a(x, dtype):
    x = np.ascontiguousarray(x, dtype=dtype)
    return x, _p(x.ctypes.data)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_threads(n: int) -> None:
    """Worker threads of the oracle's parallel loops (default: what OpenMP takes from the environment)."""
    lib().orc_set_threads(C.c_int(int(n)))


# ---- generators --------------------------------------------------------------------------------
def gen_uniform(seed: int, count: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    """count floats from std::mt19937(seed) + std::uniform_real_distribution<float>(lo, hi)."""
    out = np.empty(count, np.float32)
    lib().orc_gen_uniform(_u32(seed), _u64(count), _f32(lo), _f32(hi), _p(out.ctypes.data))
    return out


def normalize_rows(x):
    """Rows divided by their norms the way the reference's Normalize does."""
    x, px = _a(x, np.float32)
    out = np.empty_like(x)
    lib().orc_normalize_rows(px, _u64(x.shape[0]), _u64(x.shape[1]), _p(out.ctypes.data))
    return out


# ---- scalar kernels ----------------------------------------------------------------------------
def fp32_l2sqr(a, b) -> float:
    a, pa = _a(a, np.float32)
    b, pb = _a(b, np.float32)
    return float(lib().orc_fp32_l2sqr(pa, pb, _u64(a.size)))


def fp32_ip(a, b) -> float:
    a, pa = _a(a, np.float32)
    b, pb = _a(b, np.float32)
    return float(lib().orc_fp32_ip(pa, pb, _u64(a.size)))


def sq8_l2sqr(q, code, lower, diff) -> float:
    q, pq = _a(q, np.float32)
    code, pc = _a(code, np.uint8)
    lower, pl = _a(lower, np.float32)
    diff, pd = _a(diff, np.float32)
    return float(lib().orc_sq8_l2sqr(pq, pc, pl, pd, _u64(q.size)))


def sq8_ip(q, code, lower, diff) -> float:
    q, pq = _a(q, np.float32)
    code, pc = _a(code, np.uint8)
    lower, pl = _a(lower, np.float32)
    diff, pd = _a(diff, np.float32)
    return float(lib().orc_sq8_ip(pq, pc, pl, pd, _u64(q.size)))


def float_to_bf16(x) -> np.ndarray:
    x, px = _a(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_float_to_bf16_batch(px, _u64(x.size), _p(out.ctypes.data))
    return out


def bf16_to_float(x) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


# ---- SQ8 ---------------------------------------------------------------------------------------
def sq8_train(data, mode: int = 3):
    data, pd = _a(data, np.float32)
    n, d = data.shape
    lower = np.empty(d, np.float32)
    diff = np.empty(d, np.float32)
    rc = lib().orc_sq8_train(pd, _u64(n), _u64(d), _i32(mode), _p(lower.ctypes.data), _p(diff.ctypes.data))
    if rc != 0:
        raise RuntimeError(f"orc_sq8_train failed: {rc}")
    return lower, diff


def sq8_encode(data, lower, diff) -> np.ndarray:
    data, pd = _a(data, np.float32)
    lower, pl = _a(lower, np.float32)
    diff, pf = _a(diff, np.float32)
    n, d = data.shape
    codes = np.empty((n, d), np.uint8)
    lib().orc_sq8_encode(pd, _u64(n), _u64(d), pl, pf, _p(codes.ctypes.data))
    return codes


def sq8_decode(codes, lower, diff) -> np.ndarray:
    codes, pc = _a(codes, np.uint8)
    lower, pl = _a(lower, np.float32)
    diff, pf = _a(diff, np.float32)
    n, d = codes.shape
    out = np.empty((n, d), np.float32)
    lib().orc_sq8_decode(pc, _u64(n), _u64(d), pl, pf, _p(out.ctypes.data))
    return out


# ---- k-means -----------------------------------------------------------------------------------
def kmeans_assign(x, centroids, want_gap: bool = False):
    x, px = _a(x, np.float32)
    centroids, pc = _a(centroids, np.float32)
    n, d = x.shape
    k = centroids.shape[0]
    labels = np.empty(n, np.int32)
    best = np.empty(n, np.float32)
    gap = np.empty(n, np.float32)
    err = lib().orc_kmeans_assign(px, _u64(n), _u64(d), pc, _u64(k), _p(labels.ctypes.data),
                                  _p(best.ctypes.data), _p(gap.ctypes.data))
    if want_gap:
        return labels, float(err), best, gap
    return labels, float(err)


def kmeans_update(x, labels, k: int, it: int = 0):
    x, px = _a(x, np.float32)
    labels, pl = _a(labels, np.int32)
    n, d = x.shape
    centroids = np.empty((k, d), np.float32)
    counts = np.empty(k, np.int32)
    lib().orc_kmeans_update(px, _u64(n), _u64(d), pl, _u64(k), _u32(it), _p(centroids.ctypes.data),
                            _p(counts.ctypes.data))
    return centroids, counts


def kmeans_pp_init(x, k: int, seed: int):
    """k-means++ seeding with a seeded generator: (centroids [k, d], picked rows [k])."""
    x, px = _a(x, np.float32)
    n, d = x.shape
    centroids = np.empty((k, d), np.float32)
    picked = np.empty(k, np.int64)
    lib().orc_kmeans_pp_init(px, _u64(n), _u64(d), _u64(k), _u32(seed), _p(centroids.ctypes.data),
                             _p(picked.ctypes.data))
    return centroids, picked


def std_draws(seed: int, n: int, count: int, restated: bool):
    """count (index, real) pairs from the restated draws or from the C++ library itself."""
    ints = np.empty(count, np.uint64)
    reals = np.empty(count, np.float64)
    if restated:
        fn = lib().orc_std_draws
    else:
        so = HERE / "libstd_draws.so"
        if not so.exists():
            build()
        fn = C.CDLL(os.fspath(so)).std_draws
    fn.restype = None
    fn(_u32(seed), _u64(n), _u64(count), _p(ints.ctypes.data), _p(reals.ctypes.data))
    return ints, reals


def kmeans_run(x, init, iters: int, per_iter: bool = False):
    x, px = _a(x, np.float32)
    n, d = x.shape
    centroids = np.ascontiguousarray(init, np.float32).copy()
    k = centroids.shape[0]
    labels = np.empty(n, np.int32)
    hist = np.empty((iters, n), np.int32) if per_iter else None
    err = lib().orc_kmeans_run(px, _u64(n), _u64(d), _u64(k), _i32(iters), _p(centroids.ctypes.data),
                               _p(labels.ctypes.data), _p(hist.ctypes.data) if per_iter else None)
    return centroids, labels, float(err), hist


# ---- routing / scan / rerank / brute force ---------------------------------------------------
def route(q, centroids, nprobe: int, metric: int = 0):
    q, pq = _a(q, np.float32)
    centroids, pc = _a(centroids, np.float32)
    nq, d = q.shape
    ids = np.empty((nq, nprobe), np.int32)
    dists = np.empty((nq, nprobe), np.float32)
    lib().orc_route(pq, _u64(nq), _u64(d), pc, _u64(centroids.shape[0]), _u64(nprobe), _i32(metric),
                    _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def build_lists(labels: np.ndarray, nlist: int):
    """CSR inverted file for rows appended in ascending row order (IVF::Add with one thread)."""
    labels = np.asarray(labels)
    order = np.argsort(labels, kind="stable").astype(np.int64)
    sizes = np.bincount(labels, minlength=nlist).astype(np.int64)
    off = np.zeros(nlist + 1, np.int64)
    np.cumsum(sizes, out=off[1:])
    return off, order


def ivf_fp32_search(rows, list_off, inner_ids, q, probes, k: int, metric: int = 0):
    """IVF scan over fp32 buckets: rows in list order, offsets and ids as for ivf_sq8_search."""
    rows, pr = _a(rows, np.float32)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    q, pq = _a(q, np.float32)
    probes, pp = _a(probes, np.int32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_fp32_search(pr, po, pi, _u64(d), pq, _u64(nq), pp, _u64(probes.shape[1]), _i64(k), _i32(metric),
                              _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def residual_rows(rows, lists, centroids) -> np.ndarray:
    """rows - centroid of each row's list (BucketDataCell::Train with use_residual)."""
    rows, pr = _a(rows, np.float32)
    lists, pl = _a(lists, np.int32)
    centroids, pc = _a(centroids, np.float32)
    out = np.empty_like(rows)
    lib().orc_residual_rows(pr, _u64(rows.shape[0]), _u64(rows.shape[1]), pl, pc, _p(out.ctypes.data))
    return out


def sq8_residual_encode(rows, lists, centroids, lower, diff, metric: int = 0):
    """use_residual encoding: (codes of rows - centroid, per-row bias for L2)."""
    rows, pr = _a(rows, np.float32)
    lists, pl = _a(lists, np.int32)
    centroids, pc = _a(centroids, np.float32)
    lower, plo = _a(lower, np.float32)
    diff, pdf = _a(diff, np.float32)
    codes = np.empty(rows.shape, np.uint8)
    bias = np.empty(rows.shape[0], np.float32)
    lib().orc_sq8_residual_encode(pr, _u64(rows.shape[0]), _u64(rows.shape[1]), pl, pc, plo, pdf, _i32(metric),
                                  _p(codes.ctypes.data), _p(bias.ctypes.data))
    return codes, bias


def ivf_sq8_residual_search(codes, bias, list_off, inner_ids, lower, diff, centroids, q, probes, k: int, metric: int = 0):
    codes, pc = _a(codes, np.uint8)
    bias, pb = _a(bias, np.float32)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    lower, plo = _a(lower, np.float32)
    diff, pdf = _a(diff, np.float32)
    centroids, pce = _a(centroids, np.float32)
    q, pq = _a(q, np.float32)
    probes, pp = _a(probes, np.int32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_sq8_residual_search(pc, pb, po, pi, _u64(d), plo, pdf, pce, pq, _u64(nq), pp, _u64(probes.shape[1]),
                                      _i64(k), _i32(metric), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def sq8u_code_size(dim: int, metric: int = 0) -> int:
    lib().orc_sq8u_code_size.restype = C.c_uint64
    return int(lib().orc_sq8u_code_size(_u64(dim), _i32(metric)))


def sq8u_train(data, metric: int = 0) -> np.ndarray:
    """SQ8UniformQuantizer::TrainImpl: model = [lower, diff] over all dimensions (metric 2 normalises first)."""
    data, pd = _a(data, np.float32)
    model = np.empty(2, np.float32)
    assert lib().orc_sq8u_train(pd, _u64(data.shape[0]), _u64(data.shape[1]), _i32(metric), _p(model.ctypes.data)) == 0
    return model


def sq8u_encode(data, model, metric: int = 0) -> np.ndarray:
    """Code records [n, code_size]: codes, padding, then the uint64 norm (l2) or the fp32 sum (ip / cosine)."""
    data, pd = _a(data, np.float32)
    model, pm = _a(model, np.float32)
    out = np.empty((data.shape[0], sq8u_code_size(data.shape[1], metric)), np.uint8)
    lib().orc_sq8u_encode(pd, _u64(data.shape[0]), _u64(data.shape[1]), _i32(metric), pm, _p(out.ctypes.data))
    return out


def ivf_sq8u_search(codes, list_off, inner_ids, dim: int, model, q, probes, k: int, metric: int = 0):
    codes, pc = _a(codes, np.uint8)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    model, pm = _a(model, np.float32)
    q, pq = _a(q, np.float32)
    probes, pp = _a(probes, np.int32)
    nq = q.shape[0]
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_sq8u_search(pc, po, pi, _u64(dim), pm, pq, _u64(nq), pp, _u64(probes.shape[1]), _i64(k), _i32(metric),
                              _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def float_to_half(x, fmt: str) -> np.ndarray:
    """HalfPrecisionQuantizer::EncodeOneImpl element by element: "bf16" rounds half up, "fp16" clamps the
    exponent and truncates (generic::FloatToBF16 / FloatToFP16)."""
    x, px = _a(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_float_to_half_batch(px, _u64(x.size), _i32(0 if fmt == "bf16" else 1), _p(out.ctypes.data))
    return out


def half_to_float(x, fmt: str) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    fn = lib().orc_bf16_to_float if fmt == "bf16" else lib().orc_fp16_to_float
    fn.restype = C.c_float
    return np.array([fn(C.c_uint16(int(v))) for v in x.reshape(-1)], np.float32).reshape(x.shape)


def ivf_half_search(codes, list_off, inner_ids, q, probes, k: int, metric: int = 0, fmt: str = "bf16"):
    """IVF scan over bf16 / fp16 buckets: codes[n, dim] uint16 in list order; metric 0 l2, 1 ip, 2 cosine
    (the query is normalised first)."""
    codes, pc = _a(codes, np.uint16)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    q, pq = _a(q, np.float32)
    probes, pp = _a(probes, np.int32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_half_search(pc, po, pi, _u64(d), pq, _u64(nq), pp, _u64(probes.shape[1]), _i64(k), _i32(metric),
                              _i32(0 if fmt == "bf16" else 1), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def ivf_sq8_search(codes, list_off, inner_ids, lower, diff, q, probes, k: int, metric: int = 0,
                   fn=None, nthreads: int = 0):
    codes, pc = _a(codes, np.uint8)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    lower, pl = _a(lower, np.float32)
    diff, pf = _a(diff, np.float32)
    q, pq = _a(q, np.float32)
    probes, pp = _a(probes, np.int32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_sq8_search(pc, po, pi, _u64(d), pl, pf, pq, _u64(nq), pp, _u64(probes.shape[1]), _i64(k),
                             _i32(metric), fn, _i32(nthreads), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def rerank_fp32(base, q, cand, k: int, metric: int = 0):
    base, pb = _a(base, np.float32)
    q, pq = _a(q, np.float32)
    cand, pc = _a(cand, np.int64)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_rerank_fp32(pb, _u64(d), pq, _u64(nq), pc, _u64(cand.shape[1]), _i64(k), _i32(metric),
                          _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def bf_search_fp32(base, q, k: int, metric: int = 0, fn=None, nthreads: int = 0):
    base, pb = _a(base, np.float32)
    q, pq = _a(q, np.float32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_bf_search_fp32(pb, _u64(base.shape[0]), _u64(d), pq, _u64(nq), _i64(k), _i32(metric), fn,
                             _i32(nthreads), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


def bf_search_bf16(base_bf16, q, k: int, metric: int = 1, nthreads: int = 0):
    base_bf16, pb = _a(base_bf16, np.uint16)
    q, pq = _a(q, np.float32)
    nq, d = q.shape
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_bf_search_bf16(pb, _u64(base_bf16.shape[0]), _u64(d), pq, _u64(nq), _i64(k), _i32(metric),
                             _i32(nthreads), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists


# ---- RaBitQ ------------------------------------------------------------------------------------
def random_rotation(dim: int, seed: int) -> np.ndarray:
    """A fixed-seed random orthogonal matrix with determinant +1, handed to both the oracle and the
    engine (the reference draws its own from std::random_device, so it is an input here)."""
    rng = np.random.default_rng(seed)
    g = rng.standard_normal((dim, dim))
    qm, r = np.linalg.qr(g)
    qm = qm * np.sign(np.diag(r))
    if np.linalg.det(qm) < 0:
        qm[:, 0] = -qm[:, 0]
    return np.ascontiguousarray(qm, np.float32)


def rabitq_code_size(dim: int) -> int:
    return int(lib().orc_rabitq_code_size(_u64(dim)))


def rabitq_train(data, rotation) -> np.ndarray:
    data, pd = _a(data, np.float32)
    rotation, pr = _a(rotation, np.float32)
    n, d = data.shape
    centroid = np.empty(d, np.float32)
    lib().orc_rabitq_train(pd, _u64(n), _u64(d), pr, _p(centroid.ctypes.data))
    return centroid


def rabitq_encode(data, rotation, centroid, want_rotated: bool = False):
    data, pd = _a(data, np.float32)
    rotation, pr = _a(rotation, np.float32)
    centroid, pc = _a(centroid, np.float32)
    n, d = data.shape
    codes = np.empty((n, rabitq_code_size(d)), np.uint8)
    rot = np.empty((n, d), np.float32) if want_rotated else None
    lib().orc_rabitq_encode(pd, _u64(n), _u64(d), pr, pc, _p(codes.ctypes.data),
                            _p(rot.ctypes.data) if want_rotated else None)
    return (codes, rot) if want_rotated else codes


def rabitq_process_query(q, rotation, centroid) -> np.ndarray:
    q, pq = _a(q, np.float32)
    rotation, pr = _a(rotation, np.float32)
    centroid, pc = _a(centroid, np.float32)
    n, d = q.shape
    out = np.empty((n, d + 1), np.float32)
    lib().orc_rabitq_process_query(pq, _u64(n), _u64(d), pr, pc, _p(out.ctypes.data))
    return out


def ivf_rabitq_search(codes, list_off, inner_ids, dim: int, qcodes, probes, k: int, nthreads: int = 0):
    codes, pc = _a(codes, np.uint8)
    list_off, po = _a(list_off, np.int64)
    inner_ids, pi = _a(inner_ids, np.int64)
    qcodes, pq = _a(qcodes, np.float32)
    probes, pp = _a(probes, np.int32)
    nq = qcodes.shape[0]
    ids = np.empty((nq, k), np.int64)
    dists = np.empty((nq, k), np.float32)
    lib().orc_ivf_rabitq_search(pc, po, pi, _u64(dim), pq, _u64(nq), pp, _u64(probes.shape[1]), _i64(k),
                                _i32(nthreads), _p(ids.ctypes.data), _p(dists.ctypes.data))
    return ids, dists
