// Inverted-list scan kernels with fused top-k (SQ8 and 1-bit RaBitQ codes).
//
// Schedule: list-major.  The (query, probed list) pairs of a search batch are grouped by list; a
// work item is one list and up to QT of the queries that probe it.  A persistent CTA takes items
// from an atomic counter; each thread owns one code row of the list at a time, decodes it once and
// scores it against every query of the tile, whose vectors sit in shared memory.  So the codes of
// a list cross HBM once per tile (and are L2 hits for the other tiles of the same list) instead
// of once per query as in the reference's query-major loop (src/algorithm/ivf/ivf.cpp:1741-1767,
// src/datacell/bucket_datacell.h:526-572).
//
// Selection: a candidate enters the tile's per-query buffer only if its distance does not exceed
// the query's running bound -- the smaller of the k-th best of this (query, list) pair so far and
// a global per-query bound that every finished pair tightens with atomicMin.  Each pair writes
// its k best as sortable keys to its own slot; a merge kernel then keeps the k best per query.
// This yields the reference's result set (FlatBucketSearcher::Search,
// src/algorithm/ivf/flat_bucket_searcher.cpp:62-104) whatever order the items run in: a dropped
// candidate is strictly worse than k candidates that are kept.
#pragma once

#include "common.cuh"

namespace vb200 {

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_WARPS = SCAN_THREADS / 32;

struct ScanParams {
    const uint8_t* codes;        // [positions x code_stride]
    uint32_t code_stride;        // bytes, multiple of 16
    uint32_t dim;
    uint32_t dpad;               // dim rounded up (16 for SQ8, 128 for RaBitQ)
    const uint32_t* list_off;    // [nlist + 1] positions
    const uint32_t* pair_off;    // [nlist + 1] pair ranges per list
    const uint32_t* pair_q;      // [pairs] query index
    const uint32_t* pair_slot;   // [pairs] output slot (query * nprobe + probe rank)
    const uint32_t* item_off;    // [nlist + 1] exclusive prefix of tiles per list
    uint32_t nlist;
    uint32_t* item_counter;      // work queue head
    uint32_t k;
    uint32_t cap;                // per-query candidate buffer, power of two >= k + SCAN_THREADS
    uint32_t* thr_g;             // [nq] global bound, ordered distance
    uint64_t* part;              // [slots x k] partial results
    const float* queries;        // SQ8: [nq x dim]; RaBitQ: [nq x (dim + 1)] processed queries
    const float* lower;          // SQ8 model, padded to dpad with zeros
    const float* diff;
    float inv_sqrt_d;            // RaBitQ
    int metric;
};

// Per-tile selection state in shared memory.
template <int QT>
struct TileSelect {
    uint64_t* keys;   // [QT][cap]
    uint32_t* cnt;    // [QT]
    uint32_t* thr;    // [QT] ordered distance bound
    uint32_t* slot;   // [QT]
    uint32_t* qidx;   // [QT]
    uint32_t k, cap;

    __device__ __forceinline__ void
    push(int qi, float dist, uint32_t pos) {
        uint32_t u = float_to_ordered(dist);
        if (u <= thr[qi] && dist == dist) {
            uint32_t s = atomicAdd(&cnt[qi], 1u);
            keys[static_cast<uint32_t>(qi) * cap + s] = (static_cast<uint64_t>(u) << 32) | pos;
        }
    }

    // Sorts query qi's buffer (one warp), keeps the k best, tightens its bound.
    __device__ __forceinline__ void
    compact(int qi, uint32_t lane) {
        uint32_t c = cnt[qi];
        uint64_t* kq = keys + static_cast<uint32_t>(qi) * cap;
        uint32_t n2 = next_pow2(c < 2 ? 2 : c);
        for (uint32_t i = c + lane; i < n2; i += 32) {
            kq[i] = KEY_INF;
        }
        warp_bitonic_sort(kq, n2, lane);
        if (lane == 0) {
            if (c > k) {
                cnt[qi] = k;
            }
            if (c >= k) {
                uint32_t t = static_cast<uint32_t>(kq[k - 1] >> 32);
                if (t < thr[qi]) {
                    thr[qi] = t;
                }
            }
        }
        __syncwarp();
    }

    // Between passes: make sure the next SCAN_THREADS candidates fit.  Called by all threads,
    // bracketed by the caller's __syncthreads().
    __device__ __forceinline__ void
    make_room(int nqt) {
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int qi = warp; qi < nqt; qi += SCAN_WARPS) {
            if (cnt[qi] + SCAN_THREADS > cap) {
                compact(qi, lane);
            }
        }
    }

    // End of the item: write each query's k best to its slot and publish the bound.
    __device__ __forceinline__ void
    finish(int nqt, uint64_t* part, uint32_t* thr_g) {
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int qi = warp; qi < nqt; qi += SCAN_WARPS) {
            compact(qi, lane);
            uint32_t c = cnt[qi];
            const uint64_t* kq = keys + static_cast<uint32_t>(qi) * cap;
            uint64_t* dst = part + static_cast<uint64_t>(slot[qi]) * k;
            for (uint32_t i = lane; i < k; i += 32) {
                dst[i] = i < c ? kq[i] : KEY_INF;
            }
            if (lane == 0 && c >= k) {
                atomicMin(thr_g + qidx[qi], static_cast<uint32_t>(kq[k - 1] >> 32));
            }
        }
    }
};

// Fetches the next work item; returns false when the queue is empty.  All threads call it.
__device__ __forceinline__ bool
scan_next_item(const ScanParams& p, uint32_t* s_item, uint32_t& list, uint32_t& tile) {
    __syncthreads();
    const uint32_t n_items = p.item_off[p.nlist];
    if (threadIdx.x == 0) {
        s_item[0] = atomicAdd(p.item_counter, 1u);
    }
    __syncthreads();
    const uint32_t item = s_item[0];
    if (item >= n_items) {
        return false;
    }
    // Largest l with item_off[l] <= item.
    uint32_t lo = 0, hi = p.nlist;
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (p.item_off[mid] <= item) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    list = lo;
    tile = item - p.item_off[lo];
    return true;
}

template <int QT>
__device__ __forceinline__ void
tile_carve(unsigned char* smem, uint32_t cap, uint32_t float_count, float*& fbuf, TileSelect<QT>& ts) {
    ts.keys = reinterpret_cast<uint64_t*>(smem);
    uint32_t* w = reinterpret_cast<uint32_t*>(ts.keys + static_cast<size_t>(QT) * cap);
    ts.cnt = w;
    ts.thr = w + QT;
    ts.slot = w + 2 * QT;
    ts.qidx = w + 3 * QT;
    fbuf = reinterpret_cast<float*>(w + 4 * QT);
    (void)float_count;
}

template <int QT>
__host__ __device__ inline size_t
tile_smem_bytes(uint32_t cap, uint32_t float_count) {
    return static_cast<size_t>(QT) * cap * 8 + 4 * QT * 4 + static_cast<size_t>(float_count) * 4;
}

// ---------------------------------------------------------------------------------------------
// SQ8: distance of SQ8ComputeL2Sqr / SQ8ComputeIP (src/simd/kernels/sq8_compute.h:44-137):
// x = fma(code * (1/255), diff, lower); L2: sum (q - x)^2; IP: 1 - sum q * x.
// ---------------------------------------------------------------------------------------------
template <int QT, int METRIC>
__global__ void __launch_bounds__(SCAN_THREADS)
ivf_sq8_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ uint32_t s_item[1];
    TileSelect<QT> ts;
    float* fbuf;
    tile_carve<QT>(smem, p.cap, 0, fbuf, ts);
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t dpad = p.dpad;
    float* lb_s = fbuf;                 // [dpad]
    float* df_s = fbuf + dpad;          // [dpad]
    float* qs = fbuf + 2 * dpad;        // [QT][dpad]
    for (uint32_t i = threadIdx.x; i < dpad; i += SCAN_THREADS) {
        lb_s[i] = p.lower[i];
        df_s[i] = p.diff[i];
    }
    const float inv255 = 1.0f / 255.0f;

    uint32_t list, tile;
    while (scan_next_item(p, s_item, list, tile)) {
        const uint32_t pbeg = p.pair_off[list] + tile * QT;
        const uint32_t pend = p.pair_off[list + 1];
        const int nqt = static_cast<int>(min(static_cast<uint32_t>(QT), pend - pbeg));
        if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            if (qi < nqt) {
                uint32_t q = p.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = p.pair_slot[pbeg + qi];
                ts.thr[qi] = p.thr_g[q];
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                ts.thr[qi] = 0;
            }
            ts.cnt[qi] = 0;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < static_cast<uint32_t>(QT) * dpad; i += SCAN_THREADS) {
            uint32_t qi = i / dpad, d = i % dpad;
            float v = 0.f;
            if (static_cast<int>(qi) < nqt && d < p.dim) {
                v = __ldg(p.queries + static_cast<uint64_t>(ts.qidx[qi]) * p.dim + d);
            }
            qs[i] = v;
        }
        __syncthreads();

        const uint32_t lbeg = p.list_off[list];
        const uint32_t len = p.list_off[list + 1] - lbeg;
        for (uint32_t r0 = 0; r0 < len; r0 += SCAN_THREADS) {
            const uint32_t row = r0 + threadIdx.x;
            const bool valid = row < len;
            const uint8_t* code = p.codes + static_cast<uint64_t>(lbeg + (valid ? row : 0)) * p.code_stride;
            float acc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                acc[qi] = 0.f;
            }
            for (uint32_t c = 0; c < dpad; c += 16) {
                uint4 w = __ldg(reinterpret_cast<const uint4*>(code + c));
                uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                float x[16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float4 lb4 = *reinterpret_cast<const float4*>(lb_s + c + 4 * j);
                    float4 df4 = *reinterpret_cast<const float4*>(df_s + c + 4 * j);
                    x[4 * j + 0] = fmaf(__fmul_rn(static_cast<float>(ww[j] & 0xffu), inv255), df4.x, lb4.x);
                    x[4 * j + 1] = fmaf(__fmul_rn(static_cast<float>((ww[j] >> 8) & 0xffu), inv255), df4.y, lb4.y);
                    x[4 * j + 2] = fmaf(__fmul_rn(static_cast<float>((ww[j] >> 16) & 0xffu), inv255), df4.z, lb4.z);
                    x[4 * j + 3] = fmaf(__fmul_rn(static_cast<float>(ww[j] >> 24), inv255), df4.w, lb4.w);
                }
#pragma unroll
                for (int g = 0; g < QT; g += 4) {
                    if (g < nqt) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                float4 qv = *reinterpret_cast<const float4*>(qs + (g + u) * dpad + c + 4 * j);
                                if (METRIC == VB200_METRIC_L2) {
                                    float t0 = qv.x - x[4 * j + 0];
                                    float t1 = qv.y - x[4 * j + 1];
                                    float t2 = qv.z - x[4 * j + 2];
                                    float t3 = qv.w - x[4 * j + 3];
                                    acc[g + u] = fmaf(t0, t0, acc[g + u]);
                                    acc[g + u] = fmaf(t1, t1, acc[g + u]);
                                    acc[g + u] = fmaf(t2, t2, acc[g + u]);
                                    acc[g + u] = fmaf(t3, t3, acc[g + u]);
                                } else {
                                    acc[g + u] = fmaf(qv.x, x[4 * j + 0], acc[g + u]);
                                    acc[g + u] = fmaf(qv.y, x[4 * j + 1], acc[g + u]);
                                    acc[g + u] = fmaf(qv.z, x[4 * j + 2], acc[g + u]);
                                    acc[g + u] = fmaf(qv.w, x[4 * j + 3], acc[g + u]);
                                }
                            }
                        }
                    }
                }
            }
            if (valid) {
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        float dist = METRIC == VB200_METRIC_L2 ? acc[qi] : 1.0f - acc[qi];
                        ts.push(qi, dist, lbeg + row);
                    }
                }
            }
            __syncthreads();
            ts.make_room(nqt);
            __syncthreads();
        }
        ts.finish(nqt, p.part, p.thr_g);
    }
}

// ---------------------------------------------------------------------------------------------
// RaBitQ 1-bit: ComputeQueryBaseImpl (src/quantization/rabitq_quantization/
// rabitq_quantizer.cpp:1775-1860) with RaBitQFloatBinaryIP in its scalar order
// (src/simd/generic.cpp:447-471): ip = sum over d ascending of (+-1/sqrt(D)) * q_d, each product
// rounded, then added; est = ip / error; dist = bn^2 + qn^2 + (-2 * bn * qn * est).
// Shared memory holds, per query, sv[d] = (1/sqrt(D)) * q_d already rounded, so the inner loop is
// one add of +-sv[d] per dimension.
// ---------------------------------------------------------------------------------------------
template <int QT>
__global__ void __launch_bounds__(SCAN_THREADS)
ivf_rabitq_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ uint32_t s_item[1];
    __shared__ float s_qnorm[QT];
    TileSelect<QT> ts;
    float* fbuf;
    tile_carve<QT>(smem, p.cap, 0, fbuf, ts);
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t dpad = p.dpad;  // multiple of 128
    float* sv = fbuf;              // [QT][dpad]
    const uint32_t bits_bytes = ((p.dim + 7) / 8 + 3) / 4 * 4;

    uint32_t list, tile;
    while (scan_next_item(p, s_item, list, tile)) {
        const uint32_t pbeg = p.pair_off[list] + tile * QT;
        const uint32_t pend = p.pair_off[list + 1];
        const int nqt = static_cast<int>(min(static_cast<uint32_t>(QT), pend - pbeg));
        if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            if (qi < nqt) {
                uint32_t q = p.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = p.pair_slot[pbeg + qi];
                ts.thr[qi] = p.thr_g[q];
                s_qnorm[qi] = __ldg(p.queries + static_cast<uint64_t>(q) * (p.dim + 1) + p.dim);
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                ts.thr[qi] = 0;
                s_qnorm[qi] = 0.f;
            }
            ts.cnt[qi] = 0;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < static_cast<uint32_t>(QT) * dpad; i += SCAN_THREADS) {
            uint32_t qi = i / dpad, d = i % dpad;
            float v = 0.f;
            if (static_cast<int>(qi) < nqt && d < p.dim) {
                v = __fmul_rn(p.inv_sqrt_d,
                              __ldg(p.queries + static_cast<uint64_t>(ts.qidx[qi]) * (p.dim + 1) + d));
            }
            sv[i] = v;
        }
        __syncthreads();

        const uint32_t lbeg = p.list_off[list];
        const uint32_t len = p.list_off[list + 1] - lbeg;
        for (uint32_t r0 = 0; r0 < len; r0 += SCAN_THREADS) {
            const uint32_t row = r0 + threadIdx.x;
            const bool valid = row < len;
            const uint8_t* code = p.codes + static_cast<uint64_t>(lbeg + (valid ? row : 0)) * p.code_stride;
            float acc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                acc[qi] = 0.f;
            }
            for (uint32_t c = 0; c < bits_bytes; c += 4) {
                // Sign bits of 32 dimensions; bytes past the sign field are never read because
                // bits_bytes is a multiple of 4 and the loop stops there.
                uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(code + c));
                const uint32_t d0 = c * 8;
#pragma unroll
                for (int g = 0; g < QT; g += 4) {
                    if (g < nqt) {
#pragma unroll
                        for (int b4 = 0; b4 < 8; ++b4) {
                            // bit set -> +sv, clear -> -sv (flip the sign bit)
                            const uint32_t nb = ~w >> (4 * b4);
                            const uint32_t f0 = (nb & 1u) << 31, f1 = (nb & 2u) << 30;
                            const uint32_t f2 = (nb & 4u) << 29, f3 = (nb & 8u) << 28;
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                float4 s = *reinterpret_cast<const float4*>(sv + (g + u) * dpad + d0 + 4 * b4);
                                float a = acc[g + u];
                                a = __fadd_rn(a, __uint_as_float(__float_as_uint(s.x) ^ f0));
                                a = __fadd_rn(a, __uint_as_float(__float_as_uint(s.y) ^ f1));
                                a = __fadd_rn(a, __uint_as_float(__float_as_uint(s.z) ^ f2));
                                a = __fadd_rn(a, __uint_as_float(__float_as_uint(s.w) ^ f3));
                                acc[g + u] = a;
                            }
                        }
                    }
                }
            }
            if (valid) {
                float bn = __ldg(reinterpret_cast<const float*>(code + bits_bytes));
                float err = __ldg(reinterpret_cast<const float*>(code + bits_bytes + 4));
                if (static_cast<double>(fabsf(err)) < 1e-5) {  // float compared with a double literal, as in the reference
                    err = err >= 0.f ? 1.0f : -1.0f;
                }
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        float qn = s_qnorm[qi];
                        float est = __fdiv_rn(acc[qi], err);
                        float p1 = __fmul_rn(bn, bn);
                        float p2 = __fmul_rn(qn, qn);
                        float p3 = __fmul_rn(__fmul_rn(__fmul_rn(-2.0f, bn), qn), est);
                        float dist = __fadd_rn(__fadd_rn(p1, p2), p3);
                        ts.push(qi, dist, lbeg + row);
                    }
                }
            }
            __syncthreads();
            ts.make_room(nqt);
            __syncthreads();
        }
        ts.finish(nqt, p.part, p.thr_g);
    }
}

}  // namespace vb200
