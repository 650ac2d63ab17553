// Inverted-list scan kernels with fused top-k (SQ8 and 1-bit RaBitQ codes).
//
// Schedule: list-major.  The (query, probed list) pairs of a search batch are grouped by list; a
// work item is one list and up to QT of the queries that probe it.  A persistent CTA takes items
// from an atomic counter; each thread owns a few code rows of the list at a time, converts them
// once and scores them against every query of the tile, whose vectors sit in shared memory.  So the codes of
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

constexpr int SQ8_BALLS = 8;   // most covering balls a list can have for the SQ8 scan's pruning (3 .. 8 by its length)

// A work item of the scan queue: queries (pairs pbeg .. pbeg + nqt of its phase) against one list.
struct alignas(32) ScanItemDesc {
    uint32_t list;
    uint32_t pbeg;   // first pair of the item
    uint32_t nqt;    // its number of pairs
    uint32_t lbeg;   // first position of the list
    uint32_t len;    // rows of the list
    uint32_t goff;   // first 8-row group of the list in the tiled code copy (0 when there is none)
    uint32_t pad0, pad1;
};

struct ScanParams {
    const uint8_t* codes;        // [positions x code_stride]
    uint32_t code_stride;        // bytes, multiple of 16
    uint32_t dim;
    uint32_t dpad;               // dim rounded up (16 for SQ8, 128 for RaBitQ)
    const uint32_t* list_off;    // [nlist + 1] positions
    // Work items of the two phases (phase 0: every query's nearest list, phase 1: its other
    // probes), queued one after the other in a single launch.  Within a phase the lists are walked
    // in `order` (longest first), so the items that finish last are the short ones.
    const uint32_t* order;         // [nlist] list ids, longest list first
    const uint32_t* pair_off[2];   // [nlist] first pair of each list
    const uint32_t* pair_cnt[2];   // [nlist] pairs of each list
    const uint32_t* pair_q[2];     // [pairs] query index
    const uint32_t* pair_slot[2];  // [pairs] output slot (query * nprobe + probe rank)
    const uint32_t* item_off[2];   // [nlist + 1] exclusive prefix of tiles, by position in `order`
    const ScanItemDesc* item_map[2];   // [items] every work item, in queue order
    uint32_t n_phases;
    uint32_t nlist;
    uint32_t* item_counter;      // work queue head
    // Optional deadline of the search (timeout_ms): *deadline is a %globaltimer value; once it has passed no
    // further work item is handed out and *timed_out is set -- the granularity at which the reference checks
    // its timer (between buckets, src/algorithm/ivf/ivf.cpp:1747-1751).  nullptr: no deadline.
    const unsigned long long* deadline;
    unsigned long long* timed_out;
    // 0: every work item; 1: only items of lists no longer than k; 2: only items of longer lists.  A launch
    // with a class walks the whole queue with its own counter and passes over the other class's items.
    uint32_t len_class;
    uint32_t k;
    uint32_t cap;                // per-query candidate buffer, power of two >= k + SCAN_THREADS
    uint32_t* thr_g;             // [nq] global bound, ordered distance
    uint64_t* part;              // [slots x k] partial results
    uint8_t* slot_written;       // [slots] set to 1 by whoever writes a slot of `part`, or null: then the caller has
                                 // filled `part` with KEY_INF beforehand and reads all of it
    const float* queries;        // RaBitQ: [nq x (dim + 1)] processed queries
    const float* qw;             // SQ8: [nq x dpad] weights q_d * diff_d / 255, zero padded
    const float* qa;             // SQ8: [nq] per-query constant of the distance
    const float* code_norm;      // SQ8: [positions] |x|^2 of each decoded code
    float coef_b;                // SQ8: distance = qa + coef_b * |x|^2 + coef_c * dot
    float coef_c;
    float inv_sqrt_d;            // RaBitQ
    const float* pair_const;     // SQ8 with residual codes: [nq x nprobe] per-(query, list) term of the distance, by slot
    const uint8_t* qcodes;       // SQ8 uniform: [nq x qcode_stride] the queries' own code records
    uint32_t qcode_stride;
    float su_lower;              // SQ8 uniform: lower bound and (diff / 255)^2
    float su_rate;
    int metric;
    // SQ8 list pruning (both null = off): every decoded row of list l lies in one of SQ8_BALLS
    // balls (centre, radius); a query cannot have anything in the list closer than the triangle
    // inequality allows for the nearest ball, and when that is already worse than the query's
    // bound the (query, list) pair is dropped unscanned.
    const float* ball_centre;    // [nlist][SQ8_BALLS][dim]
    const float* ball_radius;    // [nlist][SQ8_BALLS], rounded up; -1 = empty ball
    const uint32_t* ball_count;  // [nlist] balls in use (the first ball_count[l] slots)
    unsigned long long* scanned; // bytes of codes actually scanned (pairs kept x list length x code size)
    // Id filter (filter_pos_inner null = none): a row is skipped when its inner id is tombstoned or
    // when bit (label & 0xFFFFFFFF) of the caller's bitset is set (BlackListFilter::CheckValid,
    // src/impl/filter/black_list_filter.cpp:25-31; deleted ids: InnerIndexInterface::create_search_filter,
    // src/algorithm/inner_index_interface.cpp:1100-1131).
    const uint32_t* filter_pos_inner;    // [positions] inner id of each stored row
    const uint32_t* deny_inner_bits;     // bitmap over inner ids, or null
    const int64_t* labels;               // [n_total] label per inner id (for the label bitset)
    const uint64_t* invalid_label_bits;  // caller's bitset over labels, or null
    uint64_t n_label_bits;
};

// True when the row at `pos` must not become a candidate.
__device__ __forceinline__ bool
scan_row_filtered(const ScanParams& p, uint32_t pos) {
    const uint32_t inner = __ldg(p.filter_pos_inner + pos);
    if (p.deny_inner_bits != nullptr && ((__ldg(p.deny_inner_bits + (inner >> 5)) >> (inner & 31u)) & 1u)) {
        return true;
    }
    if (p.invalid_label_bits != nullptr) {
        const uint64_t bit = static_cast<uint64_t>(__ldg(p.labels + inner)) & 0xFFFFFFFFull;
        if (bit < p.n_label_bits && ((__ldg(p.invalid_label_bits + (bit >> 6)) >> (bit & 63u)) & 1ull)) {
            return true;
        }
    }
    return false;
}

// Per-tile selection state in shared memory.
//
// A candidate's distance is offered as `partial + qa[qi]`: the scan kernels test
// partial <= bound - qa (one shared load, one compare) and only build the sortable key for the
// few candidates that pass.
template <int QT>
struct TileSelect {
    uint64_t* keys;   // [QT][cap]
    uint32_t* cnt;    // [QT]
    uint32_t* thr;    // [QT] ordered distance bound
    uint32_t* slot;   // [QT]
    uint32_t* qidx;   // [QT]
    float* thrq;      // [QT] bound as a float, minus qa
    float* qa;        // [QT] per-query additive constant
    uint32_t k, cap;

    __device__ __forceinline__ void
    set_bound(int qi, uint32_t u) {
        thr[qi] = u;
        // ordered values above +inf are NaN patterns: "no bound yet"
        float f = u >= 0xFF800000u ? INFINITY : ordered_to_float(u);
        thrq[qi] = f - qa[qi];
    }

    __device__ __forceinline__ void
    push(int qi, float partial, uint32_t pos) {
        if (partial <= thrq[qi]) {
            float dist = partial + qa[qi];
            uint32_t s = atomicAdd(&cnt[qi], 1u);
            keys[static_cast<uint32_t>(qi) * cap + s] = make_key(dist, pos);
        }
    }

    // The same with an id filter: only rows that beat the bound are looked up (few), so the filter
    // costs nothing on the rows the bound rejects anyway.
    __device__ __forceinline__ void
    push(const ScanParams& p, int qi, float partial, uint32_t pos) {
        if (partial <= thrq[qi]) {
            if (p.filter_pos_inner != nullptr && scan_row_filtered(p, pos)) {
                return;
            }
            float dist = partial + qa[qi];
            uint32_t s = atomicAdd(&cnt[qi], 1u);
            keys[static_cast<uint32_t>(qi) * cap + s] = make_key(dist, pos);
        }
    }

    // Sorts query qi's buffer (one warp), keeps the k best, tightens its bound.
    __device__ __forceinline__ void
    compact(int qi, uint32_t lane) {
        uint32_t c = cnt[qi];
        if (c > cap) {
            c = cap;   // offers beyond the buffer were counted but not stored (the tensor-core scan retries them)
        }
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
                    set_bound(qi, t);
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

    // The same for a kernel in which `nwarps` warps (numbered `warp`) share the selection and a round
    // offers at most `incoming` candidates per query.
    __device__ __forceinline__ void
    make_room_w(int nqt, uint32_t warp, uint32_t lane, uint32_t nwarps, uint32_t incoming) {
        for (int qi = static_cast<int>(warp); qi < nqt; qi += static_cast<int>(nwarps)) {
            if (cnt[qi] + incoming > cap) {
                compact(qi, lane);
            }
        }
    }

    // End of the item: write each query's (at most k) best to its slot and publish the bound.
    // Fewer than k survivors are written unsorted: the merge does not need order.
    __device__ __forceinline__ void
    finish(int nqt, uint64_t* part, uint32_t* thr_g, uint8_t* written = nullptr) {
        finish_w(nqt, part, thr_g, threadIdx.x >> 5, threadIdx.x & 31, SCAN_WARPS, written);
    }

    __device__ __forceinline__ void
    finish_w(int nqt, uint64_t* part, uint32_t* thr_g, uint32_t warp, uint32_t lane, uint32_t nwarps,
             uint8_t* written = nullptr) {
        for (int qi = static_cast<int>(warp); qi < nqt; qi += static_cast<int>(nwarps)) {
            if (cnt[qi] >= k) {
                compact(qi, lane);
            }
            uint32_t c = cnt[qi];
            const uint64_t* kq = keys + static_cast<uint32_t>(qi) * cap;
            uint64_t* dst = part + static_cast<uint64_t>(slot[qi]) * k;
            for (uint32_t i = lane; i < k; i += 32) {
                dst[i] = i < c ? kq[i] : KEY_INF;
            }
            if (lane == 0 && c >= k) {
                atomicMin(thr_g + qidx[qi], static_cast<uint32_t>(kq[k - 1] >> 32));
            }
            if (lane == 0 && written != nullptr) {
                written[slot[qi]] = 1;
            }
        }
    }
};

// A work item: `nqt` queries (pairs pbeg .. pbeg + nqt of phase `ph`) against one list.
struct ScanItem {
    uint32_t list;
    uint32_t pbeg;
    uint32_t nqt;
    const uint32_t* pair_q;
    const uint32_t* pair_slot;
};

// Fetches the next work item; returns false when the queue is empty.  All threads call it.
// True once the search's deadline has passed (one thread asks, per work item); records the fact.
__device__ __forceinline__ bool
scan_deadline_passed(const ScanParams& p) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    if (now <= *reinterpret_cast<const volatile unsigned long long*>(p.deadline)) {
        return false;
    }
    *reinterpret_cast<volatile unsigned long long*>(p.timed_out) = 1ull;
    return true;
}

template <int QT>
__device__ __forceinline__ bool
scan_next_item(const ScanParams& p, uint32_t* s_item, ScanItem& it) {
    __syncthreads();
    const uint32_t n0 = p.item_off[0][p.nlist];
    const uint32_t n1 = p.n_phases > 1 ? p.item_off[1][p.nlist] : 0u;
    if (threadIdx.x == 0) {
        uint32_t next = atomicAdd(p.item_counter, 1u);
        while (p.len_class != 0 && next < n0 + n1) {
            const ScanItemDesc* d = next < n0 ? p.item_map[0] + next : p.item_map[1] + (next - n0);
            const bool is_short = __ldg(&d->len) <= p.k;
            if (is_short == (p.len_class == 1u)) {
                break;
            }
            next = atomicAdd(p.item_counter, 1u);
        }
        if (p.deadline != nullptr && scan_deadline_passed(p)) {
            next = 0xFFFFFFFFu;
        }
        s_item[0] = next;
    }
    __syncthreads();
    uint32_t item = s_item[0];
    if (item >= n0 + n1) {
        return false;
    }
    const bool second = item >= n0;
    if (second) {
        item -= n0;
    }
    const uint4 head = __ldg(reinterpret_cast<const uint4*>((second ? p.item_map[1] : p.item_map[0]) + item));
    it.list = head.x;
    it.pbeg = head.y;
    it.nqt = head.z;
    it.pair_q = second ? p.pair_q[1] : p.pair_q[0];
    it.pair_slot = second ? p.pair_slot[1] : p.pair_slot[0];
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
    ts.thrq = reinterpret_cast<float*>(w + 4 * QT);
    ts.qa = reinterpret_cast<float*>(w + 5 * QT);
    fbuf = reinterpret_cast<float*>(w + 6 * QT);
    (void)float_count;
}

template <int QT>
__host__ __device__ inline size_t
tile_smem_bytes(uint32_t cap, uint32_t float_count) {
    return static_cast<size_t>(QT) * cap * 8 + 6 * QT * 4 + static_cast<size_t>(float_count) * 4;
}

// ---------------------------------------------------------------------------------------------
// SQ8 scan.
//
// Reference arithmetic (SQ8ComputeL2Sqr / SQ8ComputeIP, src/simd/kernels/sq8_compute.h:44-137):
//   x_d = fma(code_d * (1/255), diff_d, lower_d);  L2: sum (q_d - x_d)^2;  IP: 1 - sum q_d * x_d.
//
// The scan ranks candidates with an algebraically equal form that costs one FMA per
// (query, code, dimension) instead of a subtract and an FMA:
//   with c'_d = code_d - 128, s_d = diff_d / 255, mid_d = lower_d + 128 s_d:
//     x_d = c'_d s_d + mid_d,   sum q_d x_d = sum (q_d s_d) c'_d + sum q_d mid_d
//   L2: |q|^2 - 2 sum q_d mid_d  +  |x|^2  - 2 sum w_d c'_d,     w_d = q_d s_d
//   IP: 1 - sum q_d mid_d                  -   sum w_d c'_d
// w (per query) and |x|^2 (per code) are prepared outside the loop, so the inner loop is a pure
// FMA of a converted code byte with a weight from shared memory.  Its rounding differs from the
// reference's order by a few 1e-6 relative; the k + slack survivors of every query are therefore
// re-scored with the reference's exact operation order afterwards (sq8_rescore_kernel), and only
// those exact distances are returned.
//
// Register tile: a thread owns R code rows (rows t, t+128, ...) and QT accumulators per row, so
// one 128-bit shared-memory load of weights feeds 4*R FMAs.
// ---------------------------------------------------------------------------------------------
constexpr int SQ8_ROWS = 4;   // code rows per thread

template <int QT, int NR, int NG>
__device__ __forceinline__ void
sq8_tile_dots(const uint8_t* const (&cp)[SQ8_ROWS], const float* __restrict__ w_s, uint32_t dpad,
              float (&acc)[SQ8_ROWS][QT]) {
    constexpr int NQ = NG == 0 ? 1 : NG * 4;   // NG = 0: a tile with a single query (most tiles, once pairs are pruned)
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
            acc[r][qi] = 0.f;
        }
    }
    // Four dimensions per trip, not unrolled: the fully unrolled body (4*NR*NG*4 FMAs) is what has to
    // stay resident in the instruction cache (longer bodies measured slower).  The code bytes of
    // the next trip are fetched before the FMAs of this one.  w_s holds the weights as
    // [dpad/4][QT] float4, so every shared load of a trip is the trip's base plus a constant.
    uint32_t nxt[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        nxt[r] = __ldg(reinterpret_cast<const uint32_t*>(cp[r]));
    }
    const float4* wrow = reinterpret_cast<const float4*>(w_s);
#pragma unroll 1
    for (uint32_t c = 0; c < dpad; c += 4, wrow += QT) {
        float cf[NR][4];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            // byte b -> float(b) - 128 exactly: 0x4B0000bb is the float 2^23 + b
            const uint32_t raw = nxt[r];
            cf[r][0] = __uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7540)) - 8388736.0f;
            cf[r][1] = __uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7541)) - 8388736.0f;
            cf[r][2] = __uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7542)) - 8388736.0f;
            cf[r][3] = __uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7543)) - 8388736.0f;
        }
        if (c + 4 < dpad) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                nxt[r] = __ldg(reinterpret_cast<const uint32_t*>(cp[r] + c + 4));
            }
        }
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
            float4 wv = wrow[qi];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                acc[r][qi] = fmaf(cf[r][0], wv.x, acc[r][qi]);
                acc[r][qi] = fmaf(cf[r][1], wv.y, acc[r][qi]);
                acc[r][qi] = fmaf(cf[r][2], wv.z, acc[r][qi]);
                acc[r][qi] = fmaf(cf[r][3], wv.w, acc[r][qi]);
            }
        }
    }
}

// A tile with one query: the per-trip work is so small that fetching the codes one 32-bit word
// ahead leaves every trip waiting for its load.  Here the codes come 16 bytes at a time, one chunk
// ahead, so a row of 96 dimensions costs six dependent loads instead of twenty-four.
template <int QT, int NR>
__device__ __forceinline__ void
sq8_tile_dots_single(const uint8_t* const (&cp)[SQ8_ROWS], const float* __restrict__ w_s, uint32_t dpad,
                     float (&acc)[SQ8_ROWS][QT]) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        acc[r][0] = 0.f;
    }
    uint4 nxt[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        nxt[r] = __ldg(reinterpret_cast<const uint4*>(cp[r]));
    }
    const float4* wrow = reinterpret_cast<const float4*>(w_s);   // [dpad/4][QT]: slot 0 is the query
#pragma unroll 1
    for (uint32_t c = 0; c < dpad; c += 16, wrow += 4 * QT) {
        uint4 cur[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            cur[r] = nxt[r];
        }
        if (c + 16 < dpad) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                nxt[r] = __ldg(reinterpret_cast<const uint4*>(cp[r] + c + 16));
            }
        }
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float4 wv = wrow[w * QT];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t raw = w == 0 ? cur[r].x : (w == 1 ? cur[r].y : (w == 2 ? cur[r].z : cur[r].w));
                float a = acc[r][0];
                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7540)) - 8388736.0f, wv.x, a);
                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7541)) - 8388736.0f, wv.y, a);
                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7542)) - 8388736.0f, wv.z, a);
                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7543)) - 8388736.0f, wv.w, a);
                acc[r][0] = a;
            }
        }
    }
}

template <int QT, int NR>
__device__ __forceinline__ void
sq8_tile_dots_ng(int ng, const uint8_t* const (&cp)[SQ8_ROWS], const float* __restrict__ w_s,
                 uint32_t dpad, float (&acc)[SQ8_ROWS][QT]) {
    static_assert(QT == 16, "query-group dispatch is written for 16-query tiles");
    switch (ng) {
        case 0: sq8_tile_dots_single<QT, NR>(cp, w_s, dpad, acc); break;
        case 1: sq8_tile_dots<QT, NR, 1>(cp, w_s, dpad, acc); break;
        case 2: sq8_tile_dots<QT, NR, 2>(cp, w_s, dpad, acc); break;
        case 3: sq8_tile_dots<QT, NR, 3>(cp, w_s, dpad, acc); break;
        default: sq8_tile_dots<QT, NR, 4>(cp, w_s, dpad, acc); break;
    }
}

template <int QT>
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
    float* w_s = fbuf;  // [QT][dpad]

    ScanItem it;
    while (scan_next_item<QT>(p, s_item, it)) {
        const uint32_t list = it.list;
        const uint32_t pbeg = it.pbeg;
        int nqt = static_cast<int>(it.nqt);
        if (p.ball_radius != nullptr) {
            // Eight threads per query measure the query against the list's balls; the pair
            // survives unless even the nearest point of every ball is beyond the bound.
            static_assert(SCAN_THREADS == QT * 8, "eight threads per query of the tile");
            const int qi = threadIdx.x >> 3, part = threadIdx.x & 7;
            uint32_t q = 0;
            float qq = 0.f;
            const float* qv = nullptr;
            if (qi < nqt) {
                q = it.pair_q[pbeg + qi];
                qv = p.queries + static_cast<uint64_t>(q) * p.dim;
                if (p.metric != 0) {
                    for (uint32_t d = part; d < p.dim; d += 8) {
                        const float x = __ldg(qv + d);
                        qq = fmaf(x, x, qq);
                    }
                }
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                qq += __shfl_xor_sync(0xffffffffu, qq, o);
            }
            float bound = INFINITY;
            bool bounded = false;
            if (qi < nqt) {
                const uint32_t u = p.thr_g[q];
                bounded = u <= float_to_ordered(INFINITY);   // the query has a bound already
                bound = bounded ? ordered_to_float(u) : INFINITY;
            }
            bool any = !bounded;
            const uint32_t n_balls = __ldg(p.ball_count + list);
            const float* cv = p.ball_centre + static_cast<uint64_t>(list) * SQ8_BALLS * p.dim;
            for (uint32_t j = 0; j < n_balls; ++j, cv += p.dim) {
                float dot = 0.f;
                if (qi < nqt && bounded) {
                    for (uint32_t d = part; d < p.dim; d += 8) {
                        const float x = __ldg(qv + d), c = __ldg(cv + d);
                        if (p.metric == 0) {
                            const float t = x - c;
                            dot = fmaf(t, t, dot);
                        } else {
                            dot = fmaf(x, c, dot);
                        }
                    }
                }
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) {
                    dot += __shfl_xor_sync(0xffffffffu, dot, o);
                }
                const float r = __ldg(p.ball_radius + static_cast<uint64_t>(list) * SQ8_BALLS + j);
                if (r >= 0.f) {
                    // slack: the distances compared here and in the scan differ in rounding only
                    if (p.metric == 0) {
                        const float gap = sqrtf(dot) - r;
                        const float lower = gap > 0.f ? gap * gap : 0.f;
                        any = any || !(lower > bound * 1.001f + 1e-4f * dot);
                    } else {
                        const float lower = 1.0f - dot - sqrtf(qq) * r;
                        any = any || !(lower > bound + 1e-3f * (fabsf(bound) + fabsf(dot) + 1.0f));
                    }
                }
            }
            if (part == 0 && qi < QT) {
                const bool keep = qi < nqt && any;
                ts.cnt[qi] = keep ? 1u : 0u;   // borrowed as the keep flag until the tile is set up
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                // compact the kept queries to the front of the tile
                int kept = 0;
                for (int i = 0; i < nqt; ++i) {
                    if (ts.cnt[i] != 0) {
                        ts.qidx[kept] = it.pair_q[pbeg + i];
                        ts.slot[kept] = it.pair_slot[pbeg + i];
                        ++kept;
                    }
                }
                s_item[0] = static_cast<uint32_t>(kept);
                if (kept > 0 && p.scanned != nullptr) {
                    atomicAdd(p.scanned, static_cast<unsigned long long>(kept) *
                                             (p.list_off[list + 1] - p.list_off[list]) * p.dim);
                }
            }
            __syncthreads();
            nqt = static_cast<int>(s_item[0]);
            if (nqt == 0) {
                continue;
            }
            if (threadIdx.x < QT) {
                const int i = threadIdx.x;
                if (i < nqt) {
                    const uint32_t qk = ts.qidx[i];
                    ts.qa[i] = __ldg(p.qa + qk);
                    ts.set_bound(i, p.thr_g[qk]);
                } else {
                    ts.qidx[i] = 0;
                    ts.slot[i] = 0;
                    ts.qa[i] = 0.f;
                    ts.set_bound(i, 0u);
                }
                ts.cnt[i] = 0;
            }
        } else if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            if (qi < nqt) {
                uint32_t q = it.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = it.pair_slot[pbeg + qi];
                ts.qa[qi] = __ldg(p.qa + q) + (p.pair_const != nullptr ? __ldg(p.pair_const + ts.slot[qi]) : 0.f);
                ts.set_bound(qi, p.thr_g[q]);
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                ts.qa[qi] = 0.f;
                ts.set_bound(qi, 0u);
            }
            ts.cnt[qi] = 0;
        }
        const int ng = nqt == 1 ? 0 : (nqt + 3) >> 2;   // 0: the single-query body
        const uint32_t slots = nqt == 1 ? 1u : static_cast<uint32_t>(ng) * 4;
        __syncthreads();
        // weights of the tile's queries as [dpad/4][QT] float4 (zeros for the unused slots of the
        // last group of four)
        {
            const uint32_t d4n = dpad >> 2;
            float4* w4s = reinterpret_cast<float4*>(w_s);
            for (uint32_t i = threadIdx.x; i < slots * d4n; i += SCAN_THREADS) {
                uint32_t qi = i / d4n, d4 = i % d4n;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (static_cast<int>(qi) < nqt) {
                    v = __ldg(reinterpret_cast<const float4*>(p.qw + static_cast<uint64_t>(ts.qidx[qi]) * dpad) + d4);
                }
                w4s[d4 * QT + qi] = v;
            }
        }
        __syncthreads();

        const uint32_t lbeg = p.list_off[list];
        const uint32_t len = p.list_off[list + 1] - lbeg;
        for (uint32_t r0 = 0; r0 < len; r0 += SCAN_THREADS * SQ8_ROWS) {
            const uint32_t left = len - r0;
            const int nr = left >= SCAN_THREADS * SQ8_ROWS ? SQ8_ROWS
                                                           : static_cast<int>((left + SCAN_THREADS - 1) / SCAN_THREADS);
            const uint8_t* cp[SQ8_ROWS];
            bool valid[SQ8_ROWS];
#pragma unroll
            for (int r = 0; r < SQ8_ROWS; ++r) {
                uint32_t row = r0 + r * SCAN_THREADS + threadIdx.x;
                valid[r] = row < len;
                cp[r] = p.codes + static_cast<uint64_t>(lbeg + (valid[r] ? row : 0)) * p.code_stride;
            }
            float acc[SQ8_ROWS][QT];
            switch (nr) {
                case 1: sq8_tile_dots_ng<QT, 1>(ng, cp, w_s, dpad, acc); break;
                case 2: sq8_tile_dots_ng<QT, 2>(ng, cp, w_s, dpad, acc); break;
                case 3: sq8_tile_dots_ng<QT, 3>(ng, cp, w_s, dpad, acc); break;
                default: sq8_tile_dots_ng<QT, 4>(ng, cp, w_s, dpad, acc); break;
            }
            // one sub-row (at most SCAN_THREADS candidates per query) at a time, so the
            // per-query buffers never overflow
#pragma unroll
            for (int r = 0; r < SQ8_ROWS; ++r) {
                if (r < nr) {
                    if (valid[r]) {
                        const uint32_t pos = lbeg + r0 + r * SCAN_THREADS + threadIdx.x;
                        const float xb = p.coef_b * __ldg(p.code_norm + pos);
#pragma unroll
                        for (int qi = 0; qi < QT; ++qi) {
                            if (qi < nqt) {
                                ts.push(p, qi, fmaf(p.coef_c, acc[r][qi], xb), pos);
                            }
                        }
                    }
                    __syncthreads();
                    ts.make_room(nqt);
                    __syncthreads();
                }
            }
        }
        ts.finish(nqt, p.part, p.thr_g, p.slot_written);
    }
}

// The first phase when it runs alone: every work item is one query against its nearest list, a few hundred
// rows.  A CTA per item spends most of its time in barriers and set-up, so here a warp takes an item by itself:
// its lanes own NR rows each per round, the query's weights sit in the warp's slice of shared memory (every
// lane reads the same word: a broadcast), candidates that beat the bound are appended through a ballot, and
// the warp sorts its own small buffer when it fills.  The arithmetic per row is that of sq8_tile_dots_single
// (INT8 false), so the survivors are the ones the CTA kernel would keep -- or, with INT8, that of the tensor-core
// scan: the weights' three signed-byte terms against the codes as signed bytes (code ^ 0x80 = code - 128), three
// exact integer dot products per four dimensions (dp4a), combined as that kernel's epilogue combines them.
constexpr int SQ8_FIRST_WARPS = 8;

__host__ __device__ inline uint32_t
sq8_first_cap(uint32_t k) {
    uint32_t v = k + 64, c = 64;
    while (c < v) {
        c <<= 1;
    }
    return c;
}

// bytes of a warp's weight slot: the fp32 weights, or the three signed-byte terms of the tensor-core scan's split
__host__ __device__ inline uint32_t
sq8_first_weight_bytes(uint32_t dpad, uint32_t dpad32) {
    const uint32_t f = dpad * 4, b = dpad32 * 3;
    return ((f > b ? f : b) + 15u) & ~15u;
}

__host__ __device__ inline size_t
sq8_first_smem_bytes(uint32_t k, uint32_t dpad, uint32_t dpad32) {
    return static_cast<size_t>(SQ8_FIRST_WARPS) * (static_cast<size_t>(sq8_first_cap(k)) * 8 + sq8_first_weight_bytes(dpad, dpad32));
}

template <bool INT8, int NR = 2>
__global__ void __launch_bounds__(SQ8_FIRST_WARPS * 32)
ivf_sq8_first_kernel(const ScanParams p, const int8_t* __restrict__ qw8, const float* __restrict__ qscale, uint32_t dpad32) {
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cap = sq8_first_cap(p.k), k = p.k, dpad = p.dpad;
    uint64_t* kb = reinterpret_cast<uint64_t*>(smem) + static_cast<size_t>(warp) * cap;
    unsigned char* w_raw = smem + static_cast<size_t>(SQ8_FIRST_WARPS) * cap * 8 +
                           static_cast<size_t>(warp) * sq8_first_weight_bytes(dpad, dpad32);
    float* w_s = reinterpret_cast<float*>(w_raw);
    const uint32_t n_items = p.item_off[0][p.nlist];
    const uint32_t lt_mask = (1u << lane) - 1u;

    for (;;) {
        uint32_t item = 0;
        if (lane == 0) {
            item = atomicAdd(p.item_counter, 1u);
            if (p.deadline != nullptr && scan_deadline_passed(p)) {
                item = 0xFFFFFFFFu;
            }
        }
        item = __shfl_sync(0xffffffffu, item, 0);
        if (item >= n_items) {
            return;
        }
        const ScanItemDesc* desc = p.item_map[0] + item;
        const uint4 head = __ldg(reinterpret_cast<const uint4*>(desc));
        const uint32_t list = head.x, pbeg = head.y, nqt = head.z;
        const uint32_t lbeg = __ldg(p.list_off + list);
        const uint32_t len = __ldg(p.list_off + list + 1) - lbeg;
        for (uint32_t pi = 0; pi < nqt; ++pi) {
            const uint32_t q = __ldg(p.pair_q[0] + pbeg + pi);
            const uint32_t slot = __ldg(p.pair_slot[0] + pbeg + pi);
            const float qa = __ldg(p.qa + q) + (p.pair_const != nullptr ? __ldg(p.pair_const + slot) : 0.f);
            uint32_t thr = p.thr_g[q];
            float thrq = (thr >= 0xFF800000u ? INFINITY : ordered_to_float(thr)) - qa;
            uint32_t cnt = 0;
            float cq = 0.f;   // INT8: coef_c * the query's weight scale
            __syncwarp();
            if (INT8) {
                const uint4* src = reinterpret_cast<const uint4*>(qw8 + static_cast<uint64_t>(q) * 3 * dpad32);
                uint4* dst = reinterpret_cast<uint4*>(w_raw);
                for (uint32_t i = lane; i < (3 * dpad32) >> 4; i += 32) {
                    dst[i] = __ldg(src + i);
                }
                cq = p.coef_c * __ldg(qscale + q);
            } else {
                const float4* src = reinterpret_cast<const float4*>(p.qw + static_cast<uint64_t>(q) * dpad);
                float4* dst = reinterpret_cast<float4*>(w_s);
                for (uint32_t i = lane; i < (dpad >> 2); i += 32) {
                    dst[i] = __ldg(src + i);
                }
            }
            __syncwarp();
            if (lane == 0 && p.scanned != nullptr) {
                atomicAdd(p.scanned, static_cast<unsigned long long>(len) * p.dim);
            }
            // sorts the buffer, keeps the k best and tightens the bound (all lanes)
            auto compact = [&]() {
                const uint32_t n2 = next_pow2(cnt < 2 ? 2 : cnt);
                for (uint32_t i = cnt + lane; i < n2; i += 32) {
                    kb[i] = KEY_INF;
                }
                warp_bitonic_sort(kb, n2, lane);
                if (cnt >= k) {
                    const uint32_t t = static_cast<uint32_t>(kb[k - 1] >> 32);
                    if (t < thr) {
                        thr = t;
                        thrq = (t >= 0xFF800000u ? INFINITY : ordered_to_float(t)) - qa;
                    }
                    cnt = k;
                }
            };
            // NR rows per lane and round.  The first 16 bytes of the next round's rows and this round's |x|^2 are
            // requested before the round's arithmetic, so a round does not start with a trip to memory.
            constexpr uint32_t ROUND = 32u * NR;
            uint4 nxt[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t row = r * 32u + lane;
                nxt[r] = __ldg(reinterpret_cast<const uint4*>(p.codes + static_cast<uint64_t>(lbeg + (row < len ? row : 0)) * p.code_stride));
            }
            for (uint32_t r0 = 0; r0 < len; r0 += ROUND) {
                const uint8_t* cp[NR];
                bool valid[NR];
                float norm[NR], acc[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t row = r0 + r * 32u + lane;
                    valid[r] = row < len;
                    cp[r] = p.codes + static_cast<uint64_t>(lbeg + (valid[r] ? row : 0)) * p.code_stride;
                    norm[r] = valid[r] ? __ldg(p.code_norm + lbeg + row) : 0.f;
                    acc[r] = 0.f;
                }
                if (INT8) {
                    int32_t sum[NR][3];
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        sum[r][0] = sum[r][1] = sum[r][2] = 0;
                    }
#pragma unroll 1
                    for (uint32_t c = 0; c < dpad; c += 16) {
                        int32_t x[NR][4];
#pragma unroll
                        for (int r = 0; r < NR; ++r) {
                            x[r][0] = static_cast<int32_t>(nxt[r].x ^ 0x80808080u);
                            x[r][1] = static_cast<int32_t>(nxt[r].y ^ 0x80808080u);
                            x[r][2] = static_cast<int32_t>(nxt[r].z ^ 0x80808080u);
                            x[r][3] = static_cast<int32_t>(nxt[r].w ^ 0x80808080u);
                        }
                        if (c + 16 < dpad) {
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                nxt[r] = __ldg(reinterpret_cast<const uint4*>(cp[r] + c + 16));
                            }
                        } else if (r0 + ROUND < len) {
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                const uint32_t row = r0 + ROUND + r * 32u + lane;
                                nxt[r] = __ldg(reinterpret_cast<const uint4*>(p.codes + static_cast<uint64_t>(lbeg + (row < len ? row : 0)) * p.code_stride));
                            }
                        }
#pragma unroll
                        for (int t = 0; t < 3; ++t) {
                            const uint4 wv = *reinterpret_cast<const uint4*>(w_raw + t * dpad32 + c);
                            const int32_t wt[4] = {static_cast<int32_t>(wv.x), static_cast<int32_t>(wv.y), static_cast<int32_t>(wv.z),
                                                   static_cast<int32_t>(wv.w)};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
#pragma unroll
                                for (int r = 0; r < NR; ++r) {
                                    sum[r][t] = __dp4a(x[r][j], wt[j], sum[r][t]);
                                }
                            }
                        }
                    }
                    // sum_d w_d (code_d - 128) / s = A1 + (254 A2 + A3) / 254^2, as the tensor-core scan's epilogue
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        acc[r] = fmaf(static_cast<float>(sum[r][1] * 254 + sum[r][2]), 1.0f / 64516.0f, static_cast<float>(sum[r][0]));
                    }
                } else {
                    const float4* wrow = reinterpret_cast<const float4*>(w_s);
#pragma unroll 1
                    for (uint32_t c = 0; c < dpad; c += 16, wrow += 4) {
                        uint4 cur[NR];
#pragma unroll
                        for (int r = 0; r < NR; ++r) {
                            cur[r] = nxt[r];
                        }
                        if (c + 16 < dpad) {
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                nxt[r] = __ldg(reinterpret_cast<const uint4*>(cp[r] + c + 16));
                            }
                        } else if (r0 + ROUND < len) {
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                const uint32_t row = r0 + ROUND + r * 32u + lane;
                                nxt[r] = __ldg(reinterpret_cast<const uint4*>(p.codes + static_cast<uint64_t>(lbeg + (row < len ? row : 0)) * p.code_stride));
                            }
                        }
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            const float4 wv = wrow[w];
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                const uint32_t raw = w == 0 ? cur[r].x : (w == 1 ? cur[r].y : (w == 2 ? cur[r].z : cur[r].w));
                                float a = acc[r];
                                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7540)) - 8388736.0f, wv.x, a);
                                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7541)) - 8388736.0f, wv.y, a);
                                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7542)) - 8388736.0f, wv.z, a);
                                a = fmaf(__uint_as_float(__byte_perm(raw, 0x4B000000u, 0x7543)) - 8388736.0f, wv.w, a);
                                acc[r] = a;
                            }
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < NR; ++h) {
                    const uint32_t pos = lbeg + r0 + h * 32u + lane;
                    float partial = 0.f;
                    bool pass = false;
                    if (valid[h]) {
                        partial = fmaf(INT8 ? cq : p.coef_c, acc[h], p.coef_b * norm[h]);
                        pass = partial <= thrq;
                        if (pass && p.filter_pos_inner != nullptr && scan_row_filtered(p, pos)) {
                            pass = false;
                        }
                    }
                    const uint32_t mask = __ballot_sync(0xffffffffu, pass);
                    if (mask != 0) {
                        if (cnt + 32 > cap) {
                            compact();
                        }
                        if (pass) {
                            kb[cnt + __popc(mask & lt_mask)] = make_key(partial + qa, pos);
                        }
                        cnt += __popc(mask);
                        __syncwarp();
                    }
                }
            }
            if (cnt >= k) {
                compact();
            }
            __syncwarp();
            uint64_t* dst = p.part + static_cast<uint64_t>(slot) * k;
            for (uint32_t i = lane; i < k; i += 32) {
                dst[i] = i < cnt ? kb[i] : KEY_INF;
            }
            if (lane == 0 && cnt >= k) {
                atomicMin(p.thr_g + q, static_cast<uint32_t>(kb[k - 1] >> 32));
            }
            if (lane == 0 && p.slot_written != nullptr) {
                p.slot_written[slot] = 1;
            }
        }
    }
}

// Exact SQ8 distances of the survivors, in the reference's operation order (one thread per
// candidate walks the dimensions upward: SQ8ComputeL2Sqr / SQ8ComputeIP with Width 1), then a
// sort by (distance, position).  cand/out payloads are code positions.
__global__ void __launch_bounds__(128)
sq8_rescore_kernel(const float* __restrict__ queries, uint32_t dim, const uint8_t* __restrict__ codes,
                   uint32_t code_stride, const float* __restrict__ lower, const float* __restrict__ diff,
                   const uint64_t* __restrict__ cand, uint32_t ncand, uint32_t n2, uint32_t k, int metric,
                   uint64_t* __restrict__ out, const float* __restrict__ res_bias, const float* __restrict__ centroids,
                   const uint32_t* __restrict__ list_off, uint32_t nlist) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    // the query and the quantizer's two vectors, staged once: the candidates' chains read them from shared memory
    float* qs = reinterpret_cast<float*>(keys + n2);   // [3][dim]: query, lower, diff
    float* los = qs + dim;
    float* dis = los + dim;
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        qs[d] = __ldg(queries + static_cast<uint64_t>(blockIdx.x) * dim + d);
        los[d] = __ldg(lower + d);
        dis[d] = __ldg(diff + d);
    }
    __syncthreads();
    const float* q = qs;
    const uint64_t* cq = cand + static_cast<uint64_t>(blockIdx.x) * ncand;
    const float inv255 = 1.0f / 255.0f;
    for (uint32_t i = threadIdx.x; i < n2; i += blockDim.x) {
        uint64_t key = KEY_INF;
        if (i < ncand && cq[i] != KEY_INF) {
            uint32_t pos = static_cast<uint32_t>(cq[i]);
            const uint8_t* c = codes + static_cast<uint64_t>(pos) * code_stride;
            float s = 0.f;
            // the same chain over d ascending; the code bytes arrive sixteen at a time (rows are 16-byte aligned)
            for (uint32_t d0 = 0; d0 < dim; d0 += 16) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(c + d0));
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
                const uint32_t left = dim - d0 < 16 ? dim - d0 : 16;
#pragma unroll
                for (uint32_t j = 0; j < 16; ++j) {
                    if (j < left) {
                        const uint32_t d = d0 + j;
                        const float byte = static_cast<float>((words[j >> 2] >> ((j & 3u) * 8)) & 0xFFu);
                        const float x = fmaf(__fmul_rn(byte, inv255), dis[d], los[d]);
                        if (metric == VB200_METRIC_L2) {
                            const float t = __fsub_rn(q[d], x);
                            s = fmaf(t, t, s);
                        } else {
                            s = fmaf(q[d], x, s);
                        }
                    }
                }
            }
            if (metric != VB200_METRIC_L2) {
                s = __fsub_rn(1.0f, s);
            }
            if (res_bias != nullptr) {
                // residual codes (BucketDataCell::ScanBucketById, src/datacell/bucket_datacell.h:552-566): the
                // row's bias leaves first (L2), then 2 * IP(q, centroid) (L2) or IP(q, centroid) (IP)
                uint32_t lo = 0, hi = nlist;   // the list that holds pos
                while (hi - lo > 1) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (__ldg(list_off + mid) <= pos) {
                        lo = mid;
                    } else {
                        hi = mid;
                    }
                }
                const float* cen = centroids + static_cast<uint64_t>(lo) * dim;
                float ipd = 0.f;
                for (uint32_t d = 0; d < dim; ++d) {
                    ipd = fmaf(q[d], __ldg(cen + d), ipd);
                }
                if (metric == VB200_METRIC_L2) {
                    ipd = __fmul_rn(ipd, 2.0f);
                    s = __fsub_rn(s, __ldg(res_bias + pos));
                }
                s = __fsub_rn(s, ipd);
            }
            key = make_key(s, pos);
        }
        keys[i] = key;
    }
    block_bitonic_sort(keys, n2);
    uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        dst[i] = i < n2 ? keys[i] : KEY_INF;
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
// DIRECT: no list is longer than k (the scan depth, factor * k with reorder), so nothing can be selected
// away inside a list -- every row of a probed list is a candidate of its (query, list) slot and is written
// there as it is computed (the slots were cleared to "none" before the launch; the merge takes them in any
// order).  Without the per-query selection buffers a CTA needs only the query values in shared memory, and
// three to four times as many warps fit on an SM, which is what this latency-bound kernel lacks.
template <int QT, bool DIRECT = false>
__global__ void __launch_bounds__(SCAN_THREADS)
ivf_rabitq_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ uint32_t s_item[1];
    __shared__ float s_qnorm[QT];
    __shared__ uint32_t s_direct_q[QT], s_direct_slot[QT];
    TileSelect<QT> ts;
    float* fbuf;
    if (DIRECT) {
        fbuf = reinterpret_cast<float*>(smem);
        ts.qidx = s_direct_q;
        ts.slot = s_direct_slot;
    } else {
        tile_carve<QT>(smem, p.cap, 0, fbuf, ts);
    }
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t dpad = p.dpad;  // multiple of 128
    float* sv = fbuf;              // [QT][dpad]
    const uint32_t bits_bytes = ((p.dim + 7) / 8 + 3) / 4 * 4;

    ScanItem it;
    while (scan_next_item<QT>(p, s_item, it)) {
        const uint32_t list = it.list;
        const uint32_t pbeg = it.pbeg;
        const int nqt = static_cast<int>(it.nqt);
        if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            if (qi < nqt) {
                uint32_t q = it.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = it.pair_slot[pbeg + qi];
                if (!DIRECT) {
                    ts.qa[qi] = 0.f;
                    ts.set_bound(qi, p.thr_g[q]);
                }
                s_qnorm[qi] = __ldg(p.queries + static_cast<uint64_t>(q) * (p.dim + 1) + p.dim);
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                if (!DIRECT) {
                    ts.qa[qi] = 0.f;
                    ts.set_bound(qi, 0u);
                }
                s_qnorm[qi] = 0.f;
            }
            if (!DIRECT) {
                ts.cnt[qi] = 0;
            }
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
        // Two rows per thread: every shared-memory read of a query's four values feeds eight additions,
        // and a thread carries 2 * QT independent chains.
        for (uint32_t r0 = 0; r0 < len; r0 += 2 * SCAN_THREADS) {
            uint32_t rows[2] = {r0 + threadIdx.x, r0 + SCAN_THREADS + threadIdx.x};
            const bool valid[2] = {rows[0] < len, rows[1] < len};
            const uint8_t* code[2] = {p.codes + static_cast<uint64_t>(lbeg + (valid[0] ? rows[0] : 0)) * p.code_stride,
                                      p.codes + static_cast<uint64_t>(lbeg + (valid[1] ? rows[1] : 0)) * p.code_stride};
            float acc[2][QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                acc[0][qi] = 0.f;
                acc[1][qi] = 0.f;
            }
            for (uint32_t c = 0; c < bits_bytes; c += 4) {
                // Sign bits of 32 dimensions; bytes past the sign field are never read because
                // bits_bytes is a multiple of 4 and the loop stops there.
                const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t*>(code[0] + c));
                const uint32_t w1 = __ldg(reinterpret_cast<const uint32_t*>(code[1] + c));
                const uint32_t d0 = c * 8;
#pragma unroll
                for (int b4 = 0; b4 < 8; ++b4) {
                    // bit set -> +sv, clear -> -sv.  fma(sv, +-1, acc) rounds exactly like
                    // acc + (+-sv), and the multipliers are shared by the tile's queries.
                    const uint32_t n0 = ~w0 >> (4 * b4), n1 = ~w1 >> (4 * b4);
                    const float a0 = __uint_as_float(0x3F800000u | ((n0 & 1u) << 31));
                    const float a1 = __uint_as_float(0x3F800000u | ((n0 & 2u) << 30));
                    const float a2 = __uint_as_float(0x3F800000u | ((n0 & 4u) << 29));
                    const float a3 = __uint_as_float(0x3F800000u | ((n0 & 8u) << 28));
                    const float b0 = __uint_as_float(0x3F800000u | ((n1 & 1u) << 31));
                    const float b1 = __uint_as_float(0x3F800000u | ((n1 & 2u) << 30));
                    const float b2 = __uint_as_float(0x3F800000u | ((n1 & 4u) << 29));
                    const float b3 = __uint_as_float(0x3F800000u | ((n1 & 8u) << 28));
#pragma unroll
                    for (int qi = 0; qi < QT; ++qi) {
                        if (qi < nqt) {
                            const float4 sq = *reinterpret_cast<const float4*>(sv + qi * dpad + d0 + 4 * b4);
                            float x = acc[0][qi], y = acc[1][qi];
                            x = fmaf(sq.x, a0, x);
                            y = fmaf(sq.x, b0, y);
                            x = fmaf(sq.y, a1, x);
                            y = fmaf(sq.y, b1, y);
                            x = fmaf(sq.z, a2, x);
                            y = fmaf(sq.z, b2, y);
                            x = fmaf(sq.w, a3, x);
                            y = fmaf(sq.w, b3, y);
                            acc[0][qi] = x;
                            acc[1][qi] = y;
                        }
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (valid[h]) {
                    float bn = __ldg(reinterpret_cast<const float*>(code[h] + bits_bytes));
                    float err = __ldg(reinterpret_cast<const float*>(code[h] + bits_bytes + 4));
                    if (static_cast<double>(fabsf(err)) < 1e-5) {  // float compared with a double literal, as in the reference
                        err = err >= 0.f ? 1.0f : -1.0f;
                    }
#pragma unroll
                    for (int qi = 0; qi < QT; ++qi) {
                        if (qi < nqt) {
                            float qn = s_qnorm[qi];
                            float est = __fdiv_rn(acc[h][qi], err);
                            float p1 = __fmul_rn(bn, bn);
                            float p2 = __fmul_rn(qn, qn);
                            float p3 = __fmul_rn(__fmul_rn(__fmul_rn(-2.0f, bn), qn), est);
                            float dist = __fadd_rn(__fadd_rn(p1, p2), p3);
                            if (DIRECT) {
                                const uint32_t pos = lbeg + rows[h];
                                if (p.filter_pos_inner == nullptr || !scan_row_filtered(p, pos)) {
                                    p.part[static_cast<uint64_t>(ts.slot[qi]) * p.k + rows[h]] = make_key(dist, pos);
                                }
                            } else {
                                ts.push(p, qi, dist, lbeg + rows[h]);
                            }
                        }
                    }
                }
                if (!DIRECT) {
                    __syncthreads();
                    ts.make_room(nqt);
                    __syncthreads();
                }
            }
        }
        if (!DIRECT) {
            ts.finish(nqt, p.part, p.thr_g);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// SQ8 uniform (SQ8UniformQuantizer::ComputeImpl, src/quantization/scalar_quantization/
// sq8_uniform_quantizer.cpp:153-186): the query is encoded like a row, the inner product of the two byte codes
// is an exact integer (generic::SQ8UniformComputeCodesIP, src/simd/generic.cpp:424-433; any summation order
// gives it: four products per dp4a), and the distance is
//   L2:  (float(norm_q) + float(norm_x) - 2 * ip) * rate          with the uint64 norms stored in the records,
//   IP:  1 - (lower * (sum_q + sum_x) + rate * ip + lower * lower) with the fp32 sums stored in the records,
// each operation rounded on its own as written there.  p.dpad = bytes of a record before its trailing field.
// ---------------------------------------------------------------------------------------------
constexpr int SQ8U_QT = 8;

template <int QT>
__global__ void __launch_bounds__(SCAN_THREADS)
ivf_sq8u_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ uint32_t s_item[1];
    __shared__ float s_qfield[QT];   // float(norm) or sum of each query of the tile
    TileSelect<QT> ts;
    float* fbuf;
    tile_carve<QT>(smem, p.cap, 0, fbuf, ts);
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t words = p.dpad / 4;
    uint32_t* sq = reinterpret_cast<uint32_t*>(fbuf);   // [QT][words] the queries' code bytes
    const bool l2 = p.metric == 0;

    ScanItem it;
    while (scan_next_item<QT>(p, s_item, it)) {
        const uint32_t list = it.list;
        const uint32_t pbeg = it.pbeg;
        const int nqt = static_cast<int>(it.nqt);
        if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            ts.qa[qi] = 0.f;
            float field = 0.f;
            if (qi < nqt) {
                uint32_t q = it.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = it.pair_slot[pbeg + qi];
                ts.set_bound(qi, p.thr_g[q]);
                const uint8_t* rec = p.qcodes + static_cast<uint64_t>(q) * p.qcode_stride + p.dpad;
                field = l2 ? static_cast<float>(*reinterpret_cast<const unsigned long long*>(rec))
                           : *reinterpret_cast<const float*>(rec);
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                ts.set_bound(qi, 0u);
            }
            s_qfield[qi] = field;
            ts.cnt[qi] = 0;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < static_cast<uint32_t>(QT) * words; i += SCAN_THREADS) {
            const uint32_t qi = i / words, w = i % words;
            uint32_t v = 0;
            if (static_cast<int>(qi) < nqt) {
                v = __ldg(reinterpret_cast<const uint32_t*>(p.qcodes + static_cast<uint64_t>(ts.qidx[qi]) * p.qcode_stride) + w);
            }
            sq[i] = v;
        }
        __syncthreads();

        const uint32_t lbeg = p.list_off[list];
        const uint32_t len = p.list_off[list + 1] - lbeg;
        for (uint32_t r0 = 0; r0 < len; r0 += SCAN_THREADS) {
            const uint32_t row = r0 + threadIdx.x;
            const bool valid = row < len;
            const unsigned char* rec = p.codes + static_cast<uint64_t>(lbeg + (valid ? row : 0)) * p.code_stride;
            const uint32_t* xw = reinterpret_cast<const uint32_t*>(rec);
            uint32_t acc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                acc[qi] = 0u;
            }
            for (uint32_t w = 0; w < words; ++w) {
                const uint32_t x = __ldg(xw + w);
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        acc[qi] = __dp4a(x, sq[qi * words + w], acc[qi]);
                    }
                }
            }
            if (valid) {
                const float field = l2 ? static_cast<float>(*reinterpret_cast<const unsigned long long*>(rec + p.dpad))
                                       : *reinterpret_cast<const float*>(rec + p.dpad);
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        const float ip = static_cast<float>(static_cast<int32_t>(acc[qi]));
                        float dist;
                        if (l2) {
                            dist = __fmul_rn(__fsub_rn(__fadd_rn(s_qfield[qi], field), __fmul_rn(2.0f, ip)), p.su_rate);
                        } else {
                            const float r = __fadd_rn(__fadd_rn(__fmul_rn(p.su_lower, __fadd_rn(s_qfield[qi], field)),
                                                                __fmul_rn(p.su_rate, ip)),
                                                      __fmul_rn(p.su_lower, p.su_lower));
                            dist = __fsub_rn(1.0f, r);
                        }
                        ts.push(p, qi, dist, lbeg + row);
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
// fp32 buckets (base_quantization_type "fp32", the reference's default): rows are stored as they
// came, distances are the reference's own chains (FP32Quantizer::ComputeDistImpl,
// src/quantization/fp32_quantizer.cpp:163-190): L2 = sum of fma(t, t, acc) with t = x_d - q_d in
// ascending d, IP = 1 - sum of fma(x_d, q_d, acc).  Values are final: no re-scoring follows.
// One thread per row, 8-query tiles staged in shared memory, the shared scheduler and selection.
// ---------------------------------------------------------------------------------------------
constexpr int FP32_QT = 8;

// Half-precision buckets (base_quantization_type "bf16" / "fp16"; HalfPrecisionQuantizer,
// src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123): rows and query are both encoded
// to 16 bits, the distance is the fp32 chain over the widened values (src/simd/kernels/half_compute.h:31-94).
// bf16: FloatToBF16 adds 0x8000 and truncates; fp16: FloatToFP16 clamps the exponent to [-14, 15] and
// truncates the mantissa -- no zero, denormal or infinity encodings -- and FP16ToFloat rebiases
// (src/simd/generic.cpp:191-228).
constexpr int SCAN_FMT_FP32 = 0, SCAN_FMT_BF16 = 1, SCAN_FMT_FP16 = 2;

template <int FMT>
__device__ __forceinline__ uint16_t
half_encode(float v) {
    const uint32_t bits = __float_as_uint(v);
    if (FMT == SCAN_FMT_BF16) {
        return static_cast<uint16_t>((bits + 0x8000u) >> 16);
    }
    const uint32_t sign = bits >> 31;
    int32_t exp = static_cast<int32_t>((bits >> 23) & 0xFFu) - 127;
    exp = exp > 15 ? 15 : (exp < -14 ? -14 : exp);
    return static_cast<uint16_t>((sign << 15) | (static_cast<uint32_t>(exp + 15) << 10) | ((bits & 0x007FFFFFu) >> 13));
}

template <int FMT>
__device__ __forceinline__ float
half_decode(uint32_t h) {
    if (FMT == SCAN_FMT_BF16) {
        return __uint_as_float(h << 16);
    }
    const uint32_t sign = (h >> 15) & 1u;
    const uint32_t exp = ((h >> 10) & 0x1Fu) + 112u;   // - 15 + 127
    return __uint_as_float((sign << 31) | (exp << 23) | ((h & 0x3FFu) << 13));
}

template <int QT, int FMT = SCAN_FMT_FP32>
__global__ void __launch_bounds__(SCAN_THREADS)
ivf_fp32_scan_kernel(const ScanParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ uint32_t s_item[1];
    TileSelect<QT> ts;
    float* fbuf;
    tile_carve<QT>(smem, p.cap, 0, fbuf, ts);
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t dpad = p.dpad;  // dim rounded up to 4
    float* sv = fbuf;              // [QT][dpad]

    ScanItem it;
    while (scan_next_item<QT>(p, s_item, it)) {
        const uint32_t list = it.list;
        const uint32_t pbeg = it.pbeg;
        const int nqt = static_cast<int>(it.nqt);
        if (threadIdx.x < QT) {
            int qi = threadIdx.x;
            ts.qa[qi] = 0.f;
            if (qi < nqt) {
                uint32_t q = it.pair_q[pbeg + qi];
                ts.qidx[qi] = q;
                ts.slot[qi] = it.pair_slot[pbeg + qi];
                ts.set_bound(qi, p.thr_g[q]);
            } else {
                ts.qidx[qi] = 0;
                ts.slot[qi] = 0;
                ts.set_bound(qi, 0u);
            }
            ts.cnt[qi] = 0;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < static_cast<uint32_t>(QT) * dpad; i += SCAN_THREADS) {
            uint32_t qi = i / dpad, d = i % dpad;
            float v = 0.f;
            if (static_cast<int>(qi) < nqt && d < p.dim) {
                v = __ldg(p.queries + static_cast<uint64_t>(ts.qidx[qi]) * p.dim + d);
                if (FMT != SCAN_FMT_FP32) {
                    v = half_decode<FMT>(half_encode<FMT>(v));   // the query is encoded like a row
                }
            }
            sv[i] = v;
        }
        __syncthreads();

        const uint32_t lbeg = p.list_off[list];
        const uint32_t len = p.list_off[list + 1] - lbeg;
        for (uint32_t r0 = 0; r0 < len; r0 += SCAN_THREADS) {
            const uint32_t row = r0 + threadIdx.x;
            const bool valid = row < len;
            const unsigned char* row_ptr = p.codes + static_cast<uint64_t>(lbeg + (valid ? row : 0)) * p.code_stride;
            const float4* x4 = reinterpret_cast<const float4*>(row_ptr);
            const uint2* h4 = reinterpret_cast<const uint2*>(row_ptr);
            float acc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; ++qi) {
                acc[qi] = 0.f;
            }
            for (uint32_t d4 = 0; d4 < (dpad >> 2); ++d4) {
                float4 x;
                if (FMT == SCAN_FMT_FP32) {
                    x = __ldg(x4 + d4);   // padding columns hold zeros on both sides
                } else {
                    // four 16-bit codes; columns past dim count as zero on both sides (the fp16 decoding of
                    // padding bits is not zero)
                    const uint2 h = __ldg(h4 + d4);
                    const uint32_t d0 = 4 * d4;
                    x.x = d0 < p.dim ? half_decode<FMT>(h.x & 0xFFFFu) : 0.f;
                    x.y = d0 + 1 < p.dim ? half_decode<FMT>(h.x >> 16) : 0.f;
                    x.z = d0 + 2 < p.dim ? half_decode<FMT>(h.y & 0xFFFFu) : 0.f;
                    x.w = d0 + 3 < p.dim ? half_decode<FMT>(h.y >> 16) : 0.f;
                }
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        const float4 q = *reinterpret_cast<const float4*>(sv + qi * dpad + 4 * d4);
                        float a = acc[qi];
                        if (p.metric == 0) {
                            float t = __fsub_rn(x.x, q.x);
                            a = fmaf(t, t, a);
                            t = __fsub_rn(x.y, q.y);
                            a = fmaf(t, t, a);
                            t = __fsub_rn(x.z, q.z);
                            a = fmaf(t, t, a);
                            t = __fsub_rn(x.w, q.w);
                            a = fmaf(t, t, a);
                        } else {
                            a = fmaf(x.x, q.x, a);
                            a = fmaf(x.y, q.y, a);
                            a = fmaf(x.z, q.z, a);
                            a = fmaf(x.w, q.w, a);
                        }
                        acc[qi] = a;
                    }
                }
            }
            if (valid) {
#pragma unroll
                for (int qi = 0; qi < QT; ++qi) {
                    if (qi < nqt) {
                        const float dist = p.metric == 0 ? acc[qi] : __fsub_rn(1.0f, acc[qi]);
                        ts.push(p, qi, dist, lbeg + row);
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
