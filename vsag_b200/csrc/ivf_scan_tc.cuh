// SQ8 inverted-list scan on the tensor cores.
//
// The list-major schedule makes a work item -- one list against the queries that probe it -- a small
// integer GEMM: code rows (one byte per dimension) times the queries' weight vectors.  Here it runs
// as tcgen05.mma kind::i8 (signed 8-bit operands, exact 32-bit integer accumulation in tensor
// memory):
//
//   A  the codes of 128 consecutive rows of the list as signed bytes code - 128, read from a second,
//      tiled copy of the inverted lists in which a 128-row tile is one contiguous block already in the
//      shared-memory layout the MMA descriptor describes (K-major, no swizzle: cores of 8 rows x 16
//      bytes, the cores of an 8-row group back to back).  One bulk copy per tile, completion counted
//      on an mbarrier; two tiles in flight per CTA, two CTAs per SM.
//   B  the weights w_d = q_d * diff_d / 255 of up to 32 queries, each split into three signed-byte
//      terms w ~ s * (t1 + t2 / 254 + t3 / 254^2) with s = max|w| / 127 (residual < 1e-7 max|w| per
//      dimension), the terms side by side as 96 output columns.
//   D  [128 rows x 96] int32 in tensor memory, two accumulators so the MMAs of the next tile run
//      while this one drains.
//
// The epilogue (one thread per row) combines the three integer sums of a (row, query) into
//   sum_d w_d (code_d - 128) = s * (A1 + A2 / 254 + A3 / 254^2)
// and applies the ranking form and the bound test of the SIMT scan (ivf_scan.cuh): survivors enter
// the same per-query buffers and are re-scored afterwards in the reference's exact operation order
// (src/simd/kernels/sq8_compute.h:92-137), so returned distances do not depend on which kernel
// nominated them.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises the error flag, the CTA stops
// taking work, frees its tensor memory and returns.
#pragma once

#include "ivf_scan.cuh"
#include "tc_gemm.cuh"

namespace vb200 {

constexpr int TCS_QT = 32;                         // queries per work item
constexpr int TCS_TERMS = 3;                       // signed-byte terms per weight
constexpr int TCS_N = TCS_TERMS * TCS_QT;          // output columns per tile
constexpr int TCS_ROWS = 128;                      // code rows per tile
constexpr int TCS_EPI_WARPS = 8;                   // two per 32-lane quarter of tensor memory: 16 queries each
constexpr int TCS_EPI_THREADS = 32 * TCS_EPI_WARPS;
constexpr int TCS_THREADS = TCS_EPI_THREADS + 64;  // + one warp to issue the MMAs, one for the copies and the work queue
constexpr int TCS_MAX_STAGES = 6;                  // code tiles in flight per CTA, at most (the launch picks how many fit)
constexpr int TCS_MAX_ROUNDS = 40;                 // offer rounds a tile may take (it needs at most 128 / (cap - k) + 1)
constexpr uint32_t TCS_ACC_COLS = 128;             // tensor-memory columns reserved per accumulator

struct TcScanParams {
    ScanParams s;               // scheduler tables, selection state and the SQ8 constants of the SIMT scan
    const int8_t* codes_t;      // tiled signed codes: list after list, 8-row groups of kchunks cores (128 B each)
    const uint32_t* group_off;  // [nlist + 1] first 8-row group of each list
    uint32_t kchunks;           // 16-byte chunks per row: dim rounded up to 32, over 16
    const int8_t* qw8;          // [nq][3][16 * kchunks] the queries' weight terms
    const float* qscale;        // [nq] s of each query
    uint32_t count_scanned;     // add the items' code bytes to s.scanned
    uint32_t spin_limit;        // polls a wait may take before it gives up (TC_SPIN_LIMIT; tests pass less)
    uint32_t stages;            // code tiles in flight per CTA, 2 .. TCS_MAX_STAGES
#ifdef VB200_TCS_PROFILE
    unsigned long long* prof;   // [grid][16] cycle counters of one thread per role (diagnostic builds only)
#endif
    int* error_flag;
};

// Instruction descriptor of kind::i8: int32 accumulator, signed 8-bit A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t
umma_idesc_s8(uint32_t m, uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, 128 x N x 32, signed bytes in, int32 out.
__device__ __forceinline__ void
umma_s8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void
tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void
tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TcsItem {
    uint32_t valid, second;
    uint32_t list, pbeg, nqt, lbeg, len, goff;
};

// What the copy warp prepares for a work item while the item before it runs.
struct TcsStaged {
    uint32_t qidx[TCS_QT], slot[TCS_QT], thr[TCS_QT];
    float qa[TCS_QT], cq[TCS_QT];
};

struct TcsShared {
    uint64_t full[TCS_MAX_STAGES];    // a tile's codes have landed
    uint64_t freed[TCS_MAX_STAGES];   // the MMAs that read the stage have retired
    uint64_t acc_full[2];         // accumulator holds a finished tile
    uint64_t acc_free[2];         // accumulator drained by the epilogue threads
    uint32_t tmem_base;
    uint32_t failed;
    TcsItem item[2];              // this work item and the next
    TcsStaged staged[2];          // their queries' constants
    alignas(16) float cq[TCS_QT]; // coef_c * s of the running item's queries
};

#ifdef VB200_TCS_PROFILE
#define TCS_T0() const long long _t0 = clock64()
#define TCS_ACC(slot) prof_acc[slot] += static_cast<unsigned long long>(clock64() - _t0)
#define TCS_CNT(slot) prof_acc[slot] += 1
#else
#define TCS_T0()
#define TCS_ACC(slot)
#define TCS_CNT(slot)
#endif

// Bounded wait that also gives up as soon as another role of the CTA has failed.  Each poll may
// suspend the thread in hardware for up to a microsecond and ends as soon as the phase completes, so
// waiting threads neither spin on issue slots (the two single-thread roles share their schedulers with
// epilogue warps) nor oversleep (the epilogue warps meet at a barrier after every tile).
__device__ __forceinline__ bool
tcs_wait(uint64_t* bar, uint32_t parity, const volatile uint32_t* failed, uint32_t limit) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
            : "memory");
        if (done) {
            return true;
        }
        if ((spin & 15u) == 15u && *failed != 0) {
            return false;
        }
    }
    return false;
}

__device__ __forceinline__ void
tcs_epilogue_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(TCS_EPI_THREADS) : "memory");
}

// Barrier over the epilogue threads that also tells every one of them whether any passed `flag`.
__device__ __forceinline__ bool
tcs_epilogue_barrier_any(bool flag) {
    uint32_t out;
    asm volatile(
        "{\n.reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "bar.red.or.pred p, 1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(out)
        : "r"(flag ? 1u : 0u), "n"(TCS_EPI_THREADS)
        : "memory");
    return out != 0;
}

// Sorts a query's candidate buffer in registers and cuts it to its k smallest keys (one warp).  Element
// e of the buffer sits in register e / 32 of lane e % 32; the bitonic network exchanges registers of a
// lane when the partner is 32 or more elements away and shuffles between lanes otherwise, so a sort of
// 128 keys is 25 shuffle stages instead of 28 trips through shared memory with a warp barrier each.
// Returns the k-th smallest key (KEY_INF when the buffer holds fewer than k: nothing is cut then).
// Kept out of line: it runs once in many tiles and must not claim registers in the epilogue's loop.
template <int R>
__device__ __noinline__ uint64_t
tcs_sort_cut(uint64_t* kq, uint32_t count, uint32_t k, uint32_t lane) {
    uint64_t key[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint32_t i = r * 32 + lane;
        key[r] = i < count ? kq[i] : KEY_INF;
    }
#pragma unroll
    for (uint32_t size = 2; size <= 32u * R; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 32) {
                // partner in the same lane: registers r and r ^ (stride / 32)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int pr = r ^ static_cast<int>(stride >> 5);
                    if (pr > r) {
                        const bool up = (((static_cast<uint32_t>(r) << 5) | lane) & size) == 0;
                        const uint64_t a = key[r], b = key[pr];
                        if ((a > b) == up) {
                            key[r] = b;
                            key[pr] = a;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t e = (static_cast<uint32_t>(r) << 5) | lane;
                    const uint64_t mine = key[r];
                    const uint64_t other = __shfl_xor_sync(0xffffffffu, mine, stride);
                    const bool up = (e & size) == 0;
                    const bool lower = (lane & stride) == 0;        // this lane holds the lower index of the pair
                    const bool take_min = lower == up;
                    key[r] = take_min ? (mine < other ? mine : other) : (mine > other ? mine : other);
                }
            }
        }
    }
    if (count < k) {
        return KEY_INF;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint32_t e = (static_cast<uint32_t>(r) << 5) | lane;
        if (e < k) {
            kq[e] = key[r];
        }
    }
    uint64_t kth = 0;
    const uint32_t last = k - 1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint64_t v = __shfl_sync(0xffffffffu, key[r], last & 31u);
        if (static_cast<uint32_t>(r) == (last >> 5)) {
            kth = v;
        }
    }
    __syncwarp();
    return kth;
}

__device__ __forceinline__ uint64_t
tcs_sort_cut_any(uint64_t* kq, uint32_t count, uint32_t k, uint32_t cap, uint32_t lane) {
    if (cap <= 64) {
        return tcs_sort_cut<2>(kq, count, k, lane);
    }
    if (cap <= 128) {
        return tcs_sort_cut<4>(kq, count, k, lane);
    }
    return tcs_sort_cut<8>(kq, count, k, lane);
}

constexpr int TCS_SELECT_MAX = 8;   // keys per lane at most: buffers of up to 256 keys

// Next work item from the queue (one thread).
__device__ __forceinline__ void
tcs_fetch_item(const ScanParams& p, uint32_t n0, uint32_t n1, TcsItem* out) {
    uint32_t item = atomicAdd(p.item_counter, 1u);
    if (item >= n0 + n1 || (p.deadline != nullptr && scan_deadline_passed(p))) {
        out->valid = 0;
        return;
    }
    const bool second = item >= n0;
    if (second) {
        item -= n0;
    }
    const uint4* d = reinterpret_cast<const uint4*>((second ? p.item_map[1] : p.item_map[0]) + item);
    const uint4 head = __ldg(d), tail = __ldg(d + 1);
    out->list = head.x;
    out->pbeg = head.y;
    out->nqt = head.z;
    out->lbeg = head.w;
    out->len = tail.x;
    out->goff = tail.y;
    out->second = second ? 1u : 0u;
    out->valid = 1;
}

// The kernel.  Warps 0-7 drain the accumulators (the epilogue), warp 8 issues the MMAs, warp 9 feeds
// everything else: it takes work items from the queue one ahead, stages the next item's query
// constants and its B operand (two B buffers) and copies code tiles as stages come free, also across
// the boundary between two items, so an item starts with its operands already in shared memory.
// WIDE: code rows longer than 256 bytes in the tiled copy (see the conversion of the first integer sum below).
template <bool WIDE>
__global__ void __launch_bounds__(TCS_THREADS, 2)
ivf_sq8_scan_tc_kernel(const TcScanParams tp) {
    extern __shared__ __align__(1024) unsigned char tcs_smem[];
    unsigned char* const smem = tcs_smem;
    __shared__ TcsShared sh;
    const ScanParams& p = tp.s;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kchunks = tp.kchunks;
    const uint32_t row_bytes = kchunks * 16;                 // bytes of one code row in the tiled copy
    constexpr bool wide_sums = WIDE;                         // rows past 256 bytes: an integer sum may pass 2^22
    const uint32_t group_bytes = kchunks * 128;              // one 8-row group
    const uint32_t tile_bytes = TCS_ROWS * row_bytes;
    const uint32_t b_bytes = TCS_N * row_bytes;
    const uint32_t stages = tp.stages;
    unsigned char* a_smem = smem;                            // [stages][tile_bytes]
    unsigned char* b_smem = smem + stages * tile_bytes;      // [2][TCS_N rows][row_bytes] in core layout
    TileSelect<TCS_QT> ts;
    float* unused;
    tile_carve<TCS_QT>(b_smem + 2 * b_bytes, p.cap, 0, unused, ts);
    ts.k = p.k;
    ts.cap = p.cap;
    const uint32_t n0 = p.item_off[0][p.nlist];
    const uint32_t n1 = p.n_phases > 1 ? p.item_off[1][p.nlist] : 0u;
    const uint32_t spin_limit = tp.spin_limit;
#ifdef VB200_TCS_PROFILE
    // 0 E:wait acc  1 E:load+math  2 E:offer rounds+barrier  3 E:set-up+barrier 2  4 E:loop-top barrier  5 E:finish
    // 6 M:wait acc_free  7 M:wait full  8 M:issue  9 P:wait freed  10 P:prepare  11 P:loop-top barrier
    // 12 tiles  13 items  14 extra rounds  15 total cycles  16 E:offer loop  17 E:barrier_any  18 E:compaction+barrier  19 offers
    unsigned long long prof_acc[24] = {0};
    const long long prof_begin = clock64();
#endif

    if (tid == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.freed[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&sh.acc_full[a], 1);
            mbar_init(&sh.acc_free[a], TCS_EPI_THREADS);
        }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TCS_EPI_WARPS) {
        tmem_alloc(&sh.tmem_base, 2 * TCS_ACC_COLS);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = sh.tmem_base;
    const volatile uint32_t* failed = &sh.failed;

    // pipeline positions; every role walks the same sequence of tiles, so they stay in step
    uint32_t c_stage = 0, c_phase = 0, c_count = 0, c_ahead = 0;                  // copies (lane 0 of warp 9)
    bool c_ok = true;
    unsigned long long scanned_local = 0;   // code bytes of the items this CTA took (lane 0 of warp 9)
    uint32_t m_stage = 0, m_phase = 0, m_acc = 0, m_acc_phase = 0, m_tiles = 0;   // MMAs
    uint32_t e_tile = 0;                                                          // epilogue
    const uint32_t idesc = umma_idesc_s8(TCS_ROWS, TCS_N);
    const uint32_t ksteps = kchunks >> 1;
    // epilogue geometry: this thread's tensor-memory lane (row of the tile) and its 16 queries
    const uint32_t quarter = warp & 3u, half = (warp >> 2) & 1u;
    const uint32_t row = quarter * 32 + lane;
    const uint32_t q_first = half * 16;

    // One code tile into the next stage (lane 0 of the copy warp).
    auto copy_tile = [&](const unsigned char* src) -> bool {
        if (c_count >= stages) {
            TCS_T0();
            if (!tcs_wait(&sh.freed[c_stage], c_phase ^ 1u, failed, spin_limit)) {
                return false;
            }
            TCS_ACC(9);
        }
        mbar_expect_tx(&sh.full[c_stage], tile_bytes);
        bulk_copy_g2s(a_smem + c_stage * tile_bytes, src, tile_bytes, &sh.full[c_stage]);
        ++c_count;
        if (++c_stage == stages) {
            c_stage = 0;
            c_phase ^= 1u;
        }
        return true;
    };
    // The copy warp prepares work item `n`: description, query constants, B operand, first code tiles.
    auto prepare_item = [&](uint32_t n) {
        const uint32_t buf = n & 1u;
        if (lane == 0) {
            tcs_fetch_item(p, n0, n1, &sh.item[buf]);
        }
        __syncwarp();
        const TcsItem it = sh.item[buf];
        c_ahead = 0;
        if (it.valid == 0) {
            return;
        }
        const uint32_t* pair_q = it.second ? p.pair_q[1] : p.pair_q[0];
        const uint32_t* pair_slot = it.second ? p.pair_slot[1] : p.pair_slot[0];
        TcsStaged& st = sh.staged[buf];
        if (lane < it.nqt) {
            const uint32_t q = pair_q[it.pbeg + lane];
            st.qidx[lane] = q;
            st.slot[lane] = pair_slot[it.pbeg + lane];
            st.qa[lane] = __ldg(p.qa + q);
            st.cq[lane] = p.coef_c * __ldg(tp.qscale + q);
            st.thr[lane] = p.thr_g[q];
        } else {
            st.qidx[lane] = 0;
            st.slot[lane] = 0;
            st.qa[lane] = 0.f;
            st.cq[lane] = 0.f;
            st.thr[lane] = 0u;
        }
        __syncwarp();
        // B row n = term * TCS_QT + query slot; 16-byte chunk c of it sits at core (n / 8, c), row n % 8
        unsigned char* b_dst = b_smem + buf * b_bytes;
        const uint32_t units = TCS_N * kchunks;
        for (uint32_t u = lane; u < units; u += 32) {
            const uint32_t r = u / kchunks, c = u - r * kchunks;
            const uint32_t term = r / TCS_QT, qi = r - term * TCS_QT;
            unsigned char* dst = b_dst + (r >> 3) * group_bytes + c * 128 + (r & 7u) * 16;
            if (qi < it.nqt) {
                // asynchronous 16-byte copies: all of a lane's chunks are in flight together
                const int8_t* src = tp.qw8 + (static_cast<uint64_t>(st.qidx[qi]) * TCS_TERMS + term) * row_bytes + c * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        // the MMAs read B through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane == 0) {
            scanned_local += static_cast<unsigned long long>(it.nqt) * it.len * p.dim;
            // the item's first code tiles, as far as stages are free by the time the item before is done with them
            const uint32_t ntiles = (it.len + TCS_ROWS - 1) / TCS_ROWS;
            const unsigned char* a_src = reinterpret_cast<const unsigned char*>(tp.codes_t) +
                                         static_cast<uint64_t>(it.goff) * group_bytes;
            const uint32_t ahead = ntiles < stages ? ntiles : stages;
            for (uint32_t t = 0; t < ahead && c_ok; ++t) {
                c_ok = copy_tile(a_src + static_cast<uint64_t>(t) * tile_bytes);
                if (c_ok) {
                    ++c_ahead;
                }
            }
            if (!c_ok) {
                sh.failed = 1;
                atomicOr(tp.error_flag, 1);
            }
        }
        __syncwarp();
    };

    if (warp == TCS_EPI_WARPS + 1) {
        prepare_item(0);
    }

    for (uint32_t n_item = 0;; ++n_item) {
        {
            TCS_T0();
            __syncthreads();   // the previous item is finished by every role; this one has been prepared
            TCS_ACC(warp == TCS_EPI_WARPS + 1 ? 11 : 4);
        }
        const uint32_t buf = n_item & 1u;
        const TcsItem it = sh.item[buf];
        if (it.valid == 0 || sh.failed != 0) {
            break;
        }
        const int nqt = static_cast<int>(it.nqt);
        const uint32_t lbeg = it.lbeg, len = it.len;
        const uint32_t ntiles = (len + TCS_ROWS - 1) / TCS_ROWS;
        {
            // The candidate buffers of an item share one pool: an item with few queries gives each of them a
            // larger buffer (up to about 4k keys), which spares a query without a bound yet -- every row is a
            // candidate then -- most of its compactions.
            uint32_t c = p.cap;
            const uint32_t want = next_pow2(4 * p.k);
            while (c < want && 2 * c <= 32 * TCS_SELECT_MAX && 2 * c * it.nqt <= p.cap * TCS_QT) {
                c <<= 1;
            }
            ts.cap = c;
        }

        if (warp == TCS_EPI_WARPS + 1) {
            // ---------------- the rest of this item's code tiles, then the next item ----------------
            if (lane == 0) {
                const unsigned char* a_src = reinterpret_cast<const unsigned char*>(tp.codes_t) +
                                             static_cast<uint64_t>(it.goff) * group_bytes;
                for (uint32_t t = c_ahead; t < ntiles && c_ok; ++t) {
                    c_ok = copy_tile(a_src + static_cast<uint64_t>(t) * tile_bytes);
                }
                if (!c_ok) {
                    sh.failed = 1;
                    atomicOr(tp.error_flag, 1);
                }
            }
            __syncwarp();
            {
                TCS_T0();
                prepare_item(n_item + 1);
                TCS_ACC(10);
            }
            continue;   // the copy warp takes no part in the barriers below
        }
        TCS_T0();
        TCS_CNT(13);
        if (tid < TCS_QT) {
            // selection state of the item's queries from what the copy warp staged
            const TcsStaged& st = sh.staged[buf];
            const int qi = static_cast<int>(tid);
            ts.qidx[qi] = st.qidx[qi];
            ts.slot[qi] = st.slot[qi];
            ts.qa[qi] = st.qa[qi];
            sh.cq[qi] = st.cq[qi];
            if (qi < nqt) {
                ts.set_bound(qi, st.thr[qi]);
            } else {
                ts.thr[qi] = 0u;             // unused slots never pass the bound test
                ts.thrq[qi] = -INFINITY;
            }
            ts.cnt[qi] = 0;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(TCS_EPI_THREADS + 32) : "memory");   // epilogue warps + the MMA warp
        TCS_ACC(3);

        if (warp == TCS_EPI_WARPS) {
            // ---------------- MMA issue (one thread) ----------------
            if (lane == 0) {
                const uint64_t b_desc = umma_desc(smem_u32(b_smem + buf * b_bytes), 128, group_bytes);
                bool ok = true;
                for (uint32_t t = 0; t < ntiles && ok; ++t) {
                    if (m_tiles >= 2) {
                        TCS_T0();
                        ok = tcs_wait(&sh.acc_free[m_acc], m_acc_phase ^ 1u, failed, spin_limit);
                        TCS_ACC(6);
                        if (!ok) {
                            break;
                        }
                    }
                    {
                        TCS_T0();
                        ok = tcs_wait(&sh.full[m_stage], m_phase, failed, spin_limit);
                        TCS_ACC(7);
                    }
                    if (!ok) {
                        break;
                    }
                    TCS_T0();
                    tc_fence_after_sync();
                    const uint64_t a_desc = umma_desc(smem_u32(a_smem + m_stage * tile_bytes), 128, group_bytes);
                    const uint32_t d_tmem = tmem_base + m_acc * TCS_ACC_COLS;
                    for (uint32_t ks = 0; ks < ksteps; ++ks) {
                        // a k-step of 32 bytes = two 16-byte cores: 256 B = 16 descriptor units
                        umma_s8(d_tmem, a_desc + ks * 16, b_desc + ks * 16, idesc, ks == 0 ? 0u : 1u);
                    }
                    umma_commit(&sh.freed[m_stage]);
                    umma_commit(&sh.acc_full[m_acc]);
                    TCS_ACC(8);
                    if (++m_stage == stages) {
                        m_stage = 0;
                        m_phase ^= 1u;
                    }
                    ++m_tiles;
                    if (++m_acc == 2) {
                        m_acc = 0;
                        m_acc_phase ^= 1u;
                    }
                }
                if (!ok) {
                    sh.failed = 1;
                    atomicOr(tp.error_flag, 1);
                }
            }
            __syncwarp();
        } else {
            // ---------------- epilogue: one thread per (row of the tile, half of the queries) ----------------
            const bool any_query = static_cast<int>(q_first) < nqt;   // this warp's half holds live queries
            // one warp: query qi keeps its k best candidates, its bound becomes the k-th
            auto compact_query = [&](int qi) {
                const uint32_t have = ts.cnt[qi] < ts.cap ? ts.cnt[qi] : ts.cap;   // offers beyond the buffer were not stored
                const uint64_t kth = tcs_sort_cut_any(ts.keys + static_cast<uint32_t>(qi) * ts.cap, have, ts.k, ts.cap, lane);
                if (lane == 0) {
                    ts.cnt[qi] = have < ts.k ? have : ts.k;
                    if (kth != KEY_INF && static_cast<uint32_t>(kth >> 32) < ts.thr[qi]) {
                        ts.set_bound(qi, static_cast<uint32_t>(kth >> 32));
                    }
                }
                __syncwarp();
            };
            for (uint32_t t = 0; t < ntiles; ++t, ++e_tile) {
                const uint32_t acc = e_tile & 1u;
                const uint32_t r = t * TCS_ROWS + row;
                const bool valid = r < len;
                const uint32_t pos = lbeg + (valid ? r : 0u);
                const float xb = p.coef_b * __ldg(p.code_norm + pos);
                uint32_t pend = 0;   // bit j: this row is a candidate of query slot q_first + j that is not stored yet
                uint32_t a1[16], a2[16], a3[16];
                // sum_d w_d (code_d - 128) / s = A1 + (254 A2 + A3) / 254^2; |A1| < 2^22 (certain up to 256 dimensions:
                // 127 * 128 * 256 < 2^22) converts exactly through the float whose integer image is 1.5 * 2^23 + A1,
                // longer rows take the conversion instruction
                auto partial_of = [&](int j, float cqj) -> float {
                    const int32_t low = static_cast<int32_t>(a2[j]) * 254 + static_cast<int32_t>(a3[j]);
                    const float hi = wide_sums ? static_cast<float>(static_cast<int32_t>(a1[j]))
                                               : __int_as_float(static_cast<int32_t>(a1[j]) + 0x4B400000) - 12582912.0f;
                    const float f = fmaf(static_cast<float>(low), 1.0f / 64516.0f, hi);
                    return fmaf(cqj, f, xb);
                };
                TCS_CNT(12);
                bool ok;
                {
                    TCS_T0();
                    ok = tcs_wait(&sh.acc_full[acc], (e_tile >> 1) & 1u, failed, spin_limit);
                    ok = __all_sync(0xffffffffu, ok);
                    TCS_ACC(0);
                }
                TCS_T0();
                if (!ok) {
                    sh.failed = 1;
                } else {
                    tc_fence_after_sync();
                    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * TCS_ACC_COLS + q_first;
                    if (any_query) {
                        tmem_load_16(taddr, a1);
                        tmem_load_16(taddr + TCS_QT, a2);
                        tmem_load_16(taddr + 2 * TCS_QT, a3);
                        tmem_load_wait();
                    }
                    // the accumulator is in registers (or not needed): hand it back
                    tc_fence_before_sync();
                    mbar_arrive(&sh.acc_free[acc]);
                    if (any_query && valid) {
                        float worst = INFINITY;   // min over the queries of (distance - bound): <= 0 means a candidate
#pragma unroll
                        for (int j4 = 0; j4 < 16; j4 += 4) {
                            const float4 cq4 = *reinterpret_cast<const float4*>(&sh.cq[q_first + j4]);
                            const float4 th4 = *reinterpret_cast<const float4*>(&ts.thrq[q_first + j4]);
                            worst = fminf(worst, partial_of(j4, cq4.x) - th4.x);
                            worst = fminf(worst, partial_of(j4 + 1, cq4.y) - th4.y);
                            worst = fminf(worst, partial_of(j4 + 2, cq4.z) - th4.z);
                            worst = fminf(worst, partial_of(j4 + 3, cq4.w) - th4.w);
                        }
                        // rare once the bounds have settled
                        if (worst <= 0.f && !(p.filter_pos_inner != nullptr && scan_row_filtered(p, pos))) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                if (partial_of(j, sh.cq[q_first + j]) <= ts.thrq[q_first + j]) {   // unused slots: bound -inf
                                    pend |= 1u << j;
                                }
                            }
                        }
                    }
                }
                TCS_ACC(1);
                const long long _t1 = clock64();
                (void)_t1;
                // Offer rounds.  The threads of a warp that hold a candidate for the same query take their slots
                // in its buffer with one addition to its counter.  The buffers are small (k + 32 keys, rounded
                // up): when one is full its query is compacted -- sorted, cut to k, bound tightened -- and the
                // candidates that did not get in try again against the new bound.  One barrier per tile when
                // nothing overflows.
                for (int round = 0; round < TCS_MAX_ROUNDS; ++round) {
                    bool overflow = false;
#ifdef VB200_TCS_PROFILE
                    const long long _o0 = clock64();
#endif
                    if (pend != 0) {
                        TCS_CNT(19);
                        // query slots for which some thread of the warp that is here holds a candidate
                        const unsigned slots = __reduce_or_sync(__activemask(), pend);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (((slots >> j) & 1u) == 0) {
                                continue;
                            }
                            const int qi = static_cast<int>(q_first) + j;
                            bool want = ((pend >> j) & 1u) != 0;
                            float part = 0.f;
                            if (want) {
                                part = partial_of(j, sh.cq[qi]);
                                if (!(part <= ts.thrq[qi])) {   // the bound moved past it in a compaction
                                    want = false;
                                    pend &= ~(1u << j);
                                }
                            }
                            const unsigned here = __activemask();
                            const unsigned offering = __ballot_sync(here, want);
                            if (offering != 0) {
                                const int leader = __ffs(offering) - 1;
                                uint32_t base = 0;
                                if (static_cast<int>(lane) == leader) {
                                    base = atomicAdd(&ts.cnt[qi], static_cast<uint32_t>(__popc(offering)));
                                }
                                base = __shfl_sync(here, base, leader);
                                if (want) {
                                    const uint32_t s = base + __popc(offering & ((1u << lane) - 1u));
                                    if (s < ts.cap) {
                                        ts.keys[static_cast<uint32_t>(qi) * ts.cap + s] = make_key(part + ts.qa[qi], pos);
                                        pend &= ~(1u << j);
                                    } else {
                                        overflow = true;
                                    }
                                }
                            }
                        }
                    }
#ifdef VB200_TCS_PROFILE
                    const long long _o1 = clock64();
                    prof_acc[16] += static_cast<unsigned long long>(_o1 - _o0);
                    const bool _any = tcs_epilogue_barrier_any(overflow);
                    const long long _o2 = clock64();
                    prof_acc[17] += static_cast<unsigned long long>(_o2 - _o1);
                    if (!_any) {
                        break;
                    }
#else
                    if (!tcs_epilogue_barrier_any(overflow)) {
                        break;
                    }
#endif
                    TCS_CNT(14);
                    for (int qi = static_cast<int>(warp); qi < nqt; qi += TCS_EPI_WARPS) {
                        if (ts.cnt[qi] >= ts.cap) {
                            compact_query(qi);
                        }
                    }
                    tcs_epilogue_barrier();
#ifdef VB200_TCS_PROFILE
                    prof_acc[18] += static_cast<unsigned long long>(clock64() - _o2);
#endif
                }
                if (pend != 0) {
                    sh.failed = 1;   // cannot happen: every round stores at least cap - k candidates of a full query
                }
#ifdef VB200_TCS_PROFILE
                prof_acc[2] += static_cast<unsigned long long>(clock64() - _t1);
#endif
            }
            tcs_epilogue_barrier();   // a failed wait of any warp is visible to all of them
            {
                TCS_T0();
                if (sh.failed == 0) {
                    // every query's (at most k) best to its slot, unordered; its bound to the global table
                    for (int qi = static_cast<int>(warp); qi < nqt; qi += TCS_EPI_WARPS) {
                        if (ts.cnt[qi] > ts.k) {
                            compact_query(qi);
                        }
                        const uint32_t c = ts.cnt[qi];
                        const uint64_t* kq = ts.keys + static_cast<uint32_t>(qi) * ts.cap;
                        uint64_t* dst = p.part + static_cast<uint64_t>(ts.slot[qi]) * ts.k;
                        uint32_t worst = 0;
                        for (uint32_t i = lane; i < ts.k; i += 32) {
                            const uint64_t key = i < c ? kq[i] : KEY_INF;
                            dst[i] = key;
                            if (i < c) {
                                worst = max(worst, static_cast<uint32_t>(key >> 32));
                            }
                        }
                        if (c >= ts.k) {
                            worst = __reduce_max_sync(0xffffffffu, worst);
                            if (lane == 0) {
                                atomicMin(p.thr_g + ts.qidx[qi], worst);
                            }
                        }
                        if (lane == 0 && p.slot_written != nullptr) {
                            p.slot_written[ts.slot[qi]] = 1;
                        }
                    }
                } else if (tid == 0) {
                    atomicOr(tp.error_flag, 1);
                }
                TCS_ACC(5);
            }
        }
    }

    if (warp == TCS_EPI_WARPS + 1 && lane == 0 && tp.count_scanned != 0 && p.scanned != nullptr && scanned_local != 0) {
        atomicAdd(p.scanned, scanned_local);
    }
#ifdef VB200_TCS_PROFILE
    if (tp.prof != nullptr && lane == 0 && (warp == 0 || warp >= TCS_EPI_WARPS)) {
        prof_acc[15] = static_cast<unsigned long long>(clock64() - prof_begin);
        unsigned long long* dst = tp.prof + static_cast<size_t>(blockIdx.x) * 24;
        const int lo = warp == 0 ? 0 : (warp == TCS_EPI_WARPS ? 6 : 9), hi = warp == 0 ? 6 : (warp == TCS_EPI_WARPS ? 9 : 12);
        for (int i = lo; i < hi; ++i) {
            dst[i] = prof_acc[i];
        }
        if (warp == 0) {
            dst[12] = prof_acc[12];
            dst[13] = prof_acc[13];
            dst[14] = prof_acc[14];
            dst[15] = prof_acc[15];
            for (int i = 16; i < 24; ++i) {
                dst[i] = prof_acc[i];
            }
        }
    }
#endif
    tc_fence_before_sync();
    __syncthreads();
    if (sh.failed != 0) {
        tc_drain_pause();   // a wait gave up: let the copies and MMAs still in flight land before the CTA lets go
        __syncthreads();
    }
    if (warp == TCS_EPI_WARPS) {
        tmem_dealloc(tmem_base, 2 * TCS_ACC_COLS);
    }
}

// Shared memory of a launch: code stages, the B operand, the selection state.
inline size_t
tcs_smem_bytes(uint32_t kchunks, uint32_t cap, uint32_t stages) {
    const size_t row_bytes = static_cast<size_t>(kchunks) * 16;
    return stages * TCS_ROWS * row_bytes + 2 * TCS_N * row_bytes + tile_smem_bytes<TCS_QT>(cap, 0);
}

// Candidate buffer of a query in this kernel: k survivors plus room for a warp's worth of offers.
inline uint32_t
tcs_buffer_cap(uint32_t k) {
    const uint32_t cap = next_pow2(k + 32);
    return cap < 64 ? 64 : cap;
}

}  // namespace vb200
