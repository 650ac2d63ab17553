// tcgen05 / TMEM candidate-generation GEMM: operand pre-tiling, the kernel and its launcher.
#include "tc_gemm.cuh"

#include <cmath>
#include <cstdlib>

#include <cuda_bf16.h>

namespace vb200 {

constexpr uint32_t TC_MAX_STAGES = 6;   // operand stages in flight; the launch picks how many fit

static std::atomic<uint32_t> g_spin_limit{TC_SPIN_LIMIT};

uint32_t
tc_spin_limit() {
    return g_spin_limit.load(std::memory_order_relaxed);
}

void
tc_set_spin_limit(uint32_t polls) {
    g_spin_limit.store(polls, std::memory_order_relaxed);
}

__device__ __forceinline__ float
widen_in(float v) {
    return v;
}
__device__ __forceinline__ float
widen_in(uint16_t v) {  // bf16 bit pattern
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

// ---------------------------------------------------------------------------------------------
// pre-tiling: element (r, e) of a [rows x dim] matrix goes to
//   tile r/128, chunk e/64, core matrix ((r%128)/8, (e%64)/8), row r%8, element e%8
// so a [128 x 64] chunk is 16 KiB contiguous: 8x8-element cores of 128 B, the 8 cores of an 8-row
// group back to back (1 KiB per group).  Out-of-range rows / dimensions are zero.
// ---------------------------------------------------------------------------------------------
template <typename T, bool SPLIT>
__global__ void
tc_pretile_kernel(const T* __restrict__ src, uint64_t rows, uint32_t dim, uint32_t chunks,
                  uint16_t* __restrict__ hi, uint16_t* __restrict__ lo, uint64_t total_units) {
    uint64_t u = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 8-element core row
    if (u >= total_units) {
        return;
    }
    uint32_t rr8 = static_cast<uint32_t>(u & 7);
    uint32_t core_k = static_cast<uint32_t>((u >> 3) & 7);
    uint32_t core_r = static_cast<uint32_t>((u >> 6) & 15);
    uint64_t chunk_id = u >> 10;  // tile * chunks + chunk
    uint32_t kc = static_cast<uint32_t>(chunk_id % chunks);
    uint64_t tile = chunk_id / chunks;
    uint64_t r = tile * 128 + core_r * 8 + rr8;
    uint32_t e0 = kc * TC_KC + core_k * 8;
    uint16_t h[8], l[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float x = 0.f;
        if (r < rows && e0 + i < dim) {
            x = widen_in(src[r * dim + e0 + i]);
        }
        __nv_bfloat16 bh = __float2bfloat16_rn(x);
        h[i] = __bfloat16_as_ushort(bh);
        if (SPLIT) {
            float rest = x - __bfloat162float(bh);
            l[i] = __bfloat16_as_ushort(__float2bfloat16_rn(rest));
        }
    }
    uint4 vh = make_uint4(h[0] | (uint32_t(h[1]) << 16), h[2] | (uint32_t(h[3]) << 16),
                          h[4] | (uint32_t(h[5]) << 16), h[6] | (uint32_t(h[7]) << 16));
    reinterpret_cast<uint4*>(hi)[u] = vh;
    if (SPLIT) {
        uint4 vl = make_uint4(l[0] | (uint32_t(l[1]) << 16), l[2] | (uint32_t(l[3]) << 16),
                              l[4] | (uint32_t(l[5]) << 16), l[6] | (uint32_t(l[7]) << 16));
        reinterpret_cast<uint4*>(lo)[u] = vl;
    }
}

size_t
tc_tiled_elems(uint64_t rows, uint32_t dim) {
    uint64_t tiles = (rows + 127) / 128;
    uint64_t chunks = (dim + TC_KC - 1) / TC_KC;
    return static_cast<size_t>(tiles * chunks * TC_CHUNK_ELEMS);
}

template <typename T>
static int
pretile_launch(const T* src, uint64_t rows, uint32_t dim, uint16_t* hi, uint16_t* lo) {
    if (rows == 0) {
        return 0;
    }
    uint32_t chunks = (dim + TC_KC - 1) / TC_KC;
    uint64_t units = tc_tiled_elems(rows, dim) / 8;
    uint64_t blocks = (units + 255) / 256;
    VB_CHECK_ARG(blocks <= 0x7fffffffu, "pretile: matrix too large");
    if (lo != nullptr) {
        auto kernel = tc_pretile_kernel<T, true>;
        VB_LAUNCH(kernel, static_cast<uint32_t>(blocks), 256, 0, src, rows, dim, chunks, hi, lo, units);
    } else {
        auto kernel = tc_pretile_kernel<T, false>;
        VB_LAUNCH(kernel, static_cast<uint32_t>(blocks), 256, 0, src, rows, dim, chunks, hi, lo, units);
    }
    return 0;
}

int
tc_pretile_f32(const float* src_dev, uint64_t rows, uint32_t dim, uint16_t* hi_dev, uint16_t* lo_dev) {
    return pretile_launch<float>(src_dev, rows, dim, hi_dev, lo_dev);
}

int
tc_pretile_bf16(const uint16_t* src_dev, uint64_t rows, uint32_t dim, uint16_t* hi_dev) {
    return pretile_launch<uint16_t>(src_dev, rows, dim, hi_dev, nullptr);
}

// ---------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------
struct TcShared {
    uint64_t full[TC_MAX_STAGES];    // chunk copies landed
    uint64_t freed[TC_MAX_STAGES];   // MMAs that read the stage retired
    uint64_t a_full;             // resident-A mode: the item's A tile has landed
    uint64_t a_free;             // resident-A mode: the last MMA that reads it has retired
    uint64_t acc_full[2];        // accumulator holds a finished tile
    uint64_t acc_free[2];        // accumulator drained by the 128 epilogue threads
    uint32_t tmem_base;
    uint32_t failed;
    alignas(16) float bias[TC_EPI_WARPS][32];   // each epilogue warp's 32 bias values of its current tile
};

// Warp-cooperative: sort row `owner`'s buffer, keep its m best, tighten its threshold.  The row's
// keys are staged through this warp's shared-memory sort area (sorting in global memory is
// latency-bound: one round trip per compare-exchange stage).
__device__ __forceinline__ void
tc_compact_row(uint64_t* my_buf, uint32_t& my_cnt, float& my_thr, uint32_t owner, uint32_t lane, uint32_t m,
               uint64_t* sort_area) {
    uint64_t addr = reinterpret_cast<uint64_t>(my_buf);
    uint32_t lo = __shfl_sync(0xffffffffu, static_cast<uint32_t>(addr), owner);
    uint32_t hi = __shfl_sync(0xffffffffu, static_cast<uint32_t>(addr >> 32), owner);
    uint64_t* p = reinterpret_cast<uint64_t*>((static_cast<uint64_t>(hi) << 32) | lo);
    uint32_t c = __shfl_sync(0xffffffffu, my_cnt, owner);
    uint32_t n2 = next_pow2(c < 2 ? 2 : c);
    __syncwarp();
    for (uint32_t i = lane; i < n2; i += 32) {
        sort_area[i] = i < c ? p[i] : KEY_INF;
    }
    warp_bitonic_sort(sort_area, n2, lane);
    uint32_t keep = c < m ? c : m;
    for (uint32_t i = lane; i < keep; i += 32) {
        p[i] = sort_area[i];
    }
    if (lane == owner) {
        my_cnt = keep;
        if (c >= m) {
            my_thr = ordered_to_float(static_cast<uint32_t>(sort_area[m - 1] >> 32));
        }
    }
    __syncwarp();
}

// MODE 0: at most four candidates per row, kept sorted in registers by the row's thread (the
// k-means case); MODE 1: candidates go to per-row buffers compacted as above; MODE 2: no
// selection, the scores themselves are stored; MODE 3: every column scoring below the row's fixed
// threshold (row_bound) is appended, unsorted, to the row's output list of `cap` entries -- no
// sorting at all, the caller sizes the lists from the threshold's expected pass rate and an
// overflowing list sets bit 1 of the error flag.
template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_candidates_kernel(const TcParams p) {
    constexpr bool SMALL_M = MODE == 0;
    constexpr bool STORE = MODE == 2;
    constexpr bool THRESH = MODE == 3;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ TcShared sh;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_ops = p.n_terms == 3 ? 4u : 2u;
    const uint32_t n_terms_op = p.n_terms == 3 ? 2u : 1u;                       // bf16 terms per operand
    // resident-A mode: [A tile: chunks x terms][ring of B stages]; otherwise a ring of [A terms][B terms]
    const uint32_t a_region_bytes = p.a_resident ? p.a.chunks * n_terms_op * TC_CHUNK_BYTES : 0u;
    // wide mode: a stage holds two consecutive B tiles, term by term ([hi t][hi t+1][lo t][lo t+1]), so
    // that one 128 x 256 x 16 MMA reads both; the accumulators are 256 columns each.
    const uint32_t step = p.wide ? 2u : 1u;
    const uint32_t acc_cols = step * TC_BN;
    const uint32_t stage_bytes = ((p.a_resident ? 0u : n_terms_op) + n_terms_op * step) * TC_CHUNK_BYTES;
    (void)n_ops;
    const uint32_t chunks = p.a.chunks;
    const uint64_t m_tiles = (p.a.rows + TC_BM - 1) / TC_BM;
    const uint64_t n_tiles = (p.b.rows + TC_BN - 1) / TC_BN;
    const uint64_t n_items = m_tiles * p.n_split;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&sh.full[s], p.a_resident ? 1 : 2);   // one arrival (with its byte count) per copy thread filling it
            mbar_init(&sh.freed[s], 1);
        }
        mbar_init(&sh.a_full, 1);
        mbar_init(&sh.a_free, 1);
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(&sh.acc_full[a], 1);
            mbar_init(&sh.acc_free[a], TC_EPI_THREADS);
        }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_EPI_WARPS) {
        tmem_alloc(&sh.tmem_base, 2 * acc_cols);  // two fp32 accumulators of 128 (256 when wide) columns
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = sh.tmem_base;

    const uint32_t n_items32 = static_cast<uint32_t>(n_items);
    const uint32_t n_tiles32 = static_cast<uint32_t>(n_tiles);
    // A work item is a row tile of A against one of n_split shares of B's tiles.  Contiguous shares: share s
    // holds tiles s * tiles_per_split ..., and the items of a row tile are neighbours in the queue.
    // Interleaved shares (p.interleaved): share s holds tiles s, s + n_split, s + 2 n_split, ..., and the
    // queue walks the row tiles of one share before the next share, so the CTAs running at any moment
    // sweep B front to back together and a B tile fetched from DRAM by one of them is an L2 hit for the
    // others -- what a base far larger than L2 needs when there are many row tiles.
    const uint32_t m_tiles32 = static_cast<uint32_t>(m_tiles);
    auto open_item = [&](uint32_t item, uint32_t& mtile, uint32_t& split, uint32_t& tiles) {
        if (p.interleaved) {
            split = item / m_tiles32;
            mtile = item - split * m_tiles32;
            tiles = n_tiles32 > split ? (n_tiles32 - split + p.n_split - 1) / p.n_split : 0u;
        } else {
            mtile = item / p.n_split;
            split = item - mtile * p.n_split;
            const uint32_t t0 = split * p.tiles_per_split;
            uint32_t t1 = t0 + p.tiles_per_split;
            if (t1 > n_tiles32) {
                t1 = n_tiles32;
            }
            tiles = t1 > t0 ? t1 - t0 : 0;
        }
    };
    // B tile number u of share `split`.  With p.window > 0 (a power of two) the share is walked in windows
    // of that many tiles and every row tile starts each window at its own offset, wrapping round: the CTAs
    // that sweep a share together then ask L2 for different tiles at any moment instead of all for the same
    // lines, while a window still passes through L2 once.
    auto tile_at = [&](uint32_t split, uint32_t mtile, uint32_t tiles, uint32_t u) -> uint32_t {
        if (p.window != 0) {
            const uint32_t w0 = u & ~(p.window - 1u);
            const uint32_t len = tiles - w0 < p.window ? tiles - w0 : p.window;
            uint32_t r = (u - w0) + ((mtile * 29u) & (p.window - 1u));
            r = len == p.window ? (r & (p.window - 1u)) : r % len;
            u = w0 + r;
        }
        return p.interleaved ? split + u * p.n_split : split * p.tiles_per_split + u;
    };
    if (warp == TC_EPI_WARPS) {
        // ---------------- MMA issue (one thread) ----------------
        // Written for latency: 32-bit counters that wrap by compare instead of divide, descriptors
        // prepared once per stage.
        if (lane == 0) {
            const uint32_t idesc_one = umma_idesc_bf16(TC_BM, TC_BN), idesc_two = umma_idesc_bf16(TC_BM, 2 * TC_BN);
            // Descriptor of stage 0 / operand 0; the others differ only in the start-address field,
            // which counts 16-byte units, so they are this value plus small constants kept in registers.
            const uint64_t desc0 = umma_desc(smem_u32(smem), 128, 1024);
            const uint64_t stage_units = stage_bytes >> 4;
            const uint64_t op_units = TC_CHUNK_BYTES >> 4;
            const uint64_t ring0 = desc0 + (a_region_bytes >> 4);
            const bool a_res = p.a_resident != 0;
            uint64_t stage_desc = ring0;
            bool ok = true;
            uint32_t m_stage = 0, m_phase = 0, acc = 0, acc_phase = 0, tiles_started = 0, a_phase = 0;
            for (uint32_t item = blockIdx.x; item < n_items32 && ok; item += gridDim.x) {
                uint32_t mtile, split, tiles;
                open_item(item, mtile, split, tiles);
                if (a_res && tiles > 0) {
                    ok = mbar_wait(&sh.a_full, a_phase, p.spin_limit);
                    a_phase ^= 1u;
                    if (!ok) {
                        break;
                    }
                }
                for (uint32_t t = 0; t < tiles && ok; t += step) {
                    const uint32_t idesc = (tiles - t >= 2 && step == 2) ? idesc_two : idesc_one;
                    if (tiles_started >= 2) {
                        // the epilogue must have drained this accumulator's previous tile
                        ok = mbar_wait(&sh.acc_free[acc], acc_phase ^ 1u, p.spin_limit);
                        if (!ok) {
                            break;
                        }
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * acc_cols;
                    for (uint32_t c = 0; c < chunks && ok; ++c) {
                        ok = mbar_wait(&sh.full[m_stage], m_phase, p.spin_limit);
                        if (!ok) {
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll
                        for (uint32_t kk = 0; kk < TC_KC / 16; ++kk) {
#ifdef VB200_TC_DIAG
                            if ((p.diag & 2u) != 0) {
                                continue;
                            }
#endif
                            // a k-step of 16 elements = two 8-element cores: 256 B = 16 descriptor units
                            const uint64_t koff = kk * 16;
                            const uint32_t accumulate = (c == 0 && kk == 0) ? 0u : 1u;
                            if (p.n_terms == 3) {
                                const uint64_t a_hi = (a_res ? desc0 + c * 2 * op_units : stage_desc) + koff;
                                const uint64_t b_hi = (a_res ? stage_desc : stage_desc + 2 * op_units) + koff;
                                const uint64_t a_lo = a_hi + op_units, b_lo = b_hi + step * op_units;
                                umma_bf16(d_tmem, a_hi, b_hi, idesc, accumulate);
                                umma_bf16(d_tmem, a_hi, b_lo, idesc, 1u);
                                umma_bf16(d_tmem, a_lo, b_hi, idesc, 1u);
                            } else {
                                const uint64_t a = (a_res ? desc0 + c * op_units : stage_desc) + koff;
                                const uint64_t b = (a_res ? stage_desc : stage_desc + op_units) + koff;
                                umma_bf16(d_tmem, a, b, idesc, accumulate);
                            }
                        }
                        umma_commit(&sh.freed[m_stage]);
                        if (c + 1 == chunks) {
                            umma_commit(&sh.acc_full[acc]);
                            if (a_res && t + step >= tiles) {
                                umma_commit(&sh.a_free);   // the item's A tile may be overwritten
                            }
                        }
                        stage_desc += stage_units;
                        if (++m_stage == p.stages) {
                            m_stage = 0;
                            m_phase ^= 1u;
                            stage_desc = ring0;
                        }
                    }
                    ++tiles_started;
                    if (++acc == 2) {
                        acc = 0;
                        acc_phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                sh.failed = 1;
                atomicOr(p.error_flag, 1);
            }
        }
        __syncwarp();
    } else if (warp > TC_EPI_WARPS) {
        // ---------------- operand copies: one thread for A, one for B ----------------
        // The copy engine of an SM moves a 16 KiB bulk copy at well under the rate the MMAs eat
        // operands when a single thread issues them one after the other; two issuers overlap.
        if (lane == 0) {
            const bool is_a = warp == TC_EPI_WARPS + 1;
            const TcOperand& op = is_a ? p.a : p.b;
            const uint32_t terms = n_terms_op;
            const bool a_res = p.a_resident != 0;
            bool ok = true;
            if (is_a && a_res) {
                // the whole A tile of an item at once, into the resident region
                uint32_t a_phase = 0, n_loaded = 0;
                for (uint32_t item = blockIdx.x; item < n_items32 && ok; item += gridDim.x) {
                    uint32_t mtile, split, tiles;
                    open_item(item, mtile, split, tiles);
                    if (tiles == 0) {
                        continue;
                    }
                    if (n_loaded > 0) {
                        ok = mbar_wait(&sh.a_free, a_phase, p.spin_limit);   // previous item's MMAs are done with it
                        a_phase ^= 1u;
                        if (!ok) {
                            break;
                        }
                    }
                    mbar_expect_tx(&sh.a_full, a_region_bytes);
                    for (uint32_t c = 0; c < chunks; ++c) {
                        const size_t off = (static_cast<size_t>(mtile) * chunks + c) * TC_CHUNK_ELEMS;
                        unsigned char* dst = smem + c * terms * TC_CHUNK_BYTES;
                        bulk_copy_g2s(dst, op.hi + off, TC_CHUNK_BYTES, &sh.a_full);
                        if (terms == 2) {
                            bulk_copy_g2s(dst + TC_CHUNK_BYTES, op.lo + off, TC_CHUNK_BYTES, &sh.a_full);
                        }
                    }
                    ++n_loaded;
                }
            } else {
                // ring of stages; in resident-A mode the B thread fills whole stages
                const uint32_t op_off = (is_a || a_res) ? 0u : terms * TC_CHUNK_BYTES;   // A terms first, then B terms
                uint32_t stage = 0, phase = 0, count = 0;
                for (uint32_t item = blockIdx.x; item < n_items32 && ok; item += gridDim.x) {
                    uint32_t mtile, split, tiles;
                    open_item(item, mtile, split, tiles);
                    for (uint32_t t = 0; t < tiles && ok; t += step) {
                        const uint32_t here = is_a ? 1u : (tiles - t >= step ? step : 1u);   // B tiles of this step
                        for (uint32_t c = 0; c < chunks; ++c) {
                            if (count >= p.stages) {
                                // the stage's previous use must have been consumed by the tensor core
                                ok = mbar_wait(&sh.freed[stage], phase ^ 1u, p.spin_limit);
                                if (!ok) {
                                    break;
                                }
                            }
                            unsigned char* dst = smem + a_region_bytes + stage * stage_bytes + op_off;
                            mbar_expect_tx(&sh.full[stage], terms * here * TC_CHUNK_BYTES);
                            for (uint32_t slot = 0; slot < here; ++slot) {
                                const size_t row_tile = is_a ? mtile : tile_at(split, mtile, tiles, t + slot);
                                const size_t off = (row_tile * chunks + c) * TC_CHUNK_ELEMS;
                                const uint32_t slots = is_a ? 1u : step;   // slots per term in the stage
                                bulk_copy_g2s(dst + slot * TC_CHUNK_BYTES, op.hi + off, TC_CHUNK_BYTES, &sh.full[stage]);
                                if (terms == 2) {
                                    bulk_copy_g2s(dst + (slots + slot) * TC_CHUNK_BYTES, op.lo + off, TC_CHUNK_BYTES,
                                                  &sh.full[stage]);
                                }
                            }
                            ++count;
                            if (++stage == p.stages) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                }
            }
            if (!ok) {
                atomicOr(p.error_flag, 1);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: drain the accumulator, keep the m best per row ----------------
        const uint32_t quarter = warp & 3u;          // TMEM lanes 32 * quarter .. + 31
        const uint32_t cgroup = warp >> 2;           // columns 32 * cgroup .. + 31 of every tile
        const uint32_t row = quarter * 32 + lane;
        uint64_t* buf = p.scratch + ((static_cast<uint64_t>(blockIdx.x) * TC_BM + row) * TC_COL_GROUPS + cgroup) * p.cap;
        uint64_t* sort_area = reinterpret_cast<uint64_t*>(smem + a_region_bytes + static_cast<size_t>(p.stages) * stage_bytes) +
                              static_cast<size_t>(warp) * p.cap;
        uint64_t gtile = 0;
        bool ok = true;
        for (uint64_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            uint32_t m_tile32, split32, tiles32;
            open_item(static_cast<uint32_t>(item), m_tile32, split32, tiles32);
            const uint64_t m_tile = m_tile32, split = split32;
            const uint64_t t0 = 0, t1 = tiles32;   // the item's B tiles by their number within its share
            const uint64_t grow = m_tile * TC_BM + row;
            const bool valid_row = grow < p.a.rows;
            uint32_t cnt = 0;
            float thr = INFINITY;
            uint64_t* list = nullptr;   // THRESH: this thread's output list of the item
            if (MODE == 1 && p.row_bound != nullptr && valid_row) {
                thr = __ldg(p.row_bound + grow);   // the caller's bound: columns scoring at or above it are of no use
            }
            if (THRESH) {
                thr = valid_row ? __ldg(p.row_bound + grow) : -INFINITY;
                list = p.out + ((grow * p.n_split + split) * TC_COL_GROUPS + cgroup) * p.cap;
            }
            // bias of the warp's 32 columns: fetched one tile ahead into a register (lane = column),
            // handed to the other lanes through the warp's own shared-memory slot
            const bool has_bias = p.bias != nullptr;
            // first global column of this warp's block `half` in the tile step that starts at B tile t
            auto block_col = [&](uint64_t t, uint32_t half) -> uint64_t {
                return p.wide ? static_cast<uint64_t>(tile_at(split32, m_tile32, tiles32, static_cast<uint32_t>(t) + (cgroup >> 1))) * TC_BN +
                                    (cgroup & 1u) * 64 + half * 32
                              : static_cast<uint64_t>(tile_at(split32, m_tile32, tiles32, static_cast<uint32_t>(t))) * TC_BN + cgroup * 32;
            };
            float next_bias = 0.f;
            if (has_bias) {
                const uint64_t nn = block_col(t0, 0) + lane;
                next_bias = (t0 < t1 && nn < p.b.rows) ? __ldg(p.bias + nn) : 0.f;
            }
            // SMALL_M: the four best scores of the row, ascending, with their columns
            float bs0 = INFINITY, bs1 = INFINITY, bs2 = INFINITY, bs3 = INFINITY;
            const float margin = (SMALL_M && p.a_sq != nullptr && p.margin_scale != nullptr && valid_row)
                                     ? __ldg(p.margin_scale) * sqrtf(__ldg(p.a_sq + grow))
                                     : -1.f;
            float bound = (margin >= 0.f && p.row_bound != nullptr) ? __ldg(p.row_bound + grow) + margin : INFINITY;
            uint32_t bc0 = 0xFFFFFFFFu, bc1 = 0xFFFFFFFFu, bc2 = 0xFFFFFFFFu, bc3 = 0xFFFFFFFFu;
            for (uint64_t t = t0; t < t1 && ok; t += step, ++gtile) {
                const uint32_t acc = static_cast<uint32_t>(gtile & 1);
                ok = mbar_wait_relaxed(&sh.acc_full[acc], static_cast<uint32_t>((gtile >> 1) & 1), p.spin_limit);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    break;
                }
                tc_fence_after_sync();
                const uint32_t here = (t1 - t >= step) ? step : 1u;              // B tiles in this step
                const bool tile_present = p.wide ? (cgroup >> 1) < here : true;  // this warp's B tile exists
                for (uint32_t half = 0; half < step; ++half) {
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + acc * acc_cols +
                                       (p.wide ? cgroup * 64 + half * 32 : cgroup * 32);
                const uint64_t n0 = block_col(t, half);
                const bool whole_tile = valid_row && tile_present && n0 + 32 <= p.b.rows;
                if (has_bias) {
                    __syncwarp();
                    sh.bias[warp][lane] = next_bias;
                    const bool more = half + 1 < step || t + step < t1;
                    const uint64_t nn = (half + 1 < step ? n0 + 32 : block_col(t + step, 0)) + lane;
                    next_bias = (more && nn < p.b.rows) ? __ldg(p.bias + nn) : 0.f;
                    __syncwarp();
                }
                uint32_t r[32];
                tmem_load_32(taddr, r);
                if (half + 1 == step) {
                    // the accumulator is in registers now: hand it back before doing the selection
                    tc_fence_before_sync();
                    mbar_arrive(&sh.acc_free[acc]);
                }

                {
                    if (MODE == 1) {
                        uint32_t full = __ballot_sync(0xffffffffu, cnt + 32 > p.cap);
                        while (full != 0) {
                            uint32_t owner = __ffs(full) - 1;
                            tc_compact_row(buf, cnt, thr, owner, lane, p.m, sort_area);
                            full &= full - 1;
                        }
                    }
#ifdef VB200_TC_DIAG
                    if ((p.diag & 1u) != 0) {
                        continue;
                    }
#endif
                    const uint32_t c0 = static_cast<uint32_t>(n0);
                    // Scores of the block and their minimum first (two instructions per element);
                    // the selection code below runs only when the minimum beats the row's bound.
                    float sc[32];
                    if (__all_sync(0xffffffffu, whole_tile)) {
                        // the common case: every row and column of the block exists
                        if (has_bias) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                const float4 b4 = *reinterpret_cast<const float4*>(&sh.bias[warp][i]);
                                sc[i] = fmaf(p.alpha, __uint_as_float(r[i]), b4.x);
                                sc[i + 1] = fmaf(p.alpha, __uint_as_float(r[i + 1]), b4.y);
                                sc[i + 2] = fmaf(p.alpha, __uint_as_float(r[i + 2]), b4.z);
                                sc[i + 3] = fmaf(p.alpha, __uint_as_float(r[i + 3]), b4.w);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                sc[i] = p.alpha * __uint_as_float(r[i]);
                            }
                        }
                    } else {
                        const uint32_t cols_left = (tile_present && c0 < p.b.rows)
                                                       ? static_cast<uint32_t>(min(static_cast<uint64_t>(32), p.b.rows - c0))
                                                       : 0u;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const float4 b4 = has_bias ? *reinterpret_cast<const float4*>(&sh.bias[warp][i])
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
                            const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const bool in_range = valid_row && static_cast<uint32_t>(i + j) < cols_left;
                                sc[i + j] = in_range ? fmaf(p.alpha, __uint_as_float(r[i + j]), bb[j]) : INFINITY;
                            }
                        }
                    }
                    if (STORE) {
                        // 32 consecutive floats of this thread's row: eight 16-byte stores
                        if (valid_row && tile_present) {
                            float* dst = p.store + grow * p.store_ld + c0;
                            if (whole_tile) {
#pragma unroll
                                for (int i = 0; i < 32; i += 4) {
                                    *reinterpret_cast<float4*>(dst + i) = make_float4(sc[i], sc[i + 1], sc[i + 2], sc[i + 3]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i) {
                                    if (c0 + i < p.b.rows) {
                                        dst[i] = sc[i];
                                    }
                                }
                            }
                        }
                        continue;
                    }
                    // minimum as a tree: a serial chain of 32 dependent fminf would stall the warp
                    float m16[16], m4[4];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        m16[i] = fminf(sc[i], sc[i + 16]);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        m4[i] = fminf(fminf(m16[i], m16[i + 4]), fminf(m16[i + 8], m16[i + 12]));
                    }
                    const float mn = fminf(fminf(m4[0], m4[1]), fminf(m4[2], m4[3]));
                    if (SMALL_M) {
                        if (mn < bound) {
                            // rare path: visit only the elements that beat the bound
                            float tmp[32];
                            uint32_t hits = 0;
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                tmp[i] = sc[i];
                                hits |= (sc[i] < bound ? 1u : 0u) << i;
                            }
                            while (hits != 0) {
                                const uint32_t i = __ffs(hits) - 1;
                                hits &= hits - 1;
                                const float s = tmp[i];
                                if (s < bs3) {
                                    // insert into the ascending quadruple (bs0 <= bs1 <= bs2 <= bs3)
                                    const uint32_t col = c0 + i;
                                    if (s < bs2) {
                                        bs3 = bs2;
                                        bc3 = bc2;
                                        if (s < bs1) {
                                            bs2 = bs1;
                                            bc2 = bc1;
                                            if (s < bs0) {
                                                bs1 = bs0;
                                                bc1 = bc0;
                                                bs0 = s;
                                                bc0 = col;
                                            } else {
                                                bs1 = s;
                                                bc1 = col;
                                            }
                                        } else {
                                            bs2 = s;
                                            bc2 = col;
                                        }
                                    } else {
                                        bs3 = s;
                                        bc3 = col;
                                    }
                                }
                            }
                            // with a margin: only columns within it of the best can still win;
                            // without: anything better than the fourth best is kept
                            bound = fminf(bound, margin >= 0.f ? fminf(bs3, bs0 + margin) : bs3);
                        }
                    } else if (mn < thr
#ifdef VB200_TC_DIAG
                               && (p.diag & 4u) == 0
#endif
                    ) {
                        // few elements pass: test them in pairs through the first level of the tree
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (m16[i] < thr) {
                                if (THRESH) {
                                    if (sc[i] < thr) {
                                        if (cnt < p.cap) {
                                            list[cnt] = make_key(sc[i], c0 + i + p.col_base);
                                        }
                                        ++cnt;
                                    }
                                    if (sc[i + 16] < thr) {
                                        if (cnt < p.cap) {
                                            list[cnt] = make_key(sc[i + 16], c0 + i + 16 + p.col_base);
                                        }
                                        ++cnt;
                                    }
                                } else {
                                    if (sc[i] < thr) {
                                        buf[cnt++] = make_key(sc[i], c0 + i + p.col_base);
                                    }
                                    if (sc[i + 16] < thr) {
                                        buf[cnt++] = make_key(sc[i + 16], c0 + i + 16 + p.col_base);
                                    }
                                }
                            }
                        }
                    }
                }
                }   // half
            }
            if (!ok) {
                break;
            }
            if (STORE) {
                continue;
            }
            if (THRESH) {
                if (valid_row) {
                    p.out_count[(grow * p.n_split + split) * TC_COL_GROUPS + cgroup] = cnt;
                    if (cnt > p.cap) {
                        atomicOr(p.error_flag, 2);
                    }
                }
                continue;
            }
            if (SMALL_M) {
                if (valid_row && p.row_flags != nullptr && margin >= 0.f && bc3 != 0xFFFFFFFFu && bs3 <= bs0 + margin) {
                    // all four slots hold columns within the margin of the best: a fifth may have been turned away
                    if (atomicExch(p.row_flags + grow, 1u) == 0u) {
                        atomicAdd(p.error_flag + 1, 1);
                    }
                }
                if (valid_row) {
                    uint64_t* dst = p.out + ((grow * p.n_split + split) * TC_COL_GROUPS + cgroup) * p.m;
                    const float fs[4] = {bs0, bs1, bs2, bs3};
                    const uint32_t fc[4] = {bc0, bc1, bc2, bc3};
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        if (i < p.m) {
                            dst[i] = fc[i] == 0xFFFFFFFFu ? KEY_INF : make_key(fs[i], fc[i] + p.col_base);
                        }
                    }
                }
            } else {
                // final order of every row of this warp, then the m best go out
#ifdef VB200_TC_DIAG
                if ((p.diag & 8u) != 0) {
                    continue;
                }
#endif
                for (uint32_t owner = 0; owner < 32; ++owner) {
                    tc_compact_row(buf, cnt, thr, owner, lane, p.m, sort_area);
                    const uint64_t orow = m_tile * TC_BM + quarter * 32 + owner;
                    if (orow < p.a.rows) {
                        uint32_t c = __shfl_sync(0xffffffffu, cnt, owner);
                        uint64_t* dst = p.out + ((orow * p.n_split + split) * TC_COL_GROUPS + cgroup) * p.m;
                        for (uint32_t i = lane; i < p.m; i += 32) {
                            dst[i] = i < c ? sort_area[i] : KEY_INF;
                        }
                    }
                    __syncwarp();
                }
            }
        }
        if (!ok && lane == 0) {
            atomicOr(p.error_flag, 1);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) {
        sh.failed = static_cast<uint32_t>(*reinterpret_cast<volatile int*>(p.error_flag)) & 1u;
    }
    __syncthreads();
    if (sh.failed != 0) {
        tc_drain_pause();   // a wait gave up somewhere: let what is still in flight land before the CTA lets go
        __syncthreads();
    }
    if (warp == TC_EPI_WARPS) {
        tmem_dealloc(tmem_base, 2 * acc_cols);
    }
}

// Shared memory a launch may use for operand stages and sort areas (the rest of the 227 KiB holds
// the barriers, the bias slots and alignment slack).
constexpr size_t TC_SMEM_BUDGET = 232448 - 4096;
constexpr uint32_t TC_MIN_STAGES = 2;

static size_t
tc_stage_bytes(uint32_t n_terms) {
    return static_cast<size_t>(n_terms == 3 ? 4 : 2) * TC_CHUNK_BYTES;
}

// Largest per-row candidate buffer whose per-warp sort areas fit beside the fewest stages.
static uint32_t
tc_cap_max(uint32_t n_terms) {
    const size_t room = TC_SMEM_BUDGET - TC_MIN_STAGES * tc_stage_bytes(n_terms);
    uint32_t cap_max = 64;
    while (static_cast<size_t>(cap_max) * 2 * TC_EPI_WARPS * sizeof(uint64_t) <= room && cap_max < 1024) {
        cap_max *= 2;
    }
    return cap_max;
}

// Shared-memory plan of a launch: whether the A tile of an item stays resident (it does when it
// is at most 64 KiB, i.e. up to 128 dimensions of split fp32 or 256 of bf16: every B tile of the
// item then costs only its own bytes), and as many ring stages as fit beside it and the sort
// areas.  VB200_TC_STAGES / VB200_TC_A_RESIDENT=0 override the choices (for experiments).
static void
tc_plan(TcParams& p, size_t sort_bytes, size_t* smem_bytes) {
    const uint32_t terms = p.n_terms == 3 ? 2u : 1u;
    const size_t chunk = TC_CHUNK_BYTES;
    const size_t a_region = static_cast<size_t>(p.a.chunks) * terms * chunk;
    const char* env_res = std::getenv("VB200_TC_A_RESIDENT");
    const char* env_wide = std::getenv("VB200_TC_WIDE");
    bool resident = a_region <= 65536 && !(env_res != nullptr && env_res[0] == '0');
    auto stage_bytes = [&](bool res, bool wide) { return ((res ? 0 : terms) + terms * (wide ? 2 : 1)) * chunk; };
    auto fits = [&](bool res, bool wide, uint32_t stages) {
        return sort_bytes + (res ? a_region : 0) + stages * stage_bytes(res, wide) <= TC_SMEM_BUDGET;
    };
    if (resident && !fits(true, false, TC_MIN_STAGES)) {
        resident = false;
    }
    // Two B tiles per MMA whenever a stage stays affordable: bf16 inputs, or a resident A tile.
    bool wide = (terms == 1 || resident) && !(env_wide != nullptr && env_wide[0] == '0');
    if (wide && !fits(resident, true, TC_MIN_STAGES)) {
        wide = false;
    }
    const size_t fixed = sort_bytes + (resident ? a_region : 0);
    uint32_t stages = static_cast<uint32_t>((TC_SMEM_BUDGET - fixed) / stage_bytes(resident, wide));
    if (stages > TC_MAX_STAGES) {
        stages = TC_MAX_STAGES;
    }
    const char* env = std::getenv("VB200_TC_STAGES");
    if (env != nullptr && env[0] != 0) {
        const uint32_t want = static_cast<uint32_t>(std::atoi(env));
        if (want >= 2 && want <= stages) {
            stages = want;
        }
    }
    p.stages = stages;
    p.a_resident = resident ? 1u : 0u;
    p.wide = wide ? 1u : 0u;
    *smem_bytes = fixed + stages * stage_bytes(resident, wide) + 1024;
}

uint32_t
tc_max_candidates(uint32_t n_terms) {
    return tc_cap_max(n_terms) - 32;
}

int
tc_candidates(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
              const float* bias_dev, uint32_t m, uint32_t col_base, DevBuf<uint64_t>& out,
              uint32_t* n_split_out, const float* a_sq_dev, const float* margin_scale_dev,
              const float* row_bound_dev, uint32_t* row_flags_dev, uint32_t* n_flagged_out) {
    VB_CHECK_ARG(a.rows > 0 && b.rows > 0, "tc_candidates: empty operand");
    VB_CHECK_ARG(a.chunks == b.chunks && a.chunks > 0, "tc_candidates: operand depths differ");
    VB_CHECK_ARG(n_terms == 1 || n_terms == 3, "tc_candidates: 1 or 3 terms");
    VB_CHECK_ARG(m >= 1 && m <= 480, "tc_candidates: m out of range");
    const uint64_t m_tiles = (a.rows + TC_BM - 1) / TC_BM;
    const uint64_t n_tiles = (b.rows + TC_BN - 1) / TC_BN;
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    uint64_t n_split = (2ull * sms + m_tiles - 1) / m_tiles;
    if (n_split > n_tiles) {
        n_split = n_tiles;
    }
    if (n_split < 1) {
        n_split = 1;
    }
    uint64_t tiles_per_split = (n_tiles + n_split - 1) / n_split;
    n_split = (n_tiles + tiles_per_split - 1) / tiles_per_split;
    // A B operand far larger than L2 under many row tiles (BruteForce over millions of rows): interleaved
    // shares, so that the CTAs running together sweep B front to back together and DRAM delivers every B
    // tile about once instead of once per row tile.  The number of shares makes the item count close to a
    // whole number of waves of the grid.
    const uint64_t b_bytes = n_tiles * b.chunks * static_cast<uint64_t>(TC_CHUNK_BYTES) * (n_terms == 3 ? 2 : 1);
    bool interleaved = false;
    if (b_bytes > (uint64_t{64} << 20) && m_tiles >= 4 && n_tiles >= 64) {
        // the queue deals items round-robin and items take about equally long: pick the share count that
        // leaves the fewest CTAs idle in the last round (79 row tiles on 148 SMs: 13 shares = 6.94 rounds)
        double best_eff = 0.0;
        for (uint64_t ns = 4; ns <= 32 && ns * 8 <= n_tiles; ++ns) {
            const uint64_t count = m_tiles * ns;
            const uint64_t rounds = (count + sms - 1) / sms;
            const double eff = static_cast<double>(count) / static_cast<double>(rounds * sms);
            if (rounds >= 2 && eff > best_eff + 0.01) {
                best_eff = eff;
                n_split = ns;
                interleaved = true;
            }
        }
        if (!interleaved && m_tiles >= sms) {
            n_split = 1;
            interleaved = true;
        }
        if (interleaved) {
            tiles_per_split = (n_tiles + n_split - 1) / n_split;
        }
    }
    const uint64_t items = m_tiles * n_split;
    const uint32_t grid = static_cast<uint32_t>(items < sms ? items : sms);

    TcParams p{};
    p.a = a;
    p.b = b;
    p.n_terms = n_terms;
    p.alpha = alpha;
    p.bias = bias_dev;
    p.interleaved = interleaved ? 1u : 0u;
#ifdef VB200_TC_DIAG
    {
        const char* env = std::getenv("VB200_TC_DIAG");
        p.diag = env != nullptr ? static_cast<uint32_t>(std::atoi(env)) : 0u;
    }
#endif
    p.window = 0;
    if (interleaved) {
        p.window = 64;
        const char* env = std::getenv("VB200_TC_WINDOW");   // tuning aid: 0 or a power of two
        if (env != nullptr && env[0] != 0) {
            const uint32_t w = static_cast<uint32_t>(std::atoi(env));
            if ((w & (w - 1u)) == 0) {
                p.window = w;
            }
        }
    }
    p.a_sq = a_sq_dev;
    p.margin_scale = margin_scale_dev;
    p.row_bound = row_bound_dev;
    p.m = m;
    // Per-row candidate buffers: a few times m so compactions are rare, within what the per-warp
    // shared-memory sort areas can hold next to the operand stages.
    {
        const uint32_t cap_max = tc_cap_max(n_terms);
        uint32_t cap = next_pow2(4 * m < 64 ? 64 : 4 * m);
        if (cap > cap_max) {
            cap = cap_max;
        }
        VB_CHECK_ARG(m <= 4 || m + 32 <= cap, "tc_candidates: m = %u too large for the shared-memory sort area", m);
        p.cap = cap;
    }
    p.n_split = static_cast<uint32_t>(n_split);
    p.tiles_per_split = static_cast<uint32_t>(tiles_per_split);
    p.col_base = col_base;
    VB_TRY(ws.scratch.reserve(static_cast<size_t>(grid) * TC_BM * TC_COL_GROUPS * p.cap));
    VB_TRY(ws.error_flag.reserve(2));
    VB_TRY(out.reserve(static_cast<size_t>(a.rows) * n_split * TC_COL_GROUPS * m));
    VB_CUDA(cudaMemsetAsync(ws.error_flag.ptr, 0, 2 * sizeof(int), current_stream()));
    p.scratch = ws.scratch.ptr;
    p.out = out.ptr;
    p.error_flag = ws.error_flag.ptr;
    p.spin_limit = tc_spin_limit();
    p.row_flags = row_flags_dev;

    const bool small_m = m <= 4;
    const size_t sort_bytes = small_m ? 0 : TC_EPI_WARPS * static_cast<size_t>(p.cap) * sizeof(uint64_t);
    size_t smem = 0;
    tc_plan(p, sort_bytes, &smem);
    auto kernel = small_m ? tc_candidates_kernel<0> : tc_candidates_kernel<1>;
    VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    VB_LAUNCH(kernel, grid, TC_THREADS, smem, p);
    int flags[2] = {0, 0};
    VB_CUDA(cudaMemcpyAsync(flags, ws.error_flag.ptr, 2 * sizeof(int), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    if ((flags[0] & 1) != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "tensor-core kernel gave up on a bounded wait");
    }
    *n_split_out = static_cast<uint32_t>(n_split) * TC_COL_GROUPS;
    if (n_flagged_out != nullptr) {
        *n_flagged_out = static_cast<uint32_t>(flags[1]);
    }
    return 0;
}

int
tc_below_threshold(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
                   const float* bias_dev, const float* row_thr_dev, uint32_t expected_per_row, uint32_t max_per_row,
                   DevBuf<uint64_t>& out, DevBuf<uint32_t>& out_count, uint32_t* lists_out, uint32_t* cap_out,
                   bool* overflow_out, int* deferred_flag_dev) {
    VB_CHECK_ARG(a.rows > 0 && b.rows > 0, "tc_below_threshold: empty operand");
    VB_CHECK_ARG(a.chunks == b.chunks && a.chunks > 0, "tc_below_threshold: operand depths differ");
    VB_CHECK_ARG(n_terms == 1 || n_terms == 3, "tc_below_threshold: 1 or 3 terms");
    VB_CHECK_ARG(row_thr_dev != nullptr, "tc_below_threshold: thresholds missing");
    const uint64_t m_tiles = (a.rows + TC_BM - 1) / TC_BM;
    const uint64_t n_tiles = (b.rows + TC_BN - 1) / TC_BN;
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    // More column ranges per row tile than the sorted modes take: a list costs nothing but its
    // slots here, and short items spread evenly over the SMs.
    // The number of column ranges (at most 16: the pick kernels take 64 lists per row) that needs the fewest
    // tile steps: rounds of the persistent CTAs times the tiles of an item.
    uint64_t n_split = 1, best_cost = ~0ull;
    for (uint64_t ns = 1; ns <= 16 && ns <= n_tiles; ++ns) {
        const uint64_t tps = (n_tiles + ns - 1) / ns;
        const uint64_t ns_eff = (n_tiles + tps - 1) / tps;
        const uint64_t rounds = (m_tiles * ns_eff + sms - 1) / sms;
        const uint64_t cost = rounds * tps;
        if (cost < best_cost) {
            best_cost = cost;
            n_split = ns_eff;
        }
    }
    const uint64_t tiles_per_split = (n_tiles + n_split - 1) / n_split;
    n_split = (n_tiles + tiles_per_split - 1) / tiles_per_split;
    const uint32_t lists = static_cast<uint32_t>(n_split) * TC_COL_GROUPS;
    // list capacity: a list's expected share plus eight standard deviations of a Poisson count and a few more
    // (3.5 x the share at least), within the caller's limit per row.  An overflowing list costs its row a slow
    // exact answer, and with many short lists per row a multiple of the mean alone is passed every few thousand lists.
    const double share = static_cast<double>(expected_per_row) / lists;
    uint32_t want = static_cast<uint32_t>(share + 8.0 * std::sqrt(share) + 8.0);
    if (want < (7 * expected_per_row / 2 + lists - 1) / lists) {
        want = (7 * expected_per_row / 2 + lists - 1) / lists;
    }
    uint32_t cap = next_pow2(want);
    if (cap < 16) {
        cap = 16;
    }
    while (cap > 16 && static_cast<uint64_t>(cap) * lists > max_per_row) {
        cap >>= 1;
    }
    VB_CHECK_ARG(static_cast<uint64_t>(cap) * lists <= max_per_row, "tc_below_threshold: %u lists do not fit %u entries",
                 lists, max_per_row);
    const uint64_t items = m_tiles * n_split;
    const uint32_t grid = static_cast<uint32_t>(items < sms ? items : sms);
    TcParams p{};
    p.a = a;
    p.b = b;
    p.n_terms = n_terms;
    p.alpha = alpha;
    p.bias = bias_dev;
    p.row_bound = row_thr_dev;
    p.m = 0;
    p.cap = cap;
    p.n_split = static_cast<uint32_t>(n_split);
    p.tiles_per_split = static_cast<uint32_t>(tiles_per_split);
    VB_TRY(out.reserve(static_cast<size_t>(a.rows) * lists * cap));
    VB_TRY(out_count.reserve(static_cast<size_t>(a.rows) * lists));
    if (deferred_flag_dev == nullptr) {
        VB_TRY(ws.error_flag.reserve(2));
        VB_CUDA(cudaMemsetAsync(ws.error_flag.ptr, 0, 2 * sizeof(int), current_stream()));
    }
    p.out = out.ptr;
    p.out_count = out_count.ptr;
    p.error_flag = deferred_flag_dev != nullptr ? deferred_flag_dev : ws.error_flag.ptr;
    p.spin_limit = tc_spin_limit();
    size_t smem = 0;
    tc_plan(p, 0, &smem);
    auto kernel = tc_candidates_kernel<3>;
    VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    VB_LAUNCH(kernel, grid, TC_THREADS, smem, p);
    *lists_out = lists;
    *cap_out = cap;
    *overflow_out = false;
    if (deferred_flag_dev != nullptr) {
        return 0;
    }
    int flag = 0;
    VB_CUDA(cudaMemcpyAsync(&flag, ws.error_flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    if ((flag & 1) != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "tensor-core kernel gave up on a bounded wait");
    }
    *lists_out = lists;
    *cap_out = cap;
    *overflow_out = (flag & 2) != 0;
    return 0;
}

int
tc_scores(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
          const float* bias_dev, float* scores_dev, uint64_t ld, int* deferred_flag_dev) {
    VB_CHECK_ARG(a.rows > 0 && b.rows > 0, "tc_scores: empty operand");
    VB_CHECK_ARG(a.chunks == b.chunks && a.chunks > 0, "tc_scores: operand depths differ");
    VB_CHECK_ARG(n_terms == 1 || n_terms == 3, "tc_scores: 1 or 3 terms");
    VB_CHECK_ARG(ld >= b.rows && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(scores_dev) & 15) == 0,
                 "tc_scores: the score matrix must be 16-byte aligned with a row stride that is a multiple of 4");
    const uint64_t m_tiles = (a.rows + TC_BM - 1) / TC_BM;
    const uint64_t n_tiles = (b.rows + TC_BN - 1) / TC_BN;
    const uint32_t sms = static_cast<uint32_t>(sm_count());
    uint64_t n_split = (2ull * sms + m_tiles - 1) / m_tiles;
    if (n_split > n_tiles) {
        n_split = n_tiles;
    }
    if (n_split < 1) {
        n_split = 1;
    }
    const uint64_t tiles_per_split = (n_tiles + n_split - 1) / n_split;
    n_split = (n_tiles + tiles_per_split - 1) / tiles_per_split;
    const uint64_t items = m_tiles * n_split;
    const uint32_t grid = static_cast<uint32_t>(items < sms ? items : sms);
    TcParams p{};
    p.a = a;
    p.b = b;
    p.n_terms = n_terms;
    p.alpha = alpha;
    p.bias = bias_dev;
    p.m = 0;
    p.cap = 0;
    p.n_split = static_cast<uint32_t>(n_split);
    p.tiles_per_split = static_cast<uint32_t>(tiles_per_split);
    p.store = scores_dev;
    p.store_ld = ld;
    if (deferred_flag_dev == nullptr) {
        VB_TRY(ws.error_flag.reserve(2));
        VB_CUDA(cudaMemsetAsync(ws.error_flag.ptr, 0, 2 * sizeof(int), current_stream()));
    }
    p.error_flag = deferred_flag_dev != nullptr ? deferred_flag_dev : ws.error_flag.ptr;
    p.spin_limit = tc_spin_limit();
    size_t smem = 0;
    tc_plan(p, 0, &smem);
    auto kernel = tc_candidates_kernel<2>;
    VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    VB_LAUNCH(kernel, grid, TC_THREADS, smem, p);
    if (deferred_flag_dev != nullptr) {
        return 0;
    }
    int flag = 0;
    VB_CUDA(cudaMemcpyAsync(&flag, ws.error_flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    if ((flag & 1) != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "tensor-core kernel gave up on a bounded wait");
    }
    return 0;
}

}  // namespace vb200
