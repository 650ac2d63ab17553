// Tensor-core candidate generator: for every row of A, the `m` columns of B with the smallest
//   score(i, j) = alpha * <A_i, B_j> + bias[j]
// computed by tcgen05.mma (bf16 operands, fp32 accumulation in tensor memory) with the selection
// fused into the epilogue that drains the accumulator.  The scores are approximations whose only
// job is to nominate candidates: the callers re-score the survivors in the reference's exact fp32
// operation order (k-means labels, routing, BruteForce), so results stay bit-equal to the oracle.
//
// fp32 inputs are split into two bf16 terms, x = hi + lo with hi = bf16(x), lo = bf16(x - hi), and
// the product is taken as hi*hi + hi*lo + lo*hi (three MMAs per k-step; the dropped lo*lo term is
// ~2^-18 relative).  bf16 inputs use one term.
//
// Operands are pre-tiled in global memory so that a [128 rows x 64 k] chunk is one contiguous
// 16 KiB block already in the shared-memory layout the MMA descriptors describe (K-major, no
// swizzle: 8x8 core matrices of 128 B, cores adjacent along K 128 B apart, 8-row groups 1 KiB
// apart).  A chunk therefore moves with a single bulk copy that completes on an mbarrier.
#pragma once

#include "common.cuh"

namespace vb200 {

constexpr uint32_t TC_BM = 128;           // rows of A per tile
constexpr uint32_t TC_BN = 128;           // rows of B (output columns) per tile
constexpr uint32_t TC_KC = 64;            // k elements per chunk
constexpr uint32_t TC_CHUNK_ELEMS = 128 * TC_KC;
constexpr uint32_t TC_CHUNK_BYTES = TC_CHUNK_ELEMS * 2;   // 16 KiB
constexpr uint32_t TC_COL_GROUPS = 4;      // epilogue warps per TMEM lane quarter; each takes 32 of a tile's columns
constexpr uint32_t TC_EPI_WARPS = 4 * TC_COL_GROUPS;
constexpr uint32_t TC_EPI_THREADS = 32 * TC_EPI_WARPS;
constexpr uint32_t TC_THREADS = TC_EPI_THREADS + 96;   // + one warp each to issue the MMAs, the A copies and the B copies
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

struct TcOperand {
    const uint16_t* hi;   // [tiles][chunks][16 KiB] bf16
    const uint16_t* lo;   // same shape, nullptr when the operand has one term
    uint64_t rows;
    uint32_t chunks;      // ceil(dim / 64)
};

struct TcParams {
    TcOperand a, b;
    uint32_t n_terms;         // 1 (bf16 inputs) or 3 (split fp32 inputs)
    float alpha;
    const float* bias;        // [b.rows] or nullptr
    const float* a_sq;        // [a.rows] |A_i|^2, or nullptr            } used by the m <= 4 mode to skip
    const float* margin_scale;// device scalar: 1e-3 * max_j |B_j|, or nullptr } columns that cannot win
    const float* row_bound;   // [a.rows] a score some column is known to reach (warm start), or nullptr
    uint32_t m;               // candidates kept per row
    uint32_t cap;             // per-row buffer, power of two >= m + 32
    uint32_t stages;          // operand stages in shared memory (2 .. 6)
    uint32_t a_resident;      // 1: the A tile of a work item stays in shared memory for all its B tiles
    uint32_t wide;            // 1: two B tiles per MMA (128 x 256 x 16), 512 TMEM columns
    uint32_t n_split;         // shares of B's tiles per row tile
    uint32_t tiles_per_split; // B tiles per share when the shares are contiguous
#ifdef VB200_TC_DIAG
    uint32_t diag;            // timing experiments only: bit 0 skips the selection, bit 1 the MMAs
#endif
    uint32_t window;          // 0, or a power of two: tiles per window of the staggered walk over a share
    uint32_t interleaved;     // 1: share s holds tiles s, s + n_split, ...; the queue walks row tiles within a share
    uint64_t* scratch;        // [grid][128][TC_COL_GROUPS][cap] candidate buffers
    uint64_t* out;            // [a.rows][n_split][TC_COL_GROUPS][m] keys (ordered score << 32 | column), KEY_INF padded
                              // (threshold mode: [a.rows][n_split][TC_COL_GROUPS][cap], unsorted, with out_count)
    uint32_t* out_count;      // threshold mode: [a.rows][n_split][TC_COL_GROUPS] entries offered to each list
    uint32_t col_base;        // added to column indices in the keys
    float* store;             // score-matrix mode: [a.rows][store_ld] fp32 scores instead of candidates
    uint64_t store_ld;        // row stride of `store` in floats (multiple of 4, store 16-byte aligned)
    int* error_flag;          // [0] set non-zero if a bounded wait gave up; [1] counts the rows flagged below
    uint32_t spin_limit;      // polls a wait may take before it gives up
    uint32_t* row_flags;      // m <= 4 mode with a margin, optional: [a.rows], set to 1 for a row one of whose
                              // lists ended full of columns within the margin of its best -- a column the list
                              // had no room for might be the exact winner, so the caller decides such rows exactly
};

// A kernel whose wait ran out returns only after this pause, so that the copies and MMAs it still
// has in flight land in shared and tensor memory it still owns.
__device__ __forceinline__ void
tc_drain_pause() {
    for (int i = 0; i < 64; ++i) {
        __nanosleep(1000);
    }
}

// ---- raw PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t
smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void
mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void
mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void
mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait: returns false (and the caller bails out) if the phase never completes.
__device__ __forceinline__ bool
mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = TC_SPIN_LIMIT) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) {
            return true;
        }
    }
    return false;
}

// The same wait for the many epilogue threads: between polls they sleep, so that their polling
// does not take issue slots from the three single threads that feed the tensor core.
__device__ __forceinline__ bool
mbar_wait_relaxed(uint64_t* bar, uint32_t parity, uint32_t limit = TC_SPIN_LIMIT) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) {
            return true;
        }
        __nanosleep(128);
    }
    return false;
}

// One contiguous global -> shared bulk copy, completion counted in bytes on `bar`.
__device__ __forceinline__ void
bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void
tmem_alloc(uint32_t* slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void
tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void
tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void
tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 128 x 16, bf16 in, fp32 out.
__device__ __forceinline__ void
umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void
umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void
tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// All 128 fp32 columns of this thread's TMEM lane in one instruction (one wait instead of four).
__device__ __forceinline__ void
tmem_load_128(uint32_t taddr, uint32_t (&r)[128]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x128.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63, %64, %65, %66, %67, %68, %69, %70, %71, %72, %73, %74, %75, %76, %77, %78, %79, %80, %81, %82, %83, %84, %85, %86, %87, %88, %89, %90, %91, %92, %93, %94, %95, %96, %97, %98, %99, %100, %101, %102, %103, %104, %105, %106, %107, %108, %109, %110, %111, %112, %113, %114, %115, %116, %117, %118, %119, %120, %121, %122, %123, %124, %125, %126, %127}, [%128];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63]), "=r"(r[64]), "=r"(r[65]), "=r"(r[66]), "=r"(r[67]), "=r"(r[68]), "=r"(r[69]), "=r"(r[70]), "=r"(r[71]), "=r"(r[72]), "=r"(r[73]), "=r"(r[74]), "=r"(r[75]), "=r"(r[76]), "=r"(r[77]), "=r"(r[78]), "=r"(r[79]), "=r"(r[80]), "=r"(r[81]), "=r"(r[82]), "=r"(r[83]), "=r"(r[84]), "=r"(r[85]), "=r"(r[86]), "=r"(r[87]), "=r"(r[88]), "=r"(r[89]), "=r"(r[90]), "=r"(r[91]), "=r"(r[92]), "=r"(r[93]), "=r"(r[94]), "=r"(r[95]), "=r"(r[96]), "=r"(r[97]), "=r"(r[98]), "=r"(r[99]), "=r"(r[100]), "=r"(r[101]), "=r"(r[102]), "=r"(r[103]), "=r"(r[104]), "=r"(r[105]), "=r"(r[106]), "=r"(r[107]), "=r"(r[108]), "=r"(r[109]), "=r"(r[110]), "=r"(r[111]), "=r"(r[112]), "=r"(r[113]), "=r"(r[114]), "=r"(r[115]), "=r"(r[116]), "=r"(r[117]), "=r"(r[118]), "=r"(r[119]), "=r"(r[120]), "=r"(r[121]), "=r"(r[122]), "=r"(r[123]), "=r"(r[124]), "=r"(r[125]), "=r"(r[126]), "=r"(r[127])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, no swizzle: start address, leading-dimension byte
// offset (between the two 8-element K halves of a k-step) and stride byte offset (between 8-row
// groups), all in 16-byte units; bit 46 marks the sm_100 descriptor version.
__device__ __forceinline__ uint64_t
umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    return d;
}

// Instruction descriptor of kind::f16: fp32 accumulator, bf16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t
umma_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- host API (tc_gemm.cu) ------------------------------------------------------------------

// Polls a bounded wait of the tensor-core kernels may take before it gives up (default
// TC_SPIN_LIMIT).  Lowered only by tests that want to see the error path.
uint32_t tc_spin_limit();
void tc_set_spin_limit(uint32_t polls);

// Bytes of one pre-tiled term for `rows` x `dim`.
size_t tc_tiled_elems(uint64_t rows, uint32_t dim);
// fp32 rows -> hi (and lo when lo_dev != nullptr) bf16 terms in the tiled layout.
int tc_pretile_f32(const float* src_dev, uint64_t rows, uint32_t dim, uint16_t* hi_dev, uint16_t* lo_dev);
// bf16 rows (bit patterns) -> tiled layout.
int tc_pretile_bf16(const uint16_t* src_dev, uint64_t rows, uint32_t dim, uint16_t* hi_dev);

struct TcWorkspace {
    DevBuf<uint64_t> scratch;
    DevBuf<int> error_flag;
};

// For every row of A the m best columns of B by alpha * <a, b> + bias, as keys in
// out_dev[a_rows][n_split * TC_COL_GROUPS][m]; the number of lists per row (n_split * TC_COL_GROUPS) is
// chosen here and returned in n_split_out.
// a_sq_dev / margin_scale_dev (both optional, m <= 4 only): squared row norms of A and a device scalar
// c such that |approximate score - exact score| << c * |A_i|; columns scoring worse than the row's
// best by more than that margin are not nominated at all.  row_bound_dev (optional): with the margin
// (m <= 4), per row the exact score of some column: nothing worse than it plus the margin is visited;
// with m > 4, per row a score that columns must stay below to be of use (e.g. the m-th best score found
// in another column range): columns at or above it are not nominated.
// row_flags_dev / n_flagged_out (optional, with the margin): rows whose candidate lists may have lost a
// column within the margin (see TcParams::row_flags) are marked and counted; the array must be zeroed by
// the caller.
int tc_candidates(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
                  const float* bias_dev, uint32_t m, uint32_t col_base, DevBuf<uint64_t>& out,
                  uint32_t* n_split_out, const float* a_sq_dev = nullptr,
                  const float* margin_scale_dev = nullptr, const float* row_bound_dev = nullptr,
                  uint32_t* row_flags_dev = nullptr, uint32_t* n_flagged_out = nullptr);

// Every column of B whose score alpha * <a, b> + bias lies below the row's threshold row_thr_dev[row],
// unsorted, in out[a.rows][lists][cap] with the number offered to each list in out_count[a.rows][lists]
// (a count above cap means the list overflowed and lost entries: *overflow_out is set and the caller
// must not trust the result).  Lists are sized from expected_per_row, the number of columns the caller
// expects below a row's threshold; lists * cap never exceeds max_per_row.
// With deferred_flag_dev (two ints the caller zeroed on the stream) the call does not wait for the kernel:
// bit 0 (a bounded wait gave up) and bit 1 (some list overflowed) are OR-ed into deferred_flag_dev[0] for the
// caller to read when it next synchronises, and *overflow_out is left false.
int tc_below_threshold(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
                       const float* bias_dev, const float* row_thr_dev, uint32_t expected_per_row,
                       uint32_t max_per_row, DevBuf<uint64_t>& out, DevBuf<uint32_t>& out_count, uint32_t* lists_out,
                       uint32_t* cap_out, bool* overflow_out, int* deferred_flag_dev = nullptr);

// The whole score matrix alpha * <a, b> + bias as fp32 in scores_dev[a.rows][ld] (ld >= b.rows, a
// multiple of 4, scores_dev 16-byte aligned), from the same tensor-core pipeline.
// deferred_flag_dev: as for tc_below_threshold.
int tc_scores(TcWorkspace& ws, const TcOperand& a, const TcOperand& b, uint32_t n_terms, float alpha,
              const float* bias_dev, float* scores_dev, uint64_t ld, int* deferred_flag_dev = nullptr);

// Largest m tc_candidates accepts for the given number of terms.
uint32_t tc_max_candidates(uint32_t n_terms);

}  // namespace vb200
