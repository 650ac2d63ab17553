// IVF index: device-resident inverted lists, exact routing, the batched list-major scan
// scheduler, the partial-result merge and the fp32 rerank.
#include <algorithm>
#include <cooperative_groups.h>
#include <cub/device/device_radix_sort.cuh>

#include "dense.cuh"
#include "ivf_scan.cuh"
#include "comm.cuh"
#include "ivf_scan_tc.cuh"
#include "kmeans.cuh"
#include "rabitq.cuh"
#include "sq8.cuh"
#include "tc_gemm.cuh"

namespace vb200 {

constexpr uint32_t NONE32 = 0xFFFFFFFFu;
constexpr uint32_t ROUTE_SLACK = 8;   // extra routing candidates re-scored exactly
constexpr size_t SCALARS = 10;                // entries of the search workspace's scalar block
constexpr uint32_t ROUTE_MAX_PER_ROW = 4096;   // approximate candidates a query may bring to the final pick (32 KiB of keys)
constexpr int SQ8_QT = 16;
constexpr uint32_t SQ8_SLACK = 16;    // survivors kept beyond k for exact re-scoring
constexpr int RABITQ_QT = 4;   // 4-query tiles: twice the resident warps of 8-query tiles, which this latency-bound scan needs more than reuse

template <typename T>
static int
grow_preserve(DevBuf<T>& buf, size_t keep, size_t need) {
    if (need <= buf.cap) {
        return 0;
    }
    size_t cap = buf.cap * 2 > need ? buf.cap * 2 : need;
    DevBuf<T> bigger;
    if (bigger.reserve(cap) != 0) {
        VB_TRY(bigger.reserve(need));
    }
    if (keep > 0) {
        VB_CUDA(cudaMemcpyAsync(bigger.ptr, buf.ptr, keep * sizeof(T), cudaMemcpyDeviceToDevice,
                                current_stream()));
        VB_TRY(sync_stream());
    }
    buf = std::move(bigger);
    return 0;
}

struct SearchWorkspace {
    DevBuf<float> queries;      // staged queries / processed RaBitQ queries
    DevBuf<float> qproc;
    DevBuf<float> qw, qa;       // SQ8 per-query weights and constants
    DevBuf<int8_t> qw8;         // SQ8 tensor-core scan: the weights as three signed-byte terms, [nq][3][dpad32]
    DevBuf<float> qscale;       // [nq] their scale
    DevBuf<uint64_t> merged;    // SQ8 survivors before exact re-scoring
    DevBuf<float> scores;       // routing score slab
    DevBuf<uint64_t> cand;      // routing candidates
    DevBuf<float> route_thr;    // [nq] per-query score threshold of the routing pass
    DevBuf<uint64_t> route_keys;   // [nq][lists][cap] centroids below the threshold, unsorted
    DevBuf<uint32_t> route_cnt;    // [nq][lists]
    DevBuf<int32_t> probes;     // [nq x nprobe]
    DevBuf<float> probe_dists;
    // pair grouping, one set per scan phase (nearest list first, then the rest)
    DevBuf<uint32_t> pair_ctr;     // pair counts and scatter cursors of both phases: 4 x [nlist]
    DevBuf<uint32_t> pair_off[2];  // [nlist + 1]
    DevBuf<uint32_t> item_off[2];  // [nlist + 1]
    DevBuf<ScanItemDesc> item_map[2];  // [pairs of the phase] at most: the work items of the phase
    DevBuf<uint32_t> pair_q[2], pair_slot[2];
    DevBuf<uint32_t> first_live;  // [nq] probe rank of the first list this shard scans for the query
    DevBuf<uint8_t> pair_drop;    // [nq x nprobe] second-phase pairs pruned before grouping
    DevBuf<float> q_unit;         // cosine: the queries divided by their norms
    const vb200_filter* filter = nullptr;   // set for the duration of one filtered search
    DevBuf<uint32_t> deny_bits;   // tombstones | the caller's deny_inner_bits
    DevBuf<uint64_t> label_bits;  // device copy of the caller's label bitset
    bool pruning = false;         // the last scan dropped (query, list) pairs by the list radius
    DevBuf<float> bounds;         // [nq] per-query bounds as floats, the buffer the shards exchange
    DevBuf<uint16_t> q_hi, q_lo;  // tensor-core routing: tiled bf16 terms of the queries
    vb200_exchange_fn exchange = nullptr;   // set for the duration of one partial search
    void* exchange_arg = nullptr;
    DevBuf<float> qrot;   // RaBitQ: rotated query rows of one slice
    DevBuf<uint8_t> qcodes;   // SQ8 uniform: the queries' code records
    DevBuf<uint8_t> route_handled;  // routing: queries the warp-per-query pick answered
    DevBuf<float> pair_const;       // residual codes: per (query, probe) the centroid term of the distance
    DevBuf<uint64_t> keys_unique;   // buckets_per_data > 1: a query's postings folded to one per vector
    const float* ext_probe_dists = nullptr;   // centroid distances of caller-given probe lists (same duration)
    // sharded search: this rank's routed slice [probes | distances], the gathered probe lists and distances,
    // this rank's packed partial result [keys | labels] and the gathered ones
    DevBuf<uint32_t> sh_route_local;
    DevBuf<int32_t> sh_probes_all;
    DevBuf<float> sh_dists_all;
    DevBuf<uint64_t> sh_local, sh_all;
    DevBuf<uint32_t> thr;       // [nq]
    DevBuf<uint64_t> part;      // [nq x nprobe x k]
    DevBuf<uint64_t> keys;      // [nq x kscan]
    DevBuf<uint64_t> keys2;     // [nq x k] after rerank
    bool group_by_stages = false;   // the cooperative grouping launch was refused once: use the four-kernel form
    DevBuf<uint8_t> slot_written;   // [nq x nprobe] SQ8: which slots of `part` a scan kernel wrote
    DevBuf<uint64_t> scalars;   // [0] scan bytes, [1], [2] work-queue heads of the two phases, [3] bytes read, [4] tensor-core scan error flag,
                                // [5] the deadline passed, [6] the deadline (%globaltimer value; written by deadline_stamp_kernel)
    bool opt_no_reorder = false;   // search options of the running call (vb200_search_options)
    bool opt_deadline = false;
    DevBuf<int64_t> out_ids;
    DevBuf<float> out_dists;
};

}  // namespace vb200

using namespace vb200;

struct vb200_ivf {
    uint32_t dim = 0, nlist = 0;
    int metric = 0, quant = 0;
    bool use_reorder = false;
    uint32_t shard_rank = 0, shard_world = 1;
    uint32_t code_size = 0, code_stride = 0, dpad = 0;
    int device = 0;

    bool has_centroids = false, has_model = false, has_rotation = false;
    // cosine: rows, queries and centroids are normalised and the inner-product path does the rest
    // (ScalarQuantizer / FP32Quantizer with METRIC_TYPE_COSINE, IVFNearestPartition::Train)
    bool cosine = false;
    DevBuf<float> centroids, c_sq;
    DevBuf<float> lower, diff;           // SQ8, padded to dpad
    DevBuf<float> sq_scale, sq_mid;      // SQ8: diff/255 and lower + 128*diff/255, padded to dpad
    DevBuf<float> code_norm;             // SQ8: |decoded code|^2 per position
    // SQ8 tensor-core scan: a second copy of the lists as signed bytes (code - 128) in 8-row groups of
    // 16-byte cores, the shared-memory layout of the MMA's A operand; group_off[l] = first group of list l
    DevBuf<int8_t> codes_t;
    DevBuf<uint32_t> group_off;
    uint32_t kchunks = 0;                // 16-byte chunks per tiled row (dim rounded up to 32, over 16)
    DevBuf<float> rotation, rq_centroid; // RaBitQ

    uint64_t n_total = 0;   // rows seen (inner ids 0 .. n_total-1)
    uint64_t n_stored = 0;  // rows held by this shard
    DevBuf<uint8_t> codes;
    DevBuf<uint32_t> list_off;
    std::vector<uint32_t> list_off_host;
    uint32_t max_list_len = 0;   // the longest list this index (shard) holds
    bool balls_valid = false;    // the covering balls describe the lists as they are stored
    bool use_residual = false;       // SQ8: lists hold the codes of x - centroid (IVF use_residual)
    DevBuf<float> res_bias;          // [n_stored] L2 residual bias of every stored code (bucket_datacell.h:642-649)
    uint32_t buckets_per_data = 1;   // every vector is stored in this many of its nearest lists (IVF buckets_per_data)
    float su_lower = 0.f, su_diff = 0.f;   // SQ8 uniform model (one bound and one range for all dimensions)
    DevBuf<uint32_t> scan_order;  // list ids, longest list first: the order the scan queue walks
    DevBuf<uint32_t> tombstones;  // bitmap over inner ids: vectors removed with MARK_REMOVE
    uint64_t tomb_words = 0;
    uint64_t n_removed = 0;
    DevBuf<float> ball_centre;    // SQ8 list pruning: [nlist][SQ8_BALLS][dim] centres of the covering balls
    DevBuf<float> ball_radius;    // [nlist][SQ8_BALLS] their radii (-1: empty)
    DevBuf<uint32_t> ball_count;  // [nlist] balls in use per list
    DevBuf<float> list_radius;    // [nlist] largest distance of a decoded row from the list's centroid, rounded up
    bool prune_lists = true;
    int64_t last_scanned_bytes = 0;
    // tensor-core routing: the centroids as tiled bf16 hi/lo terms (rebuilt when they change)
    DevBuf<uint16_t> c_hi, c_lo;
    bool c_tiled = false;
    DevBuf<float> c_max_norm;     // [1] largest centroid norm
    TcWorkspace tc;
    DevBuf<uint32_t> pos_inner;
    DevBuf<int64_t> labels;
    DevBuf<float> flat;

    KMeansWorkspace kws;
    SearchWorkspace ws;
    std::mutex mu;
    int64_t last_scan_bytes = 0;
    cudaEvent_t ev_scan_begin = nullptr, ev_scan_end = nullptr;  // bracket the list-scan kernel
    bool scan_timed = false;

    ~vb200_ivf() {
        if (ev_scan_begin != nullptr) {
            cudaEventDestroy(ev_scan_begin);
        }
        if (ev_scan_end != nullptr) {
            cudaEventDestroy(ev_scan_end);
        }
    }
};

namespace vb200 {

// ---------------------------------------------------------------------------------------------
// build kernels
// ---------------------------------------------------------------------------------------------

// keys[i] = (list << 32) | i for rows this shard stores, (nlist << 32) | i otherwise; add_cnt[list]++.
__global__ void
ivf_make_keys_kernel(const int32_t* __restrict__ labels, uint64_t n, uint32_t nlist, uint32_t rank,
                     uint32_t world, uint64_t* __restrict__ keys, uint32_t* __restrict__ add_cnt) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    int32_t l = labels[i];
    uint32_t list = nlist;
    if (l >= 0 && static_cast<uint32_t>(l) < nlist && static_cast<uint32_t>(l) % world == rank) {
        list = static_cast<uint32_t>(l);
        atomicAdd(add_cnt + list, 1u);
    }
    keys[i] = (static_cast<uint64_t>(list) << 32) | static_cast<uint32_t>(i);
}

// Moves the rows already stored to their place in the regrown arrays (16 bytes per thread).
__global__ void
ivf_move_old_kernel(const uint8_t* __restrict__ old_codes, const uint32_t* __restrict__ old_inner,
                    const uint32_t* __restrict__ old_off, const uint32_t* __restrict__ new_off,
                    uint32_t nlist, uint64_t n_old, uint32_t stride16,
                    uint8_t* __restrict__ new_codes, uint32_t* __restrict__ new_inner) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= n_old * stride16) {
        return;
    }
    uint32_t p = static_cast<uint32_t>(e / stride16);
    uint32_t c = static_cast<uint32_t>(e % stride16);
    uint32_t lo = 0, hi = nlist;  // largest l with old_off[l] <= p
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (old_off[mid] <= p) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    uint32_t np = new_off[lo] + (p - old_off[lo]);
    reinterpret_cast<uint4*>(new_codes)[static_cast<uint64_t>(np) * stride16 + c] =
        reinterpret_cast<const uint4*>(old_codes)[static_cast<uint64_t>(p) * stride16 + c];
    if (c == 0) {
        new_inner[np] = old_inner[p];
    }
}

// Places lists given in the serialised inverted-file layout (per list: its codes packed at code_size
// bytes each, its inner ids) into this shard's arrays: one thread per (destination position, 16-byte
// chunk of the padded code).  Inner ids at or beyond n_total are counted in *bad and stored as NONE32.
__global__ void
ivf_import_lists_kernel(const uint8_t* __restrict__ src_codes, const int64_t* __restrict__ src_inner,
                        const uint64_t* __restrict__ src_off, const uint32_t* __restrict__ new_off,
                        uint32_t nlist, uint64_t n_kept, uint32_t code_size, uint32_t stride16,
                        uint64_t n_total, uint8_t* __restrict__ new_codes, uint32_t* __restrict__ new_inner,
                        unsigned long long* __restrict__ bad) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= n_kept * stride16) {
        return;
    }
    uint32_t np = static_cast<uint32_t>(e / stride16);
    uint32_t c = static_cast<uint32_t>(e % stride16);
    uint32_t lo = 0, hi = nlist;  // largest l with new_off[l] <= np
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (new_off[mid] <= np) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const uint64_t sp = src_off[lo] + (np - new_off[lo]);
    const uint8_t* src = src_codes + sp * code_size;
    uint8_t* dst = new_codes + (static_cast<uint64_t>(np) * stride16 + c) * 16;
#pragma unroll
    for (uint32_t b = 0; b < 16; ++b) {
        uint32_t pos = c * 16 + b;
        dst[b] = pos < code_size ? src[pos] : uint8_t{0};
    }
    if (c == 0) {
        int64_t inner = src_inner[sp];
        if (inner < 0 || static_cast<uint64_t>(inner) >= n_total) {
            atomicAdd(bad, 1ull);
            new_inner[np] = NONE32;
        } else {
            new_inner[np] = static_cast<uint32_t>(inner);
        }
    }
}

// Sorted key s -> destination position of its row: after the rows the list already held, in
// ascending row order (the append order of IVF::Add with thread_count 1, ivf.cpp:662-676).
__global__ void
ivf_place_new_kernel(const uint64_t* __restrict__ sorted_keys, uint64_t n, uint32_t nlist,
                     const uint32_t* __restrict__ new_off, const uint32_t* __restrict__ old_off,
                     const uint32_t* __restrict__ add_off, uint32_t inner_base, uint32_t per_vector,
                     uint32_t* __restrict__ dst_of_row, uint32_t* __restrict__ new_inner) {
    uint64_t s = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (s >= n) {
        return;
    }
    uint64_t key = sorted_keys[s];
    uint32_t list = static_cast<uint32_t>(key >> 32);
    uint32_t row = static_cast<uint32_t>(key);
    if (list >= nlist) {
        dst_of_row[row] = NONE32;
        return;
    }
    uint32_t old_size = old_off[list + 1] - old_off[list];
    uint32_t np = new_off[list] + old_size + static_cast<uint32_t>(s - add_off[list]);
    dst_of_row[row] = np;
    new_inner[np] = inner_base + row / per_vector;   // per_vector consecutive rows are postings of one vector
}

// scale_d = diff_d / 255, mid_d = lower_d + 128 * scale_d (zero beyond dim).
__global__ void
sq8_derive_model_kernel(const float* __restrict__ lower, const float* __restrict__ diff, uint32_t dim,
                        uint32_t dpad, float* __restrict__ scale, float* __restrict__ mid) {
    uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= dpad) {
        return;
    }
    float s = 0.f, m = 0.f;
    if (d < dim) {
        s = __fdiv_rn(diff[d], 255.0f);
        m = fmaf(128.0f, s, lower[d]);
    }
    scale[d] = s;
    mid[d] = m;
}

// fp32 buckets: row i of the batch goes, unchanged, to position dst_pos[i] (rows of foreign
// shards have no position).
__global__ void
fp32_place_rows_kernel(const float* __restrict__ x, uint64_t count, uint32_t dim, const uint32_t* __restrict__ dst_pos,
                       uint8_t* __restrict__ codes, uint32_t code_stride) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count * dim) {
        return;
    }
    const uint64_t row = e / dim;
    const uint32_t d = static_cast<uint32_t>(e % dim);
    const uint32_t pos = dst_pos[row];
    if (pos != 0xFFFFFFFFu) {
        reinterpret_cast<float*>(codes + static_cast<uint64_t>(pos) * code_stride)[d] = x[e];
    }
}

// use_residual: out[i] = x[i] - centroid of the row's list (FP32Sub, src/datacell/bucket_datacell.h:607-612, :634);
// rows without a list (another shard's) are copied as they are and never stored.
__global__ void
residual_rows_kernel(const float* __restrict__ x, uint64_t count, uint32_t dim, const int32_t* __restrict__ lists,
                     uint32_t nlist, const float* __restrict__ centroids, float* __restrict__ out) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count * dim) {
        return;
    }
    const int32_t l = lists[e / dim];
    const float c = (l >= 0 && static_cast<uint32_t>(l) < nlist) ? centroids[static_cast<uint64_t>(l) * dim + e % dim] : 0.f;
    out[e] = __fsub_rn(x[e], c);
}

// Residual codes, per stored position p of list l: bias[p] = -2 * IP(c_l, DecodeOne(code)) - IP(c_l, c_l) for L2
// (encode_vector, bucket_datacell.h:642-649; DecodeOne = code / 255 * diff + lower, scalar_quantizer.cpp:112-124;
// IP = one ascending FMA chain), and the ranking form's per-row term becomes |decoded|^2 - bias.
__global__ void
sq8_residual_bias_kernel(const uint8_t* __restrict__ codes, uint64_t n, uint32_t dim, uint32_t code_stride,
                         const float* __restrict__ lower, const float* __restrict__ diff,
                         const uint32_t* __restrict__ list_off, uint32_t nlist, const float* __restrict__ centroids,
                         int metric, float* __restrict__ bias, float* __restrict__ code_norm) {
    const uint64_t p = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p >= n) {
        return;
    }
    if (metric != VB200_METRIC_L2) {
        bias[p] = 0.f;
        return;
    }
    uint32_t lo = 0, hi = nlist;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (list_off[mid] <= p) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const float* cen = centroids + static_cast<uint64_t>(lo) * dim;
    const uint8_t* c = codes + p * code_stride;
    float ip_cd = 0.f, ip_cc = 0.f;
    for (uint32_t d = 0; d < dim; ++d) {
        const float dec = __fadd_rn(__fmul_rn(__fdiv_rn(static_cast<float>(c[d]), 255.0f), __ldg(diff + d)), __ldg(lower + d));
        const float cv = __ldg(cen + d);
        ip_cd = fmaf(cv, dec, ip_cd);
        ip_cc = fmaf(cv, cv, ip_cc);
    }
    const float b = __fsub_rn(__fmul_rn(-2.0f, ip_cd), ip_cc);
    bias[p] = b;
    code_norm[p] = code_norm[p] - b;
}

// pair_const[e] for pair e = (query, probe): -2 <q, c_l> (L2) or -<q, c_l> (IP), the centroid term of a distance
// over residual codes; used for ranking only (the exact re-scoring recomputes it in the reference's order).
__global__ void
pair_const_kernel(const int32_t* __restrict__ probes, uint64_t total, uint32_t nprobe, uint32_t nlist,
                  const float* __restrict__ queries, uint32_t dim, const float* __restrict__ centroids, int metric,
                  float* __restrict__ pair_const) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    const int32_t l = probes[e];
    float v = 0.f;
    if (l >= 0 && static_cast<uint32_t>(l) < nlist) {
        const float* q = queries + (e / nprobe) * dim;
        const float* c = centroids + static_cast<uint64_t>(l) * dim;
        float ip = 0.f;
        for (uint32_t d = 0; d < dim; ++d) {
            ip = fmaf(__ldg(q + d), __ldg(c + d), ip);
        }
        v = metric == VB200_METRIC_L2 ? -2.0f * ip : -ip;
    }
    pair_const[e] = v;
}

// out[p] = x[p / per_vector]: the rows of the postings of an add with buckets_per_data > 1.
__global__ void
repeat_rows_kernel(const float* __restrict__ x, uint64_t postings, uint32_t dim, uint32_t per_vector,
                   float* __restrict__ out) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < postings * dim) {
        out[e] = x[(e / dim) / per_vector * dim + e % dim];
    }
}

// buckets_per_data > 1: the same vector can be found in several probed lists.  keys[q][n] hold a query's n
// best postings ascending with the vector's inner id as payload; the first posting of every vector (its
// smallest distance) stays, and the k best of those go out (the de-duplication of IVF::search,
// src/algorithm/ivf/ivf.cpp:1799-1825).  One CTA per query.
__global__ void __launch_bounds__(128)
dedup_keys_kernel(const uint64_t* __restrict__ keys, uint32_t n, uint32_t k, uint64_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char dedup_smem[];
    uint64_t* kq = reinterpret_cast<uint64_t*>(dedup_smem);
    uint32_t* keep = reinterpret_cast<uint32_t*>(kq + n);
    const uint64_t* src = keys + static_cast<uint64_t>(blockIdx.x) * n;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        kq[i] = src[i];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint64_t key = kq[i];
        uint32_t first = key != KEY_INF ? 1u : 0u;
        const uint32_t id = static_cast<uint32_t>(key);
        for (uint32_t j = 0; j < i && first != 0; ++j) {
            if (static_cast<uint32_t>(kq[j]) == id && kq[j] != KEY_INF) {
                first = 0;
            }
        }
        keep[i] = first;
    }
    __syncthreads();
    if (threadIdx.x == 0) {   // n is a few hundred at most: an in-order walk keeps the ascending order
        uint32_t w = 0;
        uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
        for (uint32_t i = 0; i < n && w < k; ++i) {
            if (keep[i] != 0) {
                dst[w++] = kq[i];
            }
        }
        for (; w < k; ++w) {
            dst[w] = KEY_INF;
        }
    }
}

// The same for half-precision buckets: every element encoded to 16 bits on its way in.
template <int FMT>
__global__ void
half_place_rows_kernel(const float* __restrict__ x, uint64_t count, uint32_t dim, const uint32_t* __restrict__ dst_pos,
                       uint8_t* __restrict__ codes, uint32_t code_stride) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count * dim) {
        return;
    }
    const uint64_t row = e / dim;
    const uint32_t d = static_cast<uint32_t>(e % dim);
    const uint32_t pos = dst_pos[row];
    if (pos != 0xFFFFFFFFu) {
        reinterpret_cast<uint16_t*>(codes + static_cast<uint64_t>(pos) * code_stride)[d] = half_encode<FMT>(x[e]);
    }
}

// Tiled signed copy of the lists for the tensor-core scan: row r of list l goes to 8-row group
// group_off[l] + r / 8; its 16-byte chunk c (bytes code - 128, i.e. code ^ 0x80; zero beyond the code)
// to core c of the group, row r % 8.  One thread per (position, chunk).
__global__ void
sq8_tile_codes_kernel(const uint8_t* __restrict__ codes, uint32_t code_stride, const uint32_t* __restrict__ list_off,
                      const uint32_t* __restrict__ group_off, uint32_t nlist, uint64_t n_stored, uint32_t kchunks,
                      int8_t* __restrict__ tiled) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= n_stored * kchunks) {
        return;
    }
    const uint32_t pos = static_cast<uint32_t>(e / kchunks);
    const uint32_t c = static_cast<uint32_t>(e % kchunks);
    uint32_t lo = 0, hi = nlist;  // largest l with list_off[l] <= pos
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (list_off[mid] <= pos) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    const uint32_t r = pos - list_off[lo];
    const uint64_t g = static_cast<uint64_t>(group_off[lo]) + (r >> 3);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (c * 16 < code_stride) {
        v = __ldg(reinterpret_cast<const uint4*>(codes + static_cast<uint64_t>(pos) * code_stride + c * 16));
        v.x ^= 0x80808080u;
        v.y ^= 0x80808080u;
        v.z ^= 0x80808080u;
        v.w ^= 0x80808080u;
    }
    *reinterpret_cast<uint4*>(tiled + (g * kchunks + c) * 128 + (r & 7u) * 16) = v;
}

// code_norm[p] = sum_d x_d^2 with x_d the reference's decode fma(code * (1/255), diff, lower).
__global__ void
sq8_code_norm_kernel(const uint8_t* __restrict__ codes, uint64_t n, uint32_t dim, uint32_t code_stride,
                     const float* __restrict__ lower, const float* __restrict__ diff,
                     float* __restrict__ code_norm) {
    uint64_t p = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p >= n) {
        return;
    }
    const uint8_t* c = codes + p * code_stride;
    const float inv255 = 1.0f / 255.0f;
    float s = 0.f;
    for (uint32_t d0 = 0; d0 < dim; d0 += 16) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(c + d0));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            uint32_t d = d0 + j;
            if (d < dim) {
                float code = static_cast<float>((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
                float x = fmaf(__fmul_rn(code, inv255), __ldg(diff + d), __ldg(lower + d));
                s = fmaf(x, x, s);
            }
        }
    }
    code_norm[p] = s;
}

// Covering balls of a list for the scan's pruning: SQ8_BALLS centres per list (farthest-point
// seeds refined by two Lloyd steps over the list's decoded rows) and, per centre, the largest
// distance of a row assigned to it, rounded up.  Every row lies in the ball it is assigned to, so
// a query farther than that from every ball cannot have a neighbour in the list -- whatever the
// quality of the little clustering.  A list that holds two clusters of the data gets two small
// balls instead of one large one.  One CTA per list; empty balls have radius -1.
__device__ __forceinline__ float
sq8_row_dist(const uint8_t* __restrict__ row, uint32_t dim, const float* __restrict__ lower,
             const float* __restrict__ diff, const float* __restrict__ centre) {
    const float inv255 = 1.0f / 255.0f;
    float s = 0.f;
    for (uint32_t d0 = 0; d0 < dim; d0 += 16) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(row + d0));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            uint32_t d = d0 + j;
            if (d < dim) {
                float code = static_cast<float>((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
                float x = fmaf(__fmul_rn(code, inv255), __ldg(diff + d), __ldg(lower + d));
                float t = x - centre[d];
                s = fmaf(t, t, s);
            }
        }
    }
    return s;
}

__global__ void __launch_bounds__(128)
sq8_list_balls_kernel(const uint8_t* __restrict__ codes, uint32_t code_stride, uint32_t dim,
                      const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ old_off,
                      const float* __restrict__ lower,
                      const float* __restrict__ diff, const float* __restrict__ centroids,
                      float* __restrict__ ball_centre, float* __restrict__ ball_radius,
                      uint32_t* __restrict__ ball_count, float* __restrict__ list_radius) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* seeds = reinterpret_cast<float*>(smem_raw);              // [SQ8_BALLS][dim]
    float* sums = seeds + SQ8_BALLS * dim;                          // [SQ8_BALLS][dim]
    __shared__ unsigned long long best;                             // (ordered distance << 32) | row
    __shared__ uint32_t cnt[SQ8_BALLS];
    __shared__ uint32_t rmax[SQ8_BALLS];
    const uint32_t l = blockIdx.x, tid = threadIdx.x;
    const uint32_t beg = list_off[l], len = list_off[l + 1] - beg;
    if (old_off != nullptr && len == old_off[l + 1] - old_off[l]) {
        return;   // rows are only ever appended: a list of unchanged length keeps the balls it has
    }
    float* out_c = ball_centre + static_cast<uint64_t>(l) * SQ8_BALLS * dim;
    float* out_r = ball_radius + static_cast<uint64_t>(l) * SQ8_BALLS;
    // three balls for an ordinary list, one more per 300 rows beyond 900, eight at most: the long
    // lists are the ones that hold several clusters of the data and that many queries probe
    int n_balls = static_cast<int>((len + 299) / 300);
    n_balls = n_balls < 3 ? 3 : (n_balls > SQ8_BALLS ? SQ8_BALLS : n_balls);
    if (tid == 0) {
        ball_count[l] = len == 0 ? 0u : static_cast<uint32_t>(n_balls);
    }
    if (len == 0) {
        for (uint32_t i = tid; i < SQ8_BALLS * dim; i += blockDim.x) {
            out_c[i] = 0.f;
        }
        if (tid < SQ8_BALLS) {
            out_r[tid] = -1.0f;
        }
        if (tid == 0) {
            list_radius[l] = 0.f;
        }
        return;
    }
    const float inv255 = 1.0f / 255.0f;
    auto row_ptr = [&](uint32_t r) { return codes + static_cast<uint64_t>(beg + r) * code_stride; };
    auto decode_to = [&](uint32_t r, float* dst) {   // all threads: dst[d] = decoded row r
        const uint8_t* row = row_ptr(r);
        for (uint32_t d = tid; d < dim; d += blockDim.x) {
            dst[d] = fmaf(__fmul_rn(static_cast<float>(row[d]), inv255), __ldg(diff + d), __ldg(lower + d));
        }
    };
    // farthest-point seeding, starting from the row farthest from the list's centroid
    for (uint32_t d = tid; d < dim; d += blockDim.x) {
        sums[d] = centroids[static_cast<uint64_t>(l) * dim + d];
    }
    for (int j = 0; j < n_balls; ++j) {
        if (tid == 0) {
            best = 0ull;
        }
        __syncthreads();
        unsigned long long mine = 0ull;
        for (uint32_t r = tid; r < len; r += blockDim.x) {
            float dmin;
            if (j == 0) {
                dmin = sq8_row_dist(row_ptr(r), dim, lower, diff, sums);
            } else {
                dmin = INFINITY;
                for (int t = 0; t < j; ++t) {
                    dmin = fminf(dmin, sq8_row_dist(row_ptr(r), dim, lower, diff, seeds + t * dim));
                }
            }
            const unsigned long long key = (static_cast<unsigned long long>(__float_as_uint(dmin)) << 32) | (len - 1 - r);
            mine = key > mine ? key : mine;   // distances are non-negative: their bit patterns order like the values
        }
        atomicMax(&best, mine);
        __syncthreads();
        if (j == 0 && tid == 0) {
            // the farthest row from the list's centroid: the radius of the one ball around the centroid,
            // which costs a pair nothing to test because routing has measured |q - centroid| already
            list_radius[l] = sqrtf(__uint_as_float(static_cast<uint32_t>(best >> 32))) * 1.00001f + 1e-12f;
        }
        const uint32_t pick = len - 1 - static_cast<uint32_t>(best & 0xFFFFFFFFull);
        decode_to(pick < len ? pick : 0, seeds + j * dim);
        __syncthreads();
    }
    for (uint32_t i = n_balls * dim + tid; i < SQ8_BALLS * dim; i += blockDim.x) {
        seeds[i] = 0.f;
    }
    __syncthreads();
    // two Lloyd steps, then the radii
    for (int it = 0; it < 3; ++it) {
        const bool last = it == 2;
        for (uint32_t i = tid; i < SQ8_BALLS * dim; i += blockDim.x) {
            sums[i] = 0.f;
        }
        if (tid < SQ8_BALLS) {
            cnt[tid] = 0;
            rmax[tid] = 0;
        }
        __syncthreads();
        for (uint32_t r = tid; r < len; r += blockDim.x) {
            int arg = 0;
            float dbest = INFINITY;
            for (int t = 0; t < n_balls; ++t) {
                const float dd = sq8_row_dist(row_ptr(r), dim, lower, diff, seeds + t * dim);
                if (dd < dbest) {
                    dbest = dd;
                    arg = t;
                }
            }
            atomicAdd(&cnt[arg], 1u);
            if (last) {
                atomicMax(&rmax[arg], __float_as_uint(dbest));
            } else {
                const uint8_t* row = row_ptr(r);
                for (uint32_t d = 0; d < dim; ++d) {
                    const float x = fmaf(__fmul_rn(static_cast<float>(row[d]), inv255), __ldg(diff + d), __ldg(lower + d));
                    atomicAdd(&sums[arg * dim + d], x);
                }
            }
        }
        __syncthreads();
        if (!last) {
            for (uint32_t i = tid; i < SQ8_BALLS * dim; i += blockDim.x) {
                const uint32_t c = cnt[i / dim];
                if (c > 0) {
                    seeds[i] = sums[i] / static_cast<float>(c);
                }
            }
            __syncthreads();
        }
    }
    for (uint32_t i = tid; i < SQ8_BALLS * dim; i += blockDim.x) {
        out_c[i] = seeds[i];
    }
    if (tid < SQ8_BALLS) {
        out_r[tid] = (static_cast<int>(tid) < n_balls && cnt[tid] > 0)
                         ? sqrtf(__uint_as_float(rmax[tid])) * 1.00001f + 1e-12f
                         : -1.0f;
    }
}

// One warp per query: qw[q][d] = q_d * scale_d (zero padded) and
//   L2: qa = |q|^2 - 2 sum q_d mid_d      IP: qa = 1 - sum q_d mid_d
__global__ void __launch_bounds__(128)
sq8_query_prep_kernel(const float* __restrict__ queries, uint64_t nq, uint32_t dim, uint32_t dpad,
                      const float* __restrict__ scale, const float* __restrict__ mid, int metric,
                      float* __restrict__ qw, float* __restrict__ qa, uint32_t dpad32, int8_t* __restrict__ qw8,
                      float* __restrict__ qscale) {
    uint64_t q = static_cast<uint64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    uint32_t lane = threadIdx.x & 31;
    if (q >= nq) {
        return;
    }
    const float* src = queries + q * dim;
    float* dst = qw + q * dpad;
    float qq = 0.f, qm = 0.f;
    for (uint32_t d = lane; d < dpad; d += 32) {
        float v = d < dim ? __ldg(src + d) : 0.f;
        dst[d] = v * scale[d];
        qq = fmaf(v, v, qq);
        qm = fmaf(v, mid[d], qm);
    }
    for (int off = 16; off > 0; off >>= 1) {
        qq += __shfl_xor_sync(0xffffffffu, qq, off);
        qm += __shfl_xor_sync(0xffffffffu, qm, off);
    }
    if (lane == 0) {
        qa[q] = metric == VB200_METRIC_L2 ? fmaf(-2.0f, qm, qq) : 1.0f - qm;
    }
    if (qw8 == nullptr) {
        return;
    }
    // Tensor-core scan: w = s * (t1 + t2 / 254 + t3 / 254^2) with signed-byte terms, s = max|w| / 127.
    float wmax = 0.f;
    for (uint32_t d = lane; d < dim; d += 32) {
        wmax = fmaxf(wmax, fabsf(__ldg(src + d) * scale[d]));
    }
    for (int off = 16; off > 0; off >>= 1) {
        wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
    }
    const float s = wmax > 0.f && wmax < INFINITY ? wmax / 127.0f : 1.0f;
    int8_t* t = qw8 + q * 3 * dpad32;
    for (uint32_t d = lane; d < dpad32; d += 32) {
        const float w = d < dim ? __ldg(src + d) * scale[d] : 0.f;
        const float u = w / s;
        const float t1 = fminf(fmaxf(rintf(u), -127.f), 127.f);
        const float v2 = (u - t1) * 254.0f;
        const float t2 = fminf(fmaxf(rintf(v2), -127.f), 127.f);
        const float t3 = fminf(fmaxf(rintf((v2 - t2) * 254.0f), -127.f), 127.f);
        t[d] = static_cast<int8_t>(static_cast<int>(t1));
        t[dpad32 + d] = static_cast<int8_t>(static_cast<int>(t2));
        t[2 * dpad32 + d] = static_cast<int8_t>(static_cast<int>(t3));
    }
    if (lane == 0) {
        qscale[q] = s;
    }
}

// ---------------------------------------------------------------------------------------------
// search kernels
// ---------------------------------------------------------------------------------------------

// Re-scores the routing candidates of one query exactly and orders them: distance ascending,
// lower list id first on ties.  L2: FMA chain of (q-c)^2 over d ascending; IP: 1 - chain of q*c
// (the loop of IVF::route_buckets_only, src/algorithm/ivf/ivf.cpp:1589-1660).
__global__ void __launch_bounds__(128)
route_finalize_kernel(const float* __restrict__ queries, uint32_t dim,
                      const float* __restrict__ centroids, const uint64_t* __restrict__ cand,
                      uint32_t ncand, uint32_t n2, uint32_t nprobe, int metric,
                      int32_t* __restrict__ probes, float* __restrict__ probe_dists) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    float* qs = reinterpret_cast<float*>(keys + n2);   // the query, staged once for all candidates
    const float* q = queries + static_cast<uint64_t>(blockIdx.x) * dim;
    const uint64_t* cq = cand + static_cast<uint64_t>(blockIdx.x) * ncand;
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        qs[d] = q[d];
    }
    __syncthreads();
    const bool vec4 = (dim & 3u) == 0;   // centroid rows are then 16-byte aligned
    for (uint32_t i = threadIdx.x; i < n2; i += blockDim.x) {
        uint64_t key = KEY_INF;
        if (i < ncand && cq[i] != KEY_INF) {
            uint32_t list = static_cast<uint32_t>(cq[i]);
            const float* c = centroids + static_cast<uint64_t>(list) * dim;
            float s = 0.f;
            // one chain per candidate, dimensions in ascending order, as the reference computes it
            if (vec4) {
                const float4* c4 = reinterpret_cast<const float4*>(c);
                const float4* q4 = reinterpret_cast<const float4*>(qs);
                if (metric == VB200_METRIC_L2) {
#pragma unroll 4
                    for (uint32_t d4 = 0; d4 < (dim >> 2); ++d4) {
                        const float4 cv = __ldg(c4 + d4), qv = q4[d4];
                        float t = __fsub_rn(qv.x, cv.x);
                        s = fmaf(t, t, s);
                        t = __fsub_rn(qv.y, cv.y);
                        s = fmaf(t, t, s);
                        t = __fsub_rn(qv.z, cv.z);
                        s = fmaf(t, t, s);
                        t = __fsub_rn(qv.w, cv.w);
                        s = fmaf(t, t, s);
                    }
                } else {
#pragma unroll 4
                    for (uint32_t d4 = 0; d4 < (dim >> 2); ++d4) {
                        const float4 cv = __ldg(c4 + d4), qv = q4[d4];
                        s = fmaf(qv.x, cv.x, s);
                        s = fmaf(qv.y, cv.y, s);
                        s = fmaf(qv.z, cv.z, s);
                        s = fmaf(qv.w, cv.w, s);
                    }
                    s = __fsub_rn(1.0f, s);
                }
            } else if (metric == VB200_METRIC_L2) {
                for (uint32_t d = 0; d < dim; ++d) {
                    float t = __fsub_rn(qs[d], __ldg(c + d));
                    s = fmaf(t, t, s);
                }
            } else {
                for (uint32_t d = 0; d < dim; ++d) {
                    s = fmaf(qs[d], __ldg(c + d), s);
                }
                s = __fsub_rn(1.0f, s);
            }
            key = make_key(s, list);
        }
        keys[i] = key;
    }
    block_bitonic_sort(keys, n2);
    for (uint32_t i = threadIdx.x; i < nprobe; i += blockDim.x) {
        uint64_t key = keys[i];
        uint64_t o = static_cast<uint64_t>(blockIdx.x) * nprobe + i;
        probes[o] = key == KEY_INF ? -1 : static_cast<int32_t>(static_cast<uint32_t>(key));
        if (probe_dists != nullptr) {
            probe_dists[o] = key == KEY_INF ? INFINITY : ordered_to_float(static_cast<uint32_t>(key >> 32));
        }
    }
}

__device__ __forceinline__ bool
probe_is_live(int32_t l, uint32_t nlist, uint32_t rank, uint32_t world, const uint32_t* list_off) {
    if (l < 0 || static_cast<uint32_t>(l) >= nlist || static_cast<uint32_t>(l) % world != rank) {
        return false;
    }
    return list_off[l + 1] > list_off[l];
}

// out = tombstones | extra (either may be shorter than `words`; missing words count as zero).
__global__ void
deny_merge_kernel(const uint32_t* __restrict__ tomb, uint64_t tomb_words, const uint32_t* __restrict__ extra,
                  uint64_t extra_words, uint64_t words, uint32_t* __restrict__ out) {
    uint64_t w = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (w < words) {
        out[w] = (w < tomb_words ? tomb[w] : 0u) | (w < extra_words ? extra[w] : 0u);
    }
}

// Marks the inner ids whose label is in sorted[0..count): one thread per inner id, binary search.
__global__ void
tombstone_kernel(const int64_t* __restrict__ labels, uint64_t n_total, const int64_t* __restrict__ sorted,
                 uint64_t count, uint32_t* __restrict__ tomb, unsigned long long* __restrict__ newly) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_total) {
        return;
    }
    const int64_t label = labels[i];
    uint64_t lo = 0, hi = count;
    while (lo < hi) {
        const uint64_t mid = (lo + hi) >> 1;
        if (sorted[mid] < label) {
            lo = mid + 1;
        } else {
            hi = mid;
        }
    }
    if (lo < count && sorted[lo] == label) {
        const uint32_t bit = 1u << (i & 31u);
        if ((atomicOr(tomb + (i >> 5), bit) & bit) == 0u) {
            atomicAdd(newly, 1ull);
        }
    }
}

// first_live[q] = probe rank of the nearest list of query q that this shard holds and that is not
// empty (nprobe when there is none): the list whose scan gives the query its first bound.
__global__ void
first_live_kernel(const int32_t* __restrict__ probes, uint64_t nq, uint32_t nprobe, uint32_t nlist,
                  uint32_t rank, uint32_t world, const uint32_t* __restrict__ list_off, int nearest_only,
                  uint32_t* __restrict__ first_live) {
    uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (q >= nq) {
        return;
    }
    uint32_t pr = 0;
    while (pr < nprobe && !probe_is_live(probes[q * nprobe + pr], nlist, rank, world, list_off)) {
        ++pr;
    }
    // nearest_only (shards that exchange their bounds): only the shard that holds a query's
    // nearest list scans for it before the exchange; the others get its bound, so the first phase
    // shrinks with the number of shards instead of costing every shard one list per query.
    first_live[q] = (nearest_only && pr != 0) ? nprobe : pr;
}

// Grouping tables of the two phases: phase 0 takes every query's first live probe, phase 1 the
// others.
struct PairTables {
    uint32_t* cnt[2];       // [nlist] pairs per list
    uint32_t* cursor[2];    // [nlist] scatter cursors
    uint32_t* off[2];       // [nlist + 1] first pair of each list
    uint32_t* item_off[2];  // [nlist + 1] tile prefix by position in the scan order
    ScanItemDesc* item_map[2];  // [items] every work item
    uint32_t* q[2];         // [pairs] query
    uint32_t* slot[2];      // [pairs] output slot
};

__device__ __forceinline__ void
pair_count_one(uint64_t e, const int32_t* __restrict__ probes, uint32_t nprobe, const uint32_t* __restrict__ first_live,
               uint32_t nlist, uint32_t rank, uint32_t world, const uint32_t* __restrict__ list_off, const PairTables& t,
               uint32_t phase_sel, const uint8_t* __restrict__ drop) {
    const uint32_t e32 = static_cast<uint32_t>(e);   // (the batch holds fewer than 2^32 pairs: 32-bit division)
    const uint32_t qi = e32 / nprobe, pr = e32 - qi * nprobe;
    const uint32_t ph = pr == first_live[qi] ? 0u : 1u;
    if ((phase_sel < 2 && ph != phase_sel) || (drop != nullptr && drop[e] != 0)) {
        return;   // phase_sel 0 / 1: group that phase only; dropped pairs were pruned beforehand
    }
    int32_t l = probes[e];
    if (probe_is_live(l, nlist, rank, world, list_off)) {
        atomicAdd((ph == 0 ? t.cnt[0] : t.cnt[1]) + l, 1u);
    }
}

// After the first phase: drop[e] = 1 for every second-phase (query, list) pair that the list's
// covering balls put beyond the query's bound (the test the SIMT scan kernel makes per tile, made here
// once per pair so that pruned pairs never become work items).  Two steps per warp.  Every lane applies
// the cheap test to its own pair: the ball around the list's centroid, whose distance from the query
// routing has computed exactly -- on clustered data that settles most pairs without reading a ball
// centre.  The pairs that pass it are then measured against the list's covering balls, one ball after the
// other until one of them cannot exclude the list, four pairs at a time with eight lanes per pair, so the
// loads of a step cover 128 contiguous bytes of each centre instead of 32 separate lines; sums are reduced
// within the eight lanes.  The code bytes of the dropped pairs still count as algorithmic scan volume
// (scalars[0]).
__device__ __forceinline__ float
pair_ball_dot8(const float* __restrict__ qv, const float* __restrict__ cv, uint32_t dim, int metric, uint32_t part,
               uint32_t gmask) {
    float dot = 0.f;
    if ((dim & 3u) == 0 && ((reinterpret_cast<uintptr_t>(qv) | reinterpret_cast<uintptr_t>(cv)) & 15u) == 0) {
        const float4* q4 = reinterpret_cast<const float4*>(qv);
        const float4* c4 = reinterpret_cast<const float4*>(cv);
        for (uint32_t i = part; i < (dim >> 2); i += 8) {
            const float4 x = __ldg(q4 + i), c = __ldg(c4 + i);
            if (metric == 0) {
                float t = x.x - c.x;
                dot = fmaf(t, t, dot);
                t = x.y - c.y;
                dot = fmaf(t, t, dot);
                t = x.z - c.z;
                dot = fmaf(t, t, dot);
                t = x.w - c.w;
                dot = fmaf(t, t, dot);
            } else {
                dot = fmaf(x.x, c.x, dot);
                dot = fmaf(x.y, c.y, dot);
                dot = fmaf(x.z, c.z, dot);
                dot = fmaf(x.w, c.w, dot);
            }
        }
    } else {
        for (uint32_t d = part; d < dim; d += 8) {
            const float x = __ldg(qv + d), c = __ldg(cv + d);
            if (metric == 0) {
                const float t = x - c;
                dot = fmaf(t, t, dot);
            } else {
                dot = fmaf(x, c, dot);
            }
        }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        dot += __shfl_xor_sync(gmask, dot, o);
    }
    return dot;
}

// The same for four consecutive ball centres of a list at once (cv, cv + dim, ...): one trip to memory instead
// of four for a pair that has to look at several balls.
__device__ __forceinline__ void
pair_ball_dot8x4(const float* __restrict__ qv, const float* __restrict__ cv, uint32_t dim, int metric, uint32_t part,
                 uint32_t gmask, float (&dot)[4]) {
    dot[0] = dot[1] = dot[2] = dot[3] = 0.f;
    if ((dim & 3u) == 0 && ((reinterpret_cast<uintptr_t>(qv) | reinterpret_cast<uintptr_t>(cv)) & 15u) == 0) {
        const float4* q4 = reinterpret_cast<const float4*>(qv);
        const float4* c4 = reinterpret_cast<const float4*>(cv);
        const uint32_t row4 = dim >> 2;
        for (uint32_t i = part; i < row4; i += 8) {
            const float4 x = __ldg(q4 + i);
            float4 c[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                c[b] = __ldg(c4 + b * row4 + i);
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (metric == 0) {
                    float t = x.x - c[b].x;
                    dot[b] = fmaf(t, t, dot[b]);
                    t = x.y - c[b].y;
                    dot[b] = fmaf(t, t, dot[b]);
                    t = x.z - c[b].z;
                    dot[b] = fmaf(t, t, dot[b]);
                    t = x.w - c[b].w;
                    dot[b] = fmaf(t, t, dot[b]);
                } else {
                    dot[b] = fmaf(x.x, c[b].x, dot[b]);
                    dot[b] = fmaf(x.y, c[b].y, dot[b]);
                    dot[b] = fmaf(x.z, c[b].z, dot[b]);
                    dot[b] = fmaf(x.w, c[b].w, dot[b]);
                }
            }
        }
    } else {
        for (uint32_t d = part; d < dim; d += 8) {
            const float x = __ldg(qv + d);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float c = __ldg(cv + b * dim + d);
                if (metric == 0) {
                    const float t = x - c;
                    dot[b] = fmaf(t, t, dot[b]);
                } else {
                    dot[b] = fmaf(x, c, dot[b]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) {
            dot[b] += __shfl_xor_sync(gmask, dot[b], o);
        }
    }
}

__global__ void __launch_bounds__(256)
pair_drop_kernel(const int32_t* __restrict__ probes, uint64_t total, uint32_t nprobe,
                         const uint32_t* __restrict__ first_live, uint32_t nlist, uint32_t rank, uint32_t world,
                         const uint32_t* __restrict__ list_off, const float* __restrict__ queries, uint32_t dim,
                         const float* __restrict__ ball_centre, const float* __restrict__ ball_radius,
                         const uint32_t* __restrict__ ball_count, const uint32_t* __restrict__ thr, int metric,
                         uint32_t code_size, const float* __restrict__ probe_dists, const float* __restrict__ list_radius,
                         uint8_t* __restrict__ drop, unsigned long long* __restrict__ scalars) {
    __shared__ unsigned long long s_bytes;
    if (threadIdx.x == 0) {
        s_bytes = 0;
    }
    __syncthreads();
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31u;
    unsigned long long my_bytes = 0;   // code bytes of the pairs this lane reports dropped
    // step 1: the lane's own pair
    bool need_balls = false;
    uint32_t q = 0;
    int32_t l = 0;
    float bound = 0.f;
    if (e < total) {
        q = static_cast<uint32_t>(e) / nprobe;   // (fewer than 2^32 pairs in a batch: 32-bit division)
        const uint32_t pr = static_cast<uint32_t>(e) - q * nprobe;
        l = probes[e];
        const uint32_t t = thr[q];
        bool dropped = false;
        if (pr != first_live[q] && probe_is_live(l, nlist, rank, world, list_off) && t <= float_to_ordered(INFINITY)) {
            bound = ordered_to_float(t);
            bool beyond = false;   // the ball around the centroid already excludes the list
            if (probe_dists != nullptr && metric == 0) {
                const float dc = __ldg(probe_dists + e), big_r = __ldg(list_radius + l);
                const float gap = sqrtf(dc) - big_r;
                const float lower = gap > 0.f ? gap * gap : 0.f;
                beyond = lower > bound * 1.001f + 1e-4f * dc;
            }
            dropped = beyond;
            need_balls = !beyond;
        }
        if (!need_balls) {
            drop[e] = dropped ? 1 : 0;
            if (dropped) {
                my_bytes = static_cast<unsigned long long>(list_off[l + 1] - list_off[l]) * code_size;
            }
        }
    }
    // step 2: the warp's remaining pairs, four at a time
    uint32_t todo = __ballot_sync(0xffffffffu, need_balls);
    const uint32_t group = lane >> 3, part = lane & 7u;
    const uint32_t gmask = 0xFFu << (lane & 24u);
    while (todo != 0) {
        // the group's pair: the group-th lowest set bit of todo
        uint32_t rest = todo;
        for (uint32_t g = 0; g < group && rest != 0; ++g) {
            rest &= rest - 1;
        }
        const bool have = rest != 0;
        const uint32_t src = have ? static_cast<uint32_t>(__ffs(rest)) - 1u : 0u;
        const uint32_t pq = __shfl_sync(0xffffffffu, q, src);
        const int32_t pl = __shfl_sync(0xffffffffu, l, src);
        const float pbound = __shfl_sync(0xffffffffu, bound, src);
        if (have) {
            const float* qv = queries + static_cast<uint64_t>(pq) * dim;
            const float qq = metric != 0 ? pair_ball_dot8(qv, qv, dim, 1, part, gmask) : 0.f;
            bool beyond = false;
            if (probe_dists != nullptr && metric != 0) {
                const uint64_t pe = e - lane + src;
                const float dc = __ldg(probe_dists + pe), big_r = __ldg(list_radius + pl);
                const float lower = dc - sqrtf(qq) * big_r;   // dc = 1 - <q, centroid>
                beyond = lower > pbound + 1e-3f * (fabsf(pbound) + fabsf(1.0f - dc) + 1.0f);
            }
            bool any = false;      // some ball may hold a row within the bound
            if (!beyond) {
                static_assert(SQ8_BALLS % 4 == 0, "a list's ball slots are read four at a time");
                const uint32_t n_balls = __ldg(ball_count + pl);
                const float* cv = ball_centre + static_cast<uint64_t>(pl) * SQ8_BALLS * dim;
                // four balls per trip (every list owns SQ8_BALLS slots, so slots past n_balls may be read; they are
                // not judged)
                for (uint32_t j0 = 0; j0 < n_balls && !any; j0 += 4, cv += 4 * static_cast<size_t>(dim)) {
                    float dots[4];
                    pair_ball_dot8x4(qv, cv, dim, metric, part, gmask, dots);
#pragma unroll
                    for (uint32_t b = 0; b < 4; ++b) {
                        const uint32_t j = j0 + b;
                        const float r = j < n_balls ? __ldg(ball_radius + static_cast<uint64_t>(pl) * SQ8_BALLS + j) : -1.f;
                        if (r >= 0.f && !any) {
                            // slack: the distances compared here and in the scan differ in rounding only
                            const float dot = dots[b];
                            if (metric == 0) {
                                const float gap = sqrtf(dot) - r;
                                const float lower = gap > 0.f ? gap * gap : 0.f;
                                any = !(lower > pbound * 1.001f + 1e-4f * dot);
                            } else {
                                const float lower = 1.0f - dot - sqrtf(qq) * r;
                                any = !(lower > pbound + 1e-3f * (fabsf(pbound) + fabsf(dot) + 1.0f));
                            }
                        }
                    }
                }
            }
            if (part == 0) {
                const uint64_t pe = e - lane + src;
                drop[pe] = any ? 0 : 1;
                if (!any) {
                    my_bytes += static_cast<unsigned long long>(list_off[pl + 1] - list_off[pl]) * code_size;
                }
            }
        }
        // the four lowest set bits are done
        for (int g = 0; g < 4 && todo != 0; ++g) {
            todo &= todo - 1;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        my_bytes += __shfl_xor_sync(0xffffffffu, my_bytes, o);
    }
    if (lane == 0 && my_bytes != 0) {
        atomicAdd(&s_bytes, my_bytes);
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_bytes != 0) {
        atomicAdd(scalars, s_bytes);
    }
}

// One CTA per phase: exclusive prefixes of (pairs) and of (tiles of qt queries) over the lists
// taken in `order` (pair_off is stored by list, item_off by position in the order), plus the
// logical scan volume sum(pairs[l] * len[l]).  pair_items_kernel turns the prefixes into work items.
// A thread owns PAIR_SCAN_PER consecutive positions of a 1024 * PAIR_SCAN_PER-position slab: all its loads of
// `order` go out together, then all the gathers behind them, so a slab costs two trips to memory and one block
// scan rather than a chain of dependent gathers per 32 positions.
constexpr int PAIR_SCAN_PER = 16;

__device__ __forceinline__ void
pair_scan_block(uint32_t ph, const PairTables& tables, const uint32_t* __restrict__ list_off,
                const uint32_t* __restrict__ order, uint32_t nlist, uint32_t qt, uint32_t code_size,
                uint64_t* __restrict__ scalars) {
    const uint32_t* __restrict__ pair_cnt = ph == 0 ? tables.cnt[0] : tables.cnt[1];
    uint32_t* __restrict__ pair_off = ph == 0 ? tables.off[0] : tables.off[1];
    uint32_t* __restrict__ item_off = ph == 0 ? tables.item_off[0] : tables.item_off[1];
    __shared__ uint32_t s_pairs[33], s_items[33];   // exclusive prefixes of the warps' sums, totals in [32]
    __shared__ unsigned long long s_bytes;
    __syncthreads();   // (a CTA may run this for one phase after the other)
    if (threadIdx.x == 0) {
        s_bytes = 0;
    }
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t carry_p = 0, carry_t = 0;
    unsigned long long my_bytes = 0;
    for (uint32_t slab = 0; slab < nlist; slab += 1024u * PAIR_SCAN_PER) {
        const uint32_t p0 = slab + threadIdx.x * PAIR_SCAN_PER;
        uint32_t l[PAIR_SCAN_PER], c[PAIR_SCAN_PER];
#pragma unroll
        for (int i = 0; i < PAIR_SCAN_PER; ++i) {
            l[i] = p0 + i < nlist ? __ldg(order + p0 + i) : 0xFFFFFFFFu;
        }
        uint32_t sum_p = 0, sum_t = 0;
        uint32_t len[PAIR_SCAN_PER];
#pragma unroll
        for (int i = 0; i < PAIR_SCAN_PER; ++i) {
            const bool real = l[i] != 0xFFFFFFFFu;
            c[i] = real ? pair_cnt[l[i]] : 0u;
            len[i] = real ? __ldg(list_off + l[i] + 1) - __ldg(list_off + l[i]) : 0u;   // asked for unconditionally: no load waits for another
        }
#pragma unroll
        for (int i = 0; i < PAIR_SCAN_PER; ++i) {
            sum_p += c[i];
            sum_t += (c[i] + qt - 1) / qt;
            my_bytes += static_cast<unsigned long long>(c[i]) * len[i] * code_size;
        }
        // block-wide exclusive prefix of the threads' sums
        uint32_t ip = sum_p, it = sum_t;
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, ip, off), ut = __shfl_up_sync(0xffffffffu, it, off);
            if (lane >= static_cast<uint32_t>(off)) {
                ip += up;
                it += ut;
            }
        }
        __syncthreads();   // the previous slab's reads of s_pairs / s_items are done
        if (lane == 31) {
            s_pairs[warp] = ip;
            s_items[warp] = it;
        }
        __syncthreads();
        if (warp == 0) {
            const uint32_t vp = s_pairs[lane], vt = s_items[lane];
            uint32_t wp = vp, wt = vt;
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, wp, off), ut = __shfl_up_sync(0xffffffffu, wt, off);
                if (lane >= static_cast<uint32_t>(off)) {
                    wp += up;
                    wt += ut;
                }
            }
            s_pairs[lane] = wp - vp;
            s_items[lane] = wt - vt;
            if (lane == 31) {
                s_pairs[32] = wp;
                s_items[32] = wt;
            }
        }
        __syncthreads();
        uint32_t run_p = carry_p + s_pairs[warp] + ip - sum_p, run_t = carry_t + s_items[warp] + it - sum_t;
#pragma unroll
        for (int i = 0; i < PAIR_SCAN_PER; ++i) {
            if (l[i] != 0xFFFFFFFFu) {
                pair_off[l[i]] = run_p;
                item_off[p0 + i] = run_t;
                run_p += c[i];
                run_t += (c[i] + qt - 1) / qt;
            }
        }
        carry_p += s_pairs[32];
        carry_t += s_items[32];
    }
    for (int off = 16; off > 0; off >>= 1) {
        my_bytes += __shfl_xor_sync(0xffffffffu, my_bytes, off);
    }
    if (lane == 0 && my_bytes != 0) {
        atomicAdd(&s_bytes, my_bytes);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        pair_off[nlist] = carry_p;
        item_off[nlist] = carry_t;
        atomicAdd(reinterpret_cast<unsigned long long*>(scalars), s_bytes);  // logical scan volume, both phases
    }
}

// The work items of the scan's queue, written from the prefixes above: one thread per list position and
// phase (blockIdx.y), each writing the descriptors of its list's tiles of qt queries.
__device__ __forceinline__ void
pair_items_one(uint32_t pos, uint32_t ph, const PairTables& tables, const uint32_t* __restrict__ list_off,
               const uint32_t* __restrict__ group_off, const uint32_t* __restrict__ order, uint32_t qt) {
    const uint32_t l = order[pos];
    const uint32_t c = tables.cnt[ph][l];
    if (c == 0) {
        return;
    }
    const uint32_t t = (c + qt - 1) / qt;
    const uint32_t first_pair = tables.off[ph][l], first_item = tables.item_off[ph][pos];
    ScanItemDesc d;
    d.list = l;
    d.lbeg = list_off[l];
    d.len = list_off[l + 1] - d.lbeg;
    d.goff = group_off != nullptr ? group_off[l] : 0u;
    d.pad0 = 0;
    d.pad1 = 0;
    ScanItemDesc* __restrict__ item_map = tables.item_map[ph];
    for (uint32_t j = 0; j < t; ++j) {
        d.pbeg = first_pair + j * qt;
        d.nqt = c - j * qt < qt ? c - j * qt : qt;
        item_map[first_item + j] = d;
    }
}

__device__ __forceinline__ void
pair_scatter_one(uint64_t e, const int32_t* __restrict__ probes, uint32_t nprobe, const uint32_t* __restrict__ first_live,
                 uint32_t nlist, uint32_t rank, uint32_t world, const uint32_t* __restrict__ list_off, const PairTables& t,
                 uint32_t phase_sel, const uint8_t* __restrict__ drop) {
    const uint32_t e32 = static_cast<uint32_t>(e);
    const uint32_t qi = e32 / nprobe, pr = e32 - qi * nprobe;
    const bool first = pr == first_live[qi];
    if ((phase_sel < 2 && (first ? 0u : 1u) != phase_sel) || (drop != nullptr && drop[e] != 0)) {
        return;
    }
    int32_t l = probes[e];
    if (probe_is_live(l, nlist, rank, world, list_off)) {
        uint32_t s = (first ? t.off[0] : t.off[1])[l] + atomicAdd((first ? t.cursor[0] : t.cursor[1]) + l, 1u);
        (first ? t.q[0] : t.q[1])[s] = qi;
        (first ? t.slot[0] : t.slot[1])[s] = static_cast<uint32_t>(e);
    }
}

// The four stages as kernels of their own: the path for a context that cannot hold one CTA per SM resident (the
// cooperative launch below refuses then), and for comparisons (VB200_GROUP_COOPERATIVE=0).
__global__ void
pair_count_kernel(const int32_t* __restrict__ probes, uint64_t total, uint32_t nprobe, const uint32_t* __restrict__ first_live,
                  uint32_t nlist, uint32_t rank, uint32_t world, const uint32_t* __restrict__ list_off, PairTables t,
                  uint32_t phase_sel, const uint8_t* __restrict__ drop) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < total) {
        pair_count_one(e, probes, nprobe, first_live, nlist, rank, world, list_off, t, phase_sel, drop);
    }
}

__global__ void __launch_bounds__(1024)
pair_scan_kernel(PairTables t, const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ order, uint32_t nlist,
                 uint32_t qt, uint32_t code_size, uint64_t* __restrict__ scalars) {
    pair_scan_block(blockIdx.x, t, list_off, order, nlist, qt, code_size, scalars);
}

__global__ void
pair_items_kernel(PairTables t, const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ group_off,
                  const uint32_t* __restrict__ order, uint32_t nlist, uint32_t qt) {
    const uint32_t pos = blockIdx.x * blockDim.x + threadIdx.x;
    if (pos < nlist) {
        pair_items_one(pos, blockIdx.y, t, list_off, group_off, order, qt);
    }
}

__global__ void
pair_scatter_kernel(const int32_t* __restrict__ probes, uint64_t total, uint32_t nprobe, const uint32_t* __restrict__ first_live,
                    uint32_t nlist, uint32_t rank, uint32_t world, const uint32_t* __restrict__ list_off, PairTables t,
                    uint32_t phase_sel, const uint8_t* __restrict__ drop) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < total) {
        pair_scatter_one(e, probes, nprobe, first_live, nlist, rank, world, list_off, t, phase_sel, drop);
    }
}

// Groups the (query, probed list) pairs by list and writes the scan's work queue, in one cooperative launch:
// clear the counters | count the pairs of every list | prefix sums (one CTA per phase) | work items and the
// pairs' places, with a grid-wide barrier between the stages.  As four launches the stages cost more in launch
// and drain latency than in work.
__global__ void __launch_bounds__(1024, 1)
pair_group_kernel(const int32_t* __restrict__ probes, uint64_t total, uint32_t nprobe,
                  const uint32_t* __restrict__ first_live, uint32_t nlist, uint32_t rank, uint32_t world,
                  const uint32_t* __restrict__ list_off, const uint32_t* __restrict__ group_off,
                  const uint32_t* __restrict__ order, PairTables t, uint32_t* __restrict__ counters, uint32_t phase_sel,
                  const uint8_t* __restrict__ drop, uint32_t qt, uint32_t code_size, uint64_t* __restrict__ scalars) {
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t nthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = tid; i < 4ull * nlist; i += nthreads) {
        counters[i] = 0;
    }
    grid.sync();
    for (uint64_t e = tid; e < total; e += nthreads) {
        pair_count_one(e, probes, nprobe, first_live, nlist, rank, world, list_off, t, phase_sel, drop);
    }
    grid.sync();
    if (gridDim.x == 1) {
        pair_scan_block(0, t, list_off, order, nlist, qt, code_size, scalars);
        pair_scan_block(1, t, list_off, order, nlist, qt, code_size, scalars);
    } else if (blockIdx.x < 2) {
        pair_scan_block(blockIdx.x, t, list_off, order, nlist, qt, code_size, scalars);
    }
    grid.sync();
    for (uint64_t i = tid; i < 2ull * nlist; i += nthreads) {
        pair_items_one(static_cast<uint32_t>(i % nlist), static_cast<uint32_t>(i / nlist), t, list_off, group_off, order, qt);
    }
    for (uint64_t e = tid; e < total; e += nthreads) {
        pair_scatter_one(e, probes, nprobe, first_live, nlist, rank, world, list_off, t, phase_sel, drop);
    }
}

// Per query: the k smallest of its `per_query` partial keys, ascending.  With slot flags (slot_written, slots of
// slot_keys keys) only the slots a scan kernel wrote hold keys -- the others were never initialised -- and the
// query's written slots are listed first, so the rounds run over those alone.
constexpr uint32_t MERGE_MAX_SLOTS = 1024;

__global__ void __launch_bounds__(256)
merge_keys_kernel(const uint64_t* __restrict__ part, uint64_t per_query, uint32_t k, uint32_t cap,
                  uint64_t* __restrict__ out, const uint8_t* __restrict__ slot_written, uint32_t slot_keys) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ uint16_t s_slots[MERGE_MAX_SLOTS];
    __shared__ uint32_t s_nslots;
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    uint32_t* state = reinterpret_cast<uint32_t*>(keys + cap);
    BlockSelect sel;
    const uint64_t* src = part + static_cast<uint64_t>(blockIdx.x) * per_query;
    uint64_t n_keys = per_query;
    const uint32_t n_slots = slot_written != nullptr ? static_cast<uint32_t>(per_query / slot_keys) : 0u;
    const bool listed = slot_written != nullptr && n_slots <= MERGE_MAX_SLOTS;
    if (listed) {
        if (threadIdx.x == 0) {
            s_nslots = 0;
        }
        __syncthreads();
        const uint8_t* flags = slot_written + static_cast<uint64_t>(blockIdx.x) * n_slots;
        for (uint32_t sl = threadIdx.x; sl < n_slots; sl += blockDim.x) {
            if (flags[sl] != 0) {
                s_slots[atomicAdd(&s_nslots, 1u)] = static_cast<uint16_t>(sl);   // any order: the selection sorts
            }
        }
        __syncthreads();
        n_keys = static_cast<uint64_t>(s_nslots) * slot_keys;
    }
    sel.init(keys, state, k, cap);
    for (uint64_t base = 0; base < n_keys; base += blockDim.x) {
        sel.make_room(blockDim.x);
        uint64_t thr = sel.threshold();
        uint64_t i = base + threadIdx.x;
        if (i < n_keys) {
            bool present = true;
            uint64_t at = i;
            if (listed) {
                at = static_cast<uint64_t>(s_slots[i / slot_keys]) * slot_keys + i % slot_keys;
            } else if (slot_written != nullptr) {
                present = slot_written[(static_cast<uint64_t>(blockIdx.x) * per_query + i) / slot_keys] != 0;
            }
            if (present) {
                uint64_t key = __ldg(src + at);
                if (key != KEY_INF) {
                    sel.offer(key, thr);
                }
            }
        }
    }
    uint32_t cnt = sel.finish();
    uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        dst[i] = i < cnt ? keys[i] : KEY_INF;
    }
}

// Replaces each key's payload (a code position) by the inner id stored there.
__global__ void
keys_pos_to_inner_kernel(uint64_t* __restrict__ keys, uint64_t total,
                         const uint32_t* __restrict__ pos_inner) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    uint64_t key = keys[e];
    if (key != KEY_INF) {
        keys[e] = (key & 0xFFFFFFFF00000000ull) | pos_inner[static_cast<uint32_t>(key)];
    }
}

// FlattenReorder::Reorder, simple path (src/impl/reorder/flatten_reorder.cpp:76-118): one CTA per
// query recomputes every candidate against its fp32 row (one warp per candidate) and keeps k.
__global__ void __launch_bounds__(256)
rerank_kernel(const float* __restrict__ queries, uint32_t dim, const float* __restrict__ flat,
              const uint64_t* __restrict__ cand, uint32_t ncand, uint32_t n2, uint32_t k, int metric,
              uint64_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    const float* q = queries + static_cast<uint64_t>(blockIdx.x) * dim;
    const uint64_t* cq = cand + static_cast<uint64_t>(blockIdx.x) * ncand;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (uint32_t i = threadIdx.x; i < n2; i += blockDim.x) {
        keys[i] = KEY_INF;
    }
    __syncthreads();
    for (uint32_t c = warp; c < ncand; c += nwarps) {
        uint64_t key = cq[c];
        if (key == KEY_INF) {
            continue;
        }
        uint32_t inner = static_cast<uint32_t>(key);
        const float* x = flat + static_cast<uint64_t>(inner) * dim;
        float s = 0.f;
        for (uint32_t d = lane; d < dim; d += 32) {
            float a = __ldg(q + d), b = __ldg(x + d);
            if (metric == VB200_METRIC_L2) {
                float t = a - b;
                s = fmaf(t, t, s);
            } else {
                s = fmaf(a, b, s);
            }
        }
        for (int off = 16; off > 0; off >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, off);
        }
        if (lane == 0) {
            float dist = metric == VB200_METRIC_L2 ? s : 1.0f - s;
            keys[c] = make_key(dist, inner);
        }
    }
    block_bitonic_sort(keys, n2);
    uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        dst[i] = i < n2 ? keys[i] : KEY_INF;
    }
}

// keys (payload = inner id) -> user labels and distances.
__global__ void
keys_to_results_kernel(const uint64_t* __restrict__ keys, uint64_t total,
                       const int64_t* __restrict__ labels, int64_t* __restrict__ ids,
                       float* __restrict__ dists) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    uint64_t key = keys[e];
    if (key == KEY_INF) {
        ids[e] = -1;
        dists[e] = INFINITY;
    } else {
        ids[e] = labels[static_cast<uint32_t>(key)];
        dists[e] = ordered_to_float(static_cast<uint32_t>(key >> 32));
    }
}

// Cross-shard merge input: labels gathered beside the keys; payload = index into the gathered
// arrays so the label can be fetched after selection.
__global__ void
tag_partials_kernel(const uint64_t* __restrict__ keys, uint32_t parts, uint64_t part_stride, uint64_t nq, uint32_t k,
                    uint64_t* __restrict__ tagged) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    uint64_t total = static_cast<uint64_t>(parts) * nq * k;
    if (e >= total) {
        return;
    }
    // input [part][q][i] (parts part_stride keys apart) -> output [q][part][i]
    uint64_t part = e / (nq * k);
    uint64_t rem = e % (nq * k);
    uint64_t q = rem / k, i = rem % k;
    uint64_t src = part * part_stride + rem;
    uint64_t key = keys[src];
    uint64_t o = (q * parts + part) * k + i;
    tagged[o] = key == KEY_INF ? KEY_INF : ((key & 0xFFFFFFFF00000000ull) | static_cast<uint32_t>(src));
}

static int
launch_merge(const uint64_t* part, uint64_t nq, uint64_t per_query, uint32_t k, uint64_t* out,
             const uint8_t* slot_written = nullptr, uint32_t slot_keys = 1) {
    uint32_t cap = next_pow2(k + 256);
    size_t smem = cap * sizeof(uint64_t) + 16;
    if (smem > 48 * 1024) {
        VB_CUDA(cudaFuncSetAttribute(merge_keys_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
    }
    VB_LAUNCH(merge_keys_kernel, static_cast<uint32_t>(nq), 256, smem, part, per_query, k, cap, out, slot_written, slot_keys);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// routing
// ---------------------------------------------------------------------------------------------
// out[0] = sqrt(max_j sq[j]); one CTA.
__global__ void __launch_bounds__(256)
max_row_norm_kernel(const float* __restrict__ sq, uint32_t n, float* __restrict__ out) {
    __shared__ float part[8];
    float m = 0.f;
    for (uint32_t j = threadIdx.x; j < n; j += blockDim.x) {
        m = fmaxf(m, sq[j]);
    }
    for (int off = 16; off > 0; off >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    }
    if ((threadIdx.x & 31) == 0) {
        part[threadIdx.x >> 5] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            m = fmaxf(m, part[w]);
        }
        out[0] = sqrtf(m);
    }
}

// Block-wide helpers for the two routing kernels below (256 threads).
constexpr int ROUTE_THREADS = 256;

__device__ __forceinline__ float
route_block_min(float v, float* red) {
    for (int off = 16; off > 0; off >>= 1) {
        v = fminf(v, __shfl_xor_sync(0xffffffffu, v, off));
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
        red[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < ROUTE_THREADS / 32; ++w) {
        m = fminf(m, red[w]);
    }
    return m;
}

__device__ __forceinline__ float
route_block_max(float v, float* red) {
    return -route_block_min(-v, red);
}

// Given hist[256] and a 1-based rank, finds the bin the rank-th smallest element falls into and the
// rank it has inside that bin (warp 0 computes, everyone gets the result after the barriers).
__device__ __forceinline__ void
route_find_bin(const uint32_t* hist, uint32_t rank, uint32_t* s_bin, uint32_t* s_rank_in_bin) {
    __syncthreads();
    if (threadIdx.x < 32) {
        const uint32_t lane = threadIdx.x;
        uint32_t local[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            local[i] = hist[lane * 8 + i];
            sum += local[i];
        }
        uint32_t incl = sum;
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= static_cast<uint32_t>(off)) {
                incl += v;
            }
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        const uint32_t want = rank < total ? rank : total;   // fewer elements than the rank: the last one
        uint32_t run = incl - sum;
        if (want > run && want <= incl) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (want > run && want <= run + local[i]) {
                    *s_bin = lane * 8 + i;
                    *s_rank_in_bin = want - run;
                }
                run += local[i];
            }
        }
        if (total == 0 && lane == 0) {
            *s_bin = 0;
            *s_rank_in_bin = 0;
        }
    }
    __syncthreads();
}

// thr[q] = a score that at least ncand of query q's `sample` approximate scores (scores[q][0 .. sample))
// do not exceed -- one of those scores, at most a few ranks above the ncand-th smallest -- plus a margin
// of 1e-3 |q| max|c| that covers the rounding of the tensor-core scores on both sides: at least ncand
// centroids score below it exactly, so every one of the query's ncand nearest centroids scores below
// it approximately.  One CTA per query: two rounds of a 256-bin histogram over the range of the scores
// still in question (bins follow the values' own range, so a narrow spread does not pile them into one
// bin), then the largest score of the bins taken.
// ROUTE_THR_PER_THREAD: scores a thread holds, sample / ROUTE_THREADS rounded up (sample <= 4096).
template <int ROUTE_THR_PER_THREAD>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_threshold_kernel(const float* __restrict__ scores, uint32_t sample, uint32_t ncand, const float* __restrict__ queries,
                       uint32_t dim, const float* __restrict__ c_max_norm, float* __restrict__ thr) {
    __shared__ uint32_t hist[256];
    __shared__ float red[ROUTE_THREADS / 32];
    __shared__ uint32_t s_bin, s_rank;
    const uint64_t q = blockIdx.x;
    const uint32_t tid = threadIdx.x;
    float v[ROUTE_THR_PER_THREAD];
    uint8_t bin1[ROUTE_THR_PER_THREAD];
    float mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_THR_PER_THREAD; ++i) {
        const uint32_t c = tid + i * ROUTE_THREADS;
        const float x = c < sample ? __ldg(scores + q * sample + c) : NAN;
        v[i] = x;
        if (x == x) {   // NaN scores take no part
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
    }
    float qq = 0.f;
    for (uint32_t d = tid; d < dim; d += ROUTE_THREADS) {
        const float x = __ldg(queries + q * dim + d);
        qq = fmaf(x, x, qq);
    }
    // sum of the per-thread partial norms
    for (int off = 16; off > 0; off >>= 1) {
        qq += __shfl_xor_sync(0xffffffffu, qq, off);
    }
    __shared__ float s_qq[ROUTE_THREADS / 32];
    if ((tid & 31) == 0) {
        s_qq[tid >> 5] = qq;
    }
    mn = route_block_min(mn, red);
    mx = route_block_max(mx, red);
    float bound = mx;   // everything, when the scores do not spread (or there are fewer than ncand of them)
    if (mx > mn && mx < INFINITY && mn > -INFINITY) {
        // first pass: bins over [mn, mx]
        hist[tid] = 0;
        __syncthreads();
        const float scale1 = 255.0f / (mx - mn);
#pragma unroll
        for (int i = 0; i < ROUTE_THR_PER_THREAD; ++i) {
            uint32_t b = 255;
            if (v[i] == v[i]) {
                const float t = (v[i] - mn) * scale1;
                b = t >= 255.0f ? 255u : static_cast<uint32_t>(t);
                atomicAdd(&hist[b], 1u);
            }
            bin1[i] = static_cast<uint8_t>(b);
        }
        route_find_bin(hist, ncand, &s_bin, &s_rank);
        const uint32_t b1 = s_bin, rank2 = s_rank;
        // second pass: the scores of bin b1 alone, over their own range
        float mn2 = INFINITY, mx2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < ROUTE_THR_PER_THREAD; ++i) {
            if (v[i] == v[i] && bin1[i] == b1) {
                mn2 = fminf(mn2, v[i]);
                mx2 = fmaxf(mx2, v[i]);
            }
        }
        mn2 = route_block_min(mn2, red);
        mx2 = route_block_max(mx2, red);
        float pick = -INFINITY;   // the largest score taken from bin b1
        if (mx2 > mn2) {
            hist[tid] = 0;
            __syncthreads();
            const float scale2 = 255.0f / (mx2 - mn2);
            uint8_t bin2[ROUTE_THR_PER_THREAD];
#pragma unroll
            for (int i = 0; i < ROUTE_THR_PER_THREAD; ++i) {
                bin2[i] = 255;
                if (v[i] == v[i] && bin1[i] == b1) {
                    const float t = (v[i] - mn2) * scale2;
                    const uint32_t b = t >= 255.0f ? 255u : static_cast<uint32_t>(t);
                    bin2[i] = static_cast<uint8_t>(b);
                    atomicAdd(&hist[b], 1u);
                }
            }
            route_find_bin(hist, rank2, &s_bin, &s_rank);
            const uint32_t b2 = s_bin;
#pragma unroll
            for (int i = 0; i < ROUTE_THR_PER_THREAD; ++i) {
                if (v[i] == v[i] && bin1[i] == b1 && bin2[i] <= b2) {
                    pick = fmaxf(pick, v[i]);
                }
            }
        } else {
            pick = mx2;   // the bin holds one value (possibly many times)
        }
        bound = route_block_max(pick, red);
    }
    if (tid == 0) {
        float total = 0.f;
        for (int w = 0; w < ROUTE_THREADS / 32; ++w) {
            total += s_qq[w];
        }
        thr[q] = bound + 1e-3f * sqrtf(total) * __ldg(c_max_norm);
    }
}

// Exact routing distance of a query (in shared memory) to one centroid: L2 as an FMA chain of (q-c)^2 over the
// dimensions ascending, IP as 1 - the chain of q*c (the loop of IVF::route_buckets_only,
// src/algorithm/ivf/ivf.cpp:1589-1660).
__device__ __forceinline__ float
route_exact_score(const float* __restrict__ qs, const float* __restrict__ c, uint32_t dim, int metric) {
    float s = 0.f;
    if ((dim & 3u) == 0) {   // centroid rows are then 16-byte aligned: four dimensions per load, several loads in flight
        const float4* c4 = reinterpret_cast<const float4*>(c);
        const float4* q4 = reinterpret_cast<const float4*>(qs);
        if (metric == VB200_METRIC_L2) {
#pragma unroll 8
            for (uint32_t d4 = 0; d4 < (dim >> 2); ++d4) {
                const float4 cv = __ldg(c4 + d4), qv = q4[d4];
                float t = __fsub_rn(qv.x, cv.x);
                s = fmaf(t, t, s);
                t = __fsub_rn(qv.y, cv.y);
                s = fmaf(t, t, s);
                t = __fsub_rn(qv.z, cv.z);
                s = fmaf(t, t, s);
                t = __fsub_rn(qv.w, cv.w);
                s = fmaf(t, t, s);
            }
        } else {
#pragma unroll 8
            for (uint32_t d4 = 0; d4 < (dim >> 2); ++d4) {
                const float4 cv = __ldg(c4 + d4), qv = q4[d4];
                s = fmaf(qv.x, cv.x, s);
                s = fmaf(qv.y, cv.y, s);
                s = fmaf(qv.z, cv.z, s);
                s = fmaf(qv.w, cv.w, s);
            }
            s = __fsub_rn(1.0f, s);
        }
    } else if (metric == VB200_METRIC_L2) {
        for (uint32_t d = 0; d < dim; ++d) {
            const float t = __fsub_rn(qs[d], __ldg(c + d));
            s = fmaf(t, t, s);
        }
    } else {
        for (uint32_t d = 0; d < dim; ++d) {
            s = fmaf(qs[d], __ldg(c + d), s);
        }
        s = __fsub_rn(1.0f, s);
    }
    return s;
}

// Four such distances at once (each chain in the same order as route_exact_score): the four chains' loads and
// FMAs interleave, which a thread working through them one after the other cannot do.  c[j] null: +inf.
__device__ __forceinline__ void
route_exact_score4(const float* __restrict__ qs, const float* const (&c)[4], uint32_t dim, int metric, float (&out)[4]) {
    if ((dim & 3u) != 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[j] = c[j] != nullptr ? route_exact_score(qs, c[j], dim, metric) : INFINITY;
        }
        return;
    }
    const float4* q4 = reinterpret_cast<const float4*>(qs);
    const float* safe = c[0] != nullptr ? c[0] : (c[1] != nullptr ? c[1] : (c[2] != nullptr ? c[2] : c[3]));
    const float4* c4[4];
    float s[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        c4[j] = reinterpret_cast<const float4*>(c[j] != nullptr ? c[j] : safe);
        s[j] = 0.f;
    }
    if (safe == nullptr) {
        out[0] = out[1] = out[2] = out[3] = INFINITY;
        return;
    }
#pragma unroll 4
    for (uint32_t d4 = 0; d4 < (dim >> 2); ++d4) {
        const float4 qv = q4[d4];
        float4 cv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            cv[j] = __ldg(c4[j] + d4);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (metric == VB200_METRIC_L2) {
                float t = __fsub_rn(qv.x, cv[j].x);
                s[j] = fmaf(t, t, s[j]);
                t = __fsub_rn(qv.y, cv[j].y);
                s[j] = fmaf(t, t, s[j]);
                t = __fsub_rn(qv.z, cv[j].z);
                s[j] = fmaf(t, t, s[j]);
                t = __fsub_rn(qv.w, cv[j].w);
                s[j] = fmaf(t, t, s[j]);
            } else {
                s[j] = fmaf(qv.x, cv[j].x, s[j]);
                s[j] = fmaf(qv.y, cv[j].y, s[j]);
                s[j] = fmaf(qv.z, cv[j].z, s[j]);
                s[j] = fmaf(qv.w, cv[j].w, s[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        out[j] = c[j] == nullptr ? INFINITY : (metric == VB200_METRIC_L2 ? s[j] : __fsub_rn(1.0f, s[j]));
    }
}

// One CTA per query: gathers the query's centroids below its threshold from their lists, takes the
// ncand best by approximate score, re-scores them exactly -- L2: FMA chain of (q-c)^2 over d
// ascending; IP: 1 - chain of q*c (the loop of IVF::route_buckets_only,
// src/algorithm/ivf/ivf.cpp:1589-1660) -- and writes the nprobe nearest, distance ascending, lower
// list id first on ties.  The ncand best come from a histogram over the candidates' score range (the bin
// that holds the ncand-th and everything below it, a few more than ncand keys), sorted as 64-bit keys so
// that equal scores keep the lower list id; only if that set does not fit the small sort buffer (a
// pile of equal scores) are all candidates sorted.
// Bitonic sort of 32 * R keys held R per lane (element e = 32 * r + lane lives in key[r] of lane e % 32):
// compare-exchanges inside a lane when the partner is 32 or more elements away, shuffles otherwise; ascending.
template <int R>
__device__ __forceinline__ void
warp_sort_registers(uint64_t (&key)[R], uint32_t lane) {
#pragma unroll
    for (uint32_t size = 2; size <= 32u * R; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 32) {
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
                    const bool lower = (lane & stride) == 0;
                    const bool take_min = lower == up;
                    key[r] = take_min ? (mine < other ? mine : other) : (mine > other ? mine : other);
                }
            }
        }
    }
}

// buf[0 .. 32 R) sorted ascending through registers (one warp).
template <int R>
__device__ __noinline__ void
warp_sort_buffer(uint64_t* buf, uint32_t lane) {
    uint64_t key[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        key[r] = buf[r * 32 + lane];
    }
    warp_sort_registers<R>(key, lane);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        buf[r * 32 + lane] = key[r];
    }
    __syncwarp();
}

// route_pick_kernel for the common case, one warp per query and no block-wide barrier: a query whose lists hold at
// most 512 candidates (288 expected for nprobe 64) has them sorted through registers, the
// ncand <= 128 best re-scored exactly, one chain per lane, and sorted again.  handled[q] = 1 tells route_pick_kernel
// (launched afterwards over all queries) to leave the query alone.
constexpr uint32_t ROUTE_WARP_KEYS = 512;

__global__ void __launch_bounds__(256, 5)   // 40 warps per SM: the sort's registers just fit
route_pick_warp_kernel(const float* __restrict__ queries, uint64_t nq, uint32_t dim, const float* __restrict__ centroids,
                       const uint64_t* __restrict__ lists_keys, const uint32_t* __restrict__ lists_cnt, uint32_t lists,
                       uint32_t cap, uint32_t ncand, uint32_t nprobe, int metric, int32_t* __restrict__ probes,
                       float* __restrict__ probe_dists, uint8_t* __restrict__ handled) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t q = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
    if (q >= nq) {
        return;
    }
    uint64_t* buf = reinterpret_cast<uint64_t*>(smem_raw) + static_cast<size_t>(warp) * ROUTE_WARP_KEYS;
    float* qs = reinterpret_cast<float*>(reinterpret_cast<uint64_t*>(smem_raw) + static_cast<size_t>(blockDim.x >> 5) * ROUTE_WARP_KEYS) +
                static_cast<size_t>(warp) * dim;
    // exclusive prefix of the (clamped) list counts, two lists per lane
    const uint32_t l0 = 2 * lane, l1 = 2 * lane + 1;
    uint32_t c0 = l0 < lists ? lists_cnt[q * lists + l0] : 0u;
    uint32_t c1 = l1 < lists ? lists_cnt[q * lists + l1] : 0u;
    const bool lost = __any_sync(0xffffffffu, c0 > cap || c1 > cap);   // a list overflowed: route_pick_kernel's business
    c0 = c0 < cap ? c0 : cap;
    c1 = c1 < cap ? c1 : cap;
    uint32_t incl = c0 + c1;
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= static_cast<uint32_t>(off)) {
            incl += v;
        }
    }
    const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
    if (lost || total > ROUTE_WARP_KEYS || total < ncand) {   // (fewer than ncand: the threshold came out too low)
        if (lane == 0) {
            handled[q] = 0;
        }
        return;
    }
    const uint32_t before = incl - c0 - c1;
    for (uint32_t d = lane; d < dim; d += 32) {
        qs[d] = queries[q * dim + d];
    }
    for (uint32_t i = total + lane; i < ROUTE_WARP_KEYS; i += 32) {
        buf[i] = KEY_INF;
    }
    // every lane copies its two lists (short: a few entries each)
    {
        const uint64_t* src0 = lists_keys + (q * lists + l0) * cap;
        for (uint32_t i = 0; i < c0; ++i) {
            buf[before + i] = src0[i];
        }
        const uint64_t* src1 = lists_keys + (q * lists + l1) * cap;
        for (uint32_t i = 0; i < c1; ++i) {
            buf[before + c0 + i] = src1[i];
        }
    }
    __syncwarp();
    // Only the ncand best are wanted, so most of the keys need no sorting: a pivot from a 32-key sample -- the key
    // at 1.6 times the rank that would cut off ncand, plus two -- is counted against all keys, and when between
    // ncand and 256 keys lie at or below it those alone are compacted to the front and sorted.  The set of the
    // ncand smallest is the same either way (keys are distinct: the list id is their low word).
    uint32_t n_keys = total;
    if (total > 128) {
        uint64_t sample[1] = {buf[(lane * total) >> 5]};
        warp_sort_registers<1>(sample, lane);
        uint32_t r = (ncand * 32u * 8u / 5u) / total + 2u;
        r = r > 31u ? 31u : r;
        const uint64_t pivot = __shfl_sync(0xffffffffu, sample[0], r);
        uint32_t below = 0;
        for (uint32_t i = lane; i < ROUTE_WARP_KEYS; i += 32) {
            below += __popc(__ballot_sync(0xffffffffu, i < total && buf[i] <= pivot));
        }
        if (below >= ncand && below <= 256) {
            uint32_t cnt = 0;
            for (uint32_t i = lane; i < ROUTE_WARP_KEYS; i += 32) {   // all lanes take the same number of trips
                const uint64_t key = i < total ? buf[i] : KEY_INF;
                const bool keep = key <= pivot && i < total;
                const uint32_t mask = __ballot_sync(0xffffffffu, keep);
                __syncwarp();
                if (keep) {
                    buf[cnt + __popc(mask & ((1u << lane) - 1u))] = key;   // at or before its own place
                }
                cnt += __popc(mask);
                __syncwarp();
            }
            const uint32_t pad = cnt <= 128 ? 128u : 256u;
            for (uint32_t i = cnt + lane; i < pad; i += 32) {
                buf[i] = KEY_INF;
            }
            __syncwarp();
            n_keys = cnt;
        }
    }
    if (n_keys <= 128) {
        warp_sort_buffer<4>(buf, lane);
    } else if (n_keys <= 256) {
        warp_sort_buffer<8>(buf, lane);
    } else {
        warp_sort_buffer<16>(buf, lane);
    }
    // exact distances of the ncand best by approximate score, one chain per lane, dimensions ascending
    uint64_t exact[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t e = r * 32 + lane;
        uint64_t mine = KEY_INF;
        if (e < ncand && e < n_keys) {
            const uint32_t list = static_cast<uint32_t>(buf[e]);
            const float s = route_exact_score(qs, centroids + static_cast<uint64_t>(list) * dim, dim, metric);
            mine = make_key(s, list);
        }
        exact[r] = mine;
    }
    warp_sort_registers<4>(exact, lane);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t i = r * 32 + lane;
        if (i < nprobe) {
            const uint64_t key = exact[r];
            const uint64_t o = q * nprobe + i;
            probes[o] = key == KEY_INF ? -1 : static_cast<int32_t>(static_cast<uint32_t>(key));
            if (probe_dists != nullptr) {
                probe_dists[o] = key == KEY_INF ? INFINITY : ordered_to_float(static_cast<uint32_t>(key >> 32));
            }
        }
    }
    if (lane == 0) {
        handled[q] = 1;
    }
}

constexpr uint32_t ROUTE_PICK_SMALL = 512;   // keys the small sort takes

// One query (q) by the whole CTA.
__device__ __forceinline__ void
route_pick_one(const uint64_t q, const float* __restrict__ queries, uint32_t dim, const float* __restrict__ centroids,
               const uint64_t* __restrict__ lists_keys, const uint32_t* __restrict__ lists_cnt, uint32_t lists,
               uint32_t cap, uint32_t ncand, uint32_t nprobe, int metric, int32_t* __restrict__ probes,
               float* __restrict__ probe_dists, uint32_t nlist) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ uint32_t s_off[65];
    __shared__ uint32_t s_lost, s_state[3];
    __shared__ uint32_t hist[256];
    __shared__ float red[ROUTE_THREADS / 32];
    __shared__ uint32_t s_bin, s_rank, s_taken;
    const uint32_t slots = next_pow2(lists * cap > ROUTE_PICK_SMALL ? lists * cap : ROUTE_PICK_SMALL);
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);   // [slots] gathered candidates
    uint64_t* small = keys + slots;                            // [ROUTE_PICK_SMALL]
    float* qs = reinterpret_cast<float*>(small + ROUTE_PICK_SMALL);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (uint32_t d = tid; d < dim; d += blockDim.x) {
        qs[d] = queries[q * dim + d];
    }
    if (tid < 32) {
        // exclusive prefix of the (clamped) list counts, two lists per lane
        const uint32_t l0 = 2 * tid, l1 = 2 * tid + 1;
        uint32_t c0 = l0 < lists ? lists_cnt[q * lists + l0] : 0u;
        uint32_t c1 = l1 < lists ? lists_cnt[q * lists + l1] : 0u;
        const bool lost = __any_sync(0xffffffffu, c0 > cap || c1 > cap);
        if (tid == 0) {
            s_lost = lost ? 1u : 0u;
        }
        c0 = c0 < cap ? c0 : cap;
        c1 = c1 < cap ? c1 : cap;
        uint32_t incl = c0 + c1;
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
            if (tid >= static_cast<uint32_t>(off)) {
                incl += v;
            }
        }
        const uint32_t before = incl - c0 - c1;
        if (l0 < lists) {
            s_off[l0] = before;
        }
        if (l1 < lists) {
            s_off[l1] = before + c0;
        }
        if (tid == 31) {
            s_off[lists] = incl;
        }
        if (tid == 0) {
            s_taken = 0;
        }
    }
    __syncthreads();
    if (s_lost != 0 || s_off[lists] < ncand) {
        // One of the query's lists overflowed (its scores lie far from what the centroid sample predicted), so
        // candidates were lost -- or the threshold came out so low that fewer than ncand centroids passed.  The query is answered from scratch instead: exact distances to every centroid,
        // the nprobe nearest kept by a streaming selection.  Rare, and decided here, so the host never has to
        // wait for the candidate pass to know.
        BlockSelect sel;
        sel.init(keys, s_state, nprobe, next_pow2(nprobe + blockDim.x));
        // four centroids per thread and trip, so four chains of loads and FMAs are in flight at once
        for (uint32_t base = 0; base < nlist; base += 4 * blockDim.x) {
            float sc[4];
            const float* rows[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t c = base + j * blockDim.x + tid;
                rows[j] = c < nlist ? centroids + static_cast<uint64_t>(c) * dim : nullptr;
            }
            route_exact_score4(qs, rows, dim, metric, sc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t c = base + j * blockDim.x + tid;
                sel.make_room(blockDim.x);
                const uint64_t bound = sel.threshold();
                if (c < nlist) {
                    sel.offer(make_key(sc[j], c), bound);
                }
            }
        }
        const uint32_t found = sel.finish();
        for (uint32_t i = tid; i < nprobe; i += blockDim.x) {
            const uint64_t key = i < found ? keys[i] : KEY_INF;
            const uint64_t o = q * nprobe + i;
            probes[o] = key == KEY_INF ? -1 : static_cast<int32_t>(static_cast<uint32_t>(key));
            if (probe_dists != nullptr) {
                probe_dists[o] = key == KEY_INF ? INFINITY : ordered_to_float(static_cast<uint32_t>(key >> 32));
            }
        }
        return;
    }
    const uint32_t total = s_off[lists];
    float mn = INFINITY, mx = -INFINITY;
    for (uint32_t l = warp; l < lists; l += blockDim.x >> 5) {
        const uint32_t beg = s_off[l], c = s_off[l + 1] - beg;
        const uint64_t* src = lists_keys + (q * lists + l) * cap;
        for (uint32_t i = lane; i < c; i += 32) {
            const uint64_t key = src[i];
            keys[beg + i] = key;
            const float sc = ordered_to_float(static_cast<uint32_t>(key >> 32));
            mn = fminf(mn, sc);
            mx = fmaxf(mx, sc);
        }
    }
    mn = route_block_min(mn, red);
    mx = route_block_max(mx, red);
    uint32_t n_small = 0;
    bool use_small = false;
    if (total > ncand && mx > mn) {
        hist[tid] = 0;
        __syncthreads();
        const float scale = 255.0f / (mx - mn);
        for (uint32_t i = tid; i < total; i += blockDim.x) {
            const float t = (ordered_to_float(static_cast<uint32_t>(keys[i] >> 32)) - mn) * scale;
            atomicAdd(&hist[t >= 255.0f ? 255u : static_cast<uint32_t>(t)], 1u);
        }
        route_find_bin(hist, ncand, &s_bin, &s_rank);
        const uint32_t b_last = s_bin;
        for (uint32_t i = tid; i < total; i += blockDim.x) {
            const uint64_t key = keys[i];
            const float t = (ordered_to_float(static_cast<uint32_t>(key >> 32)) - mn) * scale;
            const uint32_t b = t >= 255.0f ? 255u : static_cast<uint32_t>(t);
            if (b <= b_last) {
                const uint32_t at = atomicAdd(&s_taken, 1u);
                if (at < ROUTE_PICK_SMALL) {
                    small[at] = key;
                }
            }
        }
        __syncthreads();
        n_small = s_taken;
        use_small = n_small <= ROUTE_PICK_SMALL;
    }
    uint64_t* sorted = keys;
    uint32_t n_sorted;
    if (use_small) {
        n_sorted = next_pow2(n_small < 2 ? 2 : n_small);
        for (uint32_t i = n_small + tid; i < n_sorted; i += blockDim.x) {
            small[i] = KEY_INF;
        }
        block_bitonic_sort(small, n_sorted);
        sorted = small;
    } else {
        n_sorted = next_pow2(total < 2 ? 2 : total);
        for (uint32_t i = total + tid; i < n_sorted; i += blockDim.x) {
            keys[i] = KEY_INF;
        }
        block_bitonic_sort(keys, n_sorted);
    }
    // exact distances of the ncand best (one chain per candidate, dimensions in ascending order)
    const uint32_t m2 = next_pow2(ncand < 2 ? 2 : ncand);
    uint64_t mine = KEY_INF;
    if (tid < ncand && tid < n_sorted && sorted[tid] != KEY_INF) {
        const uint32_t list = static_cast<uint32_t>(sorted[tid]);
        const float s = route_exact_score(qs, centroids + static_cast<uint64_t>(list) * dim, dim, metric);
        mine = make_key(s, list);
    }
    __syncthreads();
    if (tid < m2) {
        small[tid] = mine;
    }
    block_bitonic_sort(small, m2);
    for (uint32_t i = tid; i < nprobe; i += blockDim.x) {
        const uint64_t key = i < m2 ? small[i] : KEY_INF;
        const uint64_t o = q * nprobe + i;
        probes[o] = key == KEY_INF ? -1 : static_cast<int32_t>(static_cast<uint32_t>(key));
        if (probe_dists != nullptr) {
            probe_dists[o] = key == KEY_INF ? INFINITY : ordered_to_float(static_cast<uint32_t>(key >> 32));
        }
    }
}

// A CTA takes `per_block` consecutive queries one after the other and passes over those route_pick_warp_kernel
// answered (handled[q] != 0): nearly all of them, which is why the queries are not given a CTA each.
__global__ void __launch_bounds__(ROUTE_THREADS)
route_pick_kernel(const float* __restrict__ queries, uint64_t nq, uint32_t per_block, uint32_t dim,
                  const float* __restrict__ centroids, const uint64_t* __restrict__ lists_keys,
                  const uint32_t* __restrict__ lists_cnt, uint32_t lists, uint32_t cap, uint32_t ncand, uint32_t nprobe,
                  int metric, int32_t* __restrict__ probes, float* __restrict__ probe_dists,
                  const uint8_t* __restrict__ handled, uint32_t nlist) {
    for (uint32_t i = 0; i < per_block; ++i) {
        const uint64_t q = static_cast<uint64_t>(blockIdx.x) * per_block + i;
        if (q >= nq) {
            return;
        }
        if (handled != nullptr && handled[q] != 0) {
            continue;
        }
        __syncthreads();   // the previous query's shared memory is no longer read
        route_pick_one(q, queries, dim, centroids, lists_keys, lists_cnt, lists, cap, ncand, nprobe, metric, probes, probe_dists,
                       nlist);
    }
}

// The workspace's scalar block, zeroed when it is first allocated (entry 8, the routing passes' flag, is read at
// the end of every search whether or not that search routed).
static int
reserve_scalars(SearchWorkspace& ws) {
    if (ws.scalars.cap >= SCALARS) {
        return 0;
    }
    VB_TRY(ws.scalars.reserve(SCALARS));
    VB_CUDA(cudaMemsetAsync(ws.scalars.ptr, 0, SCALARS * sizeof(uint64_t), current_stream()));
    return 0;
}

// After a synchronisation: fails if a tensor-core routing pass of the call reported a wait that gave up.
static int
route_flag_check(uint64_t flag_word) {
    if ((flag_word & 1u) != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "tensor-core kernel gave up on a bounded wait");
    }
    return 0;
}

// For callers that only route: waits for the stream and reads the flag.
static int
route_sync_and_check(SearchWorkspace& ws) {
    uint64_t word = 0;
    VB_CUDA(cudaMemcpyAsync(&word, ws.scalars.ptr + 8, sizeof(word), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    return route_flag_check(word);
}

static int
ivf_route_device(vb200_ivf* ix, const float* q_dev, uint64_t nq, uint32_t nprobe, int32_t* probes_dev,
                 float* dists_dev) {
    SearchWorkspace& ws = ix->ws;
    VB_TRY(reserve_scalars(ws));
    int* route_flag = reinterpret_cast<int*>(ws.scalars.ptr + 8);
    VB_CUDA(cudaMemsetAsync(route_flag, 0, sizeof(uint64_t), current_stream()));
    const uint32_t nlist = ix->nlist;
    uint32_t ncand = nprobe + ROUTE_SLACK < nlist ? nprobe + ROUTE_SLACK : nlist;
    VB_CHECK_ARG(ncand <= 1024, "scan_buckets_count %u is too large (limit %u)", nprobe,
                 1024 - ROUTE_SLACK);
    VB_TRY(ws.cand.reserve(nq * ncand));
    const bool l2 = ix->metric == VB200_METRIC_L2;
    const uint64_t ld = (static_cast<uint64_t>(nlist) + 3) / 4 * 4;
    if (tensor_cores_enabled() && nq >= 256 && nlist >= 1024 && nq * ld <= (uint64_t{1} << 30)) {
        // Scores from the tcgen05 kernel (split-bf16, good to ~1e-5 relative) nominate the
        // candidates; the exact re-scoring below orders them and drops the slack, as on the
        // SIMT path.
        const uint32_t chunks = (ix->dim + TC_KC - 1) / TC_KC;
        if (!ix->c_tiled) {
            const size_t elems = tc_tiled_elems(nlist, ix->dim);
            VB_TRY(ix->c_hi.reserve(elems));
            VB_TRY(ix->c_lo.reserve(elems));
            VB_TRY(tc_pretile_f32(ix->centroids.ptr, nlist, ix->dim, ix->c_hi.ptr, ix->c_lo.ptr));
            VB_TRY(ix->c_max_norm.reserve(1));
            VB_LAUNCH(max_row_norm_kernel, 1, 256, 0, ix->c_sq.ptr, nlist, ix->c_max_norm.ptr);
            ix->c_tiled = true;
        }
        const size_t q_elems = tc_tiled_elems(nq, ix->dim);
        VB_TRY(ws.q_hi.reserve(q_elems));
        VB_TRY(ws.q_lo.reserve(q_elems));
        VB_TRY(tc_pretile_f32(q_dev, nq, ix->dim, ws.q_hi.ptr, ws.q_lo.ptr));
        TcOperand a{ws.q_hi.ptr, ws.q_lo.ptr, nq, chunks};
        TcOperand b{ix->c_hi.ptr, ix->c_lo.ptr, nlist, chunks};
        // Large list counts: no score matrix.  The scores against a sample of the centroids (the first
        // `sample` of them; centroid numbering carries no geometry) give each query a threshold; one pass
        // of the tensor-core kernel over all centroids then keeps, unsorted, only what scores below it --
        // about rank * nlist / sample per query -- and one small kernel per query orders those and
        // re-scores the best exactly.
        // The threshold is the score of rank `rank` in the sample, chosen so that about four times ncand
        // centroids are expected below it.  With rank = ncand that many are certain; with a smaller sample
        // and a lower rank they are only very likely, and a query that ends up with fewer than ncand is
        // answered exactly by route_pick_kernel like one whose lists overflowed.
        uint32_t sample = 0, rank = 0;
        for (uint32_t s = 1024; s <= 4096 && sample == 0; s *= 2) {
            uint64_t r = (4ull * ncand * s + nlist - 1) / nlist;   // (3x and 5x measured slower: exact fallbacks, longer sorts)
            r = r < 16 ? 16 : r;
            r = r > ncand ? ncand : r;
            const uint64_t expected = r * nlist / s;
            if (4ull * s <= nlist && s >= 4 * ncand && 5 * expected / 2 <= ROUTE_MAX_PER_ROW) {
                sample = s;
                rank = static_cast<uint32_t>(r);
            }
        }
        if (sample != 0 && ncand <= 256) {
            const float alpha = l2 ? -2.0f : -1.0f;
            const float* bias = l2 ? ix->c_sq.ptr : nullptr;
            TcOperand bs{ix->c_hi.ptr, ix->c_lo.ptr, sample, chunks};
            VB_TRY(ws.scores.reserve(nq * sample));
            // No wait for either tensor-core pass: what they report (a bounded wait that gave up) is OR-ed into
            // ws.scalars[8], which every caller reads when it synchronises at the end of its call; a query whose
            // candidate lists overflowed is answered exactly by route_pick_kernel itself.
            VB_TRY(tc_scores(ix->tc, a, bs, 3, alpha, bias, ws.scores.ptr, sample, route_flag));
            VB_TRY(ws.route_thr.reserve(nq));
            auto thr_kernel = sample <= 4 * ROUTE_THREADS ? route_threshold_kernel<4>
                                                          : (sample <= 8 * ROUTE_THREADS ? route_threshold_kernel<8> : route_threshold_kernel<16>);
            VB_LAUNCH(thr_kernel, static_cast<uint32_t>(nq), ROUTE_THREADS, 0, ws.scores.ptr, sample, rank,
                      q_dev, ix->dim, ix->c_max_norm.ptr, ws.route_thr.ptr);
            uint32_t lists = 0, cap = 0;
            bool overflow = false;
            const uint32_t expected = static_cast<uint32_t>(static_cast<uint64_t>(rank) * nlist / sample);
            const uint32_t n_keep = next_pow2(nprobe + ROUTE_THREADS);   // the exact fallback's selection buffer
            VB_TRY(tc_below_threshold(ix->tc, a, b, 3, alpha, bias, ws.route_thr.ptr, expected, ROUTE_MAX_PER_ROW,
                                      ws.route_keys, ws.route_cnt, &lists, &cap, &overflow, route_flag));
            if (lists <= 64 && n_keep <= ROUTE_PICK_SMALL) {
                const uint32_t slots = next_pow2(lists * cap > ROUTE_PICK_SMALL ? lists * cap : ROUTE_PICK_SMALL);
                const size_t smem = (static_cast<size_t>(slots) + ROUTE_PICK_SMALL) * sizeof(uint64_t) + ix->dim * sizeof(float);
                if (smem > 48 * 1024) {
                    VB_CUDA(cudaFuncSetAttribute(route_pick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem)));
                }
                // queries with few candidates (nearly all) are answered by a warp each; the block-per-query kernel
                // takes what is left
                const uint8_t* handled = nullptr;
                const size_t warp_smem = 8 * (ROUTE_WARP_KEYS * sizeof(uint64_t) + ix->dim * sizeof(float));
                if (ncand <= 128 && nprobe <= 128 && warp_smem <= 200 * 1024) {
                    VB_TRY(ws.route_handled.reserve(nq));
                    if (warp_smem > 48 * 1024) {
                        VB_CUDA(cudaFuncSetAttribute(route_pick_warp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(warp_smem)));
                    }
                    VB_LAUNCH(route_pick_warp_kernel, static_cast<uint32_t>((nq + 7) / 8), 256, warp_smem, q_dev, nq, ix->dim,
                              ix->centroids.ptr, ws.route_keys.ptr, ws.route_cnt.ptr, lists, cap, ncand, nprobe, ix->metric,
                              probes_dev, dists_dev, ws.route_handled.ptr);
                    handled = ws.route_handled.ptr;
                }
                const uint32_t per_block = handled != nullptr ? 8u : 1u;   // with the warp kernel in front, few queries are left
                VB_LAUNCH(route_pick_kernel, static_cast<uint32_t>((nq + per_block - 1) / per_block), 256, smem, q_dev, nq, per_block,
                          ix->dim, ix->centroids.ptr, ws.route_keys.ptr, ws.route_cnt.ptr, lists, cap, ncand, nprobe, ix->metric,
                          probes_dev, dists_dev, handled, nlist);
                return 0;
            }
            VB_TRY(sync_stream());   // (more lists than the pick kernels take: the score-matrix path below)
        }
        VB_TRY(ws.scores.reserve(nq * ld));
        VB_TRY(tc_scores(ix->tc, a, b, 3, l2 ? -2.0f : -1.0f, l2 ? ix->c_sq.ptr : nullptr, ws.scores.ptr, ld));
        VB_TRY(select_rows(ws.scores.ptr, nq, nlist, ld, ncand, 0, ws.cand.ptr, ncand));
    } else {
        uint64_t slab = (uint64_t{256} << 20) / nlist;  // rows of a 1 GiB score slab
        if (slab < 1) {
            slab = 1;
        }
        if (slab > nq) {
            slab = nq;
        }
        VB_TRY(ws.scores.reserve(slab * nlist));
        for (uint64_t b = 0; b < nq; b += slab) {
            uint64_t n = nq - b < slab ? nq - b : slab;
            VB_TRY(dense_scores_f32(q_dev + b * ix->dim, n, ix->centroids.ptr, nlist, ix->dim,
                                    l2 ? -2.0f : -1.0f, l2 ? ix->c_sq.ptr : nullptr, ws.scores.ptr, nlist));
            VB_TRY(select_rows(ws.scores.ptr, n, nlist, nlist, ncand, 0, ws.cand.ptr + b * ncand, ncand));
        }
    }
    uint32_t n2 = next_pow2(ncand < 2 ? 2 : ncand);
    VB_LAUNCH(route_finalize_kernel, static_cast<uint32_t>(nq), 128, n2 * sizeof(uint64_t) + ix->dim * sizeof(float), q_dev,
              ix->dim, ix->centroids.ptr, ws.cand.ptr, ncand, n2, nprobe, ix->metric, probes_dev,
              dists_dev);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------------------------
// Per-query bounds leave as plain distances (+inf = none yet) so that ranks can take their
// minimum with an ordinary float all-reduce, and come back the same way.
__global__ void
bounds_to_float_kernel(const uint32_t* __restrict__ thr, uint64_t nq, float* __restrict__ bounds) {
    uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (q < nq) {
        const uint32_t u = thr[q];
        bounds[q] = u > float_to_ordered(INFINITY) ? INFINITY : ordered_to_float(u);
    }
}

__global__ void
bounds_from_float_kernel(const float* __restrict__ bounds, uint64_t nq, uint32_t* __restrict__ thr) {
    uint64_t q = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (q < nq) {
        const float b = bounds[q];
        if (b < INFINITY) {   // NaN and +inf carry no information
            const uint32_t u = float_to_ordered(b);
            if (u < thr[q]) {
                thr[q] = u;
            }
        }
    }
}

template <typename Kernel>
static int
launch_scan(Kernel kernel, const ScanParams& p, size_t smem) {
    if (smem > 40 * 1024) {   // the kernels' static shared memory counts against the 48 KiB default too
        VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
    }
    int per_sm = 0;
    VB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SCAN_THREADS, smem));
    if (per_sm < 1) {
        VB_FAIL(VB200_INVALID_ARGUMENT,
                "scan tile needs %zu bytes of shared memory, more than one SM has", smem);
    }
    uint32_t grid = static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(per_sm);
    VB_LAUNCH(kernel, grid, SCAN_THREADS, smem, p);
    return 0;
}

// VB200_SCAN_PROFILE=1: device time of the scan's sections from CUDA events, averaged over 20 calls after the
// first three and printed to stderr (a diagnostic; the events are recorded on the search's stream and read at
// the next call, after that call's own work has been queued behind them).
struct ScanProfile {
    static constexpr int N = 8;
    cudaEvent_t ev[N + 1] = {};
    double acc[N] = {};
    int calls = 0, pending = 0;
    bool on = false, init = false;
    void begin(cudaStream_t st) {
        if (!init) {
            const char* e = std::getenv("VB200_SCAN_PROFILE");
            on = e != nullptr && e[0] == '1';
            init = true;
            if (on) {
                for (auto& x : ev) {
                    cudaEventCreate(&x);
                }
            }
        }
        if (!on) {
            return;
        }
        if (pending > 0 && cudaEventSynchronize(ev[pending]) == cudaSuccess && ++calls > 3) {
            for (int i = 0; i < pending; ++i) {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
                acc[i] += ms;
            }
            if ((calls - 3) % 20 == 0) {
                std::fprintf(stderr, "scan-prof: prep %.3f first %.3f exchange %.3f drop %.3f group %.3f second %.3f merge %.3f tail %.3f ms\n",
                             acc[0] / 20, acc[1] / 20, acc[2] / 20, acc[3] / 20, acc[4] / 20, acc[5] / 20, acc[6] / 20, acc[7] / 20);
                for (auto& a : acc) {
                    a = 0;
                }
            }
        }
        pending = 0;
        cudaEventRecord(ev[0], st);
    }
    void mark(cudaStream_t st) {
        if (on && pending < N) {
            cudaEventRecord(ev[++pending], st);
        }
    }
};
static ScanProfile g_scan_profile;

// Scans the probed lists of every query and leaves, per query, the kscan best as keys
// (payload = inner id) in ws.keys.
static int
ivf_scan_device(vb200_ivf* ix, const float* q_dev, uint64_t nq, uint32_t kfinal, uint32_t nprobe,
                const int32_t* probes_dev, const float* probe_dists_dev) {
    SearchWorkspace& ws = ix->ws;
    const bool sq8 = ix->quant == VB200_QUANT_SQ8;
    // SQ8 ranks with a re-associated distance and re-scores a few more survivors exactly.
    const uint32_t kscan = sq8 ? kfinal + SQ8_SLACK : kfinal;
    const uint32_t nlist = ix->nlist;
    const uint64_t total = nq * nprobe;
    VB_CHECK_ARG(total < 0xFFFFFFFFull, "query batch too large: %llu probes",
                 static_cast<unsigned long long>(total));
    VB_CHECK_ARG(kfinal >= 1 && kscan <= 1024 - SCAN_THREADS, "k = %u out of range [1, %u]", kfinal,
                 1024 - SCAN_THREADS - (sq8 ? SQ8_SLACK : 0));
    const bool flat_rows = ix->quant == VB200_QUANT_FP32 || ix->quant == VB200_QUANT_BF16 || ix->quant == VB200_QUANT_FP16;
    const int qt = ix->quant == VB200_QUANT_SQ8 ? SQ8_QT
                   : (flat_rows ? FP32_QT : (ix->quant == VB200_QUANT_SQ8_UNIFORM ? SQ8U_QT : RABITQ_QT));

    // Phase 0 scans every query's nearest list (of those this shard holds), phase 1 the other
    // probes: after phase 0 the per-query bound is already close to final, so almost nothing
    // enters the buffers later.
    const uint32_t n_phases = nprobe > 1 ? 2 : 1;
    for (uint32_t ph = 0; ph < 2; ++ph) {
        const uint64_t cap_pairs = ph == 0 ? nq : total;
        VB_TRY(ws.pair_off[ph].reserve(nlist + 1));
        VB_TRY(ws.item_off[ph].reserve(nlist + 1));
        VB_TRY(ws.item_map[ph].reserve(cap_pairs));
        VB_TRY(ws.pair_q[ph].reserve(cap_pairs));
        VB_TRY(ws.pair_slot[ph].reserve(cap_pairs));
    }
    VB_TRY(ws.thr.reserve(nq));
    VB_TRY(ws.part.reserve(total * kscan));
    VB_TRY(ws.keys.reserve(nq * kfinal));
    VB_TRY(reserve_scalars(ws));
    if (sq8) {
        VB_TRY(ws.qw.reserve(nq * ix->dpad));
        VB_TRY(ws.qa.reserve(nq));
        VB_TRY(ws.merged.reserve(nq * kscan));
    }
    cudaStream_t st = current_stream();
    g_scan_profile.begin(st);
    VB_CUDA(cudaMemsetAsync(ws.scalars.ptr, 0, 6 * sizeof(uint64_t), st));   // not [6]: the deadline is stamped before routing
    VB_CUDA(cudaMemsetAsync(ws.thr.ptr, 0xFF, nq * sizeof(uint32_t), st));
    if (sq8) {
        // the SQ8 kernels flag the slots they write: one byte per (query, probe) to clear instead of the slots themselves
        VB_TRY(ws.slot_written.reserve(total));
        VB_CUDA(cudaMemsetAsync(ws.slot_written.ptr, 0, total, st));
    } else {
        VB_CUDA(cudaMemsetAsync(ws.part.ptr, 0xFF, total * kscan * sizeof(uint64_t), st));
    }
    const uint32_t blocks = static_cast<uint32_t>((total + 255) / 256);
    VB_TRY(ws.first_live.reserve(nq));
    VB_LAUNCH(first_live_kernel, static_cast<uint32_t>((nq + 255) / 256), 256, 0, probes_dev, nq, nprobe, nlist,
              ix->shard_rank, ix->shard_world, ix->list_off.ptr,
              (ws.exchange != nullptr && ix->shard_world > 1) ? 1 : 0, ws.first_live.ptr);
    VB_TRY(ws.pair_ctr.reserve(4 * static_cast<size_t>(nlist)));
    PairTables tables{};
    for (uint32_t ph = 0; ph < 2; ++ph) {
        tables.cnt[ph] = ws.pair_ctr.ptr + static_cast<size_t>(ph) * nlist;
        tables.cursor[ph] = ws.pair_ctr.ptr + static_cast<size_t>(2 + ph) * nlist;
        tables.off[ph] = ws.pair_off[ph].ptr;
        tables.item_off[ph] = ws.item_off[ph].ptr;
        tables.item_map[ph] = ws.item_map[ph].ptr;
        tables.q[ph] = ws.pair_q[ph].ptr;
        tables.slot[ph] = ws.pair_slot[ph].ptr;
    }
    // Groups the pairs of one phase (0 / 1) or of both (2) by list; `drop` marks pruned pairs.
    auto group_pairs = [&](uint32_t phase_sel, const uint8_t* drop, uint32_t queries_per_item) -> int {
        const int32_t* a_probes = probes_dev;
        uint64_t a_total = total;
        uint32_t a_nprobe = nprobe, a_nlist = nlist, a_rank = ix->shard_rank, a_world = ix->shard_world, a_sel = phase_sel,
                 a_qt = queries_per_item, a_code = ix->code_size;
        const uint32_t* a_first = ws.first_live.ptr;
        const uint32_t* a_off = ix->list_off.ptr;
        const uint32_t* a_goff = ix->group_off.ptr;
        const uint32_t* a_order = ix->scan_order.ptr;
        PairTables a_tables = tables;
        uint32_t* a_ctr = ws.pair_ctr.ptr;
        const uint8_t* a_drop = drop;
        uint64_t* a_scalars = ws.scalars.ptr;
        void* args[] = {&a_probes, &a_total, &a_nprobe, &a_first, &a_nlist, &a_rank, &a_world, &a_off, &a_goff, &a_order,
                        &a_tables, &a_ctr, &a_sel, &a_drop, &a_qt, &a_code, &a_scalars};
        // every CTA of a cooperative launch must be resident: one per SM
        static const bool cooperative_off =
            std::getenv("VB200_GROUP_COOPERATIVE") != nullptr && std::getenv("VB200_GROUP_COOPERATIVE")[0] == '0';
        if (!cooperative_off && !ws.group_by_stages) {
            const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(pair_group_kernel),
                                                              dim3(static_cast<uint32_t>(sm_count())), dim3(1024), args, 0, st);
            if (e == cudaSuccess) {
                g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
                return 0;
            }
            if (e != cudaErrorCooperativeLaunchTooLarge && e != cudaErrorNotSupported) {
                VB_CUDA(e);
            }
            (void)cudaGetLastError();        // the refusal is not an error of this call
            ws.group_by_stages = true;       // this context cannot hold the grid: stage by stage from now on
        }
        VB_CUDA(cudaMemsetAsync(ws.pair_ctr.ptr, 0, 4 * static_cast<size_t>(nlist) * sizeof(uint32_t), st));
        VB_LAUNCH(pair_count_kernel, blocks, 256, 0, probes_dev, total, nprobe, ws.first_live.ptr, nlist, ix->shard_rank,
                  ix->shard_world, ix->list_off.ptr, tables, phase_sel, drop);
        VB_LAUNCH(pair_scan_kernel, 2, 1024, 0, tables, ix->list_off.ptr, ix->scan_order.ptr, nlist, queries_per_item,
                  ix->code_size, ws.scalars.ptr);
        VB_LAUNCH(pair_items_kernel, dim3((nlist + 255) / 256, 2), 256, 0, tables, ix->list_off.ptr, ix->group_off.ptr,
                  ix->scan_order.ptr, nlist, queries_per_item);
        VB_LAUNCH(pair_scatter_kernel, blocks, 256, 0, probes_dev, total, nprobe, ws.first_live.ptr, nlist, ix->shard_rank,
                  ix->shard_world, ix->list_off.ptr, tables, phase_sel, drop);
        return 0;
    };
    // SQ8 with list pruning: the first phase runs alone, then the pairs its bounds rule out are
    // dropped before the second phase is grouped, so they never become work items.
    const bool pruning = sq8 && ix->prune_lists && ix->ball_radius.ptr != nullptr && !ix->use_residual;
    const uint32_t scan_cap = next_pow2(kscan + SCAN_THREADS);
    const bool tc_scan = sq8 && !ix->use_residual && tensor_cores_enabled() && ix->codes_t.ptr != nullptr && ix->kchunks > 0 &&
                         tcs_buffer_cap(kscan) <= 32 * TCS_SELECT_MAX &&
                         tcs_smem_bytes(ix->kchunks, tcs_buffer_cap(kscan), 2) + 4096 <= 227 * 1024;
    const bool split_phases = n_phases == 2 && (ws.exchange != nullptr || pruning);
    // SQ8 work items run on the tensor cores (32 queries per item).  That kernel does not test the lists'
    // covering balls tile by tile as the SIMT kernel does: with list pruning on, the pairs of the second
    // phase have just been tested against the bounds of the first (pair_drop_kernel), which are close to
    // final, and a first phase has no bounds to test against.
    // A first phase that runs alone (pruning on) is a few thousand items of one or two queries: 32-query tiles
    // are nearly empty there and the SIMT kernel's single-query body is the faster one; VB200_TC_FIRST=1 keeps it
    // on the tensor cores (for comparisons).
    static const bool tc_first_forced = std::getenv("VB200_TC_FIRST") != nullptr && std::getenv("VB200_TC_FIRST")[0] == '1';
    const bool tc_first = tc_scan && (!(split_phases && pruning) || tc_first_forced), tc_second = tc_scan;
    // ... and when every item is a single query anyway, a warp per item beats a CTA per item (VB200_WARP_FIRST=0: off)
    static const bool warp_first_off = std::getenv("VB200_WARP_FIRST") != nullptr && std::getenv("VB200_WARP_FIRST")[0] == '0';
    // (the warps rank with the tensor-core scan's integer weight terms when those are prepared anyway, so both
    // phases nominate with one arithmetic; VB200_FIRST_INT8=0: the SIMT scan's fp32 weights instead)
    static const bool first_int8 = !(std::getenv("VB200_FIRST_INT8") != nullptr && std::getenv("VB200_FIRST_INT8")[0] == '0');
    const uint32_t first_dpad32 = (tc_scan && first_int8) ? ix->kchunks * 16 : 0u;
    const bool warp_first = sq8 && split_phases && pruning && !tc_first && !warp_first_off && kscan <= 192 &&
                            sq8_first_smem_bytes(kscan, ix->dpad, first_dpad32) <= 96 * 1024;
    const uint32_t qt_first = warp_first ? 1u : (tc_first ? TCS_QT : static_cast<uint32_t>(qt));
    const uint32_t qt_second = tc_second ? TCS_QT : static_cast<uint32_t>(qt);
    VB_TRY(group_pairs(split_phases ? 0u : 2u, nullptr, qt_first));

    ScanParams p{};
    p.codes = ix->codes.ptr;
    p.code_stride = ix->code_stride;
    p.dim = ix->dim;
    p.dpad = ix->dpad;
    p.list_off = ix->list_off.ptr;
    p.nlist = nlist;
    p.k = kscan;
    p.cap = scan_cap;
    p.thr_g = ws.thr.ptr;
    p.part = ws.part.ptr;
    p.slot_written = sq8 ? ws.slot_written.ptr : nullptr;
    p.queries = q_dev;
    p.qw = ws.qw.ptr;
    p.qa = ws.qa.ptr;
    p.code_norm = ix->code_norm.ptr;
    p.coef_b = ix->metric == VB200_METRIC_L2 ? 1.0f : 0.0f;
    p.coef_c = ix->metric == VB200_METRIC_L2 ? -2.0f : -1.0f;
    p.inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(ix->dim));
    p.qcodes = ws.qcodes.ptr;
    p.qcode_stride = ix->code_stride;
    p.su_lower = ix->su_lower;
    p.su_rate = static_cast<float>((static_cast<double>(ix->su_diff) / 255.0) * (static_cast<double>(ix->su_diff) / 255.0));
    p.metric = ix->metric;
    ws.pruning = sq8 && ix->prune_lists && ix->ball_radius.ptr != nullptr && !ix->use_residual;
    if (sq8 && ix->use_residual) {
        // the covering balls describe decoded residuals, not vectors: no list pruning, SIMT scan only
        VB_TRY(ws.pair_const.reserve(total));
        VB_LAUNCH(pair_const_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, probes_dev, total, nprobe, nlist, q_dev,
                  ix->dim, ix->centroids.ptr, ix->metric, ws.pair_const.ptr);
        p.pair_const = ws.pair_const.ptr;
    }
    if (ws.pruning) {
        p.ball_centre = ix->ball_centre.ptr;
        p.ball_radius = ix->ball_radius.ptr;
        p.ball_count = ix->ball_count.ptr;
    }
    p.scanned = reinterpret_cast<unsigned long long*>(ws.scalars.ptr + 3);
    {
        // id filter: tombstones and / or the caller's filter of this search
        const vb200_filter* f = ws.filter;
        const bool user_deny = f != nullptr && f->deny_inner_bits != nullptr && f->n_inner_bits > 0;
        const bool user_labels = f != nullptr && f->invalid_label_bits != nullptr && f->n_label_bits > 0;
        if (ix->n_removed > 0 || user_deny || user_labels) {
            p.filter_pos_inner = ix->pos_inner.ptr;
            p.labels = ix->labels.ptr;
            if (user_deny) {
                const uint64_t words = (ix->n_total + 31) / 32;
                const uint64_t extra_words = (f->n_inner_bits + 31) / 32;
                DevInput<uint32_t> extra;
                VB_TRY(extra.bind(f->deny_inner_bits, extra_words));
                VB_TRY(ws.deny_bits.reserve(words));
                VB_LAUNCH(deny_merge_kernel, static_cast<uint32_t>((words + 255) / 256), 256, 0, ix->tombstones.ptr,
                          ix->tomb_words, extra.ptr, extra_words, words, ws.deny_bits.ptr);
                VB_TRY(sync_stream());   // `extra` may be a staging copy that ends with this scope
                p.deny_inner_bits = ws.deny_bits.ptr;
            } else if (ix->n_removed > 0) {
                p.deny_inner_bits = ix->tombstones.ptr;
            }
            if (user_labels) {
                const uint64_t words = (f->n_label_bits + 63) / 64;
                VB_TRY(ws.label_bits.reserve(words));
                VB_CUDA(cudaMemcpyAsync(ws.label_bits.ptr, f->invalid_label_bits, words * sizeof(uint64_t),
                                        cudaMemcpyDefault, st));
                p.invalid_label_bits = ws.label_bits.ptr;
                p.n_label_bits = f->n_label_bits;
            }
        }
    }
    if (sq8) {
        const uint32_t dpad32 = ix->kchunks * 16;
        if (tc_scan) {
            VB_TRY(ws.qw8.reserve(nq * 3 * dpad32));
            VB_TRY(ws.qscale.reserve(nq));
        }
        VB_LAUNCH(sq8_query_prep_kernel, static_cast<uint32_t>((nq + 3) / 4), 128, 0, q_dev, nq, ix->dim,
                  ix->dpad, ix->sq_scale.ptr, ix->sq_mid.ptr, ix->metric, ws.qw.ptr, ws.qa.ptr, dpad32,
                  tc_scan ? ws.qw8.ptr : nullptr, tc_scan ? ws.qscale.ptr : nullptr);
    }
    VB_CUDA(cudaEventRecord(ix->ev_scan_begin, st));
    g_scan_profile.mark(st);   // prep
    auto launch_phases = [&](uint32_t first, uint32_t count, uint32_t queue_slot, bool on_tensor_cores,
                             bool warp_items = false) -> int {
        for (uint32_t i = 0; i < 2; ++i) {
            const uint32_t src = i < count ? first + i : first;
            p.pair_off[i] = ws.pair_off[src].ptr;
            p.pair_cnt[i] = tables.cnt[src];
            p.pair_q[i] = ws.pair_q[src].ptr;
            p.pair_slot[i] = ws.pair_slot[src].ptr;
            p.item_off[i] = ws.item_off[src].ptr;
            p.item_map[i] = ws.item_map[src].ptr;
        }
        p.n_phases = count;
        p.item_counter = reinterpret_cast<uint32_t*>(ws.scalars.ptr + queue_slot);
        p.deadline = ws.opt_deadline ? reinterpret_cast<const unsigned long long*>(ws.scalars.ptr + 6) : nullptr;
        p.timed_out = reinterpret_cast<unsigned long long*>(ws.scalars.ptr + 5);
        if (sq8 && on_tensor_cores) {
            TcScanParams tp{};
            tp.s = p;
            tp.s.ball_centre = nullptr;   // this kernel tests no balls
            tp.s.ball_radius = nullptr;
            tp.s.ball_count = nullptr;
            tp.s.cap = tcs_buffer_cap(p.k);   // this kernel's buffers are small: a full one is compacted and the offer retried
            tp.codes_t = ix->codes_t.ptr;
            tp.group_off = ix->group_off.ptr;
            tp.kchunks = ix->kchunks;
            tp.qw8 = ws.qw8.ptr;
            tp.qscale = ws.qscale.ptr;
            tp.count_scanned = ws.pruning ? 1u : 0u;
            tp.spin_limit = tc_spin_limit();
            tp.error_flag = reinterpret_cast<int*>(ws.scalars.ptr + 4);
            // Two CTAs per SM when they fit (each holds 256 of the SM's 512 tensor-memory columns), with as many
            // code tiles in flight as the shared memory left allows; the CTAs are persistent and pull items
            // from one queue, so a CTA that has to wait for a free slot simply finds less work left.
            const size_t sm_bytes = 228 * 1024, reserve = 4096;   // static shared memory and the per-CTA reserve
            uint32_t per_sm = 2, stages = 2;
            if (2 * (tcs_smem_bytes(ix->kchunks, tp.s.cap, 2) + reserve) > sm_bytes) {
                per_sm = 1;
            }
            while (stages < TCS_MAX_STAGES &&
                   per_sm * (tcs_smem_bytes(ix->kchunks, tp.s.cap, stages + 1) + reserve) <= sm_bytes - (per_sm == 1 ? 1024 : 0)) {
                ++stages;
            }
            tp.stages = stages;
            const size_t smem = tcs_smem_bytes(ix->kchunks, tp.s.cap, stages);
#ifdef VB200_TCS_PROFILE
            static DevBuf<unsigned long long> prof_buf;
            VB_TRY(prof_buf.reserve(static_cast<size_t>(sm_count()) * 2 * 24));
            VB_CUDA(cudaMemsetAsync(prof_buf.ptr, 0, static_cast<size_t>(sm_count()) * 2 * 24 * sizeof(unsigned long long), st));
            tp.prof = prof_buf.ptr;
#endif
            auto tc_kernel = ix->kchunks * 16 > 256 ? ivf_sq8_scan_tc_kernel<true> : ivf_sq8_scan_tc_kernel<false>;
            VB_CUDA(cudaFuncSetAttribute(tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            VB_CUDA(cudaFuncSetAttribute(tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared));
            VB_LAUNCH(tc_kernel, static_cast<uint32_t>(sm_count()) * per_sm, TCS_THREADS, smem, tp);
#ifdef VB200_TCS_PROFILE
            {
                const size_t n_cta = static_cast<size_t>(sm_count()) * per_sm;
                std::vector<unsigned long long> h(n_cta * 24);
                VB_CUDA(cudaMemcpyAsync(h.data(), prof_buf.ptr, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
                VB_TRY(sync_stream());
                double sum[24] = {0};
                for (size_t c = 0; c < n_cta; ++c) {
                    for (int i = 0; i < 24; ++i) {
                        sum[i] += static_cast<double>(h[c * 24 + i]);
                    }
                }
                std::fprintf(stderr, "tcs-prof ctas=%zu stages=%u cap=%u :", n_cta, stages, tp.s.cap);
                for (int i = 0; i < 24; ++i) {
                    std::fprintf(stderr, " %.0f", sum[i] / static_cast<double>(n_cta));
                }
                std::fprintf(stderr, "\n");
            }
#endif
            return 0;
        }
        if (sq8 && warp_items) {
            const bool int8 = first_dpad32 != 0;
            const size_t smem = sq8_first_smem_bytes(p.k, ix->dpad, first_dpad32);
            auto kernel = int8 ? ivf_sq8_first_kernel<true, 3> : ivf_sq8_first_kernel<false, 2>;   // rows per lane: measured best
            if (smem > 40 * 1024) {
                VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            }
            int per_sm = 0;
            VB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, SQ8_FIRST_WARPS * 32, smem));
            if (per_sm < 1) {
                VB_FAIL(VB200_INTERNAL_ERROR, "the first-phase scan does not fit an SM with %zu bytes of shared memory", smem);
            }
            VB_LAUNCH(kernel, static_cast<uint32_t>(sm_count()) * static_cast<uint32_t>(per_sm), SQ8_FIRST_WARPS * 32, smem, p,
                      int8 ? ws.qw8.ptr : static_cast<const int8_t*>(nullptr),
                      int8 ? ws.qscale.ptr : static_cast<const float*>(nullptr), first_dpad32);
            return 0;
        }
        if (sq8) {
            size_t smem = tile_smem_bytes<SQ8_QT>(p.cap, SQ8_QT * ix->dpad);
            return launch_scan(ivf_sq8_scan_kernel<SQ8_QT>, p, smem);
        }
        if (flat_rows) {
            size_t smem = tile_smem_bytes<FP32_QT>(p.cap, FP32_QT * ix->dpad);
            if (ix->quant == VB200_QUANT_BF16) {
                return launch_scan(ivf_fp32_scan_kernel<FP32_QT, SCAN_FMT_BF16>, p, smem);
            }
            if (ix->quant == VB200_QUANT_FP16) {
                return launch_scan(ivf_fp32_scan_kernel<FP32_QT, SCAN_FMT_FP16>, p, smem);
            }
            return launch_scan(ivf_fp32_scan_kernel<FP32_QT>, p, smem);
        }
        if (ix->quant == VB200_QUANT_SQ8_UNIFORM) {
            size_t smem = tile_smem_bytes<SQ8U_QT>(p.cap, SQ8U_QT * (ix->dpad / 4));
            return launch_scan(ivf_sq8u_scan_kernel<SQ8U_QT>, p, smem);
        }
        // Lists no longer than the scan depth need no selection (every probed row is a candidate): their items
        // go to the kernel variant without selection buffers, the longer lists' items to the one with them.
        // Each launch walks the whole queue with a counter of its own.
        const size_t direct_smem = static_cast<size_t>(RABITQ_QT) * ix->dpad * sizeof(float);
        if (ix->max_list_len <= p.k) {
            return launch_scan(ivf_rabitq_scan_kernel<RABITQ_QT, true>, p, direct_smem);
        }
        p.len_class = 2;
        size_t smem = tile_smem_bytes<RABITQ_QT>(p.cap, RABITQ_QT * ix->dpad);
        VB_TRY(launch_scan(ivf_rabitq_scan_kernel<RABITQ_QT>, p, smem));
        VB_CUDA(cudaMemsetAsync(ws.scalars.ptr + 7, 0, sizeof(uint64_t), st));
        p.len_class = 1;
        p.item_counter = reinterpret_cast<uint32_t*>(ws.scalars.ptr + 7);
        const int rc = launch_scan(ivf_rabitq_scan_kernel<RABITQ_QT, true>, p, direct_smem);
        p.len_class = 0;
        return rc;
    };
    p.order = ix->scan_order.ptr;
    if (split_phases) {
        VB_TRY(launch_phases(0, 1, 1, tc_first, warp_first));
        g_scan_profile.mark(st);   // first
        if (ws.exchange != nullptr) {
            // Sharded search: after the owner of each query's nearest list has scanned it, the
            // shards agree on the tightest bound any of them found, so the remaining lists are
            // pruned as sharply as on one GPU.  The exchange itself (an all-reduce with MIN over
            // bounds[nq]) belongs to the caller, who owns the communicator; it must be ordered
            // with the stream it is handed.
            VB_TRY(ws.bounds.reserve(nq));
            const uint32_t qblocks = static_cast<uint32_t>((nq + 255) / 256);
            VB_LAUNCH(bounds_to_float_kernel, qblocks, 256, 0, ws.thr.ptr, nq, ws.bounds.ptr);
            const int rc = ws.exchange(ws.bounds.ptr, nq, static_cast<void*>(st), ws.exchange_arg);
            if (rc != 0) {
                VB_FAIL(VB200_INTERNAL_ERROR, "the bound exchange callback failed with status %d", rc);
            }
            VB_LAUNCH(bounds_from_float_kernel, qblocks, 256, 0, ws.bounds.ptr, nq, ws.thr.ptr);
        }
        g_scan_profile.mark(st);   // exchange
        const uint8_t* drop = nullptr;
        if (pruning) {
            VB_TRY(ws.pair_drop.reserve(total));
            VB_LAUNCH(pair_drop_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, probes_dev, total, nprobe,
                      ws.first_live.ptr, nlist, ix->shard_rank, ix->shard_world, ix->list_off.ptr, q_dev, ix->dim,
                      ix->ball_centre.ptr, ix->ball_radius.ptr, ix->ball_count.ptr, ws.thr.ptr, ix->metric,
                      ix->code_size, probe_dists_dev, ix->list_radius.ptr,
                      ws.pair_drop.ptr, reinterpret_cast<unsigned long long*>(ws.scalars.ptr));
            drop = ws.pair_drop.ptr;
        }
        g_scan_profile.mark(st);   // drop
        VB_TRY(group_pairs(1u, drop, qt_second));
        g_scan_profile.mark(st);   // group
        VB_TRY(launch_phases(1, 1, 2, tc_second));
        g_scan_profile.mark(st);   // second
    } else {
        VB_TRY(launch_phases(0, n_phases, 1, tc_first));
    }
    VB_CUDA(cudaEventRecord(ix->ev_scan_end, st));
    ix->scan_timed = true;
    if (sq8) {
        VB_TRY(launch_merge(ws.part.ptr, nq, static_cast<uint64_t>(nprobe) * kscan, kscan, ws.merged.ptr, ws.slot_written.ptr, kscan));
        uint32_t n2 = next_pow2(kscan < 2 ? 2 : kscan);
        const size_t rescore_smem = n2 * sizeof(uint64_t) + 3 * ix->dim * sizeof(float);
        if (rescore_smem > 48 * 1024) {
            VB_CUDA(cudaFuncSetAttribute(sq8_rescore_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(rescore_smem)));
        }
        VB_LAUNCH(sq8_rescore_kernel, static_cast<uint32_t>(nq), 128, rescore_smem, q_dev, ix->dim,
                  ix->codes.ptr, ix->code_stride, ix->lower.ptr, ix->diff.ptr, ws.merged.ptr, kscan, n2,
                  kfinal, ix->metric, ws.keys.ptr, ix->use_residual ? ix->res_bias.ptr : static_cast<const float*>(nullptr),
                  ix->centroids.ptr, ix->list_off.ptr, nlist);
    } else {
        VB_TRY(launch_merge(ws.part.ptr, nq, static_cast<uint64_t>(nprobe) * kscan, kscan, ws.keys.ptr));
    }
    const uint64_t nkeys = nq * kfinal;
    VB_LAUNCH(keys_pos_to_inner_kernel, static_cast<uint32_t>((nkeys + 255) / 256), 256, 0, ws.keys.ptr,
              nkeys, ix->pos_inner.ptr);
    g_scan_profile.mark(st);   // merge
    return 0;
}

static int
check_search_ready(vb200_ivf* ix, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(queries != nullptr || nq == 0, "query pointer is null");
    VB_CHECK_ARG(k >= 1, "k must be positive");
    VB_CHECK_ARG(nprobe >= 1, "scan_buckets_count must be positive");
    if (!ix->has_centroids || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index is not trained");
    }
    return 0;
}

// Full pipeline up to per-query keys with inner-id payloads (k of them, ascending) in *keys_out.
static int
ivf_search_keys(vb200_ivf* ix, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe,
                float factor, const int32_t* bucket_ids, const uint64_t** keys_out) {
    SearchWorkspace& ws = ix->ws;
    if (nprobe > ix->nlist) {
        nprobe = ix->nlist;  // clamp like IVF::create_search_param (ivf.cpp:1573-1575)
    }
    uint32_t kscan = k;
    const bool rerank = ix->use_reorder && !ws.opt_no_reorder;
    if (rerank) {
        VB_CHECK_ARG(factor > 0.0f, "factor must be positive when use_reorder is true, got %f", factor);
        kscan = static_cast<uint32_t>(static_cast<int64_t>(factor * static_cast<float>(k)));
        if (kscan < 1) {
            kscan = 1;
        }
    }
    // buckets_per_data > 1: the scan looks for that many times as many postings, duplicates of a vector are
    // folded afterwards (IVF::search scales topk before and de-duplicates after, ivf.cpp:1722-1727, :1799-1825)
    const uint32_t kunique = kscan;
    if (ix->buckets_per_data > 1) {
        VB_CHECK_ARG(static_cast<uint64_t>(kscan) * ix->buckets_per_data <= 1024,
                     "k = %u with buckets_per_data = %u is too large (limit 1024 postings per query)", k,
                     ix->buckets_per_data);
        kscan *= ix->buckets_per_data;
    }
    // queries on the device
    const float* q_dev = queries;
    if (!is_device_pointer(queries)) {
        VB_TRY(ws.queries.reserve(nq * ix->dim));
        VB_CUDA(cudaMemcpyAsync(ws.queries.ptr, queries, nq * ix->dim * sizeof(float),
                                cudaMemcpyHostToDevice, current_stream()));
        q_dev = ws.queries.ptr;
    }
    if (ix->cosine) {
        VB_TRY(ws.q_unit.reserve(nq * ix->dim));
        VB_TRY(normalize_rows_f32(q_dev, nq, ix->dim, ws.q_unit.ptr));
        q_dev = ws.q_unit.ptr;
    }
    // probes
    VB_TRY(ws.probes.reserve(nq * nprobe));
    const float* probe_dists = nullptr;   // exact centroid distances of the probes, when routing ran here
    if (bucket_ids != nullptr) {
        VB_CUDA(cudaMemcpyAsync(ws.probes.ptr, bucket_ids, nq * nprobe * sizeof(int32_t),
                                cudaMemcpyDefault, current_stream()));
        probe_dists = ws.ext_probe_dists;   // the caller routed elsewhere and brought the distances along
    } else {
        VB_TRY(ws.probe_dists.reserve(nq * nprobe));
        VB_TRY(ivf_route_device(ix, q_dev, nq, nprobe, ws.probes.ptr, ws.probe_dists.ptr));
        probe_dists = ws.probe_dists.ptr;
    }
    // codec-specific query transform
    const float* q_scan = q_dev;
    if (ix->quant == VB200_QUANT_RABITQ) {
        VB_TRY(ws.qproc.reserve(nq * (ix->dim + 1)));
        VB_TRY(rabitq_process_query_device(q_dev, nq, ix->dim, ix->rotation.ptr, ix->rq_centroid.ptr,
                                           ws.qproc.ptr, &ws.qrot));
        q_scan = ws.qproc.ptr;
    }
    if (ix->quant == VB200_QUANT_SQ8_UNIFORM) {
        // ProcessQueryImpl: the query becomes a code record of its own
        VB_TRY(ws.qcodes.reserve(nq * ix->code_stride));
        VB_TRY(sq8u_encode_device(q_dev, nq, ix->dim, ix->metric == VB200_METRIC_L2 ? 1 : 0, ix->su_lower, ix->su_diff,
                                  nullptr, ws.qcodes.ptr, ix->code_stride));
    }
    VB_TRY(ivf_scan_device(ix, q_scan, nq, kscan, nprobe, ws.probes.ptr, probe_dists));
    if (ix->buckets_per_data > 1) {
        VB_TRY(ws.keys_unique.reserve(nq * kunique));
        VB_LAUNCH(dedup_keys_kernel, static_cast<uint32_t>(nq), 128, kscan * (sizeof(uint64_t) + sizeof(uint32_t)),
                  ws.keys.ptr, kscan, kunique, ws.keys_unique.ptr);
        VB_CUDA(cudaMemcpyAsync(ws.keys.ptr, ws.keys_unique.ptr, nq * kunique * sizeof(uint64_t), cudaMemcpyDeviceToDevice,
                                current_stream()));
        kscan = kunique;
    }
    const uint64_t* keys = ws.keys.ptr;
    if (rerank) {
        VB_TRY(ws.keys2.reserve(nq * k));
        uint32_t n2 = next_pow2(kscan < 2 ? 2 : kscan);
        VB_LAUNCH(rerank_kernel, static_cast<uint32_t>(nq), 256, n2 * sizeof(uint64_t), q_dev, ix->dim,
                  ix->flat.ptr, ws.keys.ptr, kscan, n2, k, ix->metric, ws.keys2.ptr);
        keys = ws.keys2.ptr;
    } else if (kscan != k) {
        VB_FAIL(VB200_INTERNAL_ERROR, "scan depth mismatch");
    }
    *keys_out = keys;
    return 0;
}

}  // namespace vb200

// =============================================================================================
// C ABI
// =============================================================================================

// The scan's work queue hands out the longest lists first so that the last items to finish are
// short ones.  Recomputed from the host copy of the offsets whenever the lists change.
static int
ivf_refresh_scan_order(vb200_ivf* ix) {
    const uint32_t nlist = ix->nlist;
    std::vector<uint32_t> order(nlist);
    for (uint32_t l = 0; l < nlist; ++l) {
        order[l] = l;
    }
    const std::vector<uint32_t>& off = ix->list_off_host;
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
        return off[a + 1] - off[a] > off[b + 1] - off[b];
    });
    VB_TRY(ix->scan_order.reserve(nlist));
    VB_CUDA(cudaMemcpyAsync(ix->scan_order.ptr, order.data(), nlist * sizeof(uint32_t), cudaMemcpyHostToDevice,
                            current_stream()));
    return sync_stream();
}

extern "C" int
vb200_ivf_create(uint32_t dim, int metric, uint32_t nlist, int quant, int use_reorder,
                 vb200_ivf_t* out) {
    VB_CHECK_ARG(out != nullptr, "null output handle");
    VB_CHECK_ARG(dim > 0, "dim must be positive");
    VB_CHECK_ARG(nlist >= 1, "buckets_count must be at least 1");
    VB_CHECK_ARG(quant == VB200_QUANT_SQ8 || quant == VB200_QUANT_RABITQ || quant == VB200_QUANT_FP32 ||
                     quant == VB200_QUANT_BF16 || quant == VB200_QUANT_FP16 || quant == VB200_QUANT_SQ8_UNIFORM,
                 "base_quantization_type must be fp32, sq8 or rabitq for this engine (got %d)", quant);
    VB_CHECK_ARG(metric == VB200_METRIC_L2 || metric == VB200_METRIC_IP || metric == VB200_METRIC_COSINE,
                 "metric_type must be l2, ip or cosine (got %d)", metric);
    VB_CHECK_ARG(!(quant == VB200_QUANT_RABITQ && metric != VB200_METRIC_L2),
                 "rabitq buckets support metric l2 only");
    int ndev = vb200_device_count();
    if (ndev <= 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "no CUDA device available; this engine has no CPU path");
    }
    vb200_ivf* ix = new (std::nothrow) vb200_ivf();
    if (ix == nullptr) {
        VB_FAIL(VB200_NO_ENOUGH_MEMORY, "out of host memory");
    }
    ix->dim = dim;
    ix->metric = metric;
    ix->nlist = nlist;
    ix->quant = quant;
    if (metric == VB200_METRIC_COSINE) {
        ix->metric = VB200_METRIC_IP;
        ix->cosine = true;
    }
    ix->use_reorder = use_reorder != 0;
    cudaGetDevice(&ix->device);
    if (quant == VB200_QUANT_SQ8) {
        ix->code_size = dim;
        ix->dpad = (dim + 15) / 16 * 16;
        ix->code_stride = ix->dpad;
    } else if (quant == VB200_QUANT_FP32) {
        ix->code_size = dim * 4;
        ix->dpad = (dim + 3) / 4 * 4;
        ix->code_stride = ix->dpad * 4;
        ix->has_model = true;   // nothing to train beyond the centroids
    } else if (quant == VB200_QUANT_BF16 || quant == VB200_QUANT_FP16) {
        ix->code_size = dim * 2;
        ix->dpad = (dim + 7) / 8 * 8;       // rows start on 16-byte boundaries
        ix->code_stride = ix->dpad * 2;
        ix->has_model = true;   // HalfPrecisionQuantizer::TrainImpl has nothing to learn
    } else if (quant == VB200_QUANT_SQ8_UNIFORM) {
        const int is_l2 = ix->metric == VB200_METRIC_L2 ? 1 : 0;   // cosine was mapped to IP above
        ix->code_size = sq8u_code_size(dim, is_l2);
        ix->dpad = ix->code_size - (is_l2 ? 8u : 4u);   // bytes of a record before its trailing field
        ix->code_stride = (ix->code_size + 15) / 16 * 16;
    } else {
        ix->code_size = rabitq_code_size(dim);
        ix->dpad = rabitq_bits_bytes(dim) * 8;
        ix->code_stride = (ix->code_size + 15) / 16 * 16;
    }
    ix->list_off_host.assign(nlist + 1, 0);
    int s = ix->list_off.reserve(nlist + 1);
    if (s == 0 && (cudaEventCreate(&ix->ev_scan_begin) != cudaSuccess ||
                   cudaEventCreate(&ix->ev_scan_end) != cudaSuccess)) {
        set_last_error(VB200_INTERNAL_ERROR, "cudaEventCreate failed");
        s = VB200_INTERNAL_ERROR;
    }
    if (s == 0) {
        cudaError_t e = cudaMemset(ix->list_off.ptr, 0, (nlist + 1) * sizeof(uint32_t));
        if (e != cudaSuccess) {
            set_last_error(VB200_INTERNAL_ERROR, "cudaMemset failed: %s", cudaGetErrorString(e));
            s = VB200_INTERNAL_ERROR;
        }
    }
    if (s != 0) {
        delete ix;
        return s;
    }
    *out = ix;
    return 0;
}

extern "C" int
vb200_ivf_destroy(vb200_ivf_t ix) {
    delete ix;
    return 0;
}

extern "C" int
vb200_ivf_set_shard(vb200_ivf_t ix, uint32_t rank, uint32_t world) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(world >= 1 && rank < world, "bad shard %u of %u", rank, world);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "set_shard must precede the first add");
    }
    VB_CHECK_ARG(world == 1 || ix->buckets_per_data == 1, "an index with buckets_per_data > 1 cannot be sharded");
    ix->shard_rank = rank;
    ix->shard_world = world;
    return 0;
}

static int
ivf_refresh_centroid_norms(vb200_ivf* ix) {
    VB_TRY(ix->c_sq.reserve(ix->nlist));
    VB_TRY(row_sqnorm_f32(ix->centroids.ptr, ix->nlist, ix->dim, ix->c_sq.ptr));
    ix->c_tiled = false;
    ix->has_centroids = true;
    return 0;
}

extern "C" int
vb200_ivf_set_centroids(vb200_ivf_t ix, const float* centroids) {
    VB_CHECK_ARG(ix != nullptr && centroids != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "centroids cannot change after vectors were added");
    }
    const size_t n = static_cast<size_t>(ix->nlist) * ix->dim;
    VB_TRY(ix->centroids.reserve(n));
    VB_CUDA(cudaMemcpyAsync(ix->centroids.ptr, centroids, n * sizeof(float), cudaMemcpyDefault,
                            current_stream()));
    VB_TRY(ivf_refresh_centroid_norms(ix));
    return sync_stream();
}

extern "C" int
vb200_ivf_get_centroids(vb200_ivf_t ix, float* centroids) {
    VB_CHECK_ARG(ix != nullptr && centroids != nullptr, "null pointer");
    if (!ix->has_centroids) {
        VB_FAIL(VB200_WRONG_STATUS, "index has no centroids yet");
    }
    VB_TRY(copy_out(centroids, ix->centroids.ptr, static_cast<size_t>(ix->nlist) * ix->dim));
    return sync_stream();
}

static int
ivf_store_sq8_model(vb200_ivf* ix, const float* lower_any, const float* diff_any) {
    VB_TRY(ix->lower.reserve(ix->dpad));
    VB_TRY(ix->diff.reserve(ix->dpad));
    cudaStream_t st = current_stream();
    VB_CUDA(cudaMemsetAsync(ix->lower.ptr, 0, ix->dpad * sizeof(float), st));
    VB_CUDA(cudaMemsetAsync(ix->diff.ptr, 0, ix->dpad * sizeof(float), st));
    VB_CUDA(cudaMemcpyAsync(ix->lower.ptr, lower_any, ix->dim * sizeof(float), cudaMemcpyDefault, st));
    VB_CUDA(cudaMemcpyAsync(ix->diff.ptr, diff_any, ix->dim * sizeof(float), cudaMemcpyDefault, st));
    VB_TRY(ix->sq_scale.reserve(ix->dpad));
    VB_TRY(ix->sq_mid.reserve(ix->dpad));
    VB_LAUNCH(sq8_derive_model_kernel, (ix->dpad + 127) / 128, 128, 0, ix->lower.ptr, ix->diff.ptr, ix->dim,
              ix->dpad, ix->sq_scale.ptr, ix->sq_mid.ptr);
    ix->has_model = true;
    return 0;
}

extern "C" int
vb200_ivf_set_sq8_model(vb200_ivf_t ix, const float* lower, const float* diff) {
    VB_CHECK_ARG(ix != nullptr && lower != nullptr && diff != nullptr, "null pointer");
    VB_CHECK_ARG(ix->quant == VB200_QUANT_SQ8, "index is not sq8");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "quantizer model cannot change after vectors were added");
    }
    VB_TRY(ivf_store_sq8_model(ix, lower, diff));
    return sync_stream();
}

extern "C" int
vb200_ivf_get_sq8_model(vb200_ivf_t ix, float* lower, float* diff) {
    VB_CHECK_ARG(ix != nullptr && lower != nullptr && diff != nullptr, "null pointer");
    if (ix->quant != VB200_QUANT_SQ8 || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index has no sq8 model");
    }
    VB_TRY(copy_out(lower, ix->lower.ptr, ix->dim));
    VB_TRY(copy_out(diff, ix->diff.ptr, ix->dim));
    return sync_stream();
}

extern "C" int
vb200_ivf_set_use_residual(vb200_ivf_t ix, int use_residual) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(use_residual == 0 || ix->quant == VB200_QUANT_SQ8,
                 "use_residual is served for sq8 buckets only");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0 || (ix->quant == VB200_QUANT_SQ8 && ix->has_model && (use_residual != 0) != ix->use_residual)) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "use_residual must be chosen before the quantizer is trained");
    }
    ix->use_residual = use_residual != 0;
    return 0;
}

extern "C" int
vb200_ivf_set_buckets_per_data(vb200_ivf_t ix, uint32_t buckets_per_data) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(buckets_per_data >= 1 && buckets_per_data <= ix->nlist && buckets_per_data <= 16,
                 "buckets_per_data must lie in [1, min(buckets_count, 16)], got %u", buckets_per_data);
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "buckets_per_data cannot change after vectors were added");
    }
    VB_CHECK_ARG(buckets_per_data == 1 || ix->shard_world == 1,
                 "buckets_per_data > 1 is not served on a sharded index (a vector's lists may live on different shards)");
    ix->buckets_per_data = buckets_per_data;
    return 0;
}

extern "C" int
vb200_ivf_set_sq8_uniform_model(vb200_ivf_t ix, float lower, float diff) {
    VB_CHECK_ARG(ix != nullptr, "null pointer");
    VB_CHECK_ARG(ix->quant == VB200_QUANT_SQ8_UNIFORM, "index is not sq8_uniform");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "quantizer model cannot change after vectors were added");
    }
    ix->su_lower = lower;
    ix->su_diff = diff;
    ix->has_model = true;
    return 0;
}

extern "C" int
vb200_ivf_get_sq8_uniform_model(vb200_ivf_t ix, float* lower, float* diff) {
    VB_CHECK_ARG(ix != nullptr && lower != nullptr && diff != nullptr, "null pointer");
    if (ix->quant != VB200_QUANT_SQ8_UNIFORM || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index has no sq8_uniform model");
    }
    *lower = ix->su_lower;
    *diff = ix->su_diff;
    return 0;
}

extern "C" int
vb200_ivf_set_rabitq_rotation(vb200_ivf_t ix, const float* rotation) {
    VB_CHECK_ARG(ix != nullptr && rotation != nullptr, "null pointer");
    VB_CHECK_ARG(ix->quant == VB200_QUANT_RABITQ, "index is not rabitq");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "quantizer model cannot change after vectors were added");
    }
    const size_t n = static_cast<size_t>(ix->dim) * ix->dim;
    VB_TRY(ix->rotation.reserve(n));
    VB_CUDA(cudaMemcpyAsync(ix->rotation.ptr, rotation, n * sizeof(float), cudaMemcpyDefault,
                            current_stream()));
    ix->has_rotation = true;
    return sync_stream();
}

extern "C" int
vb200_ivf_set_rabitq_centroid(vb200_ivf_t ix, const float* centroid) {
    VB_CHECK_ARG(ix != nullptr && centroid != nullptr, "null pointer");
    VB_CHECK_ARG(ix->quant == VB200_QUANT_RABITQ, "index is not rabitq");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "quantizer model cannot change after vectors were added");
    }
    if (!ix->has_rotation) {
        VB_FAIL(VB200_WRONG_STATUS, "set the rotation before the centroid");
    }
    VB_TRY(ix->rq_centroid.reserve(ix->dim));
    VB_CUDA(cudaMemcpyAsync(ix->rq_centroid.ptr, centroid, ix->dim * sizeof(float), cudaMemcpyDefault,
                            current_stream()));
    ix->has_model = true;
    return sync_stream();
}

extern "C" int
vb200_ivf_get_rabitq_centroid(vb200_ivf_t ix, float* centroid) {
    VB_CHECK_ARG(ix != nullptr && centroid != nullptr, "null pointer");
    if (ix->quant != VB200_QUANT_RABITQ || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index has no rabitq model");
    }
    VB_TRY(copy_out(centroid, ix->rq_centroid.ptr, ix->dim));
    return sync_stream();
}

extern "C" int
vb200_ivf_train(vb200_ivf_t ix, const float* data, uint64_t count, int kmeans_iters, const float* init) {
    VB_CHECK_ARG(ix != nullptr && data != nullptr, "null pointer");
    VB_CHECK_ARG(count >= ix->nlist, "k cannot be larger than count (%u lists, %llu rows)", ix->nlist,
                 static_cast<unsigned long long>(count));
    VB_CHECK_ARG(kmeans_iters >= 0, "iteration count must not be negative");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total != 0) {
        VB_FAIL(VB200_INDEX_NOT_EMPTY, "train must precede add");
    }
    if (ix->quant == VB200_QUANT_RABITQ && !ix->has_rotation) {
        VB_FAIL(VB200_WRONG_STATUS, "rabitq index needs its rotation matrix before training");
    }
    DevInput<float> x;
    VB_TRY(x.bind(data, count * ix->dim));
    ix->kws.forget_points();
    const size_t kd = static_cast<size_t>(ix->nlist) * ix->dim;
    VB_TRY(ix->centroids.reserve(kd));
    const float* seed = init != nullptr ? init : x.ptr;
    VB_CUDA(cudaMemcpyAsync(ix->centroids.ptr, seed, kd * sizeof(float), cudaMemcpyDefault,
                            current_stream()));
    DevBuf<int32_t> lab;
    VB_TRY(lab.reserve(count));
    for (int it = 0; it < kmeans_iters; ++it) {
        VB_TRY(kmeans_assign_device(ix->kws, x.ptr, count, ix->dim, ix->centroids.ptr, ix->nlist,
                                    lab.ptr, nullptr, it > 0 ? lab.ptr : nullptr));
        VB_TRY(kmeans_update_device(ix->kws, x.ptr, count, ix->dim, lab.ptr, ix->nlist,
                                    static_cast<uint32_t>(it), ix->centroids.ptr));
    }
    DevBuf<float> unit_rows;
    const float* x_model = x.ptr;   // what the bucket quantizer trains on
    if (ix->cosine) {
        // k-means runs on the rows as given, its centroids are normalised afterwards
        // (ivf_nearest_partition.cpp:81-85); the quantizer sees normalised rows
        // (scalar_quantization_trainer.cpp:139-141).
        VB_TRY(normalize_rows_f32(ix->centroids.ptr, ix->nlist, ix->dim, ix->centroids.ptr));
        if (ix->quant == VB200_QUANT_SQ8 || ix->quant == VB200_QUANT_SQ8_UNIFORM) {
            VB_TRY(unit_rows.reserve(count * ix->dim));
            VB_TRY(normalize_rows_f32(x.ptr, count, ix->dim, unit_rows.ptr));
            x_model = unit_rows.ptr;
        }
    }
    VB_TRY(ivf_refresh_centroid_norms(ix));
    DevBuf<float> residuals;
    if (ix->quant == VB200_QUANT_SQ8 && ix->use_residual) {
        // BucketDataCell::Train (src/datacell/bucket_datacell.h:593-614): the quantizer learns from the rows minus
        // the centroid of their nearest bucket
        VB_TRY(lab.reserve(count));
        if (ix->metric == VB200_METRIC_L2) {
            ix->kws.forget_points();
            VB_TRY(kmeans_assign_device(ix->kws, x_model, count, ix->dim, ix->centroids.ptr, ix->nlist, lab.ptr, nullptr));
            ix->kws.forget_points();
        } else {
            VB_TRY(dense_argmin_f32(x_model, count, ix->centroids.ptr, ix->nlist, ix->dim, -1.0f, nullptr, lab.ptr, nullptr));
        }
        VB_TRY(residuals.reserve(count * ix->dim));
        VB_LAUNCH(residual_rows_kernel, static_cast<uint32_t>((count * ix->dim + 255) / 256), 256, 0, x_model, count, ix->dim,
                  lab.ptr, ix->nlist, ix->centroids.ptr, residuals.ptr);
        x_model = residuals.ptr;
    }
    if (ix->quant == VB200_QUANT_SQ8) {
        DevBuf<float> model;
        VB_TRY(model.reserve(2 * static_cast<size_t>(ix->dim)));
        VB_TRY(sq8_train_device(x_model, count, ix->dim, VB200_SQ_TRAIN_TRUNC_BOUND, model.ptr,
                                model.ptr + ix->dim));
        VB_TRY(ivf_store_sq8_model(ix, model.ptr, model.ptr + ix->dim));
    } else if (ix->quant == VB200_QUANT_RABITQ) {
        VB_TRY(ix->rq_centroid.reserve(ix->dim));
        VB_TRY(rabitq_train_device(x.ptr, count, ix->dim, ix->rotation.ptr, ix->rq_centroid.ptr));
        ix->has_model = true;
    } else if (ix->quant == VB200_QUANT_SQ8_UNIFORM) {
        DevBuf<float> model;
        VB_TRY(model.reserve(2));
        VB_TRY(sq8u_train_device(x_model, count, ix->dim, model.ptr));
        float host_model[2] = {0.f, 0.f};
        VB_CUDA(cudaMemcpy(host_model, model.ptr, sizeof(host_model), cudaMemcpyDeviceToHost));
        ix->su_lower = host_model[0];
        ix->su_diff = host_model[1];
        ix->has_model = true;
    }
    return sync_stream();
}

// Labels and (for reorder) the fp32 rows of `count` new vectors, by inner id, after the ones the index
// holds; tombstone words for the new ids.  n_total itself is advanced by ivf_commit_lists.
static int
ivf_append_row_data(vb200_ivf* ix, const int64_t* ids, const float* rows_dev, uint64_t count) {
    cudaStream_t st = current_stream();
    const uint32_t dim = ix->dim;
    const uint64_t words = (ix->n_total + count + 31) / 32;
    if (words > ix->tomb_words) {
        DevBuf<uint32_t> bigger;
        const uint64_t cap = words * 2;
        VB_TRY(bigger.reserve(cap));
        VB_CUDA(cudaMemsetAsync(bigger.ptr, 0, cap * sizeof(uint32_t), st));
        if (ix->tomb_words > 0) {
            VB_CUDA(cudaMemcpyAsync(bigger.ptr, ix->tombstones.ptr, ix->tomb_words * sizeof(uint32_t),
                                    cudaMemcpyDeviceToDevice, st));
        }
        VB_TRY(sync_stream());
        ix->tombstones = std::move(bigger);
        ix->tomb_words = cap;
    }
    VB_TRY(grow_preserve(ix->labels, ix->n_total, ix->n_total + count));
    VB_CUDA(cudaMemcpyAsync(ix->labels.ptr + ix->n_total, ids, count * sizeof(int64_t),
                            cudaMemcpyDefault, st));
    if (ix->use_reorder) {
        VB_TRY(grow_preserve(ix->flat, ix->n_total * dim, (ix->n_total + count) * dim));
        VB_CUDA(cudaMemcpyAsync(ix->flat.ptr + ix->n_total * dim, rows_dev, count * dim * sizeof(float),
                                cudaMemcpyDeviceToDevice, st));
    }
    return 0;
}

// What every change of the lists recomputes (SQ8: the norm of every decoded code and the covering
// balls of every list), then the new arrays replace the old ones.
static int
ivf_commit_lists(vb200_ivf* ix, DevBuf<uint8_t>& new_codes, DevBuf<uint32_t>& new_inner,
                 DevBuf<uint32_t>& new_off_dev, const std::vector<uint32_t>& new_off, uint64_t n_new_stored,
                 uint64_t n_total_new) {
    const uint32_t nlist = ix->nlist, dim = ix->dim, stride = ix->code_stride;
    DevBuf<float> new_norm;
    if (ix->quant == VB200_QUANT_SQ8 && n_new_stored > 0) {
        VB_TRY(new_norm.reserve(n_new_stored));
        VB_LAUNCH(sq8_code_norm_kernel, static_cast<uint32_t>((n_new_stored + 127) / 128), 128, 0,
                  new_codes.ptr, n_new_stored, dim, stride, ix->lower.ptr, ix->diff.ptr, new_norm.ptr);
        if (ix->use_residual) {
            VB_TRY(ix->res_bias.reserve(n_new_stored));
            VB_LAUNCH(sq8_residual_bias_kernel, static_cast<uint32_t>((n_new_stored + 127) / 128), 128, 0, new_codes.ptr,
                      n_new_stored, dim, stride, ix->lower.ptr, ix->diff.ptr, new_off_dev.ptr, nlist, ix->centroids.ptr,
                      ix->metric, ix->res_bias.ptr, new_norm.ptr);
        }
    }
    if (ix->quant == VB200_QUANT_SQ8) {
        VB_TRY(ix->ball_centre.reserve(static_cast<size_t>(nlist) * SQ8_BALLS * dim));
        VB_TRY(ix->ball_radius.reserve(static_cast<size_t>(nlist) * SQ8_BALLS));
        VB_TRY(ix->ball_count.reserve(nlist));
        VB_TRY(ix->list_radius.reserve(nlist));
        const size_t balls_smem = 2 * static_cast<size_t>(SQ8_BALLS) * dim * sizeof(float);
        VB_CHECK_ARG(balls_smem <= 200 * 1024, "dim too large for the list-ball kernel");
        if (balls_smem > 48 * 1024) {
            VB_CUDA(cudaFuncSetAttribute(sq8_list_balls_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(balls_smem)));
        }
        // only the lists that grew get new balls (an add of a few rows must not cost a pass over the index)
        const uint32_t* old_off = ix->balls_valid ? ix->list_off.ptr : nullptr;
        VB_LAUNCH(sq8_list_balls_kernel, nlist, 128, balls_smem, new_codes.ptr, stride, dim, new_off_dev.ptr, old_off,
                  ix->lower.ptr, ix->diff.ptr, ix->centroids.ptr, ix->ball_centre.ptr, ix->ball_radius.ptr,
                  ix->ball_count.ptr, ix->list_radius.ptr);
        ix->balls_valid = true;
    }
    DevBuf<int8_t> new_tiled;
    DevBuf<uint32_t> new_group_off;
    if (ix->quant == VB200_QUANT_SQ8 && n_new_stored > 0 && dim <= 512) {
        // the tiled signed copy the tensor-core scan reads (a 128-row tile past a list's end runs into the
        // next list or into 16 groups of padding; those rows are masked by the list length)
        const uint32_t kchunks = (dim + 31) / 32 * 2;
        std::vector<uint32_t> goff(nlist + 1);
        uint64_t run = 0;
        for (uint32_t l = 0; l < nlist; ++l) {
            goff[l] = static_cast<uint32_t>(run);
            run += (new_off[l + 1] - new_off[l] + 7) / 8;
        }
        goff[nlist] = static_cast<uint32_t>(run);
        VB_CHECK_ARG(run + 16 < 0xFFFFFFFFull, "too many rows for the tiled code copy");
        const size_t bytes = static_cast<size_t>(run + 16) * kchunks * 128;
        VB_TRY(new_tiled.reserve(bytes));
        VB_TRY(new_group_off.reserve(nlist + 1));
        VB_CUDA(cudaMemsetAsync(new_tiled.ptr, 0, bytes, current_stream()));
        VB_CUDA(cudaMemcpyAsync(new_group_off.ptr, goff.data(), (nlist + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                current_stream()));
        const uint64_t work = n_new_stored * kchunks;
        VB_LAUNCH(sq8_tile_codes_kernel, static_cast<uint32_t>((work + 255) / 256), 256, 0, new_codes.ptr, stride,
                  new_off_dev.ptr, new_group_off.ptr, nlist, n_new_stored, kchunks, new_tiled.ptr);
        VB_TRY(sync_stream());   // goff is a local
        ix->kchunks = kchunks;
    }
    VB_TRY(sync_stream());
    ix->codes_t = std::move(new_tiled);
    ix->group_off = std::move(new_group_off);
    ix->code_norm = std::move(new_norm);
    ix->codes = std::move(new_codes);
    ix->pos_inner = std::move(new_inner);
    ix->list_off = std::move(new_off_dev);
    ix->list_off_host = new_off;
    ix->max_list_len = 0;
    for (size_t l = 0; l + 1 < new_off.size(); ++l) {
        ix->max_list_len = std::max(ix->max_list_len, new_off[l + 1] - new_off[l]);
    }
    ix->n_stored = n_new_stored;
    ix->n_total = n_total_new;
    return ivf_refresh_scan_order(ix);
}

extern "C" int
vb200_ivf_add(vb200_ivf_t ix, const float* data, uint64_t count, const int64_t* ids,
              const int32_t* labels_in) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(data != nullptr && ids != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (!ix->has_centroids || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index is not trained");
    }
    VB_CHECK_ARG((ix->n_total + count) * ix->buckets_per_data < 0xFFFFFFFFull, "index would exceed 2^32-1 postings");
    const uint32_t nlist = ix->nlist, dim = ix->dim;
    cudaStream_t st = current_stream();

    DevInput<float> x;
    VB_TRY(x.bind(data, count * dim));
    DevBuf<float> unit_rows;
    const float* xr = x.ptr;   // the rows as the index stores and scores them
    if (ix->cosine) {
        VB_TRY(unit_rows.reserve(count * dim));
        VB_TRY(normalize_rows_f32(x.ptr, count, dim, unit_rows.ptr));
        xr = unit_rows.ptr;
    }
    // 1. list of every posting.  With buckets_per_data = b > 1 a vector is stored in its b nearest lists
    // (IVF::Add, src/algorithm/ivf/ivf.cpp:607, :659-676): posting p = b * row + j is row's j-th nearest list,
    // and from here on the postings are the "rows" that are sorted, placed and encoded.
    const uint32_t per_vector = ix->buckets_per_data;
    const uint64_t n_rows = count;            // vectors of this call
    count *= per_vector;                      // postings of this call
    VB_CHECK_ARG(count < 0xFFFFFFFFull, "too many postings in one add");
    DevBuf<int32_t> lab;
    DevBuf<float> posting_rows, route_dists;
    VB_TRY(lab.reserve(count));
    if (labels_in != nullptr) {
        VB_CUDA(cudaMemcpyAsync(lab.ptr, labels_in, count * sizeof(int32_t), cudaMemcpyDefault, st));
    } else if (per_vector > 1) {
        VB_TRY(route_dists.reserve(count));
        VB_TRY(ivf_route_device(ix, xr, n_rows, per_vector, lab.ptr, route_dists.ptr));
        VB_TRY(route_sync_and_check(ix->ws));
    } else {
        if (ix->metric == VB200_METRIC_L2) {
            // the k-means assignment (tensor-core candidates + exact pick when large enough)
            ix->kws.forget_points();
            VB_TRY(kmeans_assign_device(ix->kws, xr, count, dim, ix->centroids.ptr, nlist, lab.ptr, nullptr));
            ix->kws.forget_points();
        } else {
            VB_TRY(dense_argmin_f32(xr, count, ix->centroids.ptr, nlist, dim, -1.0f, nullptr, lab.ptr, nullptr));
        }
    }
    const float* x_rows = xr;                 // one row per vector: labels, reorder rows
    if (per_vector > 1) {
        VB_TRY(posting_rows.reserve(count * dim));
        VB_LAUNCH(repeat_rows_kernel, static_cast<uint32_t>((count * dim + 255) / 256), 256, 0, xr, count, dim, per_vector,
                  posting_rows.ptr);
        xr = posting_rows.ptr;
    }
    // 2. sort rows by (list, row)
    DevBuf<uint64_t> keys, sorted;
    DevBuf<uint32_t> add_cnt;
    VB_TRY(keys.reserve(count));
    VB_TRY(sorted.reserve(count));
    VB_TRY(add_cnt.reserve(nlist + 1));
    VB_CUDA(cudaMemsetAsync(add_cnt.ptr, 0, (nlist + 1) * sizeof(uint32_t), st));
    VB_LAUNCH(ivf_make_keys_kernel, static_cast<uint32_t>((count + 255) / 256), 256, 0, lab.ptr, count,
              nlist, ix->shard_rank, ix->shard_world, keys.ptr, add_cnt.ptr);
    {
        int end_bit = 33;
        while ((uint64_t{1} << (end_bit - 32)) <= nlist) {
            ++end_bit;
        }
        size_t tmp_bytes = 0;
        VB_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, tmp_bytes, keys.ptr, sorted.ptr,
                                               static_cast<int64_t>(count), 0, end_bit, st));
        DevBuf<uint8_t> tmp;
        VB_TRY(tmp.reserve(tmp_bytes > 0 ? tmp_bytes : 1));
        VB_CUDA(cub::DeviceRadixSort::SortKeys(tmp.ptr, tmp_bytes, keys.ptr, sorted.ptr,
                                               static_cast<int64_t>(count), 0, end_bit, st));
        g_kernel_launches.fetch_add(1);
        VB_TRY(sync_stream());
    }
    // 3. new offsets (host side; nlist entries)
    std::vector<uint32_t> add_host(nlist + 1), add_off(nlist + 1), new_off(nlist + 1);
    VB_CUDA(cudaMemcpyAsync(add_host.data(), add_cnt.ptr, (nlist + 1) * sizeof(uint32_t),
                            cudaMemcpyDeviceToHost, st));
    VB_TRY(sync_stream());
    uint64_t run_add = 0, run_new = 0;
    for (uint32_t l = 0; l < nlist; ++l) {
        add_off[l] = static_cast<uint32_t>(run_add);
        new_off[l] = static_cast<uint32_t>(run_new);
        run_add += add_host[l];
        run_new += (ix->list_off_host[l + 1] - ix->list_off_host[l]) + add_host[l];
    }
    add_off[nlist] = static_cast<uint32_t>(run_add);
    new_off[nlist] = static_cast<uint32_t>(run_new);
    const uint64_t n_new_stored = run_new;
    DevBuf<uint32_t> add_off_dev, new_off_dev;
    VB_TRY(add_off_dev.reserve(nlist + 1));
    VB_TRY(new_off_dev.reserve(nlist + 1));
    VB_CUDA(cudaMemcpyAsync(add_off_dev.ptr, add_off.data(), (nlist + 1) * sizeof(uint32_t),
                            cudaMemcpyHostToDevice, st));
    VB_CUDA(cudaMemcpyAsync(new_off_dev.ptr, new_off.data(), (nlist + 1) * sizeof(uint32_t),
                            cudaMemcpyHostToDevice, st));
    // 4. regrown arrays
    DevBuf<uint8_t> new_codes;
    DevBuf<uint32_t> new_inner, dst_of_row;
    const uint32_t stride = ix->code_stride;
    VB_TRY(new_codes.reserve((n_new_stored > 0 ? n_new_stored : 1) * stride));
    VB_TRY(new_inner.reserve(n_new_stored > 0 ? n_new_stored : 1));
    VB_TRY(dst_of_row.reserve(count));
    VB_CUDA(cudaMemsetAsync(new_codes.ptr, 0, (n_new_stored > 0 ? n_new_stored : 1) * stride, st));
    if (ix->n_stored > 0) {
        uint64_t work = ix->n_stored * (stride / 16);
        VB_LAUNCH(ivf_move_old_kernel, static_cast<uint32_t>((work + 255) / 256), 256, 0, ix->codes.ptr,
                  ix->pos_inner.ptr, ix->list_off.ptr, new_off_dev.ptr, nlist, ix->n_stored, stride / 16,
                  new_codes.ptr, new_inner.ptr);
    }
    VB_LAUNCH(ivf_place_new_kernel, static_cast<uint32_t>((count + 255) / 256), 256, 0, sorted.ptr, count,
              nlist, new_off_dev.ptr, ix->list_off.ptr, add_off_dev.ptr,
              static_cast<uint32_t>(ix->n_total), per_vector, dst_of_row.ptr, new_inner.ptr);
    // 5. encode the new rows in place
    if (ix->quant == VB200_QUANT_SQ8) {
        DevBuf<float> residuals;
        const float* to_encode = xr;
        if (ix->use_residual) {
            VB_TRY(residuals.reserve(count * dim));
            VB_LAUNCH(residual_rows_kernel, static_cast<uint32_t>((count * dim + 255) / 256), 256, 0, xr, count, dim, lab.ptr,
                      nlist, ix->centroids.ptr, residuals.ptr);
            to_encode = residuals.ptr;
        }
        VB_TRY(sq8_encode_device(to_encode, count, dim, ix->lower.ptr, ix->diff.ptr, dst_of_row.ptr,
                                 new_codes.ptr, stride));
        VB_TRY(sync_stream());   // `residuals` ends with this scope
    } else if (ix->quant == VB200_QUANT_FP32) {
        VB_LAUNCH(fp32_place_rows_kernel, static_cast<uint32_t>((count * dim + 255) / 256), 256, 0, xr, count, dim,
                  dst_of_row.ptr, new_codes.ptr, stride);
    } else if (ix->quant == VB200_QUANT_SQ8_UNIFORM) {
        VB_TRY(sq8u_encode_device(xr, count, dim, ix->metric == VB200_METRIC_L2 ? 1 : 0, ix->su_lower, ix->su_diff,
                                  dst_of_row.ptr, new_codes.ptr, stride));
    } else if (ix->quant == VB200_QUANT_BF16) {
        VB_LAUNCH(half_place_rows_kernel<SCAN_FMT_BF16>, static_cast<uint32_t>((count * dim + 255) / 256), 256, 0, xr, count,
                  dim, dst_of_row.ptr, new_codes.ptr, stride);
    } else if (ix->quant == VB200_QUANT_FP16) {
        VB_LAUNCH(half_place_rows_kernel<SCAN_FMT_FP16>, static_cast<uint32_t>((count * dim + 255) / 256), 256, 0, xr, count,
                  dim, dst_of_row.ptr, new_codes.ptr, stride);
    } else {
        VB_TRY(rabitq_encode_device(xr, count, dim, ix->rotation.ptr, ix->rq_centroid.ptr,
                                    dst_of_row.ptr, new_codes.ptr, stride));
    }
    // 6. labels and (for reorder) the fp32 rows, by inner id; tombstone words for the new ids
    VB_TRY(ivf_append_row_data(ix, ids, x_rows, n_rows));
    // 7. per-list derived data, then commit
    return ivf_commit_lists(ix, new_codes, new_inner, new_off_dev, new_off, n_new_stored, ix->n_total + n_rows);
}

extern "C" int
vb200_ivf_remove(vb200_ivf_t ix, const int64_t* labels, uint64_t count, uint64_t* removed) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    if (removed != nullptr) {
        *removed = 0;
    }
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(labels != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n_total == 0) {
        return 0;
    }
    std::vector<int64_t> sorted(count);
    VB_CUDA(cudaMemcpy(sorted.data(), labels, count * sizeof(int64_t), cudaMemcpyDefault));
    std::sort(sorted.begin(), sorted.end());
    DevBuf<int64_t> sorted_dev;
    DevBuf<unsigned long long> newly;
    VB_TRY(sorted_dev.reserve(count));
    VB_TRY(newly.reserve(1));
    cudaStream_t st = current_stream();
    VB_CUDA(cudaMemcpyAsync(sorted_dev.ptr, sorted.data(), count * sizeof(int64_t), cudaMemcpyHostToDevice, st));
    VB_CUDA(cudaMemsetAsync(newly.ptr, 0, sizeof(unsigned long long), st));
    VB_LAUNCH(tombstone_kernel, static_cast<uint32_t>((ix->n_total + 255) / 256), 256, 0, ix->labels.ptr, ix->n_total,
              sorted_dev.ptr, count, ix->tombstones.ptr, newly.ptr);
    unsigned long long n_new = 0;
    VB_CUDA(cudaMemcpyAsync(&n_new, newly.ptr, sizeof(n_new), cudaMemcpyDeviceToHost, st));
    VB_TRY(sync_stream());
    ix->n_removed += n_new;
    if (removed != nullptr) {
        *removed = n_new;
    }
    return 0;
}

extern "C" int64_t
vb200_ivf_num_elements(vb200_ivf_t ix) {
    return ix == nullptr ? 0 : static_cast<int64_t>(ix->n_total - ix->n_removed);
}

extern "C" int64_t
vb200_ivf_memory_usage(vb200_ivf_t ix) {
    if (ix == nullptr) {
        return 0;
    }
    return static_cast<int64_t>(ix->codes.bytes() + ix->codes_t.bytes() + ix->pos_inner.bytes() + ix->labels.bytes() +
                                ix->flat.bytes() + ix->centroids.bytes() + ix->rotation.bytes() +
                                ix->list_off.bytes());
}

extern "C" int
vb200_ivf_set_lists(vb200_ivf_t ix, const int64_t* list_sizes, const uint8_t* codes, const int64_t* inner_ids,
                    const int64_t* labels, uint64_t n_total, const float* rows) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(list_sizes != nullptr && labels != nullptr, "null pointer");
    VB_CHECK_ARG(!is_device_pointer(list_sizes), "list_sizes is read on the host");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (!ix->has_centroids || !ix->has_model) {
        VB_FAIL(VB200_WRONG_STATUS, "index is not trained");
    }
    if (ix->n_total != 0) {
        VB_FAIL(VB200_WRONG_STATUS, "lists can only be loaded into an empty index");
    }
    VB_CHECK_ARG(n_total > 0 && n_total < 0xFFFFFFFFull, "n_total must be in [1, 2^32-2]");
    VB_CHECK_ARG(!ix->use_reorder || rows != nullptr, "an index with reorder needs the fp32 rows");
    const uint32_t nlist = ix->nlist, dim = ix->dim, stride = ix->code_stride;
    std::vector<uint64_t> src_off(nlist + 1);
    std::vector<uint32_t> new_off(nlist + 1);
    uint64_t run_src = 0, run_new = 0;
    for (uint32_t l = 0; l < nlist; ++l) {
        VB_CHECK_ARG(list_sizes[l] >= 0, "negative list size");
        src_off[l] = run_src;
        new_off[l] = static_cast<uint32_t>(run_new);
        run_src += static_cast<uint64_t>(list_sizes[l]);
        if (l % ix->shard_world == ix->shard_rank) {
            run_new += static_cast<uint64_t>(list_sizes[l]);
        }
        VB_CHECK_ARG(run_src < 0xFFFFFFFFull, "lists hold more than 2^32-2 entries");
    }
    src_off[nlist] = run_src;
    new_off[nlist] = static_cast<uint32_t>(run_new);
    VB_CHECK_ARG(run_src == 0 || (codes != nullptr && inner_ids != nullptr), "null pointer");
    const uint64_t n_kept = run_new;
    cudaStream_t st = current_stream();

    DevInput<uint8_t> src_codes;
    DevInput<int64_t> src_inner;
    VB_TRY(src_codes.bind(codes, run_src * ix->code_size));
    VB_TRY(src_inner.bind(inner_ids, run_src));
    DevBuf<uint64_t> src_off_dev;
    DevBuf<uint32_t> new_off_dev, new_inner;
    DevBuf<uint8_t> new_codes;
    DevBuf<unsigned long long> bad;
    VB_TRY(src_off_dev.reserve(nlist + 1));
    VB_TRY(new_off_dev.reserve(nlist + 1));
    VB_TRY(new_codes.reserve((n_kept > 0 ? n_kept : 1) * stride));
    VB_TRY(new_inner.reserve(n_kept > 0 ? n_kept : 1));
    VB_TRY(bad.reserve(1));
    VB_CUDA(cudaMemcpyAsync(src_off_dev.ptr, src_off.data(), (nlist + 1) * sizeof(uint64_t), cudaMemcpyHostToDevice, st));
    VB_CUDA(cudaMemcpyAsync(new_off_dev.ptr, new_off.data(), (nlist + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    VB_CUDA(cudaMemsetAsync(bad.ptr, 0, sizeof(unsigned long long), st));
    if (n_kept > 0) {
        const uint64_t work = n_kept * (stride / 16);
        VB_LAUNCH(ivf_import_lists_kernel, static_cast<uint32_t>((work + 255) / 256), 256, 0, src_codes.ptr,
                  src_inner.ptr, src_off_dev.ptr, new_off_dev.ptr, nlist, n_kept, ix->code_size, stride / 16, n_total,
                  new_codes.ptr, new_inner.ptr, bad.ptr);
    }
    unsigned long long n_bad = 0;
    VB_CUDA(cudaMemcpyAsync(&n_bad, bad.ptr, sizeof(n_bad), cudaMemcpyDeviceToHost, st));
    VB_TRY(sync_stream());
    VB_CHECK_ARG(n_bad == 0, "%llu inner ids are outside [0, n_total)", n_bad);

    DevInput<float> x;   // the rows as stored: nothing is normalised again
    if (ix->use_reorder) {
        VB_TRY(x.bind(rows, n_total * dim));
    }
    VB_TRY(ivf_append_row_data(ix, labels, x.ptr, n_total));
    return ivf_commit_lists(ix, new_codes, new_inner, new_off_dev, new_off, n_kept, n_total);
}

extern "C" int
vb200_ivf_get_rows(vb200_ivf_t ix, float* rows) {
    VB_CHECK_ARG(ix != nullptr && rows != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    VB_CHECK_ARG(ix->use_reorder, "the index keeps fp32 rows only when reorder is on");
    VB_TRY(copy_out(rows, ix->flat.ptr, ix->n_total * ix->dim));
    return sync_stream();
}

extern "C" int
vb200_ivf_get_lists(vb200_ivf_t ix, int64_t* list_sizes, uint8_t* codes, int64_t* inner_ids) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (list_sizes != nullptr) {
        for (uint32_t l = 0; l < ix->nlist; ++l) {
            list_sizes[l] = static_cast<int64_t>(ix->list_off_host[l + 1] - ix->list_off_host[l]);
        }
    }
    if (ix->n_stored == 0) {
        return 0;
    }
    if (codes != nullptr) {
        VB_CHECK_ARG(!is_device_pointer(codes), "get_lists writes host memory");
        VB_CUDA(cudaMemcpy2D(codes, ix->code_size, ix->codes.ptr, ix->code_stride, ix->code_size,
                             ix->n_stored, cudaMemcpyDeviceToHost));
    }
    if (inner_ids != nullptr) {
        std::vector<uint32_t> tmp(ix->n_stored);
        VB_CUDA(cudaMemcpy(tmp.data(), ix->pos_inner.ptr, ix->n_stored * sizeof(uint32_t),
                           cudaMemcpyDeviceToHost));
        for (uint64_t i = 0; i < ix->n_stored; ++i) {
            inner_ids[i] = tmp[i];
        }
    }
    return 0;
}

extern "C" int
vb200_ivf_route(vb200_ivf_t ix, const float* queries, uint64_t nq, uint32_t nprobe,
                int32_t* bucket_ids, float* bucket_dists) {
    VB_CHECK_ARG(ix != nullptr && bucket_ids != nullptr, "null pointer");
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(queries != nullptr, "query pointer is null");
    VB_CHECK_ARG(nprobe >= 1 && nprobe <= ix->nlist, "scan_buckets_count out of range");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (!ix->has_centroids) {
        VB_FAIL(VB200_WRONG_STATUS, "index is not trained");
    }
    DevInput<float> q;
    VB_TRY(q.bind(queries, nq * ix->dim));
    VB_TRY(ix->ws.probes.reserve(nq * nprobe));
    VB_TRY(ix->ws.probe_dists.reserve(nq * nprobe));
    const float* q_dev = q.ptr;
    if (ix->cosine) {
        VB_TRY(ix->ws.q_unit.reserve(nq * ix->dim));
        VB_TRY(normalize_rows_f32(q_dev, nq, ix->dim, ix->ws.q_unit.ptr));
        q_dev = ix->ws.q_unit.ptr;
    }
    VB_TRY(ivf_route_device(ix, q_dev, nq, nprobe, ix->ws.probes.ptr, ix->ws.probe_dists.ptr));
    VB_TRY(copy_out(bucket_ids, ix->ws.probes.ptr, nq * nprobe));
    if (bucket_dists != nullptr) {
        VB_TRY(copy_out(bucket_dists, ix->ws.probe_dists.ptr, nq * nprobe));
    }
    return route_sync_and_check(ix->ws);
}

extern "C" int
vb200_ivf_search(vb200_ivf_t ix, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe,
                 float factor, const int32_t* bucket_ids, int64_t* ids, float* dists) {
    return vb200_ivf_search_filtered(ix, queries, nq, k, nprobe, factor, bucket_ids, nullptr, ids, dists);
}

// *deadline = now + budget on the GPU's own clock; launched first in a search with a timeout, so the budget
// runs from the start of the call's device work.
__global__ void
deadline_stamp_kernel(unsigned long long* deadline, unsigned long long budget_ns) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    *deadline = now + budget_ns;
}

extern "C" int
vb200_ivf_search_filtered(vb200_ivf_t ix, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe,
                          float factor, const int32_t* bucket_ids, const vb200_filter* filter, int64_t* ids,
                          float* dists) {
    return vb200_ivf_search_ex(ix, queries, nq, k, nprobe, factor, bucket_ids, filter, nullptr, ids, dists, nullptr);
}

extern "C" int
vb200_ivf_search_ex(vb200_ivf_t ix, const float* queries, uint64_t nq, uint32_t k, uint32_t nprobe, float factor,
                    const int32_t* bucket_ids, const vb200_filter* filter, const vb200_search_options* options,
                    int64_t* ids, float* dists, int* timed_out) {
    if (timed_out != nullptr) {
        *timed_out = 0;
    }
    VB_TRY(check_search_ready(ix, queries, nq, k, nprobe));
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(ids != nullptr && dists != nullptr, "null output pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    SearchWorkspace& ws = ix->ws;
    struct OptionScope {   // the options hold for this call only, whatever way it ends
        SearchWorkspace& w;
        ~OptionScope() {
            w.opt_no_reorder = false;
            w.opt_deadline = false;
        }
    } option_scope{ws};
    if (options != nullptr) {
        ws.opt_no_reorder = options->enable_reorder == 0;
        // IndexSearchParameter's default is "no limit" (src/algorithm/index_search_parameter.h:53); a limit of
        // zero or less has passed as soon as the scan asks
        const double ms = options->timeout_ms;
        if (options->has_timeout != 0 && ms < 1e12) {
            VB_TRY(reserve_scalars(ws));
            const double ns = ms > 0.0 ? ms * 1e6 : 0.0;
            VB_LAUNCH(deadline_stamp_kernel, 1, 1, 0, reinterpret_cast<unsigned long long*>(ws.scalars.ptr + 6),
                      static_cast<unsigned long long>(ns));
            ws.opt_deadline = true;
        }
    }
    const uint64_t total = nq * k;
    VB_TRY(ws.out_ids.reserve(total));
    VB_TRY(ws.out_dists.reserve(total));
    if (ix->n_total == 0) {
        // Empty index: every slot padded, like the Dim=0 dataset of IndexImpl (index_impl.h:60-63).
        std::vector<int64_t> hi(total, -1);
        std::vector<float> hd(total, INFINITY);
        VB_CUDA(cudaMemcpy(ids, hi.data(), total * sizeof(int64_t), cudaMemcpyDefault));
        VB_CUDA(cudaMemcpy(dists, hd.data(), total * sizeof(float), cudaMemcpyDefault));
        ix->last_scan_bytes = 0;
        return 0;
    }
    const uint64_t* keys = nullptr;
    ws.filter = filter;
    const int search_status = ivf_search_keys(ix, queries, nq, k, nprobe, factor, bucket_ids, &keys);
    ws.filter = nullptr;
    VB_TRY(search_status);
    VB_LAUNCH(keys_to_results_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, keys, total,
              ix->labels.ptr, ws.out_ids.ptr, ws.out_dists.ptr);
    VB_TRY(copy_out(ids, ws.out_ids.ptr, total));
    VB_TRY(copy_out(dists, ws.out_dists.ptr, total));
    uint64_t scalars[SCALARS] = {};
    VB_CUDA(cudaMemcpyAsync(scalars, ws.scalars.ptr, sizeof(scalars), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    VB_TRY(route_flag_check(scalars[8]));
    ix->last_scan_bytes = static_cast<int64_t>(scalars[0]);
    ix->last_scanned_bytes = static_cast<int64_t>(ws.pruning ? scalars[3] : scalars[0]);
    if (scalars[4] != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "the tensor-core scan gave up on a bounded wait");
    }
    if (timed_out != nullptr) {
        *timed_out = scalars[5] != 0 ? 1 : 0;
    }
    return 0;
}

// keys (payload = inner id) -> keys unchanged plus the label of each entry.
__global__ void
keys_labels_kernel(const uint64_t* __restrict__ keys, uint64_t total,
                   const int64_t* __restrict__ labels, uint64_t* __restrict__ keys_out,
                   int64_t* __restrict__ labels_out) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    uint64_t key = keys[e];
    keys_out[e] = key;
    labels_out[e] = key == KEY_INF ? -1 : labels[static_cast<uint32_t>(key)];
}

extern "C" int
vb200_ivf_search_partial(vb200_ivf_t ix, const float* queries, uint64_t nq, uint32_t k,
                         uint32_t nprobe, float factor, const int32_t* bucket_ids, vb200_exchange_fn exchange,
                         void* exchange_arg, uint64_t* keys_dev, int64_t* labels_dev) {
    VB_TRY(check_search_ready(ix, queries, nq, k, nprobe));
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(keys_dev != nullptr && labels_dev != nullptr, "null output pointer");
    VB_CHECK_ARG(is_device_pointer(keys_dev) && is_device_pointer(labels_dev),
                 "partial results are written to device memory");
    std::lock_guard<std::mutex> lock(ix->mu);
    const uint64_t total = nq * k;
    if (ix->n_total == 0 || ix->n_stored == 0) {
        VB_CUDA(cudaMemsetAsync(keys_dev, 0xFF, total * sizeof(uint64_t), current_stream()));
        VB_CUDA(cudaMemsetAsync(labels_dev, 0xFF, total * sizeof(int64_t), current_stream()));
        ix->last_scan_bytes = 0;
        return sync_stream();
    }
    const uint64_t* keys = nullptr;
    ix->ws.exchange = exchange;
    ix->ws.exchange_arg = exchange_arg;
    const int search_status = ivf_search_keys(ix, queries, nq, k, nprobe, factor, bucket_ids, &keys);
    ix->ws.exchange = nullptr;
    ix->ws.exchange_arg = nullptr;
    VB_TRY(search_status);
    VB_LAUNCH(keys_labels_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, keys, total,
              ix->labels.ptr, keys_dev, labels_dev);
    uint64_t scalars[SCALARS] = {};
    VB_CUDA(cudaMemcpyAsync(scalars, ix->ws.scalars.ptr, sizeof(scalars), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    VB_TRY(route_flag_check(scalars[8]));
    ix->last_scan_bytes = static_cast<int64_t>(scalars[0]);
    ix->last_scanned_bytes = static_cast<int64_t>(ix->ws.pruning ? scalars[3] : scalars[0]);
    if (scalars[4] != 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "the tensor-core scan gave up on a bounded wait");
    }
    return 0;
}

extern "C" int64_t
vb200_ivf_last_scan_bytes(vb200_ivf_t ix) {
    return ix == nullptr ? 0 : ix->last_scan_bytes;
}

extern "C" int64_t
vb200_ivf_last_scanned_bytes(vb200_ivf_t ix) {
    return ix == nullptr ? 0 : ix->last_scanned_bytes;
}

extern "C" int
vb200_ivf_set_list_pruning(vb200_ivf_t ix, int enable) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    std::lock_guard<std::mutex> lock(ix->mu);
    ix->prune_lists = enable != 0;
    return 0;
}

extern "C" int
vb200_ivf_last_scan_ms(vb200_ivf_t ix, float* ms) {
    VB_CHECK_ARG(ix != nullptr && ms != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (!ix->scan_timed) {
        VB_FAIL(VB200_WRONG_STATUS, "no search has run on this index yet");
    }
    VB_CUDA(cudaEventSynchronize(ix->ev_scan_end));
    VB_CUDA(cudaEventElapsedTime(ms, ix->ev_scan_begin, ix->ev_scan_end));
    return 0;
}

// labels gathered beside tagged keys: payload indexes the gathered label array.
__global__ void
tagged_to_results_kernel(const uint64_t* __restrict__ keys, uint64_t total,
                         const int64_t* __restrict__ gathered_labels, int64_t* __restrict__ ids,
                         float* __restrict__ dists) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    uint64_t key = keys[e];
    if (key == KEY_INF) {
        ids[e] = -1;
        dists[e] = INFINITY;
    } else {
        ids[e] = gathered_labels[static_cast<uint32_t>(key)];
        dists[e] = ordered_to_float(static_cast<uint32_t>(key >> 32));
    }
}

namespace vb200 {

// Merge of `parts` partial results [nq][k], part p's keys at keys_all + p * part_stride and its labels at
// labels_all + p * part_stride, into ids / dists (host or device).  No host synchronisation.
int
merge_partials_device(const uint64_t* keys_all, const int64_t* labels_all, uint32_t parts, uint64_t part_stride,
                      uint64_t nq, uint32_t k, int64_t* ids, float* dists) {
    const uint64_t in_total = static_cast<uint64_t>(parts) * nq * k;
    VB_CHECK_ARG(static_cast<uint64_t>(parts) * part_stride < 0xFFFFFFFFull, "merge input too large");
    // Workspace kept between calls (a serving loop merges the same shape every step); one merge
    // at a time per process.
    static std::mutex merge_mu;
    static DevBuf<uint64_t> tagged, merged;
    static DevBuf<int64_t> out_ids;
    static DevBuf<float> out_dists;
    std::lock_guard<std::mutex> lock(merge_mu);
    VB_TRY(tagged.reserve(in_total));
    VB_TRY(merged.reserve(nq * k));
    VB_LAUNCH(tag_partials_kernel, static_cast<uint32_t>((in_total + 255) / 256), 256, 0, keys_all, parts,
              part_stride, nq, k, tagged.ptr);
    VB_TRY(launch_merge(tagged.ptr, nq, static_cast<uint64_t>(parts) * k, k, merged.ptr));
    const bool direct = is_device_pointer(ids) && is_device_pointer(dists);
    int64_t* ids_dev = ids;
    float* dists_dev = dists;
    if (!direct) {
        VB_TRY(out_ids.reserve(nq * k));
        VB_TRY(out_dists.reserve(nq * k));
        ids_dev = out_ids.ptr;
        dists_dev = out_dists.ptr;
    }
    VB_LAUNCH(tagged_to_results_kernel, static_cast<uint32_t>((nq * k + 255) / 256), 256, 0, merged.ptr,
              nq * k, labels_all, ids_dev, dists_dev);
    if (!direct) {
        VB_TRY(copy_out(ids, out_ids.ptr, nq * k));
        VB_TRY(copy_out(dists, out_dists.ptr, nq * k));
    }
    return 0;
}

}  // namespace vb200

extern "C" int
vb200_merge_partials(const uint64_t* keys_dev, const int64_t* labels_dev, uint32_t parts, uint64_t nq,
                     uint32_t k, int64_t* ids, float* dists) {
    VB_CHECK_ARG(keys_dev != nullptr && labels_dev != nullptr && ids != nullptr && dists != nullptr,
                 "null pointer");
    VB_CHECK_ARG(parts >= 1 && k >= 1 && k <= 1024, "bad merge shape");
    if (nq == 0) {
        return 0;
    }
    VB_TRY(merge_partials_device(keys_dev, labels_dev, parts, nq * k, nq, k, ids, dists));
    return sync_stream();
}

__global__ void
fill_f32_kernel(float* __restrict__ out, uint64_t n, float value) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = value;
    }
}

// Bound exchange of the sharded search: an all-reduce (MIN) over the ranks of the communicator in `arg`.
static int
exchange_bounds_over_comm(float* bounds_dev, uint64_t nq, void* cuda_stream, void* arg) {
    return comm_all_reduce_min_f32(static_cast<vb200_comm*>(arg), bounds_dev, nq, static_cast<cudaStream_t>(cuda_stream));
}

extern "C" int
vb200_ivf_search_sharded(vb200_ivf_t ix, vb200_comm_t comm, const float* queries, uint64_t nq, uint32_t k,
                         uint32_t nprobe, float factor, int64_t* ids, float* dists) {
    VB_CHECK_ARG(comm != nullptr, "null communicator");
    VB_TRY(check_search_ready(ix, queries, nq, k, nprobe));
    if (comm->world == 1) {
        return vb200_ivf_search(ix, queries, nq, k, nprobe, factor, nullptr, ids, dists);
    }
    VB_CHECK_ARG(ix->shard_world == static_cast<uint32_t>(comm->world) && ix->shard_rank == static_cast<uint32_t>(comm->rank),
                 "the index is shard %u of %u but the communicator is rank %d of %d", ix->shard_rank, ix->shard_world,
                 comm->rank, comm->world);
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(ids != nullptr && dists != nullptr, "null output pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    SearchWorkspace& ws = ix->ws;
    cudaStream_t st = current_stream();
    if (nprobe > ix->nlist) {
        nprobe = ix->nlist;
    }
    const uint32_t world = static_cast<uint32_t>(comm->world), rank = static_cast<uint32_t>(comm->rank);
    const uint64_t total = nq * k;
    // VB200_SHARD_PROFILE=1: device time of the step's sections from CUDA events, averaged and printed to
    // stderr every 20 calls after the first three (rank 0 and the last rank)
    static const bool profile = std::getenv("VB200_SHARD_PROFILE") != nullptr && std::getenv("VB200_SHARD_PROFILE")[0] == '1';
    static cudaEvent_t ev[6];
    static double acc_ms[5] = {0, 0, 0, 0, 0};
    static int n_prof = 0;
    if (profile && n_prof == 0 && ev[0] == nullptr) {
        for (auto& e : ev) {
            VB_CUDA(cudaEventCreate(&e));
        }
    }
    auto mark = [&](int i) {
        if (profile) {
            cudaEventRecord(ev[i], st);
        }
    };
    mark(0);
    // the batch on the device, once for routing and scan
    const float* q_dev = queries;
    if (!is_device_pointer(queries)) {
        VB_TRY(ws.queries.reserve(nq * ix->dim));
        VB_CUDA(cudaMemcpyAsync(ws.queries.ptr, queries, nq * ix->dim * sizeof(float), cudaMemcpyHostToDevice, st));
        q_dev = ws.queries.ptr;
    }
    // 1. this rank routes rows [lo, hi) of the batch; probe lists and their centroid distances are gathered
    const uint64_t per = (nq + world - 1) / world;
    const uint64_t lo = std::min<uint64_t>(nq, rank * per), hi = std::min<uint64_t>(nq, lo + per);
    const uint64_t slice_entries = per * nprobe;
    VB_TRY(ws.sh_route_local.reserve(2 * slice_entries));
    VB_TRY(ws.sh_probes_all.reserve(static_cast<size_t>(world) * slice_entries));
    VB_TRY(ws.sh_dists_all.reserve(static_cast<size_t>(world) * slice_entries));
    int32_t* probes_local = reinterpret_cast<int32_t*>(ws.sh_route_local.ptr);
    float* dists_local = reinterpret_cast<float*>(ws.sh_route_local.ptr + slice_entries);
    if (hi - lo < per) {
        VB_CUDA(cudaMemsetAsync(ws.sh_route_local.ptr, 0, 2 * slice_entries * sizeof(uint32_t), st));
    }
    if (hi > lo) {
        const float* q_slice = q_dev + lo * ix->dim;
        if (ix->cosine) {
            VB_TRY(ws.q_unit.reserve(nq * ix->dim));
            VB_TRY(normalize_rows_f32(q_slice, hi - lo, ix->dim, ws.q_unit.ptr));
            q_slice = ws.q_unit.ptr;
        }
        VB_TRY(ivf_route_device(ix, q_slice, hi - lo, nprobe, probes_local, dists_local));
    }
    mark(1);
    VB_TRY(comm_group_start());
    VB_TRY(comm_all_gather(comm, probes_local, ws.sh_probes_all.ptr, slice_entries * sizeof(int32_t), st));
    VB_TRY(comm_all_gather(comm, dists_local, ws.sh_dists_all.ptr, slice_entries * sizeof(float), st));
    VB_TRY(comm_group_end());
    mark(2);
    // 2. scan of the probed lists this rank owns, bounds shared between the two phases
    VB_TRY(ws.sh_local.reserve(2 * total));
    VB_TRY(ws.sh_all.reserve(static_cast<size_t>(world) * 2 * total));
    uint64_t* keys_local = ws.sh_local.ptr;
    int64_t* labels_local = reinterpret_cast<int64_t*>(ws.sh_local.ptr + total);
    if (ix->n_total == 0 || ix->n_stored == 0) {
        VB_CUDA(cudaMemsetAsync(ws.sh_local.ptr, 0xFF, 2 * total * sizeof(uint64_t), st));
        ix->last_scan_bytes = 0;
        if (nprobe > 1) {
            // the ranks that hold rows exchange their bounds between the two scan phases (a search with more
            // than one probe list has two): take part with "no bound"
            VB_TRY(ws.bounds.reserve(nq));
            VB_LAUNCH(fill_f32_kernel, static_cast<uint32_t>((nq + 255) / 256), 256, 0, ws.bounds.ptr, nq, INFINITY);
            VB_TRY(comm_all_reduce_min_f32(comm, ws.bounds.ptr, nq, st));
        }
    } else {
        const uint64_t* keys = nullptr;
        ws.exchange = exchange_bounds_over_comm;
        ws.exchange_arg = comm;
        ws.ext_probe_dists = ws.sh_dists_all.ptr;
        const int search_status = ivf_search_keys(ix, q_dev, nq, k, nprobe, factor, ws.sh_probes_all.ptr, &keys);
        ws.exchange = nullptr;
        ws.exchange_arg = nullptr;
        ws.ext_probe_dists = nullptr;
        VB_TRY(search_status);
        VB_LAUNCH(keys_labels_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, keys, total,
                  ix->labels.ptr, keys_local, labels_local);
    }
    // 3. one gather of the packed (keys, labels) and the merge, on every rank
    mark(3);
    VB_TRY(comm_all_gather(comm, ws.sh_local.ptr, ws.sh_all.ptr, 2 * total * sizeof(uint64_t), st));
    mark(4);
    VB_TRY(merge_partials_device(ws.sh_all.ptr, reinterpret_cast<const int64_t*>(ws.sh_all.ptr + total), world, 2 * total,
                                 nq, k, ids, dists));
    mark(5);
    uint64_t scalars[SCALARS] = {};
    VB_CUDA(cudaMemcpyAsync(scalars, ws.scalars.ptr, sizeof(scalars), cudaMemcpyDeviceToHost, st));
    VB_TRY(sync_stream());
    VB_TRY(route_flag_check(scalars[8]));
    static int n_calls = 0;
    if (profile && ++n_calls > 3) {   // the first three calls are a caller's warm-up
        for (int i = 0; i < 5; ++i) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
            acc_ms[i] += ms;
        }
        if (++n_prof % 20 == 0 && (rank == 0 || rank + 1 == world)) {
            std::fprintf(stderr, "shard-prof rank %u: route %.3f gather %.3f scan+exchange %.3f gather %.3f merge %.3f ms\n", rank,
                         acc_ms[0] / 20, acc_ms[1] / 20, acc_ms[2] / 20, acc_ms[3] / 20, acc_ms[4] / 20);
            for (auto& a : acc_ms) {
                a = 0;
            }
        }
    }
    if (ix->n_total != 0 && ix->n_stored != 0) {
        ix->last_scan_bytes = static_cast<int64_t>(scalars[0]);
        ix->last_scanned_bytes = static_cast<int64_t>(ws.pruning ? scalars[3] : scalars[0]);
        if (scalars[4] != 0) {
            VB_FAIL(VB200_INTERNAL_ERROR, "the tensor-core scan gave up on a bounded wait");
        }
    }
    return 0;
}
