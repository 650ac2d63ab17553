// Exact BruteForce kNN over fp32 or bf16 rows: dense score slabs select a few candidates more
// than k per query, which are then re-scored in the reference's arithmetic and ordered.
#include <algorithm>
#include <vector>

#include "dense.cuh"
#include "kmeans.cuh"
#include "comm.cuh"
#include "tc_gemm.cuh"

namespace vb200 {

constexpr uint32_t BF_SLACK = 16;                 // candidates kept beyond k before re-scoring
constexpr uint64_t BF_COL_CHUNK = uint64_t{1} << 20;
constexpr uint64_t BF_SLAB_FLOATS = uint64_t{256} << 20;  // 1 GiB of scores

// generic::FloatToBF16 (src/simd/generic.cpp:198-202): add 0x8000, keep the high half.
__global__ void
float_to_bf16_kernel(const float* __restrict__ in, uint64_t n, uint16_t* __restrict__ out) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = static_cast<uint16_t>((__float_as_uint(in[i]) + 0x8000u) >> 16);
    }
}

// One CTA per query, one thread per candidate: distance as the reference computes it for one
// row -- an FMA chain over the dimensions in ascending order
// (FP32Quantizer::ComputeDistImpl, src/quantization/fp32_quantizer.cpp:163-190;
// HalfPrecisionQuantizer, src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123)
// -- then a sort by (distance, row).
template <typename T>
__global__ void __launch_bounds__(128)
bf_rescore_kernel(const T* __restrict__ queries, uint32_t dim, const T* __restrict__ base,
                  const uint64_t* __restrict__ cand, uint32_t ncand, uint32_t n2, uint32_t k,
                  int metric, uint64_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    float* qf = reinterpret_cast<float*>(keys + n2);   // the query, widened once
    const T* q = queries + static_cast<uint64_t>(blockIdx.x) * dim;
    const uint64_t* cq = cand + static_cast<uint64_t>(blockIdx.x) * ncand;
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        qf[d] = widen(q[d]);
    }
    __syncthreads();
    constexpr uint32_t VEC = 16 / sizeof(T);           // elements per 16-byte load
    const bool wide_loads = dim % VEC == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0;
    for (uint32_t i = threadIdx.x; i < n2; i += blockDim.x) {
        uint64_t key = KEY_INF;
        // candidates with an infinite nominating score are filtered-out rows that only filled up a
        // short list: they are not results
        if (i < ncand && cq[i] != KEY_INF && static_cast<uint32_t>(cq[i] >> 32) < 0xFF800000u) {
            uint32_t row = static_cast<uint32_t>(cq[i]);
            const T* x = base + static_cast<uint64_t>(row) * dim;
            float s = 0.f;
            const bool l2 = metric == VB200_METRIC_L2;
            if (wide_loads) {
                // same chain, rows fetched sixteen bytes at a time with a few loads in flight
                const uint4* xv = reinterpret_cast<const uint4*>(x);
                const uint32_t nv = dim / VEC;
                for (uint32_t v0 = 0; v0 < nv; v0 += 4) {
                    uint4 w[4];
#pragma unroll
                    for (uint32_t u = 0; u < 4; ++u) {
                        w[u] = v0 + u < nv ? __ldg(xv + v0 + u) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (uint32_t u = 0; u < 4; ++u) {
                        if (v0 + u < nv) {
                            T e[VEC];
                            *reinterpret_cast<uint4*>(e) = w[u];
                            const float* qq = qf + (v0 + u) * VEC;
#pragma unroll
                            for (uint32_t j = 0; j < VEC; ++j) {
                                if (l2) {
                                    float t = __fsub_rn(widen(e[j]), qq[j]);
                                    s = fmaf(t, t, s);
                                } else {
                                    s = fmaf(widen(e[j]), qq[j], s);
                                }
                            }
                        }
                    }
                }
            } else if (l2) {
                for (uint32_t d = 0; d < dim; ++d) {
                    float t = __fsub_rn(widen(x[d]), qf[d]);
                    s = fmaf(t, t, s);
                }
            } else {
                for (uint32_t d = 0; d < dim; ++d) {
                    s = fmaf(widen(x[d]), qf[d], s);
                }
            }
            if (!l2) {
                s = __fsub_rn(1.0f, s);
            }
            key = make_key(s, row);
        }
        keys[i] = key;
    }
    block_bitonic_sort(keys, n2);
    uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        dst[i] = i < n2 ? keys[i] : KEY_INF;
    }
}

template <typename T>
static int
bf_rescore(const T* queries, uint64_t nq, uint32_t dim, const T* base, const uint64_t* cand, uint32_t ncand, uint32_t n2,
           uint32_t k, int metric, uint64_t* out) {
    const size_t smem = n2 * sizeof(uint64_t) + dim * sizeof(float);
    VB_CHECK_ARG(smem <= 200 * 1024, "dim = %u is too large for the exact re-scoring step", dim);
    auto kernel = bf_rescore_kernel<T>;
    if (smem > 48 * 1024) {
        VB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    VB_LAUNCH(kernel, static_cast<uint32_t>(nq), 128, smem, queries, dim, base, cand, ncand, n2, k, metric, out);
    return 0;
}

// One block per query: the k best keys of its `per_query` partial keys and, when `prev` is given, of the k
// keys an earlier call left there (prev may be `out`).  bound_out[q], when asked for, is the score of the
// k-th key found, or +inf while fewer than k exist: no key scoring at or above it can enter the k best later.
__global__ void __launch_bounds__(256)
bf_merge_kernel(const uint64_t* __restrict__ part, uint64_t per_query, const uint64_t* prev, uint32_t k, uint32_t cap,
                uint64_t* out, float* __restrict__ bound_out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    uint32_t* state = reinterpret_cast<uint32_t*>(keys + cap);
    BlockSelect sel;
    sel.init(keys, state, k, cap);
    const uint64_t* src = part + static_cast<uint64_t>(blockIdx.x) * per_query;
    const uint64_t n_prev = prev != nullptr ? k : 0;
    const uint64_t* old = prev != nullptr ? prev + static_cast<uint64_t>(blockIdx.x) * k : nullptr;
    for (uint64_t base = 0; base < per_query + n_prev; base += blockDim.x) {
        sel.make_room(blockDim.x);
        uint64_t thr = sel.threshold();
        uint64_t i = base + threadIdx.x;
        if (i < per_query + n_prev) {
            uint64_t key = i < n_prev ? old[i] : __ldg(src + (i - n_prev));
            if (key != KEY_INF) {
                sel.offer(key, thr);
            }
        }
    }
    uint32_t cnt = sel.finish();
    uint64_t* dst = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t i = threadIdx.x; i < k; i += blockDim.x) {
        dst[i] = i < cnt ? keys[i] : KEY_INF;
    }
    if (bound_out != nullptr && threadIdx.x == 0) {
        bound_out[blockIdx.x] = cnt >= k ? ordered_to_float(static_cast<uint32_t>(keys[k - 1] >> 32)) : INFINITY;
    }
}

__global__ void
bf_results_kernel(const uint64_t* __restrict__ keys, uint64_t total, const int64_t* __restrict__ labels,
                  int64_t* __restrict__ ids, float* __restrict__ dists, uint64_t* __restrict__ keys_out) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= total) {
        return;
    }
    uint64_t key = keys[e];
    if (keys_out != nullptr) {
        keys_out[e] = key;
    }
    if (key == KEY_INF) {
        ids[e] = -1;
        if (dists != nullptr) {
            dists[e] = INFINITY;
        }
    } else {
        ids[e] = labels[static_cast<uint32_t>(key)];
        if (dists != nullptr) {
            dists[e] = ordered_to_float(static_cast<uint32_t>(key >> 32));
        }
    }
}

// bias[i] = the row's score bias (its squared norm for L2, 0 for IP), or +inf when row i is
// removed or filtered out: an infinite score is never nominated.
__global__ void
bf_masked_bias_kernel(const float* __restrict__ norms, uint64_t n, const uint32_t* __restrict__ tomb,
                      const uint32_t* __restrict__ deny, uint64_t deny_bits, const int64_t* __restrict__ labels,
                      const uint64_t* __restrict__ label_bits, uint64_t n_label_bits, float* __restrict__ bias) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    bool out = tomb != nullptr && ((tomb[i >> 5] >> (i & 31u)) & 1u);
    if (!out && deny != nullptr && i < deny_bits) {
        out = (deny[i >> 5] >> (i & 31u)) & 1u;
    }
    if (!out && label_bits != nullptr) {
        const uint64_t bit = static_cast<uint64_t>(labels[i]) & 0xFFFFFFFFull;
        out = bit < n_label_bits && ((label_bits[bit >> 6] >> (bit & 63u)) & 1ull);
    }
    bias[i] = out ? INFINITY : (norms != nullptr ? norms[i] : 0.f);
}

__global__ void
bf_tombstone_kernel(const int64_t* __restrict__ labels, uint64_t n, const int64_t* __restrict__ sorted, uint64_t count,
                    uint32_t* __restrict__ tomb, unsigned long long* __restrict__ newly) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) {
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

}  // namespace vb200

using namespace vb200;

struct vb200_bf {
    uint32_t dim = 0;
    int metric = 0, quant = 0;
    // cosine: rows and queries are normalised, then it is the inner-product index
    // (FP32Quantizer / HalfPrecisionQuantizer with METRIC_TYPE_COSINE)
    bool cosine = false;
    DevBuf<float> q_unit;
    // removed rows (MARK_REMOVE) and the id filter of the running search
    DevBuf<uint32_t> tombstones;
    uint64_t tomb_words = 0, n_removed = 0;
    const vb200_filter* filter = nullptr;
    DevBuf<float> masked_bias;
    uint64_t n = 0;
    DevBuf<float> base_f32;
    DevBuf<uint16_t> base_bf16;
    DevBuf<float> norms;
    DevBuf<int64_t> labels;
    // search workspace
    DevBuf<float> q_f32, scores;
    DevBuf<uint16_t> q_bf16;
    DevBuf<uint64_t> part, cand, keys;
    // tensor-core path: the base (and per search the queries) as tiled bf16 terms
    DevBuf<uint16_t> base_hi, base_lo, q_hi, q_lo;
    bool tiled_valid = false;
    DevBuf<uint64_t> tc_out;
    DevBuf<uint64_t> sh_local, sh_all;   // sharded search: this rank's packed [keys | labels] and the gathered ones
    DevBuf<float> row_bound;   // per query: the kcand-th candidate score after the column ranges searched so far
    TcWorkspace tc;
    DevBuf<int64_t> out_ids;
    DevBuf<float> out_dists;
    std::mutex mu;
};

template <typename T>
static int
bf_grow(DevBuf<T>& buf, size_t keep, size_t need) {
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

extern "C" int
vb200_bf_create(uint32_t dim, int metric, int quant, vb200_bf_t* out) {
    VB_CHECK_ARG(out != nullptr, "null output handle");
    VB_CHECK_ARG(dim > 0, "dim must be positive");
    VB_CHECK_ARG(metric == VB200_METRIC_L2 || metric == VB200_METRIC_IP || metric == VB200_METRIC_COSINE,
                 "metric_type must be l2, ip or cosine (got %d)", metric);
    VB_CHECK_ARG(quant == VB200_QUANT_FP32 || quant == VB200_QUANT_BF16,
                 "base_quantization_type must be fp32 or bf16 for this engine (got %d)", quant);
    if (vb200_device_count() <= 0) {
        VB_FAIL(VB200_INTERNAL_ERROR, "no CUDA device available; this engine has no CPU path");
    }
    vb200_bf* ix = new (std::nothrow) vb200_bf();
    if (ix == nullptr) {
        VB_FAIL(VB200_NO_ENOUGH_MEMORY, "out of host memory");
    }
    ix->dim = dim;
    ix->metric = metric == VB200_METRIC_COSINE ? VB200_METRIC_IP : metric;
    ix->cosine = metric == VB200_METRIC_COSINE;
    ix->quant = quant;
    *out = ix;
    return 0;
}

extern "C" int
vb200_bf_destroy(vb200_bf_t ix) {
    delete ix;
    return 0;
}

static int
bf_append_labels_and_norms(vb200_bf* ix, const int64_t* ids, uint64_t count) {
    VB_TRY(bf_grow(ix->labels, ix->n, ix->n + count));
    VB_CUDA(cudaMemcpyAsync(ix->labels.ptr + ix->n, ids, count * sizeof(int64_t), cudaMemcpyDefault,
                            current_stream()));
    VB_TRY(bf_grow(ix->norms, ix->n, ix->n + count));
    if (ix->quant == VB200_QUANT_FP32) {
        VB_TRY(row_sqnorm_f32(ix->base_f32.ptr + ix->n * ix->dim, count, ix->dim, ix->norms.ptr + ix->n));
    } else {
        VB_TRY(row_sqnorm_bf16(ix->base_bf16.ptr + ix->n * ix->dim, count, ix->dim, ix->norms.ptr + ix->n));
    }
    {
        // tombstone words for the new rows
        const uint64_t words = (ix->n + count + 31) / 32;
        if (words > ix->tomb_words) {
            DevBuf<uint32_t> bigger;
            const uint64_t cap = words * 2;
            VB_TRY(bigger.reserve(cap));
            VB_CUDA(cudaMemsetAsync(bigger.ptr, 0, cap * sizeof(uint32_t), current_stream()));
            if (ix->tomb_words > 0) {
                VB_CUDA(cudaMemcpyAsync(bigger.ptr, ix->tombstones.ptr, ix->tomb_words * sizeof(uint32_t),
                                        cudaMemcpyDeviceToDevice, current_stream()));
            }
            VB_TRY(sync_stream());
            ix->tombstones = std::move(bigger);
            ix->tomb_words = cap;
        }
    }
    VB_TRY(sync_stream());
    ix->n += count;
    ix->tiled_valid = false;
    return 0;
}

extern "C" int
vb200_bf_add(vb200_bf_t ix, const float* data, uint64_t count, const int64_t* ids) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(data != nullptr && ids != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    VB_CHECK_ARG(ix->n + count < 0xFFFFFFFFull, "index would exceed 2^32-1 vectors");
    const uint64_t elems = count * ix->dim;
    if (ix->quant == VB200_QUANT_FP32 && !ix->cosine) {
        VB_TRY(bf_grow(ix->base_f32, ix->n * ix->dim, (ix->n + count) * ix->dim));
        VB_CUDA(cudaMemcpyAsync(ix->base_f32.ptr + ix->n * ix->dim, data, elems * sizeof(float),
                                cudaMemcpyDefault, current_stream()));
    } else {
        DevInput<float> x;
        VB_TRY(x.bind(data, elems));
        DevBuf<float> unit_rows;
        const float* xr = x.ptr;
        if (ix->quant == VB200_QUANT_FP32) {
            VB_TRY(bf_grow(ix->base_f32, ix->n * ix->dim, (ix->n + count) * ix->dim));
            VB_TRY(normalize_rows_f32(x.ptr, count, ix->dim, ix->base_f32.ptr + ix->n * ix->dim));
        } else {
            if (ix->cosine) {
                VB_TRY(unit_rows.reserve(elems));
                VB_TRY(normalize_rows_f32(x.ptr, count, ix->dim, unit_rows.ptr));
                xr = unit_rows.ptr;
            }
            VB_TRY(bf_grow(ix->base_bf16, ix->n * ix->dim, (ix->n + count) * ix->dim));
            uint64_t blocks = (elems + 255) / 256;
            VB_CHECK_ARG(blocks <= 0x7fffffffu, "add batch too large");
            VB_LAUNCH(float_to_bf16_kernel, static_cast<uint32_t>(blocks), 256, 0, xr, elems,
                      ix->base_bf16.ptr + ix->n * ix->dim);
        }
        VB_TRY(sync_stream());
    }
    return bf_append_labels_and_norms(ix, ids, count);
}

extern "C" int
vb200_bf_add_bf16(vb200_bf_t ix, const uint16_t* data, uint64_t count, const int64_t* ids) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(data != nullptr && ids != nullptr, "null pointer");
    VB_CHECK_ARG(ix->quant == VB200_QUANT_BF16, "index does not store bf16 rows");
    VB_CHECK_ARG(!ix->cosine, "a cosine index normalises fp32 rows before rounding them: add them with vb200_bf_add");
    std::lock_guard<std::mutex> lock(ix->mu);
    VB_CHECK_ARG(ix->n + count < 0xFFFFFFFFull, "index would exceed 2^32-1 vectors");
    VB_TRY(bf_grow(ix->base_bf16, ix->n * ix->dim, (ix->n + count) * ix->dim));
    VB_CUDA(cudaMemcpyAsync(ix->base_bf16.ptr + ix->n * ix->dim, data, count * ix->dim * sizeof(uint16_t),
                            cudaMemcpyDefault, current_stream()));
    return bf_append_labels_and_norms(ix, ids, count);
}

extern "C" int
vb200_bf_get_rows(vb200_bf_t ix, void* rows) {
    VB_CHECK_ARG(ix != nullptr && rows != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n == 0) {
        return 0;
    }
    const uint64_t elems = ix->n * ix->dim;
    if (ix->quant == VB200_QUANT_FP32) {
        VB_TRY(copy_out(static_cast<float*>(rows), ix->base_f32.ptr, elems));
    } else {
        VB_TRY(copy_out(static_cast<uint16_t*>(rows), ix->base_bf16.ptr, elems));
    }
    return sync_stream();
}

extern "C" int
vb200_bf_set_rows(vb200_bf_t ix, const void* rows, uint64_t count, const int64_t* ids) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n != 0) {
        VB_FAIL(VB200_WRONG_STATUS, "stored rows can only be loaded into an empty index");
    }
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(rows != nullptr && ids != nullptr, "null pointer");
    VB_CHECK_ARG(count < 0xFFFFFFFFull, "index would exceed 2^32-1 vectors");
    const uint64_t elems = count * ix->dim;
    if (ix->quant == VB200_QUANT_FP32) {
        VB_TRY(bf_grow(ix->base_f32, 0, elems));
        VB_CUDA(cudaMemcpyAsync(ix->base_f32.ptr, rows, elems * sizeof(float), cudaMemcpyDefault, current_stream()));
    } else {
        VB_TRY(bf_grow(ix->base_bf16, 0, elems));
        VB_CUDA(cudaMemcpyAsync(ix->base_bf16.ptr, rows, elems * sizeof(uint16_t), cudaMemcpyDefault,
                                current_stream()));
    }
    return bf_append_labels_and_norms(ix, ids, count);
}

extern "C" int64_t
vb200_bf_num_elements(vb200_bf_t ix) {
    return ix == nullptr ? 0 : static_cast<int64_t>(ix->n - ix->n_removed);
}

extern "C" int
vb200_bf_remove(vb200_bf_t ix, const int64_t* labels, uint64_t count, uint64_t* removed) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    if (removed != nullptr) {
        *removed = 0;
    }
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(labels != nullptr, "null pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    if (ix->n == 0) {
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
    VB_LAUNCH(bf_tombstone_kernel, static_cast<uint32_t>((ix->n + 255) / 256), 256, 0, ix->labels.ptr, ix->n,
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

// Leaves the k best keys (payload = row) per query in ix->keys.
static int
bf_search_keys(vb200_bf* ix, const float* queries, uint64_t nq, uint32_t k) {
    const uint32_t dim = ix->dim;
    const uint64_t n = ix->n;
    uint32_t kcand = k + BF_SLACK;
    if (kcand > n) {
        kcand = static_cast<uint32_t>(n);
    }
    VB_CHECK_ARG(kcand <= 1024, "k = %u is too large (limit %u)", k, 1024 - BF_SLACK);
    const bool l2 = ix->metric == VB200_METRIC_L2;
    const bool bf16 = ix->quant == VB200_QUANT_BF16;

    const float* q_dev = queries;
    if (!is_device_pointer(queries)) {
        VB_TRY(ix->q_f32.reserve(nq * dim));
        VB_CUDA(cudaMemcpyAsync(ix->q_f32.ptr, queries, nq * dim * sizeof(float), cudaMemcpyHostToDevice,
                                current_stream()));
        q_dev = ix->q_f32.ptr;
    }
    if (ix->cosine) {
        VB_TRY(ix->q_unit.reserve(nq * dim));
        VB_TRY(normalize_rows_f32(q_dev, nq, dim, ix->q_unit.ptr));
        q_dev = ix->q_unit.ptr;
    }
    if (bf16) {
        VB_TRY(ix->q_bf16.reserve(nq * dim));
        VB_LAUNCH(float_to_bf16_kernel, static_cast<uint32_t>((nq * dim + 255) / 256), 256, 0, q_dev,
                  nq * dim, ix->q_bf16.ptr);
    }
    // score bias per row: |x|^2 for L2, none for IP; +inf for rows that are removed or filtered out
    const float* bias_all = l2 ? ix->norms.ptr : nullptr;
    {
        const vb200_filter* f = ix->filter;
        const bool user_deny = f != nullptr && f->deny_inner_bits != nullptr && f->n_inner_bits > 0;
        const bool user_labels = f != nullptr && f->invalid_label_bits != nullptr && f->n_label_bits > 0;
        if (ix->n_removed > 0 || user_deny || user_labels) {
            DevInput<uint32_t> deny;
            DevInput<uint64_t> lbits;
            if (user_deny) {
                VB_TRY(deny.bind(f->deny_inner_bits, (f->n_inner_bits + 31) / 32));
            }
            if (user_labels) {
                VB_TRY(lbits.bind(f->invalid_label_bits, (f->n_label_bits + 63) / 64));
            }
            VB_TRY(ix->masked_bias.reserve(n));
            VB_LAUNCH(bf_masked_bias_kernel, static_cast<uint32_t>((n + 255) / 256), 256, 0, bias_all, n,
                      ix->n_removed > 0 ? ix->tombstones.ptr : nullptr, user_deny ? deny.ptr : nullptr,
                      user_deny ? f->n_inner_bits : 0, ix->labels.ptr, user_labels ? lbits.ptr : nullptr,
                      user_labels ? f->n_label_bits : 0, ix->masked_bias.ptr);
            VB_TRY(sync_stream());   // the staged bitmaps end with this scope
            bias_all = ix->masked_bias.ptr;
        }
    }
    // Large problems nominate candidates on the tensor cores; the exact re-scoring below is the
    // same either way.
    if (tensor_cores_enabled() && kcand <= tc_max_candidates(bf16 ? 1 : 3) && static_cast<double>(nq) * n * dim >= 2e10) {
        const uint32_t chunks = (dim + TC_KC - 1) / TC_KC;
        if (!ix->tiled_valid) {
            const size_t elems = tc_tiled_elems(n, dim);
            VB_TRY(ix->base_hi.reserve(elems));
            if (bf16) {
                VB_TRY(tc_pretile_bf16(ix->base_bf16.ptr, n, dim, ix->base_hi.ptr));
            } else {
                VB_TRY(ix->base_lo.reserve(elems));
                VB_TRY(tc_pretile_f32(ix->base_f32.ptr, n, dim, ix->base_hi.ptr, ix->base_lo.ptr));
            }
            ix->tiled_valid = true;
        }
        const size_t q_elems = tc_tiled_elems(nq, dim);
        VB_TRY(ix->q_hi.reserve(q_elems));
        if (bf16) {
            VB_TRY(tc_pretile_bf16(ix->q_bf16.ptr, nq, dim, ix->q_hi.ptr));
        } else {
            VB_TRY(ix->q_lo.reserve(q_elems));
            VB_TRY(tc_pretile_f32(q_dev, nq, dim, ix->q_hi.ptr, ix->q_lo.ptr));
        }
        TcOperand a{ix->q_hi.ptr, bf16 ? nullptr : ix->q_lo.ptr, nq, chunks};
        VB_TRY(ix->cand.reserve(nq * kcand));
        VB_TRY(ix->row_bound.reserve(nq));
        // The base goes through the tensor cores in a few column ranges of growing size (a first one of about
        // a thousand rows, then sixteen times as many each time).  After each range the per-query candidate
        // lists are merged and the kcand-th score so far becomes the query's bound for the next range: no
        // column at or above it can be among the kcand best, so with rows in no particular order only about
        // 16 * kcand columns per query pass the bound in a range, and the kernel's per-row buffers hardly ever
        // need compacting.  Whatever the order of the rows, the result is the same set of candidates.
        const uint64_t n_tiles = (n + TC_BN - 1) / TC_BN;
        uint64_t len = n_tiles;
        if (n_tiles >= 1024) {
            len = 2 * kcand / TC_BN + 1 < 8 ? 8 : 2 * kcand / TC_BN + 1;
        }
        const uint32_t merge_cap = next_pow2(kcand + 256);
        const size_t merge_smem = merge_cap * sizeof(uint64_t) + 16;
        for (uint64_t tile0 = 0; tile0 < n_tiles; len *= 16) {
            uint64_t tile1 = tile0 + len;
            if (tile1 >= n_tiles || n_tiles - tile1 < len) {
                tile1 = n_tiles;   // no short last range
            }
            const uint64_t row0 = tile0 * TC_BN;
            const uint64_t rows = (tile1 * TC_BN < n ? tile1 * TC_BN : n) - row0;
            const size_t off = static_cast<size_t>(tile0) * chunks * TC_CHUNK_ELEMS;
            TcOperand b{ix->base_hi.ptr + off, bf16 ? nullptr : ix->base_lo.ptr + off, rows, chunks};
            const bool first = tile0 == 0;
            uint32_t lists = 1;
            VB_TRY(tc_candidates(ix->tc, a, b, bf16 ? 1 : 3, l2 ? -2.0f : -1.0f, bias_all != nullptr ? bias_all + row0 : nullptr,
                                 kcand, static_cast<uint32_t>(row0), ix->tc_out, &lists, nullptr, nullptr,
                                 first ? nullptr : ix->row_bound.ptr));
            VB_LAUNCH(bf_merge_kernel, static_cast<uint32_t>(nq), 256, merge_smem, ix->tc_out.ptr,
                      static_cast<uint64_t>(lists) * kcand, first ? static_cast<const uint64_t*>(nullptr) : ix->cand.ptr,
                      kcand, merge_cap, ix->cand.ptr, tile1 < n_tiles ? ix->row_bound.ptr : static_cast<float*>(nullptr));
            tile0 = tile1;
        }
        VB_TRY(ix->keys.reserve(nq * k));
        uint32_t n2 = next_pow2(kcand < 2 ? 2 : kcand);
        if (bf16) {
            VB_TRY(bf_rescore(ix->q_bf16.ptr, nq, dim, ix->base_bf16.ptr, ix->cand.ptr, kcand, n2, k, ix->metric, ix->keys.ptr));
        } else {
            VB_TRY(bf_rescore(q_dev, nq, dim, ix->base_f32.ptr, ix->cand.ptr, kcand, n2, k, ix->metric, ix->keys.ptr));
        }
        return 0;
    }
    const uint64_t col_chunk = n < BF_COL_CHUNK ? n : BF_COL_CHUNK;
    const uint32_t nchunks = static_cast<uint32_t>((n + col_chunk - 1) / col_chunk);
    uint64_t q_chunk = BF_SLAB_FLOATS / col_chunk;
    if (q_chunk < 1) {
        q_chunk = 1;
    }
    if (q_chunk > nq) {
        q_chunk = nq;
    }
    VB_TRY(ix->scores.reserve(q_chunk * col_chunk));
    const uint32_t keys_ld = nchunks * kcand;
    VB_TRY(ix->part.reserve(nq * keys_ld));
    for (uint64_t qb = 0; qb < nq; qb += q_chunk) {
        const uint64_t qn = nq - qb < q_chunk ? nq - qb : q_chunk;
        for (uint32_t c = 0; c < nchunks; ++c) {
            const uint64_t c0 = static_cast<uint64_t>(c) * col_chunk;
            const uint64_t cn = n - c0 < col_chunk ? n - c0 : col_chunk;
            const float* bias = bias_all != nullptr ? bias_all + c0 : nullptr;
            const float alpha = l2 ? -2.0f : -1.0f;
            if (bf16) {
                VB_TRY(dense_scores_bf16(ix->q_bf16.ptr + qb * dim, qn, ix->base_bf16.ptr + c0 * dim, cn,
                                         dim, alpha, bias, ix->scores.ptr, cn));
            } else {
                VB_TRY(dense_scores_f32(q_dev + qb * dim, qn, ix->base_f32.ptr + c0 * dim, cn, dim, alpha,
                                        bias, ix->scores.ptr, cn));
            }
            uint32_t kc = kcand < cn ? kcand : static_cast<uint32_t>(cn);
            if (kc < kcand) {  // short tail chunk: clear its slots first
                VB_CUDA(cudaMemset2DAsync(ix->part.ptr + qb * keys_ld + static_cast<uint64_t>(c) * kcand,
                                          keys_ld * sizeof(uint64_t), 0xFF, kcand * sizeof(uint64_t), qn,
                                          current_stream()));
            }
            VB_TRY(select_rows(ix->scores.ptr, qn, cn, cn, kc, static_cast<uint32_t>(c0),
                               ix->part.ptr + qb * keys_ld + static_cast<uint64_t>(c) * kcand, keys_ld));
        }
    }
    const uint64_t* cand = ix->part.ptr;
    if (nchunks > 1) {
        VB_TRY(ix->cand.reserve(nq * kcand));
        uint32_t cap = next_pow2(kcand + 256);
        size_t smem = cap * sizeof(uint64_t) + 16;
        VB_LAUNCH(bf_merge_kernel, static_cast<uint32_t>(nq), 256, smem, ix->part.ptr,
                  static_cast<uint64_t>(keys_ld), static_cast<const uint64_t*>(nullptr), kcand, cap, ix->cand.ptr,
                  static_cast<float*>(nullptr));
        cand = ix->cand.ptr;
    }
    VB_TRY(ix->keys.reserve(nq * k));
    uint32_t n2 = next_pow2(kcand < 2 ? 2 : kcand);
    if (bf16) {
        VB_TRY(bf_rescore(ix->q_bf16.ptr, nq, dim, ix->base_bf16.ptr, cand, kcand, n2, k, ix->metric, ix->keys.ptr));
    } else {
        VB_TRY(bf_rescore(q_dev, nq, dim, ix->base_f32.ptr, cand, kcand, n2, k, ix->metric, ix->keys.ptr));
    }
    return 0;
}

static int
bf_check_search(vb200_bf* ix, const float* queries, uint64_t nq, uint32_t k) {
    VB_CHECK_ARG(ix != nullptr, "null index");
    VB_CHECK_ARG(queries != nullptr || nq == 0, "query pointer is null");
    VB_CHECK_ARG(k >= 1, "k must be positive");
    return 0;
}

extern "C" int
vb200_bf_search(vb200_bf_t ix, const float* queries, uint64_t nq, uint32_t k, int64_t* ids,
                float* dists) {
    return vb200_bf_search_filtered(ix, queries, nq, k, nullptr, ids, dists);
}

extern "C" int
vb200_bf_search_filtered(vb200_bf_t ix, const float* queries, uint64_t nq, uint32_t k, const vb200_filter* filter,
                         int64_t* ids, float* dists) {
    VB_TRY(bf_check_search(ix, queries, nq, k));
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(ids != nullptr && dists != nullptr, "null output pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    const uint64_t total = nq * k;
    if (ix->n == 0) {
        std::vector<int64_t> hi(total, -1);
        std::vector<float> hd(total, INFINITY);
        VB_CUDA(cudaMemcpy(ids, hi.data(), total * sizeof(int64_t), cudaMemcpyDefault));
        VB_CUDA(cudaMemcpy(dists, hd.data(), total * sizeof(float), cudaMemcpyDefault));
        return 0;
    }
    ix->filter = filter;
    const int search_status = bf_search_keys(ix, queries, nq, k);
    ix->filter = nullptr;
    VB_TRY(search_status);
    VB_TRY(ix->out_ids.reserve(total));
    VB_TRY(ix->out_dists.reserve(total));
    VB_LAUNCH(bf_results_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, ix->keys.ptr, total,
              ix->labels.ptr, ix->out_ids.ptr, ix->out_dists.ptr, nullptr);
    VB_TRY(copy_out(ids, ix->out_ids.ptr, total));
    VB_TRY(copy_out(dists, ix->out_dists.ptr, total));
    return sync_stream();
}

extern "C" int
vb200_bf_search_partial(vb200_bf_t ix, const float* queries, uint64_t nq, uint32_t k,
                        uint64_t* keys_dev, int64_t* labels_dev) {
    VB_TRY(bf_check_search(ix, queries, nq, k));
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(keys_dev != nullptr && labels_dev != nullptr, "null output pointer");
    VB_CHECK_ARG(is_device_pointer(keys_dev) && is_device_pointer(labels_dev),
                 "partial results are written to device memory");
    std::lock_guard<std::mutex> lock(ix->mu);
    const uint64_t total = nq * k;
    if (ix->n == 0) {
        VB_CUDA(cudaMemsetAsync(keys_dev, 0xFF, total * sizeof(uint64_t), current_stream()));
        VB_CUDA(cudaMemsetAsync(labels_dev, 0xFF, total * sizeof(int64_t), current_stream()));
        return sync_stream();
    }
    VB_TRY(bf_search_keys(ix, queries, nq, k));
    VB_LAUNCH(bf_results_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, ix->keys.ptr, total,
              ix->labels.ptr, labels_dev, nullptr, keys_dev);
    return sync_stream();
}

extern "C" int
vb200_bf_search_sharded(vb200_bf_t ix, vb200_comm_t comm, const float* queries, uint64_t nq, uint32_t k,
                        int64_t* ids, float* dists) {
    VB_CHECK_ARG(comm != nullptr, "null communicator");
    if (comm->world == 1) {
        return vb200_bf_search(ix, queries, nq, k, ids, dists);
    }
    VB_TRY(bf_check_search(ix, queries, nq, k));
    if (nq == 0) {
        return 0;
    }
    VB_CHECK_ARG(ids != nullptr && dists != nullptr, "null output pointer");
    std::lock_guard<std::mutex> lock(ix->mu);
    cudaStream_t st = current_stream();
    const uint64_t total = nq * k;
    const uint32_t world = static_cast<uint32_t>(comm->world);
    VB_TRY(ix->sh_local.reserve(2 * total));
    VB_TRY(ix->sh_all.reserve(static_cast<size_t>(world) * 2 * total));
    if (ix->n == 0) {
        VB_CUDA(cudaMemsetAsync(ix->sh_local.ptr, 0xFF, 2 * total * sizeof(uint64_t), st));
    } else {
        VB_TRY(bf_search_keys(ix, queries, nq, k));
        VB_LAUNCH(bf_results_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, ix->keys.ptr, total,
                  ix->labels.ptr, reinterpret_cast<int64_t*>(ix->sh_local.ptr + total), nullptr, ix->sh_local.ptr);
    }
    VB_TRY(comm_all_gather(comm, ix->sh_local.ptr, ix->sh_all.ptr, 2 * total * sizeof(uint64_t), st));
    VB_TRY(merge_partials_device(ix->sh_all.ptr, reinterpret_cast<const int64_t*>(ix->sh_all.ptr + total), world,
                                 2 * total, nq, k, ids, dists));
    return sync_stream();
}
