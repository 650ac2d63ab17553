/*
 * vsag_oracle.c -- CPU restatement of the VSAG hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA engine: tests, the smoke check and the benchmark's
 * CPU-baseline leg call it; nothing in the product library links, loads or calls it.
 *
 * Every function restates, in plain C, the arithmetic of one reference routine (cited by its
 * path inside the antgroup/vsag tree).  Pinning:
 *   - SQ8 encode/decode is pinned by the reference's known-answer test
 *     (src/quantization/scalar_quantization/scalar_quantizer_test.cpp:101-116);
 *   - the distance kernels (SQ8/FP32/BF16/RaBitQ/normalize) are pinned against the reference's own
 *     src/simd sources compiled unchanged into oracle/_ref (tests/test_oracle_vs_ref.py and the
 *     committed fixtures under tests/golden/);
 *   - PARITY UNPINNED: the k-means assignment GEMM.  The reference calls an external BLAS
 *     (OpenBLAS cblas_sgemm, or an AMX bf16 kernel) whose summation order is not part of the
 *     tree and is not fixed by any reference test.  This file defines the canonical order as a
 *     sequential fp32 FMA chain over the dimensions; the engine reproduces that order bit for bit.
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off).
 * -ffp-contract=off matters: every fused multiply-add below is written as fmaf() explicitly so the
 * rounding sequence is the documented one, not whatever the compiler fuses.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* Seeded generators (std::mt19937 + libstdc++ distributions), so fixtures built like the       */
/* reference's tests/fixtures/data/vector_generator.h:55-70 can be produced without C++.        */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
    uint32_t mt[624];
    int idx;
} orc_mt19937;

static void
mt_seed(orc_mt19937* s, uint32_t seed) {
    s->mt[0] = seed;
    for (int i = 1; i < 624; ++i) {
        s->mt[i] = 1812433253u * (s->mt[i - 1] ^ (s->mt[i - 1] >> 30)) + (uint32_t)i;
    }
    s->idx = 624;
}

static uint32_t
mt_next(orc_mt19937* s) {
    if (s->idx >= 624) {
        for (int i = 0; i < 624; ++i) {
            uint32_t y = (s->mt[i] & 0x80000000u) | (s->mt[(i + 1) % 624] & 0x7fffffffu);
            uint32_t v = s->mt[(i + 397) % 624] ^ (y >> 1);
            if (y & 1u) {
                v ^= 0x9908b0dfu;
            }
            s->mt[i] = v;
        }
        s->idx = 0;
    }
    uint32_t y = s->mt[s->idx++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}

/* libstdc++ std::generate_canonical<float,24>(mt19937): one 32-bit draw, float(x)/2^32, and the
 * value 1.0f (reached when float(x) rounds up to 2^32) replaced by the largest float below 1. */
static float
mt_canonical(orc_mt19937* s) {
    float r = (float)mt_next(s) / 4294967296.0f;
    if (r >= 1.0f) {
        r = nextafterf(1.0f, 0.0f);
    }
    return r;
}

/* std::uniform_real_distribution<float>(lo, hi) filled in row-major order. */
ORC_API void
orc_gen_uniform(uint32_t seed, uint64_t count, float lo, float hi, float* out) {
    orc_mt19937 s;
    mt_seed(&s, seed);
    for (uint64_t i = 0; i < count; ++i) {
        out[i] = mt_canonical(&s) * (hi - lo) + lo;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Scalar distance kernels: canonical scalar order of src/simd/generic.cpp                      */
/* ------------------------------------------------------------------------------------------ */

/* FP32ComputeL2Sqr, scalar order (src/simd/kernels/compute_l2.h:27-78 with Width 1). */
ORC_API float
orc_fp32_l2sqr(const float* a, const float* b, uint64_t dim) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float d = a[i] - b[i];
        sum = fmaf(d, d, sum);
    }
    return sum;
}

/* Normalize (src/simd/generic.cpp:875-879) row by row: norm = sqrt(FP32ComputeIP(x, x)), every
 * element divided by it; a zero norm divides by 1 (src/simd/kernels/scalar_op.h:40-42). */
ORC_API void
orc_normalize_rows(const float* x, uint64_t n, uint64_t dim, float* out) {
    for (uint64_t r = 0; r < n; ++r) {
        const float* a = x + r * dim;
        float s = 0.0f;
        for (uint64_t i = 0; i < dim; ++i) {
            s = fmaf(a[i], a[i], s);
        }
        float norm = sqrtf(s);
        if (norm == 0.0f) {
            norm = 1.0f;
        }
        for (uint64_t i = 0; i < dim; ++i) {
            out[r * dim + i] = a[i] / norm;
        }
    }
}

/* FP32ComputeIP, scalar order (src/simd/kernels/compute_ip.h:38-92 with Width 1). */
ORC_API float
orc_fp32_ip(const float* a, const float* b, uint64_t dim) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        sum = fmaf(a[i], b[i], sum);
    }
    return sum;
}

/* SQ8ComputeL2Sqr (src/simd/kernels/sq8_compute.h:92-137): decode on the fly,
 * x = fma(code * (1/255), diff, lower), d = q - x, sum = fma(d, d, sum). */
ORC_API float
orc_sq8_l2sqr(const float* q, const uint8_t* code, const float* lower, const float* diff, uint64_t dim) {
    const float inv255 = 1.0f / 255.0f;
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float normalized = (float)code[i] * inv255;
        float adjusted = fmaf(normalized, diff[i], lower[i]);
        float d = q[i] - adjusted;
        sum = fmaf(d, d, sum);
    }
    return sum;
}

/* SQ8ComputeIP (src/simd/kernels/sq8_compute.h:44-88). */
ORC_API float
orc_sq8_ip(const float* q, const uint8_t* code, const float* lower, const float* diff, uint64_t dim) {
    const float inv255 = 1.0f / 255.0f;
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float normalized = (float)code[i] * inv255;
        float adjusted = fmaf(normalized, diff[i], lower[i]);
        sum = fmaf(q[i], adjusted, sum);
    }
    return sum;
}

/* generic::FloatToBF16 (src/simd/generic.cpp:198-202): add 0x8000 and truncate, i.e. round half
 * up in magnitude, no NaN special case. */
ORC_API uint16_t
orc_float_to_bf16(float v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    return (uint16_t)((bits + 0x8000u) >> 16);
}

/* generic::BF16ToFloat (src/simd/generic.cpp:191-196). */
ORC_API float
orc_bf16_to_float(uint16_t v) {
    uint32_t bits = ((uint32_t)v) << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API void
orc_float_to_bf16_batch(const float* in, uint64_t n, uint16_t* out) {
    for (uint64_t i = 0; i < n; ++i) {
        out[i] = orc_float_to_bf16(in[i]);
    }
}

/* BF16ComputeIP (src/simd/kernels/half_compute.h:31-62): widen both sides, fp32 FMA. */
ORC_API float
orc_bf16_ip(const uint16_t* a, const uint16_t* b, uint64_t dim) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        sum = fmaf(orc_bf16_to_float(a[i]), orc_bf16_to_float(b[i]), sum);
    }
    return sum;
}

/* BF16ComputeL2Sqr (src/simd/kernels/half_compute.h:64-94). */
ORC_API float
orc_bf16_l2sqr(const uint16_t* a, const uint16_t* b, uint64_t dim) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float d = orc_bf16_to_float(a[i]) - orc_bf16_to_float(b[i]);
        sum = fmaf(d, d, sum);
    }
    return sum;
}

/* ------------------------------------------------------------------------------------------ */
/* SQ8 quantizer                                                                               */
/* ------------------------------------------------------------------------------------------ */

static int
cmp_float_asc(const void* a, const void* b) {
    float x = *(const float*)a, y = *(const float*)b;
    return (x > y) - (x < y);
}

/* ScalarQuantizationTrainer::Train (src/quantization/scalar_quantization/
 * scalar_quantization_trainer.cpp:31-146) followed by ScalarQuantizer::TrainImpl's
 * diff = upper - lower (scalar_quantizer.cpp:51-74).
 * Sampling: at most 100000 rows, row j of the sample is row (j * (2147483647 % n)) % n.
 * mode 1 = CLASSIC (min/max); mode 3 = TRUNC_BOUND (default): upper = m-th largest and
 * lower = m-th smallest sampled value with m = max(1, floor((cnt-1) * 0.001)).  The reference's
 * two bounded heaps compute exactly these order statistics for finite inputs. */
ORC_API int
orc_sq8_train(const float* data, uint64_t count, uint64_t dim, int mode, float* lower, float* diff) {
    if (data == NULL || count == 0) {
        return -1;
    }
    const uint64_t max_sample = 100000;
    uint64_t step = 2147483647ULL % count;
    uint64_t cnt = max_sample;
    if (count <= max_sample) {
        step = 1;
        cnt = count;
    }
    float* col = (float*)malloc(cnt * sizeof(float));
    if (col == NULL) {
        return -2;
    }
    uint64_t ignore = (uint64_t)((double)(cnt - 1) * 0.001);
    if (ignore < 1) {
        ignore = 1;
    }
    for (uint64_t d = 0; d < dim; ++d) {
        for (uint64_t j = 0; j < cnt; ++j) {
            col[j] = data[((j * step) % count) * dim + d];
        }
        float up, lo;
        if (mode == 1) {
            up = -FLT_MAX;
            lo = FLT_MAX;
            for (uint64_t j = 0; j < cnt; ++j) {
                up = col[j] > up ? col[j] : up;
                lo = col[j] < lo ? col[j] : lo;
            }
        } else {
            qsort(col, cnt, sizeof(float), cmp_float_asc);
            up = col[cnt - ignore];
            lo = col[ignore - 1];
        }
        lower[d] = lo;
        diff[d] = up - lo;
    }
    free(col);
    return 0;
}

/* ScalarQuantizer<metric,8>::EncodeOneImpl (scalar_quantizer.cpp:85-110) with
 * ClampScalarQuantizationDelta (scalar_quantization_utils.h:19-30). */
ORC_API void
orc_sq8_encode(const float* data,
               uint64_t count,
               uint64_t dim,
               const float* lower,
               const float* diff,
               uint8_t* codes) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)count; ++i) {
        const float* x = data + (uint64_t)i * dim;
        uint8_t* c = codes + (uint64_t)i * dim;
        for (uint64_t d = 0; d < dim; ++d) {
            float delta;
            if (diff[d] < FLT_EPSILON) {
                delta = 1.0f;
            } else {
                delta = 1.0f * (x[d] - lower[d]) / diff[d];
            }
            if (!(delta >= 0.0f)) {
                delta = 0.0f;
            } else if (delta > 0.999f) {
                delta = 1.0f;
            }
            c[d] = (uint8_t)(255.0f * delta);
        }
    }
}

/* ScalarQuantizer::DecodeOneImpl (scalar_quantizer.cpp:112-124). */
ORC_API void
orc_sq8_decode(const uint8_t* codes,
               uint64_t count,
               uint64_t dim,
               const float* lower,
               const float* diff,
               float* out) {
    for (uint64_t i = 0; i < count; ++i) {
        for (uint64_t d = 0; d < dim; ++d) {
            out[i * dim + d] = (float)codes[i * dim + d] / (256.0f - 1.0f) * diff[d] + lower[d];
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* k-means (src/impl/cluster/kmeans_cluster.cpp)                                               */
/* ------------------------------------------------------------------------------------------ */

/* find_nearest_one_with_blas (kmeans_cluster.cpp:192-305), canonical order:
 *   y_sqr[j] = chain of fmaf(c, c, .) over the dimensions           (:216-225)
 *   ip       = chain of fmaf(c_j[d], x_i[d], .)                     (the SGEMM at :262-275)
 *   score    = y_sqr[j] + (-2 * ip)   (one rounding; -2*ip is exact) (:283)
 *   label    = lowest j attaining the minimum (std::min_element, :284)
 * Returns sum over points of (min score + |x|^2) / n, accumulated in double (:281-303).
 * second[] (optional) receives the runner-up score minus the best, for near-tie reporting. */
ORC_API double
orc_kmeans_assign(const float* x,
                  uint64_t n,
                  uint64_t dim,
                  const float* centroids,
                  uint64_t k,
                  int32_t* labels,
                  float* best_score,
                  float* gap) {
    float* y_sqr = (float*)malloc(k * sizeof(float));
    for (uint64_t j = 0; j < k; ++j) {
        y_sqr[j] = orc_fp32_ip(centroids + j * dim, centroids + j * dim, dim);
    }
    double error = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : error)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const float* xi = x + (uint64_t)i * dim;
        float best = 0.0f, second = INFINITY;
        int32_t best_j = -1;
        for (uint64_t j = 0; j < k; ++j) {
            float ip = orc_fp32_ip(centroids + j * dim, xi, dim);
            float score = fmaf(-2.0f, ip, y_sqr[j]);
            if (best_j < 0 || score < best) {
                if (best_j >= 0) {
                    second = best;
                }
                best = score;
                best_j = (int32_t)j;
            } else if (score < second) {
                second = score;
            }
        }
        labels[i] = best_j;
        if (best_score != NULL) {
            best_score[i] = best;
        }
        if (gap != NULL) {
            gap[i] = second - best;
        }
        error += (double)(best + orc_fp32_ip(xi, xi, dim));
    }
    free(y_sqr);
    return error / (double)(float)n;
}

/* Centroid update (kmeans_cluster.cpp:106-172): per-cluster fp32 sums, then scale by
 * 1.0f / count.  The reference adds 1024-point partial sums in thread-completion order, so its
 * own centroids are reproducible only to rounding; here rows are added in ascending row order.
 * Empty clusters: the reference draws a random data row from std::random_device (:156-170);
 * the deterministic rule used here (and by the engine) is row (j * 2654435761 + iter) % n. */
ORC_API void
orc_kmeans_update(const float* x,
                  uint64_t n,
                  uint64_t dim,
                  const int32_t* labels,
                  uint64_t k,
                  uint32_t iter,
                  float* centroids,
                  int32_t* counts) {
    float* sums = (float*)calloc(k * dim, sizeof(float));
    memset(counts, 0, k * sizeof(int32_t));
    for (uint64_t i = 0; i < n; ++i) {
        int32_t l = labels[i];
        if (l >= 0 && (uint64_t)l < k) {
            counts[l]++;
            float* s = sums + (uint64_t)l * dim;
            const float* xi = x + i * dim;
            for (uint64_t d = 0; d < dim; ++d) {
                s[d] = s[d] + xi[d];
            }
        }
    }
    for (uint64_t j = 0; j < k; ++j) {
        if (counts[j] > 0) {
            float inv = 1.0f / (float)counts[j];
            for (uint64_t d = 0; d < dim; ++d) {
                centroids[j * dim + d] = sums[j * dim + d] * inv;
            }
        } else {
            uint64_t row = (j * 2654435761ULL + (uint64_t)iter) % n;
            memcpy(centroids + j * dim, x + row * dim, dim * sizeof(float));
        }
    }
    free(sums);
}

/* KMeansCluster::Run (kmeans_cluster.cpp:46-190) with the initial centroids supplied by the
 * caller (the reference seeds k-means++ from std::random_device, :75-82).  labels_per_iter, when
 * not NULL, receives the n labels of every iteration back to back. */
ORC_API double
orc_kmeans_run(const float* x,
               uint64_t n,
               uint64_t dim,
               uint64_t k,
               int iters,
               float* centroids,
               int32_t* labels,
               int32_t* labels_per_iter) {
    int32_t* counts = (int32_t*)malloc(k * sizeof(int32_t));
    double err = 0.0;
    for (int it = 0; it < iters; ++it) {
        err = orc_kmeans_assign(x, n, dim, centroids, k, labels, NULL, NULL);
        if (labels_per_iter != NULL) {
            memcpy(labels_per_iter + (uint64_t)it * n, labels, n * sizeof(int32_t));
        }
        orc_kmeans_update(x, n, dim, labels, k, (uint32_t)it, centroids, counts);
    }
    free(counts);
    return err;
}

/* libstdc++ std::uniform_int_distribution<uint64_t>(0, n - 1) over mt19937 for n <= 2^32: the
 * generator's range covers the request, so one 32-bit draw is scaled by the multiply-and-reject
 * method of Lemire ("Fast random integer generation in an interval", 2019). */
static uint64_t
mt_uniform_index(orc_mt19937* s, uint64_t n) {
    uint32_t range = (uint32_t)n; /* n == 2^32 wraps to 0: every draw is accepted as it is */
    if (n >= 4294967296ull) {
        return mt_next(s);
    }
    uint64_t product = (uint64_t)mt_next(s) * range;
    uint32_t low = (uint32_t)product;
    if (low < range) {
        uint32_t threshold = (uint32_t)(0u - range) % range;
        while (low < threshold) {
            product = (uint64_t)mt_next(s) * range;
            low = (uint32_t)product;
        }
    }
    return product >> 32;
}

/* libstdc++ std::uniform_real_distribution<double>(0, hi) over mt19937:
 * generate_canonical<double,53> takes two 32-bit draws, low word first, sums them in double
 * (rounding the 64-bit value to 53 bits), divides by 2^64 and replaces 1.0 by the double below. */
static double
mt_uniform_double(orc_mt19937* s, double hi) {
    double sum = (double)mt_next(s);
    sum += (double)mt_next(s) * 4294967296.0;
    double r = sum / 18446744073709551616.0;
    if (r >= 1.0) {
        r = nextafter(1.0, 0.0);
    }
    return hi * r + 0.0;
}

/* Draws exported so a test can hold them against the C++ library itself. */
ORC_API void
orc_std_draws(uint32_t seed, uint64_t n, uint64_t count, uint64_t* ints, double* reals) {
    orc_mt19937 s;
    mt_seed(&s, seed);
    for (uint64_t i = 0; i < count; ++i) {
        ints[i] = mt_uniform_index(&s, n);
        reals[i] = mt_uniform_double(&s, (double)(i + 1) * 1.5);
    }
}

/* KMeansCluster::select_initial_centroids_kmeans_plus_plus (kmeans_cluster.cpp:383-435) with the
 * generator seeded by the caller instead of std::random_device (:75-76): the first centre is a
 * uniform draw; every later one is the first row whose running sum of min squared distances
 * reaches a uniform draw from [0, total).  picked, when not NULL, receives the k row numbers. */
ORC_API void
orc_kmeans_pp_init(const float* x, uint64_t n, uint64_t dim, uint64_t k, uint32_t seed, float* centroids,
                   int64_t* picked) {
    orc_mt19937 s;
    mt_seed(&s, seed);
    float* min_d = (float*)malloc(n * sizeof(float));
    for (uint64_t i = 0; i < n; ++i) {
        min_d[i] = FLT_MAX;
    }
    uint64_t idx = mt_uniform_index(&s, n);
    memcpy(centroids, x + idx * dim, dim * sizeof(float));
    if (picked != NULL) {
        picked[0] = (int64_t)idx;
    }
    for (uint64_t c = 1; c < k; ++c) {
        const float* last = centroids + (c - 1) * dim;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < (int64_t)n; ++i) {
            float d = orc_fp32_l2sqr(x + (uint64_t)i * dim, last, dim);
            if (d < min_d[i]) {
                min_d[i] = d;
            }
        }
        double total = 0.0;
        for (uint64_t i = 0; i < n; ++i) {
            total += min_d[i];
        }
        if (total <= 0.0) {
            idx = mt_uniform_index(&s, n);
        } else {
            double threshold = mt_uniform_double(&s, total);
            double cumulative = 0.0;
            idx = n - 1;
            for (uint64_t i = 0; i < n; ++i) {
                cumulative += min_d[i];
                if (cumulative >= threshold) {
                    idx = i;
                    break;
                }
            }
        }
        memcpy(centroids + c * dim, x + idx * dim, dim * sizeof(float));
        if (picked != NULL) {
            picked[c] = (int64_t)idx;
        }
    }
    free(min_d);
}

/* ------------------------------------------------------------------------------------------ */
/* Bounded top-k with the reference's heap semantics                                           */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
    float dist;
    int64_t id;
} orc_rec;

typedef struct {
    orc_rec* a;
    int64_t size;
    int64_t cap;
} orc_heap;

static int
rec_less(orc_rec x, orc_rec y) { /* max-heap order on (dist, id) */
    return x.dist < y.dist || (x.dist == y.dist && x.id < y.id);
}

static void
heap_push(orc_heap* h, float dist, int64_t id) {
    int64_t i = h->size++;
    orc_rec r = {dist, id};
    while (i > 0) {
        int64_t p = (i - 1) / 2;
        if (!rec_less(h->a[p], r)) {
            break;
        }
        h->a[i] = h->a[p];
        i = p;
    }
    h->a[i] = r;
}

static void
heap_pop(orc_heap* h) {
    orc_rec r = h->a[--h->size];
    int64_t i = 0;
    for (;;) {
        int64_t c = 2 * i + 1;
        if (c >= h->size) {
            break;
        }
        if (c + 1 < h->size && rec_less(h->a[c], h->a[c + 1])) {
            ++c;
        }
        if (!rec_less(r, h->a[c])) {
            break;
        }
        h->a[i] = h->a[c];
        i = c;
    }
    if (h->size > 0) {
        h->a[i] = r;
    }
}

/* FlatBucketSearcher::Search's insert rule (src/algorithm/ivf/flat_bucket_searcher.cpp:62-104):
 * push when the heap holds fewer than k or dist < current top (strict), then pop down to k. */
static void
heap_offer_strict(orc_heap* h, int64_t k, float dist, int64_t id) {
    if (h->size < k || dist < h->a[0].dist) {
        heap_push(h, dist, id);
    }
    while (h->size > k) {
        heap_pop(h);
    }
}

/* StandardHeap<true,true>::Push (src/impl/heap/standard_heap.cpp:26-52), used by BruteForce:
 * a full heap drops dist > top; equal distances replace. */
static void
heap_offer_fixed(orc_heap* h, int64_t k, float dist, int64_t id) {
    if (h->size == k && dist > h->a[0].dist) {
        return;
    }
    heap_push(h, dist, id);
    if (h->size > k) {
        heap_pop(h);
    }
}

/* pack_knn_result (src/algorithm/inner_index_interface.cpp:1133-1147): pop the max-heap from the
 * back so the output is ascending; unused slots are id -1 / distance +inf like the IVF batch
 * branch (src/algorithm/ivf/ivf.cpp:2137-2210). */
static void
heap_drain(orc_heap* h, int64_t k, int64_t* ids, float* dists) {
    for (int64_t i = 0; i < k; ++i) {
        ids[i] = -1;
        dists[i] = INFINITY;
    }
    for (int64_t i = h->size - 1; i >= 0; --i) {
        ids[i] = h->a[0].id;
        dists[i] = h->a[0].dist;
        heap_pop(h);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Routing, IVF scan, rerank, brute force                                                      */
/* ------------------------------------------------------------------------------------------ */

typedef float (*orc_dist_fn)(const float*, const float*, uint64_t);
typedef float (*orc_sq8_fn)(const float*, const uint8_t*, const float*, const float*, uint64_t);

/* Exact routing: the nprobe nearest centroids in ascending distance order (ties: lower id).
 * Stands in for the reference's approximate HGraph router (src/algorithm/ivf/
 * ivf_nearest_partition.cpp:91-147) the way IVF::route_buckets_only recomputes centroid
 * distances with an exact scalar loop (src/algorithm/ivf/ivf.cpp:1589-1660).
 * metric: 0 = L2 squared, 1 = inner product (distance 1 - ip). */
ORC_API void
orc_route(const float* q,
          uint64_t nq,
          uint64_t dim,
          const float* centroids,
          uint64_t nlist,
          uint64_t nprobe,
          int metric,
          int32_t* out_ids,
          float* out_dists) {
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((nprobe + 2) * sizeof(orc_rec));
        h.cap = (int64_t)nprobe + 2;
        int64_t* ids = (int64_t*)malloc(nprobe * sizeof(int64_t));
        float* ds = (float*)malloc(nprobe * sizeof(float));
#pragma omp for schedule(dynamic, 4)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            h.size = 0;
            for (uint64_t j = 0; j < nlist; ++j) {
                float d = metric == 0 ? orc_fp32_l2sqr(q + (uint64_t)i * dim, centroids + j * dim, dim)
                                      : 1.0f - orc_fp32_ip(q + (uint64_t)i * dim, centroids + j * dim, dim);
                heap_offer_strict(&h, (int64_t)nprobe, d, (int64_t)j);
            }
            heap_drain(&h, (int64_t)nprobe, ids, ds);
            for (uint64_t p = 0; p < nprobe; ++p) {
                out_ids[(uint64_t)i * nprobe + p] = (int32_t)ids[p];
                if (out_dists != NULL) {
                    out_dists[(uint64_t)i * nprobe + p] = ds[p];
                }
            }
        }
        free(h.a);
        free(ids);
        free(ds);
    }
}

/* IVF-SQ8 search over an inverted file in CSR form:
 *   codes[list_off[l] .. list_off[l+1]) are the codes of list l in insertion order,
 *   inner_ids[] the matching ids (src/datacell/bucket_datacell.h:526-572 scan,
 *   src/algorithm/ivf/flat_bucket_searcher.cpp:26-138 selection, src/algorithm/ivf/ivf.cpp:1693-1828
 *   probe loop).  probes[q][0..nprobe) lists the buckets to scan in order (-1 = none).
 * metric 0: SQ8ComputeL2Sqr; metric 1: 1 - SQ8ComputeIP (scalar_quantizer.cpp:173-197).
 * fn == NULL uses this file's scalar kernels; a non-NULL fn lets the caller time the reference's
 * own compiled SIMD kernel inside the same loop.  nthreads <= 0 uses every core, one query per
 * worker like the reference's evaluation tool. */
ORC_API void
orc_ivf_sq8_search(const uint8_t* codes,
                   const int64_t* list_off,
                   const int64_t* inner_ids,
                   uint64_t dim,
                   const float* lower,
                   const float* diff,
                   const float* q,
                   uint64_t nq,
                   const int32_t* probes,
                   uint64_t nprobe,
                   int64_t k,
                   int metric,
                   orc_sq8_fn fn,
                   int nthreads,
                   int64_t* out_ids,
                   float* out_dists) {
    if (fn == NULL) {
        fn = metric == 0 ? orc_sq8_l2sqr : orc_sq8_ip;
    }
#ifdef _OPENMP
    if (nthreads <= 0) {
        nthreads = omp_get_max_threads();
    }
#else
    nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        h.cap = k + 2;
        float dist[32];
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            const float* qi = q + (uint64_t)i * dim;
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                int64_t b = list_off[l], e = list_off[l + 1];
                for (int64_t r = b; r < e; r += 32) { /* 32-code blocks, bucket_datacell.h:534-551 */
                    int64_t m = e - r < 32 ? e - r : 32;
                    for (int64_t t = 0; t < m; ++t) {
                        float v = fn(qi, codes + (uint64_t)(r + t) * dim, lower, diff, dim);
                        dist[t] = metric == 0 ? v : 1.0f - v;
                    }
                    for (int64_t t = 0; t < m; ++t) {
                        heap_offer_strict(&h, k, dist[t], inner_ids[r + t]);
                    }
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* use_residual (src/datacell/bucket_datacell.h): a bucket stores the codes of x - centroid.
 * Encoding (encode_vector, :621-651): residual = FP32Sub(x, c); codes = EncodeOne(residual); for L2 the row's
 * bias = -2 * IP(c, DecodeOne(codes)) - IP(c, c).  rows are the vectors as stored (normalised for cosine). */
ORC_API void
orc_sq8_residual_encode(const float* rows, uint64_t count, uint64_t dim, const int32_t* lists, const float* centroids,
                        const float* lower, const float* diff, int metric, uint8_t* codes, float* bias) {
    float* r = (float*)malloc(dim * sizeof(float));
    float* dec = (float*)malloc(dim * sizeof(float));
    for (uint64_t i = 0; i < count; ++i) {
        const float* c = centroids + (uint64_t)lists[i] * dim;
        for (uint64_t d = 0; d < dim; ++d) {
            r[d] = rows[i * dim + d] - c[d];
        }
        orc_sq8_encode(r, 1, dim, lower, diff, codes + i * dim);
        bias[i] = 0.0f;
        if (metric == 0) {
            orc_sq8_decode(codes + i * dim, 1, dim, lower, diff, dec);
            bias[i] = -2 * orc_fp32_ip(c, dec, dim) - orc_fp32_ip(c, c, dim);
        }
    }
    free(r);
    free(dec);
}

/* Residual rows of a training set (BucketDataCell::Train, :593-614): x - centroid of its nearest bucket. */
ORC_API void
orc_residual_rows(const float* rows, uint64_t count, uint64_t dim, const int32_t* lists, const float* centroids,
                  float* out) {
    for (uint64_t i = 0; i < count; ++i) {
        const float* c = centroids + (uint64_t)lists[i] * dim;
        for (uint64_t d = 0; d < dim; ++d) {
            out[i * dim + d] = rows[i * dim + d] - c[d];
        }
    }
}

/* ScanBucketById with use_residual (:526-572): the quantizer's distance between the raw query and the residual
 * code, minus the row's bias (L2), minus 2 * IP(q, c) (L2) or IP(q, c) (IP / cosine). */
ORC_API void
orc_ivf_sq8_residual_search(const uint8_t* codes,
                            const float* bias,
                            const int64_t* list_off,
                            const int64_t* inner_ids,
                            uint64_t dim,
                            const float* lower,
                            const float* diff,
                            const float* centroids,
                            const float* q,
                            uint64_t nq,
                            const int32_t* probes,
                            uint64_t nprobe,
                            int64_t k,
                            int metric,
                            int64_t* out_ids,
                            float* out_dists) {
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        h.cap = k + 2;
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            const float* qi = q + (uint64_t)i * dim;
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                float ipd = orc_fp32_ip(qi, centroids + (uint64_t)l * dim, dim);
                if (metric == 0) {
                    ipd *= 2;
                }
                for (int64_t r = list_off[l]; r < list_off[l + 1]; ++r) {
                    const uint8_t* c = codes + (uint64_t)r * dim;
                    float d = metric == 0 ? orc_sq8_l2sqr(qi, c, lower, diff, dim) : 1.0f - orc_sq8_ip(qi, c, lower, diff, dim);
                    if (metric == 0) {
                        d = d - bias[r];
                    }
                    d -= ipd;
                    heap_offer_strict(&h, k, d, inner_ids[r]);
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* The same probe loop over fp32 buckets (FP32Quantizer::ComputeDistImpl,
 * src/quantization/fp32_quantizer.cpp:163-190): rows[list_off[l] .. list_off[l+1]) are the rows of
 * list l as they were added. */
ORC_API void
orc_ivf_fp32_search(const float* rows,
                    const int64_t* list_off,
                    const int64_t* inner_ids,
                    uint64_t dim,
                    const float* q,
                    uint64_t nq,
                    const int32_t* probes,
                    uint64_t nprobe,
                    int64_t k,
                    int metric,
                    int64_t* out_ids,
                    float* out_dists) {
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        h.cap = k + 2;
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            const float* qi = q + (uint64_t)i * dim;
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                for (int64_t r = list_off[l]; r < list_off[l + 1]; ++r) {
                    const float* x = rows + (uint64_t)r * dim;
                    float d = metric == 0 ? orc_fp32_l2sqr(x, qi, dim) : 1.0f - orc_fp32_ip(x, qi, dim);
                    heap_offer_strict(&h, k, d, inner_ids[r]);
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* FlattenReorder::Reorder, simple path (src/impl/reorder/flatten_reorder.cpp:76-118): recompute
 * every candidate against the fp32 rows and keep the k best.  cand ids < 0 are skipped. */
ORC_API void
orc_rerank_fp32(const float* base,
                uint64_t dim,
                const float* q,
                uint64_t nq,
                const int64_t* cand,
                uint64_t ncand,
                int64_t k,
                int metric,
                int64_t* out_ids,
                float* out_dists) {
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            h.size = 0;
            for (uint64_t c = 0; c < ncand; ++c) {
                int64_t id = cand[(uint64_t)i * ncand + c];
                if (id < 0) {
                    continue;
                }
                float d = metric == 0 ? orc_fp32_l2sqr(q + (uint64_t)i * dim, base + (uint64_t)id * dim, dim)
                                      : 1.0f - orc_fp32_ip(q + (uint64_t)i * dim, base + (uint64_t)id * dim, dim);
                heap_offer_fixed(&h, k, d, id);
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* BruteForce::SearchWithRequest row loop (src/algorithm/bruteforce/bruteforce.cpp:481-597) over
 * fp32 rows (FP32Quantizer::ComputeDistImpl, src/quantization/fp32_quantizer.cpp:163-190):
 * metric 0 = sum (c-q)^2, metric 1 = 1 - sum c*q.  One query per worker thread. */
ORC_API void
orc_bf_search_fp32(const float* base,
                   uint64_t n,
                   uint64_t dim,
                   const float* q,
                   uint64_t nq,
                   int64_t k,
                   int metric,
                   orc_dist_fn fn,
                   int nthreads,
                   int64_t* out_ids,
                   float* out_dists) {
    if (fn == NULL) {
        fn = metric == 0 ? orc_fp32_l2sqr : orc_fp32_ip;
    }
#ifdef _OPENMP
    if (nthreads <= 0) {
        nthreads = omp_get_max_threads();
    }
#else
    nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            h.size = 0;
            for (uint64_t r = 0; r < n; ++r) {
                float v = fn(base + r * dim, q + (uint64_t)i * dim, dim);
                heap_offer_fixed(&h, k, metric == 0 ? v : 1.0f - v, (int64_t)r);
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* Same loop over bf16 codes (HalfPrecisionQuantizer<BF16Format>,
 * src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123): the query is rounded
 * to bf16 with FloatToBF16 too, products are widened to fp32. */
ORC_API void
orc_bf_search_bf16(const uint16_t* base,
                   uint64_t n,
                   uint64_t dim,
                   const float* q,
                   uint64_t nq,
                   int64_t k,
                   int metric,
                   int nthreads,
                   int64_t* out_ids,
                   float* out_dists) {
#ifdef _OPENMP
    if (nthreads <= 0) {
        nthreads = omp_get_max_threads();
    }
#else
    nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        uint16_t* qb = (uint16_t*)malloc(dim * sizeof(uint16_t));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            orc_float_to_bf16_batch(q + (uint64_t)i * dim, dim, qb);
            h.size = 0;
            for (uint64_t r = 0; r < n; ++r) {
                float v = metric == 0 ? orc_bf16_l2sqr(qb, base + r * dim, dim)
                                      : 1.0f - orc_bf16_ip(qb, base + r * dim, dim);
                heap_offer_fixed(&h, k, v, (int64_t)r);
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
        free(qb);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* SQ8 uniform: one lower bound and one range for all dimensions, integer inner products         */
/* ------------------------------------------------------------------------------------------ */

/* SQ8UniformQuantizer::TrainImpl (src/quantization/scalar_quantization/sq8_uniform_quantizer.cpp:76-100):
 * CLASSIC bounds of the sample (scalar_quantization_trainer.cpp:47-60: the largest per-dimension maximum and
 * the smallest per-dimension minimum, i.e. the extremes of the whole sample), diff = upper - lower.  Rows of
 * a cosine index are normalised before (metric 2).  model = {lower, diff}. */
ORC_API int
orc_sq8u_train(const float* data, uint64_t count, uint64_t dim, int metric, float* model) {
    if (data == NULL || count == 0) {
        return -1;
    }
    const uint64_t max_sample = 100000;
    uint64_t step = 2147483647ULL % count;
    uint64_t cnt = max_sample;
    if (count <= max_sample) {
        step = 1;
        cnt = count;
    }
    float up = -FLT_MAX, lo = FLT_MAX;
    float* row = (float*)malloc(dim * sizeof(float));
    for (uint64_t j = 0; j < cnt; ++j) {
        const float* x = data + ((j * step) % count) * dim;
        if (metric == 2) {
            orc_normalize_rows(x, 1, dim, row);
            x = row;
        }
        for (uint64_t d = 0; d < dim; ++d) {
            up = x[d] > up ? x[d] : up;
            lo = x[d] < lo ? x[d] : lo;
        }
    }
    free(row);
    model[0] = lo;
    model[1] = up - lo;
    return 0;
}

/* Code record (sq8_uniform_quantizer.cpp:32-60): the codes padded to the alignment of the trailing field,
 * then for L2 the uint64 sum of squared codes, for IP / cosine the fp32 sum of the (normalised) values. */
ORC_API uint64_t
orc_sq8u_code_size(uint64_t dim, int metric) {
    uint64_t align = metric == 0 ? 8 : 4;
    return (dim + align - 1) / align * align + align;
}

/* scalar_rate_ = (diff / 255.0) * (diff / 255.0), evaluated in double and stored as float (:96). */
ORC_API float
orc_sq8u_scalar_rate(float diff) {
    return (float)(((double)diff / 255.0) * ((double)diff / 255.0));
}

/* SQ8UniformQuantizer::EncodeOneImpl (:102-142), also used for the query (ProcessQueryImpl, :188-199). */
ORC_API void
orc_sq8u_encode(const float* data, uint64_t count, uint64_t dim, int metric, const float* model, uint8_t* codes) {
    const uint64_t cs = orc_sq8u_code_size(dim, metric);
    const float lower = model[0], diff = model[1];
    const float inv_diff = diff == 0.0f ? 0.0f : 1.0f / diff;
    float* row = (float*)malloc(dim * sizeof(float));
    for (uint64_t i = 0; i < count; ++i) {
        const float* x = data + i * dim;
        if (metric == 2) {
            orc_normalize_rows(x, 1, dim, row);
            x = row;
        }
        uint8_t* c = codes + i * cs;
        memset(c, 0, cs);
        uint64_t norm = 0;
        float sum = 0.0f;
        for (uint64_t d = 0; d < dim; ++d) {
            float delta = (x[d] - lower) * inv_diff;
            if (!(delta >= 0.0f)) {
                delta = 0.0f;
            } else if (delta > 0.999f) {
                delta = 1.0f;
            }
            uint8_t scaled = (uint8_t)(255.0f * delta);
            c[d] = scaled;
            norm += (uint64_t)scaled * (uint64_t)scaled;
            sum += x[d];
        }
        if (metric == 0) {
            memcpy(c + cs - 8, &norm, 8);
        } else {
            memcpy(c + cs - 4, &sum, 4);
        }
    }
    free(row);
}

/* generic::SQ8UniformComputeCodesIP (src/simd/generic.cpp:424-433): int32 sum of byte products. */
ORC_API float
orc_sq8u_codes_ip(const uint8_t* a, const uint8_t* b, uint64_t dim) {
    int32_t r = 0;
    for (uint64_t d = 0; d < dim; ++d) {
        r += (int32_t)a[d] * (int32_t)b[d];
    }
    return (float)r;
}

/* SQ8UniformQuantizer::ComputeImpl (:153-186). */
ORC_API float
orc_sq8u_dist(const uint8_t* q, const uint8_t* c, uint64_t dim, int metric, const float* model) {
    const uint64_t cs = orc_sq8u_code_size(dim, metric);
    const float rate = orc_sq8u_scalar_rate(model[1]);
    float result = orc_sq8u_codes_ip(q, c, dim);
    if (metric == 0) {
        uint64_t n1, n2;
        memcpy(&n1, q + cs - 8, 8);
        memcpy(&n2, c + cs - 8, 8);
        return ((float)n1 + (float)n2 - 2 * result) * rate;
    }
    float s1, s2;
    memcpy(&s1, q + cs - 4, 4);
    memcpy(&s2, c + cs - 4, 4);
    const float lower = model[0];
    result = lower * (s1 + s2) + rate * result + lower * lower;
    return 1 - result;
}

/* The probe loop over sq8_uniform buckets: the query is encoded like a row, distances are ComputeImpl's. */
ORC_API void
orc_ivf_sq8u_search(const uint8_t* codes,
                    const int64_t* list_off,
                    const int64_t* inner_ids,
                    uint64_t dim,
                    const float* model,
                    const float* q,
                    uint64_t nq,
                    const int32_t* probes,
                    uint64_t nprobe,
                    int64_t k,
                    int metric,
                    int64_t* out_ids,
                    float* out_dists) {
    const uint64_t cs = orc_sq8u_code_size(dim, metric);
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        h.cap = k + 2;
        uint8_t* qc = (uint8_t*)malloc(cs);
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            orc_sq8u_encode(q + (uint64_t)i * dim, 1, dim, metric, model, qc);
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                for (int64_t r = list_off[l]; r < list_off[l + 1]; ++r) {
                    float d = orc_sq8u_dist(qc, codes + (uint64_t)r * cs, dim, metric, model);
                    heap_offer_strict(&h, k, d, inner_ids[r]);
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
        free(qc);
    }
}

/* generic::FloatToFP16 (src/simd/generic.cpp:214-228): the exponent is clamped to [-14, 15] and the
 * mantissa truncated to 10 bits -- no rounding, no zero, denormal, infinity or NaN encodings (0.0f
 * becomes 2^-14).  Every code it writes is a normal number of IEEE half precision. */
ORC_API uint16_t
orc_float_to_fp16(float v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    uint32_t sign = (bits >> 31) & 1u;
    int32_t exp = (int32_t)((bits >> 23) & 0xFFu) - 127;
    uint32_t mantissa = bits & 0x007FFFFFu;
    if (exp > 15) {
        exp = 15;
    } else if (exp < -14) {
        exp = -14;
    }
    return (uint16_t)((sign << 15) | ((uint32_t)(exp + 15) << 10) | (mantissa >> 13));
}

/* generic::FP16ToFloat (src/simd/generic.cpp:204-212): rebias the exponent, widen the mantissa. */
ORC_API float
orc_fp16_to_float(uint16_t v) {
    uint32_t sign = (v >> 15) & 1u;
    int32_t exp = (int32_t)((v >> 10) & 0x1Fu) - 15;
    uint32_t mantissa = ((uint32_t)v & 0x3FFu) << 13;
    uint32_t bits = (sign << 31) | ((uint32_t)(exp + 127) << 23) | mantissa;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* fmt 0: bf16, 1: fp16 */
ORC_API void
orc_float_to_half_batch(const float* in, uint64_t n, int fmt, uint16_t* out) {
    for (uint64_t i = 0; i < n; ++i) {
        out[i] = fmt == 0 ? orc_float_to_bf16(in[i]) : orc_float_to_fp16(in[i]);
    }
}

static float
half_to_float(uint16_t v, int fmt) {
    return fmt == 0 ? orc_bf16_to_float(v) : orc_fp16_to_float(v);
}

/* HalfComputeIPImpl / HalfComputeL2SqrImpl in scalar width (src/simd/kernels/half_compute.h:31-94). */
ORC_API float
orc_half_ip(const uint16_t* a, const uint16_t* b, uint64_t dim, int fmt) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        sum = fmaf(half_to_float(a[i], fmt), half_to_float(b[i], fmt), sum);
    }
    return sum;
}

ORC_API float
orc_half_l2sqr(const uint16_t* a, const uint16_t* b, uint64_t dim, int fmt) {
    float sum = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float d = half_to_float(a[i], fmt) - half_to_float(b[i], fmt);
        sum = fmaf(d, d, sum);
    }
    return sum;
}

/* The probe loop over half-precision buckets (HalfPrecisionQuantizer,
 * src/quantization/scalar_quantization/half_precision_quantizer.cpp:54-123): the query is encoded like a
 * row (ProcessQueryImpl), the distance is ComputeL2Sqr or 1 - ComputeIP between the two codes.  Rows of a
 * cosine index were normalised before they were encoded; so is the query here (metric 2). */
ORC_API void
orc_ivf_half_search(const uint16_t* codes,
                    const int64_t* list_off,
                    const int64_t* inner_ids,
                    uint64_t dim,
                    const float* q,
                    uint64_t nq,
                    const int32_t* probes,
                    uint64_t nprobe,
                    int64_t k,
                    int metric,
                    int fmt,
                    int64_t* out_ids,
                    float* out_dists) {
#pragma omp parallel
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
        h.cap = k + 2;
        uint16_t* qh = (uint16_t*)malloc(dim * sizeof(uint16_t));
        float* qn = (float*)malloc(dim * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            const float* qi = q + (uint64_t)i * dim;
            if (metric == 2) {
                orc_normalize_rows(qi, 1, dim, qn);
                qi = qn;
            }
            orc_float_to_half_batch(qi, dim, fmt, qh);
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                for (int64_t r = list_off[l]; r < list_off[l + 1]; ++r) {
                    const uint16_t* x = codes + (uint64_t)r * dim;
                    float d = metric == 0 ? orc_half_l2sqr(qh, x, dim, fmt) : 1.0f - orc_half_ip(qh, x, dim, fmt);
                    heap_offer_strict(&h, k, d, inner_ids[r]);
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
        free(qh);
        free(qn);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* RaBitQ, 1 bit per dimension, fp32 query, "standard" layout                                   */
/* ------------------------------------------------------------------------------------------ */

/* Code record (src/quantization/rabitq_quantization/rabitq_quantizer.cpp:102-185):
 * ceil(D/8) sign bytes (dimension d -> byte d/8, bit d%8) padded to a multiple of 4, then the
 * fp32 norm, then the fp32 error term. */
ORC_API uint64_t
orc_rabitq_code_size(uint64_t dim) {
    return ((dim + 7) / 8 + 3) / 4 * 4 + 8;
}

/* RandomOrthogonalMatrix::Transform (src/impl/transform/random_orthogonal_transformer.cpp:59-77):
 * y = Q x, Q row-major.  The reference calls an external cblas_sgemv; the canonical order here is
 * a sequential fmaf chain per output row. */
ORC_API void
orc_rotate(const float* Q, const float* x, uint64_t dim, float* y) {
    for (uint64_t r = 0; r < dim; ++r) {
        y[r] = orc_fp32_ip(Q + r * dim, x, dim);
    }
}

/* NormalizeWithCentroid (src/simd/kernels/normalize.h:35-85), scalar order. */
ORC_API float
orc_normalize_with_centroid(const float* from, const float* centroid, float* to, uint64_t dim) {
    float norm_sq = 0.0f;
    for (uint64_t i = 0; i < dim; ++i) {
        float d = from[i] - centroid[i];
        norm_sq = fmaf(d, d, norm_sq);
    }
    float norm = norm_sq < 1e-5f ? 1.0f : sqrtf(norm_sq);
    for (uint64_t i = 0; i < dim; ++i) {
        to[i] = (from[i] - centroid[i]) / norm;
    }
    return norm;
}

/* generic::RaBitQFloatBinaryIP (src/simd/generic.cpp:447-471). */
ORC_API float
orc_rabitq_float_binary_ip(const float* v, const uint8_t* bits, uint64_t dim, float inv_sqrt_d) {
    if (dim == 0) {
        return 0.0f;
    }
    float pos, neg;
    if (inv_sqrt_d > 1e-3) {
        pos = inv_sqrt_d;
        neg = -inv_sqrt_d;
    } else {
        pos = 1.0f;
        neg = 0.0f;
    }
    float result = 0.0f;
    for (uint64_t d = 0; d < dim; ++d) {
        int bit = (bits[d / 8] >> (d % 8)) & 1;
        float b = bit ? pos : neg;
        result = result + b * v[d];
    }
    return result;
}

/* RaBitQuantizer::TrainImpl (rabitq_quantizer.cpp:209-254): centroid = running fp32 sum of the
 * rows in order, divided by count, then rotated.  Q is supplied by the caller (the reference
 * draws it from std::random_device, random_orthogonal_transformer.cpp:98-149). */
ORC_API void
orc_rabitq_train(const float* data, uint64_t count, uint64_t dim, const float* Q, float* centroid) {
    float* c = (float*)calloc(dim, sizeof(float));
    for (uint64_t i = 0; i < count; ++i) {
        for (uint64_t d = 0; d < dim; ++d) {
            c[d] += data[i * dim + d];
        }
    }
    for (uint64_t d = 0; d < dim; ++d) {
        c[d] = c[d] / (float)count;
    }
    orc_rotate(Q, c, dim, centroid);
    free(c);
}

/* RaBitQuantizer::EncodeOneInternal, 1-bit branch (rabitq_quantizer.cpp:723-857, esp. :770-772,
 * :824-850).  rotated (optional) receives the normalised rotated vectors for margin reporting. */
ORC_API void
orc_rabitq_encode(const float* data,
                  uint64_t count,
                  uint64_t dim,
                  const float* Q,
                  const float* centroid,
                  uint8_t* codes,
                  float* rotated) {
    const uint64_t cs = orc_rabitq_code_size(dim);
    const uint64_t off_norm = cs - 8, off_err = cs - 4;
    const float inv_sqrt_d = 1.0f / sqrtf((float)dim);
#pragma omp parallel
    {
        float* t = (float*)malloc(dim * sizeof(float));
        float* o = (float*)malloc(dim * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < (int64_t)count; ++i) {
            uint8_t* code = codes + (uint64_t)i * cs;
            memset(code, 0, cs);
            orc_rotate(Q, data + (uint64_t)i * dim, dim, t);
            float norm = orc_normalize_with_centroid(t, centroid, o, dim);
            for (uint64_t d = 0; d < dim; ++d) {
                if (o[d] >= 0.0f) {
                    code[d / 8] |= (uint8_t)(1u << (d % 8));
                }
            }
            float err = orc_rabitq_float_binary_ip(o, code, dim, inv_sqrt_d);
            memcpy(code + off_norm, &norm, 4);
            memcpy(code + off_err, &err, 4);
            if (rotated != NULL) {
                memcpy(rotated + (uint64_t)i * dim, o, dim * sizeof(float));
            }
        }
        free(t);
        free(o);
    }
}

/* RaBitQuantizer::ProcessQueryImpl, fp32 query (rabitq_quantizer.cpp:2130-2217): rotated and
 * normalised query, dim floats followed by the norm. */
ORC_API void
orc_rabitq_process_query(const float* q,
                         uint64_t nq,
                         uint64_t dim,
                         const float* Q,
                         const float* centroid,
                         float* out /* nq x (dim+1) */) {
#pragma omp parallel
    {
        float* t = (float*)malloc(dim * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            orc_rotate(Q, q + (uint64_t)i * dim, dim, t);
            float* o = out + (uint64_t)i * (dim + 1);
            o[dim] = orc_normalize_with_centroid(t, centroid, o, dim);
        }
        free(t);
    }
}

/* ComputeQueryBaseImpl, L2, fp32 query / 1-bit base (rabitq_quantizer.cpp:1775-1860) with l2_ube
 * (:915-922). */
ORC_API float
orc_rabitq_dist(const float* qcode, const uint8_t* code, uint64_t dim) {
    const uint64_t cs = orc_rabitq_code_size(dim);
    const float inv_sqrt_d = 1.0f / sqrtf((float)dim);
    float ip = orc_rabitq_float_binary_ip(qcode, code, dim, inv_sqrt_d);
    float qn = qcode[dim];
    float bn, err;
    memcpy(&bn, code + cs - 8, 4);
    memcpy(&err, code + cs - 4, 4);
    if (fabsf(err) < 1e-5) {
        err = err >= 0 ? 1.0f : -1.0f;
    }
    float est = ip / err;
    float p1 = bn * bn;
    float p2 = qn * qn;
    float p3 = -2 * bn * qn * est;
    return p1 + p2 + p3;
}

/* IVF scan over RaBitQ records, same probe loop and selection rule as orc_ivf_sq8_search.
 * qcodes: nq x (dim+1) from orc_rabitq_process_query. */
ORC_API void
orc_ivf_rabitq_search(const uint8_t* codes,
                      const int64_t* list_off,
                      const int64_t* inner_ids,
                      uint64_t dim,
                      const float* qcodes,
                      uint64_t nq,
                      const int32_t* probes,
                      uint64_t nprobe,
                      int64_t k,
                      int nthreads,
                      int64_t* out_ids,
                      float* out_dists) {
    const uint64_t cs = orc_rabitq_code_size(dim);
#ifdef _OPENMP
    if (nthreads <= 0) {
        nthreads = omp_get_max_threads();
    }
#else
    nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
    {
        orc_heap h;
        h.a = (orc_rec*)malloc((size_t)(k + 2) * sizeof(orc_rec));
#pragma omp for schedule(dynamic, 1)
        for (int64_t i = 0; i < (int64_t)nq; ++i) {
            const float* qi = qcodes + (uint64_t)i * (dim + 1);
            h.size = 0;
            for (uint64_t p = 0; p < nprobe; ++p) {
                int32_t l = probes[(uint64_t)i * nprobe + p];
                if (l < 0) {
                    continue;
                }
                for (int64_t r = list_off[l]; r < list_off[l + 1]; ++r) {
                    float d = orc_rabitq_dist(qi, codes + (uint64_t)r * cs, dim);
                    heap_offer_strict(&h, k, d, inner_ids[r]);
                }
            }
            heap_drain(&h, k, out_ids + (uint64_t)i * k, out_dists + (uint64_t)i * k);
        }
        free(h.a);
    }
}

/* Number of worker threads of the parallel loops from here on.  The benchmark's CPU arm sets it to the
 * cores the process may run on, so that an OMP_NUM_THREADS in the environment (torchrun exports 1)
 * does not decide how many cores the baseline gets. */
ORC_API void
orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) {
        omp_set_num_threads(n);
    }
#else
    (void)n;
#endif
}

ORC_API int
orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
