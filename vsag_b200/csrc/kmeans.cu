// k-means Lloyd iterations for IVF partition training: exact assignment through the fixed-order
// dense kernel with a fused argmin epilogue, and the centroid update.
#include "kmeans.cuh"

#include <random>

#include <cstdlib>

#include <cub/device/device_radix_sort.cuh>

#include "dense.cuh"

namespace vb200 {

// err += sum_i double(best_i + |x_i|^2); |x_i|^2 is the ascending FMA chain
// (src/impl/cluster/kmeans_cluster.cpp:281-296).
__global__ void __launch_bounds__(256)
kmeans_error_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim,
                    const float* __restrict__ best, double* __restrict__ err) {
    __shared__ double partial[8];
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    double v = 0.0;
    if (i < n) {
        const float* p = x + i * dim;
        float s = 0.f;
        for (uint32_t d = 0; d < dim; ++d) {
            float t = __ldg(p + d);
            s = fmaf(t, t, s);
        }
        v = static_cast<double>(__fadd_rn(best[i], s));
    }
    for (int off = 16; off > 0; off >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, off);
    }
    if ((threadIdx.x & 31) == 0) {
        partial[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double s = 0.0;
        for (int w = 0; w < 8; ++w) {
            s += partial[w];
        }
        atomicAdd(err, s);
    }
}

static std::atomic<int> g_tc_enabled{-1};

bool
tensor_cores_enabled() {
    int v = g_tc_enabled.load();
    if (v < 0) {
        const char* e = getenv("VB200_DISABLE_TC");
        v = (e != nullptr && e[0] != 0 && e[0] != '0') ? 0 : 1;
        g_tc_enabled.store(v);
    }
    return v == 1;
}

// Picks, among each row's candidate centroids, the one the reference's arithmetic prefers:
// score = fma(-2, <c, x>, |c|^2) with the inner product as one ascending FMA chain, lowest index
// on ties (src/impl/cluster/kmeans_cluster.cpp:262-284).  `lanes` (a power of two <= 32) threads
// share a row, one candidate each per round; the chain of a candidate stays in one thread.
__global__ void __launch_bounds__(128)
kmeans_pick_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, const float* __restrict__ centroids,
                   const float* __restrict__ c_sq, const uint64_t* __restrict__ cand, uint32_t per_row,
                   uint32_t lanes, int32_t* __restrict__ labels, float* __restrict__ best_out) {
    const uint64_t t = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t i = t / lanes;
    const uint32_t sub = static_cast<uint32_t>(t % lanes);
    const bool live = i < n;
    float best = INFINITY;
    uint32_t best_col = 0x7fffffffu;
    if (live) {
        const float* xi = x + i * dim;
        const uint64_t* ci = cand + i * per_row;
        const bool vec = (dim & 3u) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(centroids)) & 15u) == 0;
        for (uint32_t j = sub; j < per_row; j += lanes) {
            uint64_t key = ci[j];
            if (key == KEY_INF) {
                continue;
            }
            uint32_t col = static_cast<uint32_t>(key);
            const float* c = centroids + static_cast<uint64_t>(col) * dim;
            float ip = 0.f;
            if (vec) {
                for (uint32_t d = 0; d < dim; d += 4) {
                    float4 cv = __ldg(reinterpret_cast<const float4*>(c + d));
                    float4 xv = __ldg(reinterpret_cast<const float4*>(xi + d));
                    ip = fmaf(cv.x, xv.x, ip);
                    ip = fmaf(cv.y, xv.y, ip);
                    ip = fmaf(cv.z, xv.z, ip);
                    ip = fmaf(cv.w, xv.w, ip);
                }
            } else {
                for (uint32_t d = 0; d < dim; ++d) {
                    ip = fmaf(__ldg(c + d), __ldg(xi + d), ip);
                }
            }
            float score = fmaf(-2.0f, ip, __ldg(c_sq + col));
            if (score < best || (score == best && col < best_col)) {
                best = score;
                best_col = col;
            }
        }
    }
    for (uint32_t off = lanes >> 1; off > 0; off >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, off);
        uint32_t oc = __shfl_xor_sync(0xffffffffu, best_col, off);
        if (ob < best || (ob == best && oc < best_col)) {
            best = ob;
            best_col = oc;
        }
    }
    if (live && sub == 0) {
        labels[i] = best_col == 0x7fffffffu ? 0 : static_cast<int32_t>(best_col);
        if (best_out != nullptr) {
            best_out[i] = best;
        }
    }
}

// out[0] = scale * sqrt(max_j sq[j]); one CTA.
__global__ void __launch_bounds__(256)
max_norm_kernel(const float* __restrict__ sq, uint32_t k, float scale, float* __restrict__ out) {
    __shared__ float part[8];
    float m = 0.f;
    for (uint32_t j = threadIdx.x; j < k; j += blockDim.x) {
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
        out[0] = scale * sqrtf(m);
    }
}

// bound[i] = fma(-2, <c_l, x_i>, |c_l|^2) for l = the row's previous label (+inf when it has none).
__global__ void __launch_bounds__(128)
kmeans_prev_score_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, const float* __restrict__ centroids,
                         const float* __restrict__ c_sq, uint32_t k, const int32_t* __restrict__ prev,
                         float* __restrict__ bound) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    int32_t l = prev[i];
    if (l < 0 || static_cast<uint32_t>(l) >= k) {
        bound[i] = INFINITY;
        return;
    }
    const float* xi = x + i * dim;
    const float* c = centroids + static_cast<uint64_t>(l) * dim;
    float ip = 0.f;
    if ((dim & 15u) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(centroids)) & 15u) == 0) {
        // the same ascending chain, operands fetched 64 bytes ahead of it
        for (uint32_t d = 0; d < dim; d += 16) {
            float4 cv[4], xv[4];
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                cv[u] = __ldg(reinterpret_cast<const float4*>(c + d) + u);
                xv[u] = __ldg(reinterpret_cast<const float4*>(xi + d) + u);
            }
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
                ip = fmaf(cv[u].x, xv[u].x, ip);
                ip = fmaf(cv[u].y, xv[u].y, ip);
                ip = fmaf(cv[u].z, xv[u].z, ip);
                ip = fmaf(cv[u].w, xv[u].w, ip);
            }
        }
    } else {
        for (uint32_t d = 0; d < dim; ++d) {
            ip = fmaf(__ldg(c + d), __ldg(xi + d), ip);
        }
    }
    bound[i] = fmaf(-2.0f, ip, __ldg(c_sq + l));
}

// rows[c] = i for every flagged row i (order irrelevant), *count = how many.
__global__ void
kmeans_collect_flagged_kernel(const uint32_t* __restrict__ flags, uint64_t n, uint32_t* __restrict__ rows,
                              uint32_t* __restrict__ count) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n && flags[i] != 0) {
        rows[atomicAdd(count, 1u)] = static_cast<uint32_t>(i);
    }
}

__global__ void
kmeans_gather_rows_kernel(const float* __restrict__ x, uint32_t dim, const uint32_t* __restrict__ rows, uint64_t count,
                          float* __restrict__ out) {
    const uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < count * dim) {
        out[e] = x[static_cast<uint64_t>(rows[e / dim]) * dim + e % dim];
    }
}

__global__ void
kmeans_scatter_labels_kernel(const uint32_t* __restrict__ rows, uint64_t count, const int32_t* __restrict__ lab,
                             const float* __restrict__ best, int32_t* __restrict__ labels, float* __restrict__ best_out) {
    const uint64_t c = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c < count) {
        labels[rows[c]] = lab[c];
        if (best_out != nullptr) {
            best_out[rows[c]] = best[c];
        }
    }
}

constexpr uint32_t KMEANS_TC_CANDIDATES = 4;
constexpr uint64_t KMEANS_TC_SLICE = uint64_t{1} << 22;  // rows tiled at once

// Assignment through the tensor cores: candidates from the split-bf16 GEMM, winner by the exact
// rule above.  Equal to the fixed-order SIMT result whenever the true winner is among the four
// nominated centroids, i.e. unless more than three others sit within ~1e-5 relative of it.
static int
kmeans_assign_tc(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                 const float* centroids_dev, uint32_t k, int32_t* labels_dev, float* best_dev,
                 const int32_t* prev_labels_dev) {
    const uint32_t chunks = (dim + TC_KC - 1) / TC_KC;
    const size_t c_elems = tc_tiled_elems(k, dim);
    VB_TRY(ws.c_hi.reserve(c_elems));
    VB_TRY(ws.c_lo.reserve(c_elems));
    VB_TRY(tc_pretile_f32(centroids_dev, k, dim, ws.c_hi.ptr, ws.c_lo.ptr));
    TcOperand b{ws.c_hi.ptr, ws.c_lo.ptr, k, chunks};
    const uint32_t m = k < KMEANS_TC_CANDIDATES ? k : KMEANS_TC_CANDIDATES;
    // The split-bf16 scores are within ~3e-5 * |x| * |c| of the exact ones; columns more than
    // 1e-3 * |x| * max|c| behind a row's best cannot be its exact winner and are skipped.
    VB_TRY(ws.margin.reserve(1));
    VB_LAUNCH(max_norm_kernel, 1, 256, 0, ws.c_sq.ptr, k, 1e-3f, ws.margin.ptr);
    for (uint64_t r0 = 0; r0 < n; r0 += KMEANS_TC_SLICE) {
        const uint64_t rows = n - r0 < KMEANS_TC_SLICE ? n - r0 : KMEANS_TC_SLICE;
        const bool whole = rows == n;
        const bool cached = whole && ws.tiled_rows == x_dev && ws.tiled_n == n && ws.tiled_dim == dim;
        if (!cached) {
            const size_t x_elems = tc_tiled_elems(rows, dim);
            VB_TRY(ws.x_hi.reserve(x_elems));
            VB_TRY(ws.x_lo.reserve(x_elems));
            VB_TRY(tc_pretile_f32(x_dev + r0 * dim, rows, dim, ws.x_hi.ptr, ws.x_lo.ptr));
            VB_TRY(ws.x_sq.reserve(rows));
            VB_TRY(row_sqnorm_f32(x_dev + r0 * dim, rows, dim, ws.x_sq.ptr));
            ws.tiled_rows = whole ? x_dev : nullptr;
            ws.tiled_n = whole ? n : 0;
            ws.tiled_dim = dim;
        }
        TcOperand a{ws.x_hi.ptr, ws.x_lo.ptr, rows, chunks};
        const float* row_bound = nullptr;
        if (prev_labels_dev != nullptr) {
            VB_TRY(ws.row_bound.reserve(rows));
            VB_LAUNCH(kmeans_prev_score_kernel, static_cast<uint32_t>((rows + 127) / 128), 128, 0, x_dev + r0 * dim,
                      rows, dim, centroids_dev, ws.c_sq.ptr, k, prev_labels_dev + r0, ws.row_bound.ptr);
            row_bound = ws.row_bound.ptr;
        }
        uint32_t n_split = 1, n_flagged = 0;
        VB_TRY(ws.row_flags.reserve(rows));
        VB_CUDA(cudaMemsetAsync(ws.row_flags.ptr, 0, rows * sizeof(uint32_t), current_stream()));
        VB_TRY(tc_candidates(ws.tc, a, b, 3, -2.0f, ws.c_sq.ptr, m, 0, ws.cand, &n_split, ws.x_sq.ptr,
                             ws.margin.ptr, row_bound, ws.row_flags.ptr, &n_flagged));
        const uint32_t per_row = n_split * m;
        const uint32_t lanes = per_row >= 32 ? 32u : next_pow2(per_row);
        const uint64_t threads = rows * lanes;
        VB_LAUNCH(kmeans_pick_kernel, static_cast<uint32_t>((threads + 127) / 128), 128, 0, x_dev + r0 * dim, rows,
                  dim, centroids_dev, ws.c_sq.ptr, ws.cand.ptr, per_row, lanes, labels_dev + r0,
                  best_dev != nullptr ? best_dev + r0 : nullptr);
        if (n_flagged > 0) {
            // A candidate list of these rows ended full of columns within the error margin of its best (many
            // near-equal centroids, or data far from the origin): the exact winner may not have been
            // nominated.  They are decided by the fixed-order kernel over all centroids instead.
            VB_TRY(ws.flagged_rows.reserve(n_flagged));
            VB_TRY(ws.flagged_count.reserve(1));
            VB_TRY(ws.flagged_x.reserve(static_cast<size_t>(n_flagged) * dim));
            VB_TRY(ws.flagged_labels.reserve(n_flagged));
            VB_TRY(ws.flagged_best.reserve(n_flagged));
            VB_CUDA(cudaMemsetAsync(ws.flagged_count.ptr, 0, sizeof(uint32_t), current_stream()));
            VB_LAUNCH(kmeans_collect_flagged_kernel, static_cast<uint32_t>((rows + 255) / 256), 256, 0, ws.row_flags.ptr,
                      rows, ws.flagged_rows.ptr, ws.flagged_count.ptr);
            const uint64_t elems = static_cast<uint64_t>(n_flagged) * dim;
            VB_LAUNCH(kmeans_gather_rows_kernel, static_cast<uint32_t>((elems + 255) / 256), 256, 0, x_dev + r0 * dim, dim,
                      ws.flagged_rows.ptr, n_flagged, ws.flagged_x.ptr);
            VB_TRY(dense_argmin_f32(ws.flagged_x.ptr, n_flagged, centroids_dev, k, dim, -2.0f, ws.c_sq.ptr,
                                    ws.flagged_labels.ptr, ws.flagged_best.ptr));
            VB_LAUNCH(kmeans_scatter_labels_kernel, static_cast<uint32_t>((n_flagged + 255) / 256), 256, 0,
                      ws.flagged_rows.ptr, n_flagged, ws.flagged_labels.ptr, ws.flagged_best.ptr, labels_dev + r0,
                      best_dev != nullptr ? best_dev + r0 : nullptr);
        }
    }
    return 0;
}

int
kmeans_assign_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                     const float* centroids_dev, uint32_t k, int32_t* labels_dev,
                     double* mean_err_host, const int32_t* prev_labels_dev) {
    VB_TRY(ws.c_sq.reserve(k));
    VB_TRY(ws.best.reserve(n));
    VB_TRY(row_sqnorm_f32(centroids_dev, k, dim, ws.c_sq.ptr));
    if (tensor_cores_enabled() && k >= 64 && n >= 128) {
        VB_TRY(kmeans_assign_tc(ws, x_dev, n, dim, centroids_dev, k, labels_dev, ws.best.ptr, prev_labels_dev));
    } else {
        VB_TRY(dense_argmin_f32(x_dev, n, centroids_dev, k, dim, -2.0f, ws.c_sq.ptr, labels_dev,
                                ws.best.ptr));
    }
    if (mean_err_host != nullptr) {
        VB_TRY(ws.err.reserve(1));
        VB_CUDA(cudaMemsetAsync(ws.err.ptr, 0, sizeof(double), current_stream()));
        VB_LAUNCH(kmeans_error_kernel, static_cast<uint32_t>((n + 255) / 256), 256, 0, x_dev, n, dim,
                  ws.best.ptr, ws.err.ptr);
        double total = 0.0;
        VB_CUDA(cudaMemcpyAsync(&total, ws.err.ptr, sizeof(double), cudaMemcpyDeviceToHost,
                                current_stream()));
        VB_TRY(sync_stream());
        *mean_err_host = total / static_cast<double>(static_cast<float>(n));
    }
    return 0;
}

// Centroid sums in a fixed order.  The reference adds the rows of a cluster in 1024-point chunks whose
// partial sums it merges in thread-completion order (kmeans_cluster.cpp:106-172), so its own centroids
// vary from run to run in the last bits.  Here every cluster is summed in ascending row order, one
// fp32 addition per row -- the order the CPU oracle uses -- so training is reproducible bit for bit:
// rows are sorted by (label, row) with a stable radix sort, and one CTA per cluster walks its rows.

// keys[i] = label of row i (k for rows without a valid label), rows[i] = i, counts[label]++.
__global__ void
kmeans_sort_keys_kernel(const int32_t* __restrict__ labels, uint64_t n, uint32_t k, uint32_t* __restrict__ keys,
                        uint32_t* __restrict__ rows, int32_t* __restrict__ counts) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) {
        return;
    }
    const int32_t l = labels[i];
    const bool ok = l >= 0 && static_cast<uint32_t>(l) < k;
    keys[i] = ok ? static_cast<uint32_t>(l) : k;
    rows[i] = static_cast<uint32_t>(i);
    if (ok) {
        atomicAdd(counts + l, 1);
    }
}

// off[j] = number of rows in clusters before j (one CTA; k is small next to the rows).
__global__ void __launch_bounds__(1024)
kmeans_cluster_offsets_kernel(const int32_t* __restrict__ counts, uint32_t k, uint32_t* __restrict__ off) {
    __shared__ uint32_t part[1024];
    const uint32_t per = (k + 1023) / 1024;
    const uint32_t j0 = threadIdx.x * per, j1 = j0 + per < k ? j0 + per : k;
    uint32_t sum = 0;
    for (uint32_t j = j0; j < j1; ++j) {
        sum += static_cast<uint32_t>(counts[j]);
    }
    part[threadIdx.x] = sum;
    __syncthreads();
    for (uint32_t o = 1; o < 1024; o <<= 1) {
        const uint32_t v = threadIdx.x >= o ? part[threadIdx.x - o] : 0u;
        __syncthreads();
        part[threadIdx.x] += v;
        __syncthreads();
    }
    uint32_t run = part[threadIdx.x] - sum;
    for (uint32_t j = j0; j < j1; ++j) {
        off[j] = run;
        run += static_cast<uint32_t>(counts[j]);
    }
    if (threadIdx.x == 1023) {
        off[k] = part[1023];
    }
}

// sums[j][d] = ((x[r0][d] + x[r1][d]) + x[r2][d]) + ... over the rows r0 < r1 < ... of cluster j.  One CTA
// per cluster, one thread per dimension (strided when dim exceeds the CTA); the loads of eight rows are
// issued together, the additions stay in row order.
__global__ void __launch_bounds__(128)
kmeans_sum_in_order_kernel(const float* __restrict__ x, uint32_t dim, const uint32_t* __restrict__ sorted_rows,
                           const uint32_t* __restrict__ off, float* __restrict__ sums) {
    const uint32_t j = blockIdx.x;
    const uint32_t beg = off[j], end = off[j + 1];
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        float s = 0.f;
        uint32_t r = beg;
        for (; r + 8 <= end; r += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = __ldg(x + static_cast<uint64_t>(__ldg(sorted_rows + r + i)) * dim + d);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s = __fadd_rn(s, v[i]);
            }
        }
        for (; r < end; ++r) {
            s = __fadd_rn(s, __ldg(x + static_cast<uint64_t>(__ldg(sorted_rows + r)) * dim + d));
        }
        sums[static_cast<uint64_t>(j) * dim + d] = s;
    }
}

__global__ void
kmeans_finalize_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, uint32_t k,
                       uint32_t iter, const float* __restrict__ sums,
                       const int32_t* __restrict__ counts, float* __restrict__ centroids) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= static_cast<uint64_t>(k) * dim) {
        return;
    }
    uint32_t j = static_cast<uint32_t>(e / dim);
    uint32_t d = static_cast<uint32_t>(e % dim);
    int32_t c = counts[j];
    if (c > 0) {
        float inv = __fdiv_rn(1.0f, static_cast<float>(c));
        centroids[e] = __fmul_rn(sums[e], inv);
    } else {
        uint64_t row = (static_cast<uint64_t>(j) * 2654435761ull + iter) % n;
        centroids[e] = x[row * dim + d];
    }
}

int
kmeans_update_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                     const int32_t* labels_dev, uint32_t k, uint32_t iter, float* centroids_dev) {
    const size_t kd = static_cast<size_t>(k) * dim;
    VB_CHECK_ARG(n < 0xFFFFFFFFull, "kmeans update: batch too large");
    VB_TRY(ws.sums.reserve(kd));
    VB_TRY(ws.counts.reserve(k));
    VB_TRY(ws.sort_keys_in.reserve(n));
    VB_TRY(ws.sort_keys_out.reserve(n));
    VB_TRY(ws.sort_rows_in.reserve(n));
    VB_TRY(ws.sort_rows_out.reserve(n));
    VB_TRY(ws.cluster_off.reserve(static_cast<size_t>(k) + 1));
    cudaStream_t st = current_stream();
    VB_CUDA(cudaMemsetAsync(ws.counts.ptr, 0, k * sizeof(int32_t), st));
    VB_LAUNCH(kmeans_sort_keys_kernel, static_cast<uint32_t>((n + 255) / 256), 256, 0, labels_dev, n, k,
              ws.sort_keys_in.ptr, ws.sort_rows_in.ptr, ws.counts.ptr);
    {
        // stable sort by label: rows of a cluster stay in ascending order
        int end_bit = 1;
        while ((uint64_t{1} << end_bit) <= k) {
            ++end_bit;
        }
        size_t tmp_bytes = 0;
        VB_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, ws.sort_keys_in.ptr, ws.sort_keys_out.ptr,
                                                ws.sort_rows_in.ptr, ws.sort_rows_out.ptr, static_cast<int64_t>(n), 0,
                                                end_bit, st));
        VB_TRY(ws.sort_tmp.reserve(tmp_bytes > 0 ? tmp_bytes : 1));
        tmp_bytes = ws.sort_tmp.cap;
        VB_CUDA(cub::DeviceRadixSort::SortPairs(ws.sort_tmp.ptr, tmp_bytes, ws.sort_keys_in.ptr, ws.sort_keys_out.ptr,
                                                ws.sort_rows_in.ptr, ws.sort_rows_out.ptr, static_cast<int64_t>(n), 0,
                                                end_bit, st));
        g_kernel_launches.fetch_add(1);
    }
    VB_LAUNCH(kmeans_cluster_offsets_kernel, 1, 1024, 0, ws.counts.ptr, k, ws.cluster_off.ptr);
    VB_LAUNCH(kmeans_sum_in_order_kernel, k, 128, 0, x_dev, dim, ws.sort_rows_out.ptr, ws.cluster_off.ptr,
              ws.sums.ptr);
    VB_LAUNCH(kmeans_finalize_kernel, static_cast<uint32_t>((kd + 255) / 256), 256, 0, x_dev, n, dim,
              k, iter, ws.sums.ptr, ws.counts.ptr, centroids_dev);
    return 0;
}

}  // namespace vb200

using namespace vb200;

// The training entry points keep one workspace per process between calls (tiled rows, candidate lists, sort
// buffers: 1.3 GB for 1 M x 128 rows against 4096 centroids), because allocating and freeing it costs more than
// two Lloyd iterations; a second caller at the same time gets a workspace of its own.
// vb200_release_workspaces() frees the kept one.
namespace {

std::mutex g_kmeans_ws_mu;
KMeansWorkspace* g_kmeans_ws = nullptr;   // never destroyed at exit: the CUDA context may be gone by then

class WorkspaceLease {
public:
    WorkspaceLease() : kept_(g_kmeans_ws_mu.try_lock()) {
        if (kept_ && g_kmeans_ws == nullptr) {
            g_kmeans_ws = new (std::nothrow) KMeansWorkspace;
            if (g_kmeans_ws == nullptr) {
                g_kmeans_ws_mu.unlock();
                kept_ = false;
            }
        }
        if (kept_) {
            g_kmeans_ws->forget_points();   // another call's rows may have lived at the same address
        }
    }
    ~WorkspaceLease() {
        if (kept_) {
            g_kmeans_ws_mu.unlock();
        }
    }
    KMeansWorkspace& get() { return kept_ ? *g_kmeans_ws : own_; }

private:
    bool kept_;
    KMeansWorkspace own_;
};

}  // namespace

extern "C" int
vb200_release_workspaces(void) {
    std::lock_guard<std::mutex> lock(g_kmeans_ws_mu);
    delete g_kmeans_ws;
    g_kmeans_ws = nullptr;
    return 0;
}

static int
check_kmeans_args(const float* data, uint64_t count, uint32_t dim, const float* centroids, uint32_t k) {
    // Argument checks of KMeansCluster::Run (kmeans_cluster.cpp:54-65).
    VB_CHECK_ARG(k > 0, "k must be positive");
    VB_CHECK_ARG(count > 0, "count must be positive");
    VB_CHECK_ARG(data != nullptr, "datas cannot be null");
    VB_CHECK_ARG(dim > 0, "dim must be positive");
    VB_CHECK_ARG(centroids != nullptr, "centroids cannot be null");
    return 0;
}

extern "C" int
vb200_kmeans_assign(const float* data, uint64_t count, uint32_t dim, const float* centroids,
                    uint32_t k, int32_t* labels, double* mean_err) {
    VB_TRY(check_kmeans_args(data, count, dim, centroids, k));
    VB_CHECK_ARG(labels != nullptr, "labels cannot be null");
    DevInput<float> x, c;
    VB_TRY(x.bind(data, count * dim));
    VB_TRY(c.bind(centroids, static_cast<size_t>(k) * dim));
    DevBuf<int32_t> lab;
    VB_TRY(lab.reserve(count));
    KMeansWorkspace ws;
    VB_TRY(kmeans_assign_device(ws, x.ptr, count, dim, c.ptr, k, lab.ptr, mean_err));
    VB_TRY(copy_out(labels, lab.ptr, count));
    return sync_stream();
}

extern "C" int
vb200_kmeans_update(const float* data, uint64_t count, uint32_t dim, const int32_t* labels,
                    uint32_t k, uint32_t iter, float* centroids, int32_t* counts) {
    VB_TRY(check_kmeans_args(data, count, dim, centroids, k));
    VB_CHECK_ARG(labels != nullptr, "labels cannot be null");
    DevInput<float> x;
    DevInput<int32_t> lab;
    VB_TRY(x.bind(data, count * dim));
    VB_TRY(lab.bind(labels, count));
    DevBuf<float> c;
    VB_TRY(c.reserve(static_cast<size_t>(k) * dim));
    KMeansWorkspace ws;
    VB_TRY(kmeans_update_device(ws, x.ptr, count, dim, lab.ptr, k, iter, c.ptr));
    VB_TRY(copy_out(centroids, c.ptr, static_cast<size_t>(k) * dim));
    if (counts != nullptr) {
        VB_TRY(copy_out(counts, ws.counts.ptr, k));
    }
    return sync_stream();
}

extern "C" int
vb200_kmeans_train(const float* data, uint64_t count, uint32_t dim, uint32_t k, int iters,
                   float* centroids, int32_t* labels, double* mean_err) {
    VB_TRY(check_kmeans_args(data, count, dim, centroids, k));
    VB_CHECK_ARG(k <= count, "k cannot be larger than count");
    VB_CHECK_ARG(iters >= 0, "iters must not be negative");
    DevInput<float> x;
    VB_TRY(x.bind(data, count * dim));
    const size_t kd = static_cast<size_t>(k) * dim;
    DevBuf<float> c;
    VB_TRY(c.reserve(kd));
    VB_CUDA(cudaMemcpyAsync(c.ptr, centroids, kd * sizeof(float), cudaMemcpyDefault, current_stream()));
    DevBuf<int32_t> lab;
    VB_TRY(lab.reserve(count));
    WorkspaceLease lease;
    KMeansWorkspace& ws = lease.get();
    for (int it = 0; it < iters; ++it) {
        double* err = (it == iters - 1) ? mean_err : nullptr;
        VB_TRY(kmeans_assign_device(ws, x.ptr, count, dim, c.ptr, k, lab.ptr, err, it > 0 ? lab.ptr : nullptr));
        VB_TRY(kmeans_update_device(ws, x.ptr, count, dim, lab.ptr, k, static_cast<uint32_t>(it), c.ptr));
    }
    VB_TRY(copy_out(centroids, c.ptr, kd));
    if (labels != nullptr && iters > 0) {
        VB_TRY(copy_out(labels, lab.ptr, count));
    }
    return sync_stream();
}

// ---------------------------------------------------------------------------------------------
// k-means++ seeding (KMeansCluster::select_initial_centroids_kmeans_plus_plus,
// src/impl/cluster/kmeans_cluster.cpp:383-435)
// ---------------------------------------------------------------------------------------------
namespace vb200 {

constexpr uint32_t KPP_BLOCK_ROWS = 1024;   // rows per CTA of the update kernel = one partial sum

// min_d[i] = min(min_d[i], |x_i - c|^2) with the reference's per-row chain (difference, then one
// FMA per dimension in ascending order); part[b] = sum of the CTA's rows in double.  A warp
// stages 32 rows x 32 dimensions through shared memory so the global reads stay coalesced while
// every lane still walks its own row in order.
__global__ void __launch_bounds__(256)
kpp_update_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, const float* __restrict__ centroid,
                  float* __restrict__ min_d, double* __restrict__ part) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* c = reinterpret_cast<float*>(smem_raw);                       // dim
    float* tiles = c + ((dim + 31) / 32) * 32;                            // 8 warps x 32 x 33
    __shared__ double warp_sum[8];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        c[d] = centroid[d];
    }
    __syncthreads();
    float* tile = tiles + warp * (32 * 33);
    double acc = 0.0;
    const uint64_t block_row0 = static_cast<uint64_t>(blockIdx.x) * KPP_BLOCK_ROWS;
    for (uint32_t pass = 0; pass < KPP_BLOCK_ROWS / 256; ++pass) {
        const uint64_t row0 = block_row0 + (pass * 8 + warp) * 32;
        if (row0 >= n) {
            break;
        }
        float s = 0.f;
        for (uint32_t d0 = 0; d0 < dim; d0 += 32) {
            __syncwarp();
            for (uint32_t r = 0; r < 32; ++r) {
                const uint64_t row = row0 + r;
                const uint32_t d = d0 + lane;
                tile[r * 33 + lane] = (row < n && d < dim) ? __ldg(x + row * dim + d) : 0.f;
            }
            __syncwarp();
            const uint32_t lim = dim - d0 < 32 ? dim - d0 : 32;
            for (uint32_t j = 0; j < lim; ++j) {
                const float t = __fsub_rn(tile[lane * 33 + j], c[d0 + j]);
                s = fmaf(t, t, s);
            }
        }
        const uint64_t row = row0 + lane;
        if (row < n) {
            const float old = min_d[row];
            const float m = s < old ? s : old;
            min_d[row] = m;
            acc += static_cast<double>(m);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
    }
    if (lane == 0) {
        warp_sum[warp] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) {
            t += warp_sum[w];
        }
        part[blockIdx.x] = t;
    }
}

// One CTA: total of the partial sums; threshold = total * u (the uniform draw from [0, total));
// the first row whose running sum reaches it becomes centroid `slot`.  With total <= 0 (every row
// coincides with a chosen centre) nothing is picked and the round is recorded in state[0]; the
// host then finishes the seeding with uniform draws as the reference does.
__global__ void __launch_bounds__(1024)
kpp_pick_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim, const float* __restrict__ min_d,
                const double* __restrict__ part, uint32_t n_part, double u, uint32_t slot,
                float* __restrict__ centroids, int64_t* __restrict__ picked, uint32_t* __restrict__ state) {
    __shared__ double sh_scan[1024];
    __shared__ double sh_base;
    __shared__ uint32_t sh_block;
    __shared__ unsigned long long sh_row;
    const uint32_t t = threadIdx.x;
    // inclusive scan of the partial sums, each thread owning a contiguous run
    const uint32_t per = (n_part + 1023) / 1024;
    const uint32_t p0 = t * per;
    double local = 0.0;
    for (uint32_t i = p0; i < p0 + per && i < n_part; ++i) {
        local += part[i];
    }
    sh_scan[t] = local;
    __syncthreads();
    for (uint32_t off = 1; off < 1024; off <<= 1) {
        double v = t >= off ? sh_scan[t - off] : 0.0;
        __syncthreads();
        sh_scan[t] += v;
        __syncthreads();
    }
    const double total = sh_scan[1023];
    if (!(total > 0.0)) {
        if (t == 0) {
            atomicMin(state, slot);
        }
        return;
    }
    const double thr = total * u + 0.0;
    if (t == 0) {
        sh_block = 0xFFFFFFFFu;
        sh_row = ~0ull;
    }
    __syncthreads();
    // first run, then first partial sum inside it, whose inclusive sum reaches the threshold
    const double before = t > 0 ? sh_scan[t - 1] : 0.0;
    if (sh_scan[t] >= thr && !(before >= thr) && p0 < n_part) {
        const uint32_t last = p0 + per - 1 < n_part ? p0 + per - 1 : n_part - 1;
        double run = before;
        for (uint32_t i = p0; i <= last; ++i) {
            const double next = run + part[i];
            if (next >= thr || i == last) {
                sh_block = i;
                sh_base = run;
                break;
            }
            run = next;
        }
    }
    __syncthreads();
    uint64_t row_pick = n - 1;   // the reference's default when the running sum never gets there
    if (sh_block != 0xFFFFFFFFu) {
        const uint64_t row0 = static_cast<uint64_t>(sh_block) * KPP_BLOCK_ROWS;
        const uint64_t row = row0 + t;
        const double base = sh_base;
        __syncthreads();
        sh_scan[t] = row < n ? static_cast<double>(min_d[row]) : 0.0;
        __syncthreads();
        for (uint32_t off = 1; off < 1024; off <<= 1) {
            double v = t >= off ? sh_scan[t - off] : 0.0;
            __syncthreads();
            sh_scan[t] += v;
            __syncthreads();
        }
        if (row < n && base + sh_scan[t] >= thr) {
            atomicMin(&sh_row, static_cast<unsigned long long>(row));
        }
        __syncthreads();
        if (sh_row != ~0ull) {
            row_pick = sh_row;
        } else {
            // rounding kept the CTA's own running sum just below the threshold: its last row
            const uint64_t last = row0 + KPP_BLOCK_ROWS - 1;
            row_pick = last < n ? last : n - 1;
        }
    }
    for (uint32_t d = t; d < dim; d += blockDim.x) {
        centroids[static_cast<uint64_t>(slot) * dim + d] = x[row_pick * dim + d];
    }
    if (t == 0 && picked != nullptr) {
        picked[slot] = static_cast<int64_t>(row_pick);
    }
}

__global__ void
kpp_fill_kernel(float* __restrict__ min_d, uint64_t n, uint32_t* __restrict__ state) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) {
        min_d[i] = 3.402823466e+38f;
    }
    if (i == 0) {
        state[0] = 0xFFFFFFFFu;
    }
}

__global__ void
kpp_copy_row_kernel(const float* __restrict__ x, uint64_t row, uint32_t dim, uint32_t slot,
                    float* __restrict__ centroids, int64_t* __restrict__ picked) {
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        centroids[static_cast<uint64_t>(slot) * dim + d] = x[row * dim + d];
    }
    if (threadIdx.x == 0 && picked != nullptr) {
        picked[slot] = static_cast<int64_t>(row);
    }
}

// centroids_dev[k x dim] and (optionally) picked_dev[k] on the device.  The generator and its
// distributions are the C++ library's, exactly the objects the reference draws from; only the
// seed is the caller's (the reference takes it from std::random_device).
int
kmeans_pp_init_device(const float* x_dev, uint64_t n, uint32_t dim, uint32_t k, uint32_t seed,
                      float* centroids_dev, int64_t* picked_dev) {
    VB_CHECK_ARG(n > 0 && k > 0 && k <= n, "k cannot be larger than count");
    const uint32_t n_part = static_cast<uint32_t>((n + KPP_BLOCK_ROWS - 1) / KPP_BLOCK_ROWS);
    DevBuf<float> min_d;
    DevBuf<double> part;
    DevBuf<uint32_t> state;
    VB_TRY(min_d.reserve(n));
    VB_TRY(part.reserve(n_part));
    VB_TRY(state.reserve(1));
    VB_LAUNCH(kpp_fill_kernel, static_cast<uint32_t>((n + 255) / 256), 256, 0, min_d.ptr, n, state.ptr);
    std::mt19937 gen(seed);
    std::uniform_int_distribution<uint64_t> any_row(0, n - 1);
    VB_LAUNCH(kpp_copy_row_kernel, 1, 128, 0, x_dev, any_row(gen), dim, 0u, centroids_dev, picked_dev);
    const size_t smem = (static_cast<size_t>((dim + 31) / 32) * 32 + 8 * 32 * 33) * sizeof(float);
    VB_CHECK_ARG(smem <= 200 * 1024, "dim too large for the seeding kernel");
    VB_CUDA(cudaFuncSetAttribute(kpp_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)));
    std::uniform_real_distribution<double> unit(0.0, 1.0);
    for (uint32_t c = 1; c < k; ++c) {
        VB_LAUNCH(kpp_update_kernel, n_part, 256, smem, x_dev, n, dim,
                  centroids_dev + static_cast<size_t>(c - 1) * dim, min_d.ptr, part.ptr);
        VB_LAUNCH(kpp_pick_kernel, 1, 1024, 0, x_dev, n, dim, min_d.ptr, part.ptr, n_part, unit(gen), c,
                  centroids_dev, picked_dev, state.ptr);
    }
    uint32_t first_flat = 0xFFFFFFFFu;
    VB_CUDA(cudaMemcpyAsync(&first_flat, state.ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost, current_stream()));
    VB_TRY(sync_stream());
    if (first_flat < k) {
        // From that round on every row coincides with a chosen centre, so the total stays zero and
        // the reference draws a uniform row each round.  Replay the generator up to there (each
        // earlier round consumed one real draw) and finish the same way.
        std::mt19937 replay(seed);
        (void)any_row(replay);
        for (uint32_t c = 1; c < first_flat; ++c) {
            (void)unit(replay);
        }
        for (uint32_t c = first_flat; c < k; ++c) {
            VB_LAUNCH(kpp_copy_row_kernel, 1, 128, 0, x_dev, any_row(replay), dim, c, centroids_dev, picked_dev);
        }
        VB_TRY(sync_stream());
    }
    return 0;
}

}  // namespace vb200

extern "C" int
vb200_kmeans_init(const float* data, uint64_t count, uint32_t dim, uint32_t k, uint32_t seed, float* centroids,
                  int64_t* picked) {
    VB_TRY(check_kmeans_args(data, count, dim, centroids, k));
    VB_CHECK_ARG(k <= count, "k cannot be larger than count");
    DevInput<float> x;
    VB_TRY(x.bind(data, count * dim));
    DevBuf<float> c;
    DevBuf<int64_t> rows;
    VB_TRY(c.reserve(static_cast<size_t>(k) * dim));
    VB_TRY(rows.reserve(k));
    VB_TRY(kmeans_pp_init_device(x.ptr, count, dim, k, seed, c.ptr, rows.ptr));
    VB_TRY(copy_out(centroids, c.ptr, static_cast<size_t>(k) * dim));
    if (picked != nullptr) {
        VB_TRY(copy_out(picked, rows.ptr, k));
    }
    return sync_stream();
}

// ---------------------------------------------------------------------------------------------
// Assignment without any allocation
// ---------------------------------------------------------------------------------------------
// Some callers must not reach the CUDA allocator at all: a serving thread that holds a fixed
// memory budget and cannot tolerate the device-wide synchronisation cudaMalloc/cudaFree imply, or
// a host that has handed all remaining device memory to another pool.  For them the centroid
// norms -- the only scratch the assignment needs -- live in this fixed array, which every GPU that
// loads the library holds (256 KiB) until the process exits.
constexpr uint32_t NOALLOC_MAX_K = 65536;
static __device__ __align__(256) float g_noalloc_centroid_sq[NOALLOC_MAX_K];

// Device address of the array above, looked up once per device with that device current.  In host
// code the symbol itself is only a stand-in; kernels must be given the address this returns.
static int
noalloc_scratch(float** out) {
    static std::mutex mu;
    static float* cached[64] = {nullptr};
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    VB_CHECK_ARG(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        VB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_centroid_sq));
        cached[dev] = static_cast<float*>(p);
    }
    *out = cached[dev];
    return 0;
}

extern "C" int
vb200_kmeans_assign_noalloc(const float* data_dev, uint64_t count, uint32_t dim,
                            const float* centroids_dev, uint32_t k, int32_t* labels_dev) {
    VB_TRY(check_kmeans_args(data_dev, count, dim, centroids_dev, k));
    VB_CHECK_ARG(labels_dev != nullptr, "labels cannot be null");
    VB_CHECK_ARG(k <= NOALLOC_MAX_K, "k = %u exceeds the %u centroids the fixed scratch array holds", k,
                 NOALLOC_MAX_K);
    VB_CHECK_ARG(is_device_pointer(data_dev) && is_device_pointer(centroids_dev) &&
                     is_device_pointer(labels_dev),
                 "this entry point stages nothing: data, centroids and labels must be device pointers");
    // the scratch array used below is the current device's copy
    VB_CHECK_ARG(is_pointer_on_current_device(data_dev) && is_pointer_on_current_device(centroids_dev) &&
                     is_pointer_on_current_device(labels_dev),
                 "data, centroids and labels must live on the device that is current on the calling thread");
    float* c_sq = nullptr;
    VB_TRY(noalloc_scratch(&c_sq));
    // Every call rewrites entries [0, k) before reading them, so nothing has to be cleared.
    VB_TRY(row_sqnorm_f32(centroids_dev, k, dim, c_sq));
    VB_TRY(dense_argmin_f32(data_dev, count, centroids_dev, k, dim, -2.0f, c_sq, labels_dev, nullptr));
    return sync_stream();
}

extern "C" int
vb200_debug_set_wait_limit(int32_t polls) {
    tc_set_spin_limit(polls < 0 ? TC_SPIN_LIMIT : static_cast<uint32_t>(polls));
    return 0;
}

extern "C" int
vb200_set_tensor_cores(int enable) {
    g_tc_enabled.store(enable != 0 ? 1 : 0);
    return 0;
}
