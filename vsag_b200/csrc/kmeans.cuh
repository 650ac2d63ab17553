// Device-pointer entry points of the k-means trainer shared with the IVF index.
#pragma once

#include "common.cuh"
#include "tc_gemm.cuh"

namespace vb200 {

struct KMeansWorkspace {
    DevBuf<float> c_sq;     // |c_j|^2
    DevBuf<float> best;     // best score per point
    DevBuf<float> sums;     // k x dim accumulators
    DevBuf<int32_t> counts; // k
    // centroid update in a fixed order: rows sorted by (label, row), the first row of each cluster
    DevBuf<uint32_t> sort_keys_in, sort_keys_out, sort_rows_in, sort_rows_out, cluster_off;
    DevBuf<uint8_t> sort_tmp;
    DevBuf<double> err;     // 1
    // tensor-core path: tiled bf16 terms of the points (kept while the same rows are assigned
    // again, i.e. across Lloyd iterations) and of the centroids, candidates, kernel scratch
    DevBuf<uint16_t> x_hi, x_lo, c_hi, c_lo;
    DevBuf<float> x_sq;       // |x_i|^2 of the tiled rows
    DevBuf<float> margin;     // 1e-3 * max_j |c_j|
    DevBuf<float> row_bound;  // score of each row against its previous centroid (warm start)
    // rows whose tensor-core candidate lists may have lost a column (flagged by the kernel) are decided by
    // the fixed-order kernel over all centroids
    DevBuf<uint32_t> row_flags, flagged_rows, flagged_count;
    DevBuf<float> flagged_x, flagged_best;
    DevBuf<int32_t> flagged_labels;
    const float* tiled_rows = nullptr;
    uint64_t tiled_n = 0;
    uint32_t tiled_dim = 0;
    DevBuf<uint64_t> cand;
    TcWorkspace tc;
    void
    forget_points() {
        tiled_rows = nullptr;
        tiled_n = 0;
    }
};

// True unless the environment variable VB200_DISABLE_TC is set to a non-zero value: the
// tensor-core candidate kernels are the default, the fixed-order SIMT kernels the cross-check.
bool tensor_cores_enabled();

// k-means++ seeding on the device; see vb200_kmeans_init.  picked_dev may be null.
int kmeans_pp_init_device(const float* x_dev, uint64_t n, uint32_t dim, uint32_t k, uint32_t seed,
                          float* centroids_dev, int64_t* picked_dev);

// labels_dev[i] = argmin_j |c_j|^2 - 2 <c_j, x_i> (lowest j on ties).  mean_err_host optional.
// prev_labels_dev (optional, may alias labels_dev): the labels of the previous Lloyd iteration; the
// tensor-core path uses them to skip centroids that cannot beat a row's previous one.
int kmeans_assign_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                         const float* centroids_dev, uint32_t k, int32_t* labels_dev,
                         double* mean_err_host, const int32_t* prev_labels_dev = nullptr);

// centroids_dev <- per-cluster means; empty clusters take row (j * 2654435761 + iter) % n.
int kmeans_update_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                         const int32_t* labels_dev, uint32_t k, uint32_t iter, float* centroids_dev);

}  // namespace vb200
