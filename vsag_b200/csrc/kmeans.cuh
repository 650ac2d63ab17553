// Device-pointer entry points of the k-means trainer shared with the IVF index.
#pragma once

#include "common.cuh"

namespace vb200 {

struct KMeansWorkspace {
    DevBuf<float> c_sq;     // |c_j|^2
    DevBuf<float> best;     // best score per point
    DevBuf<float> sums;     // k x dim accumulators
    DevBuf<int32_t> counts; // k
    DevBuf<double> err;     // 1
};

// labels_dev[i] = argmin_j |c_j|^2 - 2 <c_j, x_i> (lowest j on ties).  mean_err_host optional.
int kmeans_assign_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                         const float* centroids_dev, uint32_t k, int32_t* labels_dev,
                         double* mean_err_host);

// centroids_dev <- per-cluster means; empty clusters take row (j * 2654435761 + iter) % n.
int kmeans_update_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                         const int32_t* labels_dev, uint32_t k, uint32_t iter, float* centroids_dev);

}  // namespace vb200
