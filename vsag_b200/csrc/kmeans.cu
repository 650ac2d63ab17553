// k-means Lloyd iterations for IVF partition training: exact assignment through the fixed-order
// dense kernel with a fused argmin epilogue, and the centroid update.
#include "kmeans.cuh"

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

int
kmeans_assign_device(KMeansWorkspace& ws, const float* x_dev, uint64_t n, uint32_t dim,
                     const float* centroids_dev, uint32_t k, int32_t* labels_dev,
                     double* mean_err_host) {
    VB_TRY(ws.c_sq.reserve(k));
    VB_TRY(ws.best.reserve(n));
    VB_TRY(row_sqnorm_f32(centroids_dev, k, dim, ws.c_sq.ptr));
    VB_TRY(dense_argmin_f32(x_dev, n, centroids_dev, k, dim, -2.0f, ws.c_sq.ptr, labels_dev,
                            ws.best.ptr));
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

// sums[label][d..d+3] += x[i][d..d+3]; one thread per (point, group of up to 4 dimensions).
__global__ void
kmeans_accumulate_kernel(const float* __restrict__ x, uint64_t n, uint32_t dim,
                         const int32_t* __restrict__ labels, uint32_t k, float* __restrict__ sums,
                         int32_t* __restrict__ counts) {
    const uint32_t groups = (dim + 3) / 4;
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= n * groups) {
        return;
    }
    uint64_t i = e / groups;
    uint32_t g = static_cast<uint32_t>(e % groups);
    int32_t l = labels[i];
    if (l < 0 || static_cast<uint32_t>(l) >= k) {
        return;
    }
    if (g == 0) {
        atomicAdd(counts + l, 1);
    }
    const float* p = x + i * dim;
    float* s = sums + static_cast<uint64_t>(l) * dim;
    for (uint32_t d = g * 4; d < dim && d < g * 4 + 4; ++d) {
        atomicAdd(s + d, __ldg(p + d));
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
    VB_TRY(ws.sums.reserve(kd));
    VB_TRY(ws.counts.reserve(k));
    VB_CUDA(cudaMemsetAsync(ws.sums.ptr, 0, kd * sizeof(float), current_stream()));
    VB_CUDA(cudaMemsetAsync(ws.counts.ptr, 0, k * sizeof(int32_t), current_stream()));
    const uint64_t groups = (dim + 3) / 4;
    uint64_t blocks = (n * groups + 255) / 256;
    VB_CHECK_ARG(blocks <= 0x7fffffffu, "kmeans update: batch too large");
    VB_LAUNCH(kmeans_accumulate_kernel, static_cast<uint32_t>(blocks), 256, 0, x_dev, n, dim,
              labels_dev, k, ws.sums.ptr, ws.counts.ptr);
    VB_LAUNCH(kmeans_finalize_kernel, static_cast<uint32_t>((kd + 255) / 256), 256, 0, x_dev, n, dim,
              k, iter, ws.sums.ptr, ws.counts.ptr, centroids_dev);
    return 0;
}

}  // namespace vb200

using namespace vb200;

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
    KMeansWorkspace ws;
    for (int it = 0; it < iters; ++it) {
        double* err = (it == iters - 1) ? mean_err : nullptr;
        VB_TRY(kmeans_assign_device(ws, x.ptr, count, dim, c.ptr, k, lab.ptr, err));
        VB_TRY(kmeans_update_device(ws, x.ptr, count, dim, lab.ptr, k, static_cast<uint32_t>(it), c.ptr));
    }
    VB_TRY(copy_out(centroids, c.ptr, kd));
    if (labels != nullptr && iters > 0) {
        VB_TRY(copy_out(labels, lab.ptr, count));
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
    float* c_sq = nullptr;
    VB_TRY(noalloc_scratch(&c_sq));
    // Every call rewrites entries [0, k) before reading them, so nothing has to be cleared.
    VB_TRY(row_sqnorm_f32(centroids_dev, k, dim, c_sq));
    VB_TRY(dense_argmin_f32(data_dev, count, centroids_dev, k, dim, -2.0f, c_sq, labels_dev, nullptr));
    return sync_stream();
}
