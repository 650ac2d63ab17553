// Dense inner-product kernels with a fixed summation order.
//
// Every <row, column> inner product is one fp32 FMA chain over the dimensions in ascending order,
// starting from 0 -- the order the CPU oracle defines for the reference's BLAS call sites
// (k-means assignment, src/impl/cluster/kmeans_cluster.cpp:262-275; RaBitQ rotation,
// src/impl/transform/random_orthogonal_transformer.cpp:59-77).  A register-tiled SIMT GEMM keeps
// that order for free: each thread owns its accumulators and walks k upward.
#pragma once

#include "common.cuh"

namespace vb200 {

constexpr int DENSE_BM = 128;
constexpr int DENSE_BN = 128;
constexpr int DENSE_BK = 16;
constexpr int DENSE_THREADS = 256;
constexpr int DENSE_PAD = 4;

enum DenseEpilogue { DENSE_STORE = 0, DENSE_ARGMIN = 1 };

__device__ __forceinline__ float
widen(float v) {
    return v;
}
__device__ __forceinline__ float
widen(uint16_t v) {  // bf16 bit pattern -> fp32 (generic::BF16ToFloat, src/simd/generic.cpp:191-196)
    return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

// Loads a [128 x 16] tile of a row-major matrix into shared memory transposed ([16][128+pad]),
// zero-filling outside rows < nrows, k < dim.
template <typename T, bool VEC>
__device__ __forceinline__ void
dense_load_tile(const T* __restrict__ M, uint64_t nrows, uint32_t dim, uint64_t row0, uint32_t k0,
                float (*S)[DENSE_BM + DENSE_PAD]) {
    if constexpr (VEC && sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int f = threadIdx.x + i * DENSE_THREADS;
            int r = f >> 2, kq = (f & 3) * 4;
            uint64_t row = row0 + r;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < nrows && k0 + kq < dim) {  // dim % 4 == 0 on this path
                v = __ldg(reinterpret_cast<const float4*>(M + row * dim + k0 + kq));
            }
            S[kq + 0][r] = v.x;
            S[kq + 1][r] = v.y;
            S[kq + 2][r] = v.z;
            S[kq + 3][r] = v.w;
        }
    } else if constexpr (VEC && sizeof(T) == 2) {
        int f = threadIdx.x;
        int r = f >> 1, kh = (f & 1) * 8;
        uint64_t row = row0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < nrows && k0 + kh < dim) {  // dim % 8 == 0 on this path
            v = __ldg(reinterpret_cast<const uint4*>(M + row * dim + k0 + kh));
        }
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            S[kh + 2 * j + 0][r] = __uint_as_float(w[j] << 16);
            S[kh + 2 * j + 1][r] = __uint_as_float(w[j] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < (DENSE_BM * DENSE_BK) / DENSE_THREADS; ++i) {
            int f = threadIdx.x + i * DENSE_THREADS;
            int r = f / DENSE_BK, kk = f % DENSE_BK;
            uint64_t row = row0 + r;
            float v = 0.f;
            if (row < nrows && k0 + kk < dim) {
                v = widen(M[row * dim + k0 + kk]);
            }
            S[kk][r] = v;
        }
    }
}

// out(i, j) = fma(alpha, <A_i, B_j>, bias[j])      (bias == nullptr -> 0)
//   DENSE_STORE : written to out[i * ld + j]
//   DENSE_ARGMIN: labels[i] = lowest j attaining the minimum over all j, best[i] the minimum
// grid.x = row tiles; grid.y = column-tile groups of `tiles_per_cta` (ARGMIN: one group).
template <typename TA, typename TB, int EPI, bool VEC>
__global__ void __launch_bounds__(DENSE_THREADS)
dense_kernel(const TA* __restrict__ A, uint64_t m, const TB* __restrict__ B, uint64_t n,
             uint32_t dim, float alpha, const float* __restrict__ bias, float* __restrict__ out,
             uint64_t ld, int32_t* __restrict__ labels, float* __restrict__ best_out,
             uint32_t tiles_per_cta) {
    __shared__ __align__(16) float As[DENSE_BK][DENSE_BM + DENSE_PAD];
    __shared__ __align__(16) float Bs[DENSE_BK][DENSE_BN + DENSE_PAD];

    const int tx = threadIdx.x & 15;
    const int ty = threadIdx.x >> 4;
    const uint64_t row0 = static_cast<uint64_t>(blockIdx.x) * DENSE_BM;
    const uint64_t n_tiles = (n + DENSE_BN - 1) / DENSE_BN;
    const uint64_t t_begin = static_cast<uint64_t>(blockIdx.y) * tiles_per_cta;
    uint64_t t_end = t_begin + tiles_per_cta;
    if (t_end > n_tiles) {
        t_end = n_tiles;
    }

    float best[8];
    uint32_t best_col[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        best[i] = INFINITY;
        best_col[i] = 0x7fffffffu;
    }

    for (uint64_t t = t_begin; t < t_end; ++t) {
        const uint64_t col0 = t * DENSE_BN;
        float acc[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc[i][j] = 0.f;
            }
        }
        for (uint32_t k0 = 0; k0 < dim; k0 += DENSE_BK) {
            dense_load_tile<TA, VEC>(A, m, dim, row0, k0, As);
            dense_load_tile<TB, VEC>(B, n, dim, col0, k0, Bs);
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < DENSE_BK; ++kk) {
                float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
                float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
                float4 b0 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
                float4 b1 = *reinterpret_cast<const float4*>(&Bs[kk][64 + tx * 4]);
                float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    }
                }
            }
            __syncthreads();
        }
        // epilogue
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint64_t col = col0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (col >= n) {
                continue;
            }
            float bj = bias != nullptr ? __ldg(bias + col) : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float score = fmaf(alpha, acc[i][j], bj);
                if constexpr (EPI == DENSE_STORE) {
                    uint64_t row = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
                    if (row < m) {
                        out[row * ld + col] = score;
                    }
                } else {
                    uint32_t c32 = static_cast<uint32_t>(col);
                    if (score < best[i] || (score == best[i] && c32 < best_col[i])) {
                        best[i] = score;
                        best_col[i] = c32;
                    }
                }
            }
        }
    }

    if constexpr (EPI == DENSE_ARGMIN) {
        // The 16 threads that share `ty` sit in one half-warp.
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                float ob = __shfl_xor_sync(0xffffffffu, best[i], off);
                uint32_t oc = __shfl_xor_sync(0xffffffffu, best_col[i], off);
                if (ob < best[i] || (ob == best[i] && oc < best_col[i])) {
                    best[i] = ob;
                    best_col[i] = oc;
                }
            }
            uint64_t row = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
            if (tx == 0 && row < m) {
                labels[row] = best_col[i] == 0x7fffffffu ? 0 : static_cast<int32_t>(best_col[i]);
                if (best_out != nullptr) {
                    best_out[row] = best[i];
                }
            }
        }
    }
}

// ---- host wrappers (dense.cu) ---------------------------------------------------------------

// out[m x n] (leading dimension ld) = fma(alpha, A B^T, bias).
int dense_scores_f32(const float* A, uint64_t m, const float* B, uint64_t n, uint32_t dim,
                     float alpha, const float* bias, float* out, uint64_t ld);
int dense_scores_bf16(const uint16_t* A, uint64_t m, const uint16_t* B, uint64_t n, uint32_t dim,
                      float alpha, const float* bias, float* out, uint64_t ld);
// labels[i] = argmin_j fma(alpha, <A_i, B_j>, bias[j]).
int dense_argmin_f32(const float* A, uint64_t m, const float* B, uint64_t n, uint32_t dim,
                     float alpha, const float* bias, int32_t* labels, float* best);
// sq[i] = FMA chain of M_i[d]^2 over d ascending.
int row_sqnorm_f32(const float* M, uint64_t rows, uint32_t dim, float* sq);
// out[r] = in[r] / |in[r]| (rows of norm 0 stay as they are); in == out is allowed.  The cosine metric is
// the inner product of rows and queries normalised this way.
int normalize_rows_f32(const float* in, uint64_t rows, uint32_t dim, float* out);
int row_sqnorm_bf16(const uint16_t* M, uint64_t rows, uint32_t dim, float* sq);

// For each row of scores[m x n] (leading dimension ld): the `k` smallest as keys
// (ordered score << 32 | column + col_base), ascending, KEY_INF padded.  k <= 1024.
int select_rows(const float* scores, uint64_t m, uint64_t n, uint64_t ld, uint32_t k,
                uint32_t col_base, uint64_t* keys_out, uint32_t keys_ld);

}  // namespace vb200
