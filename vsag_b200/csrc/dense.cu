// Host wrappers for the fixed-order dense kernels, the row-wise top-k selector and the library
// state (error text, stream, launch counter).
#include "dense.cuh"

namespace vb200 {

// ---------------------------------------------------------------------------------------------
// library state
// ---------------------------------------------------------------------------------------------
static thread_local int tl_err_code = 0;
static thread_local char tl_err_msg[1024] = {0};
static thread_local cudaStream_t tl_stream = nullptr;
std::atomic<uint64_t> g_kernel_launches{0};

void
set_last_error(int code, const char* fmt, ...) {
    tl_err_code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_err_msg, sizeof(tl_err_msg), fmt, ap);
    va_end(ap);
}

int
last_error_code() {
    return tl_err_code;
}

cudaStream_t
current_stream() {
    return tl_stream;
}

int
sm_count() {
    // per device ordinal: grids are sized for the device the calling thread has current
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return 148;
    }
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148;
        }
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

bool
is_device_pointer(const void* p) {
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

bool
is_pointer_on_current_device(const void* p) {
    cudaPointerAttributes attr;
    int dev = -1;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (attr.type == cudaMemoryTypeManaged) {
        return true;
    }
    return attr.type == cudaMemoryTypeDevice && attr.device == dev;
}

// ---------------------------------------------------------------------------------------------
// dense wrappers
// ---------------------------------------------------------------------------------------------
template <typename T>
static bool
vec_ok(const T* A, const T* B, uint32_t dim) {
    const uint32_t per = 16 / sizeof(T);
    return dim % per == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(B) & 15) == 0;
}

template <typename T>
static int
dense_scores_impl(const T* A, uint64_t m, const T* B, uint64_t n, uint32_t dim, float alpha,
                  const float* bias, float* out, uint64_t ld) {
    if (m == 0 || n == 0) {
        return 0;
    }
    const uint64_t row_tiles = (m + DENSE_BM - 1) / DENSE_BM;
    const uint64_t col_tiles = (n + DENSE_BN - 1) / DENSE_BN;
    // Enough column groups to fill the machine a few times over, never more than 65535.
    uint64_t want_ctas = static_cast<uint64_t>(sm_count()) * 8;
    uint64_t groups = (want_ctas + row_tiles - 1) / row_tiles;
    if (groups > col_tiles) {
        groups = col_tiles;
    }
    if (groups < 1) {
        groups = 1;
    }
    uint32_t tiles_per_cta = static_cast<uint32_t>((col_tiles + groups - 1) / groups);
    groups = (col_tiles + tiles_per_cta - 1) / tiles_per_cta;
    VB_CHECK_ARG(groups <= 65535 && row_tiles <= 0x7fffffffu, "dense_scores: shape too large");
    dim3 grid(static_cast<uint32_t>(row_tiles), static_cast<uint32_t>(groups));
    auto kernel = vec_ok(A, B, dim) ? dense_kernel<T, T, DENSE_STORE, true>
                                    : dense_kernel<T, T, DENSE_STORE, false>;
    VB_LAUNCH(kernel, grid, DENSE_THREADS, 0, A, m, B, n, dim, alpha, bias, out, ld, nullptr, nullptr,
              tiles_per_cta);
    return 0;
}

int
dense_scores_f32(const float* A, uint64_t m, const float* B, uint64_t n, uint32_t dim, float alpha,
                 const float* bias, float* out, uint64_t ld) {
    return dense_scores_impl<float>(A, m, B, n, dim, alpha, bias, out, ld);
}

int
dense_scores_bf16(const uint16_t* A, uint64_t m, const uint16_t* B, uint64_t n, uint32_t dim,
                  float alpha, const float* bias, float* out, uint64_t ld) {
    return dense_scores_impl<uint16_t>(A, m, B, n, dim, alpha, bias, out, ld);
}

int
dense_argmin_f32(const float* A, uint64_t m, const float* B, uint64_t n, uint32_t dim, float alpha,
                 const float* bias, int32_t* labels, float* best) {
    if (m == 0) {
        return 0;
    }
    VB_CHECK_ARG(n > 0 && n < 0x7fffffffu, "dense_argmin: bad column count");
    const uint64_t row_tiles = (m + DENSE_BM - 1) / DENSE_BM;
    const uint64_t col_tiles = (n + DENSE_BN - 1) / DENSE_BN;
    VB_CHECK_ARG(row_tiles <= 0x7fffffffu, "dense_argmin: too many rows");
    dim3 grid(static_cast<uint32_t>(row_tiles), 1);
    auto kernel = vec_ok(A, B, dim) ? dense_kernel<float, float, DENSE_ARGMIN, true>
                                    : dense_kernel<float, float, DENSE_ARGMIN, false>;
    VB_LAUNCH(kernel, grid, DENSE_THREADS, 0, A, m, B, n, dim, alpha, bias, nullptr, 0, labels, best,
              static_cast<uint32_t>(col_tiles));
    return 0;
}

template <typename T>
__global__ void
row_sqnorm_kernel(const T* __restrict__ M, uint64_t rows, uint32_t dim, float* __restrict__ sq) {
    uint64_t r = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= rows) {
        return;
    }
    const T* p = M + r * dim;
    float s = 0.f;
    for (uint32_t d = 0; d < dim; ++d) {
        float v = widen(p[d]);
        s = fmaf(v, v, s);
    }
    sq[r] = s;
}

int
row_sqnorm_f32(const float* M, uint64_t rows, uint32_t dim, float* sq) {
    if (rows == 0) {
        return 0;
    }
    VB_LAUNCH(row_sqnorm_kernel<float>, static_cast<uint32_t>((rows + 127) / 128), 128, 0, M, rows,
              dim, sq);
    return 0;
}

int
row_sqnorm_bf16(const uint16_t* M, uint64_t rows, uint32_t dim, float* sq) {
    if (rows == 0) {
        return 0;
    }
    VB_LAUNCH(row_sqnorm_kernel<uint16_t>, static_cast<uint32_t>((rows + 127) / 128), 128, 0, M,
              rows, dim, sq);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Normalize (src/simd/generic.cpp:875-879): norm = sqrt(sum of fma(x_d, x_d, acc)) in ascending d,
// every element divided by it (by 1 when the norm is 0, src/simd/kernels/scalar_op.h:40-42).
// One warp per row: the row is staged in shared memory, lane 0 walks the chain, all lanes divide.
// in == out is allowed.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
normalize_rows_kernel(const float* __restrict__ in, uint64_t rows, uint32_t dim, float* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* stage = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(threadIdx.x >> 5) * dim;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= rows) {
        return;
    }
    const float* src = in + row * dim;
    for (uint32_t d = lane; d < dim; d += 32) {
        stage[d] = src[d];
    }
    __syncwarp();
    float norm = 0.f;
    if (lane == 0) {
        float s = 0.f;
        for (uint32_t d = 0; d < dim; ++d) {
            s = fmaf(stage[d], stage[d], s);
        }
        norm = __fsqrt_rn(s);
        if (norm == 0.f) {
            norm = 1.0f;
        }
    }
    norm = __shfl_sync(0xffffffffu, norm, 0);
    float* dst = out + row * dim;
    for (uint32_t d = lane; d < dim; d += 32) {
        dst[d] = __fdiv_rn(stage[d], norm);
    }
}

int
normalize_rows_f32(const float* in, uint64_t rows, uint32_t dim, float* out) {
    if (rows == 0) {
        return 0;
    }
    const size_t smem = 4 * static_cast<size_t>(dim) * sizeof(float);
    VB_CHECK_ARG(smem <= 200 * 1024, "dim too large to normalise on the device");
    if (smem > 48 * 1024) {
        VB_CUDA(cudaFuncSetAttribute(normalize_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
    }
    VB_LAUNCH(normalize_rows_kernel, static_cast<uint32_t>((rows + 3) / 4), 128, smem, in, rows, dim, out);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// row-wise top-k over a materialised score matrix
// ---------------------------------------------------------------------------------------------
constexpr int SELECT_THREADS = 256;

__global__ void __launch_bounds__(SELECT_THREADS)
select_rows_kernel(const float* __restrict__ scores, uint64_t n, uint64_t ld, uint32_t k,
                   uint32_t cap, uint32_t col_base, uint64_t* __restrict__ keys_out,
                   uint32_t keys_ld) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);
    uint32_t* state = reinterpret_cast<uint32_t*>(keys + cap);
    BlockSelect sel;
    sel.init(keys, state, k, cap);
    const float* row = scores + static_cast<uint64_t>(blockIdx.x) * ld;
    // Four rounds' worth of scores are loaded together so that their latency overlaps, and a
    // round costs one barrier unless some thread actually has a candidate (after the first few
    // hundred columns almost none does).
    constexpr int ROUNDS = 4;
    uint64_t thr = sel.threshold();
    for (uint64_t base = 0; base < n; base += SELECT_THREADS * ROUNDS) {
        uint64_t key[ROUNDS];
#pragma unroll
        for (int u = 0; u < ROUNDS; ++u) {
            const uint64_t c = base + static_cast<uint64_t>(u) * SELECT_THREADS + threadIdx.x;
            key[u] = KEY_INF;
            if (c < n) {
                const float s = __ldg(row + c);
                if (s == s) {  // NaN scores are never candidates
                    key[u] = make_key(s, static_cast<uint32_t>(c) + col_base);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < ROUNDS; ++u) {
            if (__syncthreads_or(key[u] < thr)) {
                sel.make_room(SELECT_THREADS);
                thr = sel.threshold();
                sel.offer(key[u], thr);
            }
        }
    }
    uint32_t cnt = sel.finish();
    uint64_t* dst = keys_out + static_cast<uint64_t>(blockIdx.x) * keys_ld;
    for (uint32_t i = threadIdx.x; i < k; i += SELECT_THREADS) {
        dst[i] = i < cnt ? keys[i] : KEY_INF;
    }
}

// Long rows, modest k: instead of streaming the row through a selector that re-sorts its buffer
// every few hundred candidates, find the value range of the row, histogram it, read off the bin
// that holds the k-th smallest score, collect everything up to that bin (a little more than k
// keys) and sort once.  A row whose scores do not spread (or are not finite) takes the streaming
// path instead.
constexpr int HIST_BINS = 2048;
constexpr uint32_t HIST_CAP = 1024;   // keys collected at most; also the streaming path's buffer

__device__ __forceinline__ uint32_t
hist_bin(float s, float mn, float scale) {
    if (!(s > mn)) {
        return 0;
    }
    const float t = (s - mn) * scale;
    return t >= static_cast<float>(HIST_BINS - 1) ? HIST_BINS - 1 : static_cast<uint32_t>(t);
}

__global__ void __launch_bounds__(SELECT_THREADS)
select_rows_hist_kernel(const float* __restrict__ scores, uint64_t n, uint64_t ld, uint32_t k,
                        uint32_t col_base, uint64_t* __restrict__ keys_out, uint32_t keys_ld) {
    __shared__ uint32_t hist[HIST_BINS];
    __shared__ __align__(16) uint64_t keys[HIST_CAP];
    __shared__ uint32_t state[4];
    __shared__ uint32_t scan[SELECT_THREADS];
    __shared__ float red_mn[SELECT_THREADS / 32], red_mx[SELECT_THREADS / 32];
    __shared__ uint32_t pick_bin, pick_count;
    const uint32_t tid = threadIdx.x;
    const float* row = scores + static_cast<uint64_t>(blockIdx.x) * ld;
    uint64_t* dst = keys_out + static_cast<uint64_t>(blockIdx.x) * keys_ld;

    // range of the finite scores, from every fourth stretch of the row: scores outside the sampled
    // range fall into the first or the last bin, which only matters to the choice of the path below
    float mn = INFINITY, mx = -INFINITY;
    for (uint64_t c = tid; c < n; c += 4 * SELECT_THREADS) {
        const float s = __ldg(row + c);
        if (fabsf(s) < INFINITY) {
            mn = fminf(mn, s);
            mx = fmaxf(mx, s);
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((tid & 31) == 0) {
        red_mn[tid >> 5] = mn;
        red_mx[tid >> 5] = mx;
    }
    for (uint32_t b = tid; b < HIST_BINS; b += SELECT_THREADS) {
        hist[b] = 0;
    }
    if (tid == 0) {
        pick_bin = 0xFFFFFFFFu;
        pick_count = 0;
        state[3] = 0;
    }
    __syncthreads();
    mn = red_mn[0];
    mx = red_mx[0];
    for (int w = 1; w < SELECT_THREADS / 32; ++w) {
        mn = fminf(mn, red_mn[w]);
        mx = fmaxf(mx, red_mx[w]);
    }
    const float scale = static_cast<float>(HIST_BINS - 1) / (mx - mn);
    const bool spread = mx > mn && scale > 0.f && scale < INFINITY;
    if (spread) {
        for (uint64_t c = tid; c < n; c += SELECT_THREADS) {
            const float s = __ldg(row + c);
            if (s == s) {
                atomicAdd(&hist[hist_bin(s, mn, scale)], 1u);
            }
        }
        __syncthreads();
        // inclusive scan of the bins, eight per thread
        constexpr int PER = HIST_BINS / SELECT_THREADS;
        uint32_t local[PER];
        uint32_t sum = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            sum += hist[tid * PER + i];
            local[i] = sum;
        }
        scan[tid] = sum;
        __syncthreads();
        for (uint32_t off = 1; off < SELECT_THREADS; off <<= 1) {
            const uint32_t v = tid >= off ? scan[tid - off] : 0;
            __syncthreads();
            scan[tid] += v;
            __syncthreads();
        }
        const uint32_t before = scan[tid] - sum;
        const uint32_t total = scan[SELECT_THREADS - 1];
        if (total <= k) {
            if (tid == 0) {
                pick_bin = HIST_BINS - 1;
                pick_count = total;
            }
        } else if (before < k && before + sum >= k) {
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                if (before + local[i] >= k) {
                    pick_bin = tid * PER + i;
                    pick_count = before + local[i];
                    break;
                }
            }
        }
        __syncthreads();
        const uint32_t last_bin = pick_bin, count = pick_count;
        if (count <= HIST_CAP) {
            for (uint64_t c = tid; c < n; c += SELECT_THREADS) {
                const float s = __ldg(row + c);
                if (s == s && hist_bin(s, mn, scale) <= last_bin) {
                    keys[atomicAdd(&state[3], 1u)] = make_key(s, static_cast<uint32_t>(c) + col_base);
                }
            }
            const uint32_t n2 = next_pow2(count < 2 ? 2 : count);
            __syncthreads();
            for (uint32_t i = count + tid; i < n2; i += SELECT_THREADS) {
                keys[i] = KEY_INF;
            }
            block_bitonic_sort(keys, n2);
            for (uint32_t i = tid; i < k; i += SELECT_THREADS) {
                dst[i] = i < count ? keys[i] : KEY_INF;
            }
            return;
        }
    }
    // streaming path
    __syncthreads();
    BlockSelect sel;
    sel.init(keys, state, k, HIST_CAP);
    uint64_t thr = sel.threshold();
    for (uint64_t base = 0; base < n; base += SELECT_THREADS) {
        const uint64_t c = base + tid;
        uint64_t key = KEY_INF;
        if (c < n) {
            const float s = __ldg(row + c);
            if (s == s) {
                key = make_key(s, static_cast<uint32_t>(c) + col_base);
            }
        }
        if (__syncthreads_or(key < thr)) {
            sel.make_room(SELECT_THREADS);
            thr = sel.threshold();
            sel.offer(key, thr);
        }
    }
    const uint32_t cnt = sel.finish();
    for (uint32_t i = tid; i < k; i += SELECT_THREADS) {
        dst[i] = i < cnt ? keys[i] : KEY_INF;
    }
}

int
select_rows(const float* scores, uint64_t m, uint64_t n, uint64_t ld, uint32_t k, uint32_t col_base,
            uint64_t* keys_out, uint32_t keys_ld) {
    if (m == 0) {
        return 0;
    }
    VB_CHECK_ARG(k >= 1 && k <= 1024, "select_rows: k must be in [1, 1024], got %u", k);
    VB_CHECK_ARG(m <= 0x7fffffffu, "select_rows: too many rows");
    if (n >= 4096 && k + SELECT_THREADS <= HIST_CAP) {
        VB_LAUNCH(select_rows_hist_kernel, static_cast<uint32_t>(m), SELECT_THREADS, 0, scores, n, ld, k, col_base,
                  keys_out, keys_ld);
        return 0;
    }
    uint32_t cap = next_pow2(k + SELECT_THREADS);
    size_t smem = cap * sizeof(uint64_t) + 4 * sizeof(uint32_t);
    VB_LAUNCH(select_rows_kernel, static_cast<uint32_t>(m), SELECT_THREADS, smem, scores, n, ld, k,
              cap, col_base, keys_out, keys_ld);
    return 0;
}

}  // namespace vb200

// ---------------------------------------------------------------------------------------------
// C ABI: library state
// ---------------------------------------------------------------------------------------------
extern "C" int
vb200_last_error(char* buf, size_t buf_len) {
    if (buf != nullptr && buf_len > 0) {
        strncpy(buf, vb200::tl_err_msg, buf_len - 1);
        buf[buf_len - 1] = 0;
    }
    return vb200::tl_err_code;
}

extern "C" int
vb200_set_stream(void* cuda_stream) {
    vb200::tl_stream = static_cast<cudaStream_t>(cuda_stream);
    return 0;
}

extern "C" uint64_t
vb200_kernel_launches(void) {
    return vb200::g_kernel_launches.load();
}

extern "C" int
vb200_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        VB_FAIL(VB200_INTERNAL_ERROR, "no CUDA device: %s", cudaGetErrorString(e));
    }
    return n;
}
