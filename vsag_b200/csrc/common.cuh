// Shared plumbing for the sm_100a engine: status codes, error text, launch accounting, device
// buffers, host/device pointer staging and the ordered-key helpers every top-k kernel uses.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "../../include/vsag_b200.h"

namespace vb200 {

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
struct Status {
    int code;
    std::string msg;
};

void set_last_error(int code, const char* fmt, ...);
int last_error_code();

#define VB_FAIL(code, ...)                     \
    do {                                       \
        ::vb200::set_last_error(code, __VA_ARGS__); \
        return code;                           \
    } while (0)

#define VB_CHECK_ARG(cond, ...)                    \
    do {                                           \
        if (!(cond)) {                             \
            VB_FAIL(VB200_INVALID_ARGUMENT, __VA_ARGS__); \
        }                                          \
    } while (0)

#define VB_CUDA(expr)                                                                       \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess) {                                                            \
            int _c = (_e == cudaErrorMemoryAllocation) ? VB200_NO_ENOUGH_MEMORY             \
                                                       : VB200_INTERNAL_ERROR;              \
            VB_FAIL(_c, "%s failed at %s:%d: %s", #expr, __FILE__, __LINE__,                \
                    cudaGetErrorString(_e));                                                \
        }                                                                                   \
    } while (0)

#define VB_TRY(expr)        \
    do {                    \
        int _s = (expr);    \
        if (_s != 0) {      \
            return _s;      \
        }                   \
    } while (0)

// ---------------------------------------------------------------------------------------------
// stream + launch accounting
// ---------------------------------------------------------------------------------------------
cudaStream_t current_stream();
extern std::atomic<uint64_t> g_kernel_launches;

// Every kernel of this library is launched through this macro so the launch counter that
// vb200_kernel_launches() reports is a count, not an estimate.
#define VB_LAUNCH(kernel, grid, block, smem, ...)                                          \
    do {                                                                                   \
        kernel<<<(grid), (block), (smem), ::vb200::current_stream()>>>(__VA_ARGS__);       \
        ::vb200::g_kernel_launches.fetch_add(1, std::memory_order_relaxed);                \
        VB_CUDA(cudaGetLastError());                                                       \
    } while (0)

int sm_count();

// ---------------------------------------------------------------------------------------------
// device memory
// ---------------------------------------------------------------------------------------------
template <typename T>
struct DevBuf {
    T* ptr = nullptr;
    size_t cap = 0;  // elements
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : ptr(o.ptr), cap(o.cap) {
        o.ptr = nullptr;
        o.cap = 0;
    }
    DevBuf& operator=(DevBuf&& o) noexcept {
        if (this != &o) {
            release();
            ptr = o.ptr;
            cap = o.cap;
            o.ptr = nullptr;
            o.cap = 0;
        }
        return *this;
    }
    ~DevBuf() {
        release();
    }
    void release() {
        if (ptr != nullptr) {
            cudaFree(ptr);
        }
        ptr = nullptr;
        cap = 0;
    }
    // Grow-only reservation; contents are not preserved.
    int reserve(size_t n) {
        if (n <= cap) {
            return 0;
        }
        release();
        if (n == 0) {
            return 0;
        }
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, n * sizeof(T));
        if (e != cudaSuccess) {
            cudaGetLastError();
            VB_FAIL(VB200_NO_ENOUGH_MEMORY, "cudaMalloc of %zu bytes failed: %s", n * sizeof(T),
                    cudaGetErrorString(e));
        }
        ptr = static_cast<T*>(p);
        cap = n;
        return 0;
    }
    size_t bytes() const {
        return cap * sizeof(T);
    }
};

// Pinned host staging buffer (grow-only).
struct PinnedBuf {
    void* ptr = nullptr;
    size_t cap = 0;
    ~PinnedBuf() {
        if (ptr != nullptr) {
            cudaFreeHost(ptr);
        }
    }
    int reserve(size_t bytes) {
        if (bytes <= cap) {
            return 0;
        }
        if (ptr != nullptr) {
            cudaFreeHost(ptr);
            ptr = nullptr;
            cap = 0;
        }
        cudaError_t e = cudaMallocHost(&ptr, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            ptr = nullptr;
            VB_FAIL(VB200_NO_ENOUGH_MEMORY, "cudaMallocHost of %zu bytes failed", bytes);
        }
        cap = bytes;
        return 0;
    }
};

// True when `p` points into device (or managed) memory; host memory of any kind otherwise.
bool is_device_pointer(const void* p);
// True when `p` is device memory of the device current on the calling thread (or managed memory).
bool is_pointer_on_current_device(const void* p);

// A read-only view of caller data on the device: device pointers are used in place, host
// pointers are copied into an owned buffer on the current stream.
template <typename T>
struct DevInput {
    const T* ptr = nullptr;
    DevBuf<T> owned;
    int bind(const T* src, size_t n) {
        if (n == 0 || src == nullptr) {
            ptr = nullptr;
            return 0;
        }
        if (is_device_pointer(src)) {
            ptr = src;
            return 0;
        }
        VB_TRY(owned.reserve(n));
        VB_CUDA(cudaMemcpyAsync(owned.ptr, src, n * sizeof(T), cudaMemcpyHostToDevice,
                                current_stream()));
        ptr = owned.ptr;
        return 0;
    }
};

// Copies `n` elements from device memory to a caller pointer that may be host or device.
template <typename T>
int
copy_out(T* dst, const T* src_dev, size_t n) {
    if (n == 0 || dst == nullptr) {
        return 0;
    }
    cudaMemcpyKind kind = is_device_pointer(dst) ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
    VB_CUDA(cudaMemcpyAsync(dst, src_dev, n * sizeof(T), kind, current_stream()));
    return 0;
}

inline int
sync_stream() {
    VB_CUDA(cudaStreamSynchronize(current_stream()));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

// Monotone map float -> uint32: a < b  <=>  ordered(a) < ordered(b) (with -0 < +0).
__device__ __forceinline__ uint32_t
float_to_ordered(float f) {
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float
ordered_to_float(uint32_t u) {
    uint32_t b = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(b);
}

__device__ __forceinline__ uint64_t
make_key(float dist, uint32_t payload) {
    return (static_cast<uint64_t>(float_to_ordered(dist)) << 32) | payload;
}

constexpr uint64_t KEY_INF = 0xFFFFFFFFFFFFFFFFull;

__host__ __device__ __forceinline__ uint32_t
next_pow2(uint32_t v) {
    uint32_t p = 1;
    while (p < v) {
        p <<= 1;
    }
    return p;
}

// Bitonic sort (ascending) of n2 (a power of two) 64-bit keys in shared memory by one warp.
__device__ __forceinline__ void
warp_bitonic_sort(uint64_t* keys, uint32_t n2, uint32_t lane) {
    for (uint32_t size = 2; size <= n2; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            __syncwarp();
            for (uint32_t t = lane; t < (n2 >> 1); t += 32) {
                uint32_t i = 2 * t - (t & (stride - 1));
                uint32_t j = i + stride;
                bool up = (i & size) == 0;
                uint64_t a = keys[i], b = keys[j];
                if ((a > b) == up) {
                    keys[i] = b;
                    keys[j] = a;
                }
            }
        }
    }
    __syncwarp();
}

// Bitonic sort (ascending) of n2 (a power of two) keys in shared memory by the whole CTA.
// Every thread of the CTA must call it.
__device__ __forceinline__ void
block_bitonic_sort(uint64_t* keys, uint32_t n2) {
    for (uint32_t size = 2; size <= n2; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (uint32_t t = threadIdx.x; t < (n2 >> 1); t += blockDim.x) {
                uint32_t i = 2 * t - (t & (stride - 1));
                uint32_t j = i + stride;
                bool up = (i & size) == 0;
                uint64_t a = keys[i], b = keys[j];
                if ((a > b) == up) {
                    keys[i] = b;
                    keys[j] = a;
                }
            }
        }
    }
    __syncthreads();
}

// Streaming top-k selector for one CTA.  Keys are offered in rounds; a key survives only if it is
// below the running k-th smallest.  Shared memory: cap keys (cap a power of two,
// cap >= k + per_round) plus two words of state.
struct BlockSelect {
    uint64_t* keys;
    uint32_t* state;  // [0] = count, [1..2] = threshold key (lo, hi)
    uint32_t k;
    uint32_t cap;

    __device__ void
    init(uint64_t* keys_smem, uint32_t* state_smem, uint32_t k_, uint32_t cap_) {
        keys = keys_smem;
        state = state_smem;
        k = k_;
        cap = cap_;
        if (threadIdx.x == 0) {
            state[0] = 0;
            state[1] = 0xFFFFFFFFu;
            state[2] = 0xFFFFFFFFu;
        }
        __syncthreads();
    }
    __device__ __forceinline__ uint64_t
    threshold() const {
        return (static_cast<uint64_t>(state[2]) << 32) | state[1];
    }
    // Call before a round in which the CTA will offer at most `incoming` keys.
    __device__ void
    make_room(uint32_t incoming) {
        __syncthreads();
        uint32_t held = state[0];
        __syncthreads();
        if (held + incoming > cap) {
            compact();
        }
    }
    __device__ __forceinline__ void
    offer(uint64_t key, uint64_t thr) {
        if (key < thr) {
            uint32_t slot = atomicAdd(&state[0], 1u);
            keys[slot] = key;
        }
    }
    // Sorts what is held, keeps the k smallest and tightens the threshold.
    __device__ void
    compact() {
        __syncthreads();
        uint32_t cnt = state[0];
        uint32_t n2 = next_pow2(cnt < 2 ? 2 : cnt);
        for (uint32_t i = cnt + threadIdx.x; i < n2; i += blockDim.x) {
            keys[i] = KEY_INF;
        }
        block_bitonic_sort(keys, n2);
        if (threadIdx.x == 0) {
            if (cnt > k) {
                state[0] = k;
            }
            if (cnt >= k) {
                uint64_t t = keys[k - 1];
                state[1] = static_cast<uint32_t>(t);
                state[2] = static_cast<uint32_t>(t >> 32);
            }
        }
        __syncthreads();
    }
    // After finish(), keys[0 .. min(count,k)) are the result in ascending order.
    __device__ uint32_t
    finish() {
        compact();
        return state[0];
    }
};

#endif  // __CUDACC__

}  // namespace vb200
