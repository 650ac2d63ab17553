// SQ8 scalar quantizer on the GPU: bound training (order statistics by radix select) and the
// bit-exact encoder.
#include "sq8.cuh"

namespace vb200 {

// ---------------------------------------------------------------------------------------------
// training
// ---------------------------------------------------------------------------------------------

// keys[d * cnt + j] = ordered(data[((j * step) % count) * dim + d]); one column per dimension.
__global__ void
sq8_sample_kernel(const float* __restrict__ data, uint64_t count, uint32_t dim, uint64_t step,
                  uint32_t cnt, uint32_t* __restrict__ keys) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= static_cast<uint64_t>(cnt) * dim) {
        return;
    }
    uint32_t j = static_cast<uint32_t>(e / dim);
    uint32_t d = static_cast<uint32_t>(e % dim);
    uint64_t row = (static_cast<uint64_t>(j) * step) % count;
    keys[static_cast<uint64_t>(d) * cnt + j] = float_to_ordered(__ldg(data + row * dim + d));
}

// Value of rank `rank` (0 = smallest) among cnt ordered keys: 4 passes of an 8-bit radix select.
__device__ uint32_t
block_radix_select(const uint32_t* __restrict__ keys, uint32_t cnt, uint32_t rank, uint32_t* hist,
                   uint32_t* bcast) {
    uint32_t prefix = 0, mask = 0;
    for (int pass = 3; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (uint32_t b = threadIdx.x; b < 256; b += blockDim.x) {
            hist[b] = 0;
        }
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < cnt; j += blockDim.x) {
            uint32_t key = keys[j];
            if ((key & mask) == prefix) {
                atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t cum = 0, digit = 255;
            for (uint32_t b = 0; b < 256; ++b) {
                if (rank < cum + hist[b]) {
                    digit = b;
                    break;
                }
                cum += hist[b];
            }
            bcast[0] = digit;
            bcast[1] = rank - cum;
        }
        __syncthreads();
        prefix |= bcast[0] << shift;
        mask |= 0xffu << shift;
        rank = bcast[1];
        __syncthreads();
    }
    return prefix;
}

// One CTA per dimension.  lower = value of rank (ignore-1), upper = value of rank (cnt-ignore):
// the ignore-th smallest / largest sample, which is what the reference's two bounded heaps hold
// on top after the pass (scalar_quantization_trainer.cpp:89-121).  ignore = 1 gives min / max.
__global__ void __launch_bounds__(256)
sq8_bounds_kernel(const uint32_t* __restrict__ keys, uint32_t cnt, uint32_t ignore,
                  float* __restrict__ lower, float* __restrict__ diff) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t bcast[2];
    const uint32_t* col = keys + static_cast<uint64_t>(blockIdx.x) * cnt;
    uint32_t lo_key = block_radix_select(col, cnt, ignore - 1, hist, bcast);
    uint32_t up_key = block_radix_select(col, cnt, cnt - ignore, hist, bcast);
    if (threadIdx.x == 0) {
        float lo = ordered_to_float(lo_key);
        float up = ordered_to_float(up_key);
        lower[blockIdx.x] = lo;
        diff[blockIdx.x] = __fsub_rn(up, lo);
    }
}

int
sq8_train_device(const float* data_dev, uint64_t count, uint32_t dim, int mode, float* lower_dev,
                 float* diff_dev) {
    VB_CHECK_ARG(count > 0 && dim > 0, "sq8 train: empty input");
    VB_CHECK_ARG(mode == VB200_SQ_TRAIN_CLASSIC || mode == VB200_SQ_TRAIN_TRUNC_BOUND,
                 "sq8 train: unknown mode %d", mode);
    const uint64_t max_sample = 100000;
    uint64_t step = 2147483647ull % count;
    uint32_t cnt = static_cast<uint32_t>(max_sample);
    if (count <= max_sample) {
        step = 1;
        cnt = static_cast<uint32_t>(count);
    }
    uint32_t ignore = 1;
    if (mode == VB200_SQ_TRAIN_TRUNC_BOUND) {
        ignore = static_cast<uint32_t>(static_cast<double>(cnt - 1) * 0.001);
        if (ignore < 1) {
            ignore = 1;
        }
    }
    DevBuf<uint32_t> keys;
    VB_TRY(keys.reserve(static_cast<size_t>(cnt) * dim));
    uint64_t total = static_cast<uint64_t>(cnt) * dim;
    VB_LAUNCH(sq8_sample_kernel, static_cast<uint32_t>((total + 255) / 256), 256, 0, data_dev, count,
              dim, step, cnt, keys.ptr);
    VB_LAUNCH(sq8_bounds_kernel, dim, 256, 0, keys.ptr, cnt, ignore, lower_dev, diff_dev);
    VB_TRY(sync_stream());
    return 0;
}

// ---------------------------------------------------------------------------------------------
// SQ8 uniform
// ---------------------------------------------------------------------------------------------

// extremes[0] = min, extremes[1] = max (as ordered keys) over the sampled rows' values.
__global__ void __launch_bounds__(256)
sq8u_extremes_kernel(const float* __restrict__ data, uint64_t count, uint32_t dim, uint64_t step, uint32_t cnt,
                     uint32_t* __restrict__ extremes) {
    __shared__ uint32_t s_lo[8], s_hi[8];
    uint32_t lo = 0xFFFFFFFFu, hi = 0u;
    const uint64_t total = static_cast<uint64_t>(cnt) * dim;
    for (uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < total;
         e += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint64_t j = e / dim;
        const uint32_t d = static_cast<uint32_t>(e % dim);
        const uint64_t row = (j * step) % count;
        const uint32_t key = float_to_ordered(__ldg(data + row * dim + d));
        lo = key < lo ? key : lo;
        hi = key > hi ? key : hi;
    }
    for (int off = 16; off > 0; off >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, off));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, off));
    }
    if ((threadIdx.x & 31) == 0) {
        s_lo[threadIdx.x >> 5] = lo;
        s_hi[threadIdx.x >> 5] = hi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            lo = min(lo, s_lo[w]);
            hi = max(hi, s_hi[w]);
        }
        atomicMin(extremes, lo);
        atomicMax(extremes + 1, hi);
    }
}

__global__ void
sq8u_model_kernel(const uint32_t* __restrict__ extremes, float* __restrict__ model) {
    const float lo = ordered_to_float(extremes[0]), up = ordered_to_float(extremes[1]);
    model[0] = lo;
    model[1] = __fsub_rn(up, lo);   // diff_ -= lower_bound_ (:95)
}

int
sq8u_train_device(const float* data_dev, uint64_t count, uint32_t dim, float* model_dev) {
    VB_CHECK_ARG(count > 0 && dim > 0, "sq8_uniform train: empty input");
    const uint64_t max_sample = 100000;
    uint64_t step = 2147483647ull % count;
    uint32_t cnt = static_cast<uint32_t>(max_sample);
    if (count <= max_sample) {
        step = 1;
        cnt = static_cast<uint32_t>(count);
    }
    DevBuf<uint32_t> extremes;
    VB_TRY(extremes.reserve(2));
    const uint32_t init[2] = {0xFFFFFFFFu, 0u};
    VB_CUDA(cudaMemcpyAsync(extremes.ptr, init, sizeof(init), cudaMemcpyHostToDevice, current_stream()));
    const uint64_t total = static_cast<uint64_t>(cnt) * dim;
    const uint32_t blocks = static_cast<uint32_t>(std::min<uint64_t>((total + 255) / 256, 4096));
    VB_LAUNCH(sq8u_extremes_kernel, blocks, 256, 0, data_dev, count, dim, step, cnt, extremes.ptr);
    VB_LAUNCH(sq8u_model_kernel, 1, 1, 0, extremes.ptr, model_dev);
    return sync_stream();
}

// One warp per row.  EncodeOneImpl (:102-142) operation by operation: inv_diff = 1 / diff (0 when diff is 0),
// delta = (x - lower) * inv_diff, clamp, truncate 255 * delta; norm = integer sum of squared codes; sum = the
// values added one after the other in fp32 (lane 0 walks the row for it: the order is part of the result).
__global__ void __launch_bounds__(128)
sq8u_encode_kernel(const float* __restrict__ data, uint64_t count, uint32_t dim, int metric_is_l2, float lower,
                   float inv_diff, const uint32_t* __restrict__ dst_pos, uint8_t* __restrict__ codes,
                   uint32_t code_stride, uint32_t code_size) {
    const uint64_t i = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    if (i >= count) {
        return;
    }
    uint64_t p = i;
    if (dst_pos != nullptr) {
        const uint32_t t = dst_pos[i];
        if (t == 0xFFFFFFFFu) {
            return;
        }
        p = t;
    }
    const float* x = data + i * dim;
    uint8_t* c = codes + p * code_stride;
    unsigned long long norm = 0;
    for (uint32_t d = lane; d < code_size - (metric_is_l2 ? 8u : 4u); d += 32) {
        uint8_t scaled = 0;
        if (d < dim) {
            float delta = __fmul_rn(__fsub_rn(__ldg(x + d), lower), inv_diff);
            if (!(delta >= 0.0f)) {
                delta = 0.0f;
            } else if (delta > 0.999f) {
                delta = 1.0f;
            }
            scaled = static_cast<uint8_t>(__fmul_rn(255.0f, delta));
        }
        c[d] = scaled;
        norm += static_cast<unsigned long long>(scaled) * scaled;
    }
    for (int off = 16; off > 0; off >>= 1) {
        norm += __shfl_xor_sync(0xffffffffu, norm, off);
    }
    if (lane == 0) {
        if (metric_is_l2) {
            *reinterpret_cast<unsigned long long*>(c + code_size - 8) = norm;
        } else {
            float sum = 0.f;
            for (uint32_t d = 0; d < dim; ++d) {
                sum = __fadd_rn(sum, __ldg(x + d));
            }
            *reinterpret_cast<float*>(c + code_size - 4) = sum;
        }
    }
}

int
sq8u_encode_device(const float* data_dev, uint64_t count, uint32_t dim, int metric_is_l2, float lower, float diff,
                   const uint32_t* dst_pos_dev, uint8_t* codes_dev, uint32_t code_stride) {
    if (count == 0) {
        return 0;
    }
    const float inv_diff = diff == 0.0f ? 0.0f : 1.0f / diff;
    const uint64_t threads = count * 32;
    VB_LAUNCH(sq8u_encode_kernel, static_cast<uint32_t>((threads + 127) / 128), 128, 0, data_dev, count, dim,
              metric_is_l2, lower, inv_diff, dst_pos_dev, codes_dev, code_stride, sq8u_code_size(dim, metric_is_l2));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// encoding
// ---------------------------------------------------------------------------------------------

// codes[dst(i) * code_stride + d] = encode(data[i * dim + d]) with dst(i) = dst_pos[i] when
// `dst_pos` is given (0xFFFFFFFF = row not stored), else i.  Arithmetic mirrors
// ScalarQuantizer::EncodeOneImpl (scalar_quantizer.cpp:98-106) operation by operation: IEEE
// subtract, IEEE divide, clamp, multiply by 255, truncate.
__global__ void
sq8_encode_kernel(const float* __restrict__ data, uint64_t count, uint32_t dim,
                  const float* __restrict__ lower, const float* __restrict__ diff,
                  const uint32_t* __restrict__ dst_pos, uint8_t* __restrict__ codes,
                  uint32_t code_stride) {
    uint64_t e = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count * dim) {
        return;
    }
    uint64_t i = e / dim;
    uint32_t d = static_cast<uint32_t>(e % dim);
    uint64_t p = i;
    if (dst_pos != nullptr) {
        uint32_t t = dst_pos[i];
        if (t == 0xFFFFFFFFu) {
            return;
        }
        p = t;
    }
    float x = __ldg(data + e);
    float df = __ldg(diff + d);
    float delta;
    if (df < 1.1920928955078125e-07f) {  // std::numeric_limits<float>::epsilon()
        delta = 1.0f;
    } else {
        delta = __fdiv_rn(__fsub_rn(x, __ldg(lower + d)), df);
    }
    if (!(delta >= 0.0f)) {
        delta = 0.0f;
    } else if (delta > 0.999f) {
        delta = 1.0f;
    }
    float scaled = __fmul_rn(255.0f, delta);
    codes[p * code_stride + d] = static_cast<uint8_t>(static_cast<uint32_t>(scaled));
}

int
sq8_encode_device(const float* data_dev, uint64_t count, uint32_t dim, const float* lower_dev,
                  const float* diff_dev, const uint32_t* dst_pos_dev, uint8_t* codes_dev,
                  uint32_t code_stride) {
    if (count == 0) {
        return 0;
    }
    uint64_t total = count * dim;
    uint64_t blocks = (total + 255) / 256;
    VB_CHECK_ARG(blocks <= 0x7fffffffu, "sq8 encode: batch too large");
    VB_LAUNCH(sq8_encode_kernel, static_cast<uint32_t>(blocks), 256, 0, data_dev, count, dim,
              lower_dev, diff_dev, dst_pos_dev, codes_dev, code_stride);
    return 0;
}

}  // namespace vb200

using namespace vb200;

extern "C" int
vb200_sq8_train(const float* data, uint64_t count, uint32_t dim, int mode, float* lower, float* diff) {
    VB_CHECK_ARG(data != nullptr && lower != nullptr && diff != nullptr, "sq8 train: null pointer");
    VB_CHECK_ARG(count > 0 && dim > 0, "sq8 train: empty input");
    DevBuf<float> out;
    VB_TRY(out.reserve(2 * static_cast<size_t>(dim)));
    if (is_device_pointer(data)) {
        VB_TRY(sq8_train_device(data, count, dim, mode, out.ptr, out.ptr + dim));
    } else {
        // Only the sampled rows cross the bus: gather them on the host first.
        const uint64_t max_sample = 100000;
        uint64_t step = 2147483647ull % count;
        uint64_t cnt = max_sample;
        if (count <= max_sample) {
            step = 1;
            cnt = count;
        }
        std::vector<float> sample;
        try {
            sample.resize(cnt * dim);
        } catch (const std::bad_alloc&) {
            VB_FAIL(VB200_NO_ENOUGH_MEMORY, "sq8 train: host sample allocation failed");
        }
        for (uint64_t j = 0; j < cnt; ++j) {
            memcpy(sample.data() + j * dim, data + ((j * step) % count) * dim, dim * sizeof(float));
        }
        DevInput<float> in;
        VB_TRY(in.bind(sample.data(), cnt * dim));
        // The gathered sample has at most 100000 rows, so the device path takes it whole.
        VB_TRY(sq8_train_device(in.ptr, cnt, dim, mode, out.ptr, out.ptr + dim));
    }
    VB_TRY(copy_out(lower, out.ptr, dim));
    VB_TRY(copy_out(diff, out.ptr + dim, dim));
    return sync_stream();
}

extern "C" int
vb200_sq8_encode(const float* data, uint64_t count, uint32_t dim, const float* lower,
                 const float* diff, uint8_t* codes) {
    VB_CHECK_ARG(dim > 0, "sq8 encode: dim must be positive");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(data != nullptr && lower != nullptr && diff != nullptr && codes != nullptr,
                 "sq8 encode: null pointer");
    DevInput<float> lo, df;
    VB_TRY(lo.bind(lower, dim));
    VB_TRY(df.bind(diff, dim));
    const bool out_dev = is_device_pointer(codes);
    // Host batches are staged in slices so the device footprint stays bounded.
    const uint64_t slice = is_device_pointer(data) ? count : (uint64_t{1} << 22);
    DevBuf<uint8_t> out;
    DevInput<float> in;
    for (uint64_t b = 0; b < count; b += slice) {
        uint64_t n = count - b < slice ? count - b : slice;
        VB_TRY(in.bind(data + b * dim, n * dim));
        uint8_t* dst = codes + b * dim;
        if (!out_dev) {
            VB_TRY(out.reserve(n * dim));
            dst = out.ptr;
        }
        VB_TRY(sq8_encode_device(in.ptr, n, dim, lo.ptr, df.ptr, nullptr, dst, dim));
        if (!out_dev) {
            VB_TRY(copy_out(codes + b * dim, out.ptr, n * dim));
        }
        VB_TRY(sync_stream());
    }
    return 0;
}
