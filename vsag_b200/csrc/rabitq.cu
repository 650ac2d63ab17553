// 1-bit RaBitQ: training (centroid), encoder and query transform.  The rotation y = Qx runs
// through the fixed-order dense kernel, so every rotated coordinate is the same ascending FMA chain
// the CPU oracle defines for the reference's Sgemv call
// (src/impl/transform/random_orthogonal_transformer.cpp:59-77).
#include "rabitq.cuh"

#include "dense.cuh"

namespace vb200 {

// mean[d] = (((x_0d + x_1d) + x_2d) + ...) / count in fp32: the running sum over the rows in their
// given order that RaBitQuantizer::TrainImpl keeps (rabitq_quantizer.cpp:229-243), so the centroid -- and
// with it every sign bit of every code -- is the one a reference build computes from the same rows.  One
// thread per column; the loads of sixteen rows are issued together, the additions stay in row order.
__global__ void __launch_bounds__(32)
column_mean_in_order_kernel(const float* __restrict__ data, uint64_t count, uint32_t dim, float* __restrict__ mean) {
    const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= dim) {
        return;
    }
    const float* p = data + d;
    float s = 0.f;
    uint64_t r = 0;
    for (; r + 16 <= count; r += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            v[j] = __ldg(p + (r + j) * dim);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            s = __fadd_rn(s, v[j]);
        }
    }
    for (; r < count; ++r) {
        s = __fadd_rn(s, __ldg(p + r * dim));
    }
    mean[d] = __fdiv_rn(s, static_cast<float>(count));
}

int
rabitq_train_device(const float* data_dev, uint64_t count, uint32_t dim, const float* rotation_dev,
                    float* centroid_dev) {
    VB_CHECK_ARG(count > 0, "rabitq train: empty input");
    DevBuf<float> mean;
    VB_TRY(mean.reserve(dim));
    VB_LAUNCH(column_mean_in_order_kernel, (dim + 31) / 32, 32, 0, data_dev, count, dim, mean.ptr);
    VB_TRY(dense_scores_f32(mean.ptr, 1, rotation_dev, dim, dim, 1.0f, nullptr, centroid_dev, dim));
    return sync_stream();
}

// One thread per rotated row t[dim] (row stride ld): NormalizeWithCentroid in scalar order
// (src/simd/kernels/normalize.h:35-85), then either the sign bits + norm + error record of
// EncodeOneInternal's 1-bit branch (rabitq_quantizer.cpp:824-850) or the processed query.
template <bool QUERY>
__global__ void
rabitq_pack_kernel(const float* __restrict__ t, uint64_t count, uint32_t dim,
                   const float* __restrict__ centroid, float inv_sqrt_d,
                   const uint32_t* __restrict__ dst_pos, uint8_t* __restrict__ codes,
                   uint32_t code_stride, float* __restrict__ qout) {
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) {
        return;
    }
    const float* row = t + i * dim;
    float norm_sq = 0.f;
    for (uint32_t d = 0; d < dim; ++d) {
        float df = __fsub_rn(row[d], __ldg(centroid + d));
        norm_sq = fmaf(df, df, norm_sq);
    }
    float norm = norm_sq < 1e-5f ? 1.0f : __fsqrt_rn(norm_sq);
    if (QUERY) {
        float* o = qout + i * (dim + 1);
        for (uint32_t d = 0; d < dim; ++d) {
            o[d] = __fdiv_rn(__fsub_rn(row[d], __ldg(centroid + d)), norm);
        }
        o[dim] = norm;
        return;
    }
    uint64_t p = i;
    if (dst_pos != nullptr) {
        uint32_t q = dst_pos[i];
        if (q == 0xFFFFFFFFu) {
            return;
        }
        p = q;
    }
    uint8_t* code = codes + p * code_stride;
    const uint32_t bits_bytes = ((dim + 7) / 8 + 3) / 4 * 4;
    float err = 0.f;
    for (uint32_t w0 = 0; w0 < bits_bytes; w0 += 4) {
        uint32_t word = 0;
        for (uint32_t b = 0; b < 32; ++b) {
            uint32_t d = w0 * 8 + b;
            if (d < dim) {
                float o = __fdiv_rn(__fsub_rn(row[d], __ldg(centroid + d)), norm);
                bool bit = o >= 0.0f;
                if (bit) {
                    word |= 1u << b;
                }
                // RaBitQFloatBinaryIP, scalar order: result += (bit ? +s : -s) * o, product rounded.
                err = __fadd_rn(err, __fmul_rn(bit ? inv_sqrt_d : -inv_sqrt_d, o));
            }
        }
        *reinterpret_cast<uint32_t*>(code + w0) = word;
    }
    *reinterpret_cast<float*>(code + bits_bytes) = norm;
    *reinterpret_cast<float*>(code + bits_bytes + 4) = err;
    for (uint32_t b = bits_bytes + 8; b < code_stride; b += 4) {
        *reinterpret_cast<uint32_t*>(code + b) = 0u;
    }
}

constexpr uint64_t RABITQ_SLICE_FLOATS = uint64_t{64} << 20;  // 256 MiB of rotated rows

int
rabitq_encode_device(const float* data_dev, uint64_t count, uint32_t dim, const float* rotation_dev,
                     const float* centroid_dev, const uint32_t* dst_pos_dev, uint8_t* codes_dev,
                     uint32_t code_stride) {
    if (count == 0) {
        return 0;
    }
    uint64_t slice = RABITQ_SLICE_FLOATS / dim;
    if (slice < 1) {
        slice = 1;
    }
    if (slice > count) {
        slice = count;
    }
    DevBuf<float> t;
    VB_TRY(t.reserve(slice * dim));
    const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(dim));
    for (uint64_t b = 0; b < count; b += slice) {
        uint64_t n = count - b < slice ? count - b : slice;
        VB_TRY(dense_scores_f32(data_dev + b * dim, n, rotation_dev, dim, dim, 1.0f, nullptr, t.ptr, dim));
        const uint32_t* dst = dst_pos_dev != nullptr ? dst_pos_dev + b : nullptr;
        uint8_t* codes = dst_pos_dev != nullptr ? codes_dev : codes_dev + b * code_stride;
        VB_LAUNCH(rabitq_pack_kernel<false>, static_cast<uint32_t>((n + 63) / 64), 64, 0, t.ptr, n, dim,
                  centroid_dev, inv_sqrt_d, dst, codes, code_stride, nullptr);
    }
    return sync_stream();
}

int
rabitq_process_query_device(const float* q_dev, uint64_t count, uint32_t dim,
                            const float* rotation_dev, const float* centroid_dev, float* out_dev,
                            DevBuf<float>* scratch) {
    if (count == 0) {
        return 0;
    }
    uint64_t slice = RABITQ_SLICE_FLOATS / dim;
    if (slice < 1) {
        slice = 1;
    }
    if (slice > count) {
        slice = count;
    }
    // rotated rows of one slice: the caller's buffer when it has one to keep between calls (a search must not
    // allocate and free, nor wait for the device, in the middle of its step)
    DevBuf<float> own;
    DevBuf<float>& t = scratch != nullptr ? *scratch : own;
    VB_TRY(t.reserve(slice * dim));
    for (uint64_t b = 0; b < count; b += slice) {
        uint64_t n = count - b < slice ? count - b : slice;
        VB_TRY(dense_scores_f32(q_dev + b * dim, n, rotation_dev, dim, dim, 1.0f, nullptr, t.ptr, dim));
        VB_LAUNCH(rabitq_pack_kernel<true>, static_cast<uint32_t>((n + 63) / 64), 64, 0, t.ptr, n, dim,
                  centroid_dev, 0.f, nullptr, nullptr, 0, out_dev + b * (dim + 1));
    }
    return scratch != nullptr ? 0 : sync_stream();   // `own` is freed on return: its work must be done
}

}  // namespace vb200

using namespace vb200;

extern "C" uint64_t
vb200_rabitq_code_size(uint32_t dim) {
    return rabitq_code_size(dim);
}

extern "C" int
vb200_rabitq_train(const float* data, uint64_t count, uint32_t dim, const float* rotation,
                   float* centroid) {
    VB_CHECK_ARG(data != nullptr && rotation != nullptr && centroid != nullptr, "rabitq train: null pointer");
    VB_CHECK_ARG(count > 0 && dim > 0, "rabitq train: empty input");
    DevInput<float> x, rot;
    VB_TRY(x.bind(data, count * dim));
    VB_TRY(rot.bind(rotation, static_cast<size_t>(dim) * dim));
    DevBuf<float> c;
    VB_TRY(c.reserve(dim));
    VB_TRY(rabitq_train_device(x.ptr, count, dim, rot.ptr, c.ptr));
    VB_TRY(copy_out(centroid, c.ptr, dim));
    return sync_stream();
}

extern "C" int
vb200_rabitq_encode(const float* data, uint64_t count, uint32_t dim, const float* rotation,
                    const float* centroid, uint8_t* codes) {
    VB_CHECK_ARG(dim > 0, "rabitq encode: dim must be positive");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(data != nullptr && rotation != nullptr && centroid != nullptr && codes != nullptr,
                 "rabitq encode: null pointer");
    DevInput<float> x, rot, cen;
    VB_TRY(x.bind(data, count * dim));
    VB_TRY(rot.bind(rotation, static_cast<size_t>(dim) * dim));
    VB_TRY(cen.bind(centroid, dim));
    const uint32_t cs = rabitq_code_size(dim);
    DevBuf<uint8_t> out;
    VB_TRY(out.reserve(count * cs));
    VB_TRY(rabitq_encode_device(x.ptr, count, dim, rot.ptr, cen.ptr, nullptr, out.ptr, cs));
    VB_TRY(copy_out(codes, out.ptr, count * cs));
    return sync_stream();
}

extern "C" int
vb200_rabitq_process_query(const float* queries, uint64_t count, uint32_t dim, const float* rotation,
                           const float* centroid, float* out) {
    VB_CHECK_ARG(dim > 0, "rabitq query: dim must be positive");
    if (count == 0) {
        return 0;
    }
    VB_CHECK_ARG(queries != nullptr && rotation != nullptr && centroid != nullptr && out != nullptr,
                 "rabitq query: null pointer");
    DevInput<float> q, rot, cen;
    VB_TRY(q.bind(queries, count * dim));
    VB_TRY(rot.bind(rotation, static_cast<size_t>(dim) * dim));
    VB_TRY(cen.bind(centroid, dim));
    DevBuf<float> o;
    VB_TRY(o.reserve(count * (dim + 1)));
    VB_TRY(rabitq_process_query_device(q.ptr, count, dim, rot.ptr, cen.ptr, o.ptr, nullptr));
    VB_TRY(copy_out(out, o.ptr, count * (dim + 1)));
    return sync_stream();
}
