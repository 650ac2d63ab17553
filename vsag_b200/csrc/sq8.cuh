// Device-pointer entry points of the SQ8 quantizer shared with the IVF index.
#pragma once

#include "common.cuh"

namespace vb200 {

// lower_dev[dim], diff_dev[dim] from device-resident rows; synchronises the stream.
int sq8_train_device(const float* data_dev, uint64_t count, uint32_t dim, int mode, float* lower_dev,
                     float* diff_dev);

// Encodes `count` rows; row i is written at codes_dev + dst(i) * code_stride where dst(i) =
// dst_pos_dev[i] (0xFFFFFFFF = skip the row) or i when dst_pos_dev is NULL.  Asynchronous.
int sq8_encode_device(const float* data_dev, uint64_t count, uint32_t dim, const float* lower_dev,
                      const float* diff_dev, const uint32_t* dst_pos_dev, uint8_t* codes_dev,
                      uint32_t code_stride);

// --- SQ8 uniform (SQ8UniformQuantizer, src/quantization/scalar_quantization/sq8_uniform_quantizer.cpp) ---

// Bytes of one code record: codes padded to the trailing field's alignment, then the uint64 sum of squared
// codes (L2) or the fp32 sum of the values (IP / cosine) (sq8_uniform_quantizer.cpp:32-60).
inline uint32_t
sq8u_code_size(uint32_t dim, int metric_is_l2) {
    const uint32_t align = metric_is_l2 ? 8u : 4u;
    return (dim + align - 1) / align * align + align;
}

// model_dev = {lower, diff}: the extremes of the (at most 100000-row) sample over all dimensions
// (TrainImpl, :76-100).  Synchronises the stream.
int sq8u_train_device(const float* data_dev, uint64_t count, uint32_t dim, float* model_dev);

// Encodes rows (or queries: ProcessQueryImpl encodes the query like a row) into code records; destinations
// as for sq8_encode_device.  Asynchronous.
int sq8u_encode_device(const float* data_dev, uint64_t count, uint32_t dim, int metric_is_l2, float lower, float diff,
                       const uint32_t* dst_pos_dev, uint8_t* codes_dev, uint32_t code_stride);

}  // namespace vb200
