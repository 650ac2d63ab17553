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

}  // namespace vb200
