// Device-pointer entry points of the 1-bit RaBitQ quantizer shared with the IVF index.
#pragma once

#include "common.cuh"

namespace vb200 {

inline uint32_t
rabitq_bits_bytes(uint32_t dim) {
    return ((dim + 7) / 8 + 3) / 4 * 4;
}
inline uint32_t
rabitq_code_size(uint32_t dim) {
    return rabitq_bits_bytes(dim) + 8;
}

// centroid_dev[dim] = rotation * mean(rows).
int rabitq_train_device(const float* data_dev, uint64_t count, uint32_t dim,
                        const float* rotation_dev, float* centroid_dev);

// Encodes `count` rows; row i goes to codes_dev + dst(i) * code_stride, dst(i) = dst_pos_dev[i]
// (0xFFFFFFFF = skip) or i.  Rows are rotated in slices through an internal scratch buffer.
int rabitq_encode_device(const float* data_dev, uint64_t count, uint32_t dim,
                         const float* rotation_dev, const float* centroid_dev,
                         const uint32_t* dst_pos_dev, uint8_t* codes_dev, uint32_t code_stride);

// out_dev[count x (dim + 1)]: rotated, centred, normalised rows followed by the norm.  With `scratch` (a
// buffer the caller keeps between calls) nothing is allocated and the call does not wait for the device.
int rabitq_process_query_device(const float* q_dev, uint64_t count, uint32_t dim,
                                const float* rotation_dev, const float* centroid_dev,
                                float* out_dev, DevBuf<float>* scratch);

}  // namespace vb200
