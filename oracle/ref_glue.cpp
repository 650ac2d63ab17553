// Test infrastructure only: C entry points over the reference's own SIMD kernels, which
// oracle/Makefile compiles unchanged from the reference tree (src/simd/*.cpp) into
// oracle/_ref/libvsag_ref_simd.so.  Used to pin oracle/vsag_oracle.c and, in the benchmark, as the
// reference's CPU distance kernels.  Nothing in the product library links against this.
#include <cstdint>

#include "simd/bf16_simd.h"
#include "simd/fp16_simd.h"
#include "simd/fp32_simd.h"
#include "simd/normalize.h"
#include "simd/rabitq_simd.h"
#include "simd/simd_status.h"
#include "simd/sq8_simd.h"
#include "simd/sq8_uniform_simd.h"

extern "C" {

// Runtime-dispatched variants (what production calls; src/simd/simd_dispatch.h:113-135).
float ref_SQ8ComputeL2Sqr(const float* q, const uint8_t* c, const float* lb, const float* diff, uint64_t d) {
    return vsag::SQ8ComputeL2Sqr(q, c, lb, diff, d);
}
float ref_SQ8ComputeIP(const float* q, const uint8_t* c, const float* lb, const float* diff, uint64_t d) {
    return vsag::SQ8ComputeIP(q, c, lb, diff, d);
}
float ref_FP32ComputeL2Sqr(const float* a, const float* b, uint64_t d) {
    return vsag::FP32ComputeL2Sqr(a, b, d);
}
float ref_FP32ComputeIP(const float* a, const float* b, uint64_t d) {
    return vsag::FP32ComputeIP(a, b, d);
}
float ref_BF16ComputeIP(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::BF16ComputeIP(a, b, d);
}
float ref_BF16ComputeL2Sqr(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::BF16ComputeL2Sqr(a, b, d);
}
float ref_RaBitQFloatBinaryIP(const float* v, const uint8_t* bits, uint64_t d, float inv_sqrt_d) {
    return vsag::RaBitQFloatBinaryIP(v, bits, d, inv_sqrt_d);
}
float ref_NormalizeWithCentroid(const float* from, const float* centroid, float* to, uint64_t d) {
    return vsag::NormalizeWithCentroid(from, centroid, to, d);
}

// Canonical scalar variants (src/simd/generic.cpp).
float ref_generic_SQ8ComputeL2Sqr(const float* q, const uint8_t* c, const float* lb, const float* diff, uint64_t d) {
    return vsag::generic::SQ8ComputeL2Sqr(q, c, lb, diff, d);
}
float ref_generic_SQ8ComputeIP(const float* q, const uint8_t* c, const float* lb, const float* diff, uint64_t d) {
    return vsag::generic::SQ8ComputeIP(q, c, lb, diff, d);
}
float ref_generic_FP32ComputeL2Sqr(const float* a, const float* b, uint64_t d) {
    return vsag::generic::FP32ComputeL2Sqr(a, b, d);
}
float ref_generic_FP32ComputeIP(const float* a, const float* b, uint64_t d) {
    return vsag::generic::FP32ComputeIP(a, b, d);
}
float ref_generic_BF16ComputeIP(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::generic::BF16ComputeIP(a, b, d);
}
float ref_generic_RaBitQFloatBinaryIP(const float* v, const uint8_t* bits, uint64_t d, float inv_sqrt_d) {
    return vsag::generic::RaBitQFloatBinaryIP(v, bits, d, inv_sqrt_d);
}
float ref_generic_NormalizeWithCentroid(const float* from, const float* centroid, float* to, uint64_t d) {
    return vsag::generic::NormalizeWithCentroid(from, centroid, to, d);
}
float ref_SQ8UniformComputeCodesIP(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::SQ8UniformComputeCodesIP(a, b, d);
}
uint16_t ref_FloatToFP16(float v) {
    return vsag::generic::FloatToFP16(v);
}
float ref_FP16ToFloat(uint16_t v) {
    return vsag::generic::FP16ToFloat(v);
}
float ref_FP16ComputeIP(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::FP16ComputeIP(a, b, d);
}
float ref_FP16ComputeL2Sqr(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::FP16ComputeL2Sqr(a, b, d);
}
float ref_generic_FP16ComputeL2Sqr(const uint8_t* a, const uint8_t* b, uint64_t d) {
    return vsag::generic::FP16ComputeL2Sqr(a, b, d);
}
uint16_t ref_FloatToBF16(float v) {
    return vsag::generic::FloatToBF16(v);
}
float ref_BF16ToFloat(uint16_t v) {
    return vsag::generic::BF16ToFloat(v);
}
int ref_supports_avx512(void) {
    return vsag::SimdStatus::SupportAVX512() ? 1 : 0;
}
}
