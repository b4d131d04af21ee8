/* Host quantisation codec ABI, version 1.  Replaces the reference's
 * backend/include/tinyinfer_host_codec.h:8-22 (implementation backend/host_codec.cpp);
 * implemented in tinyinfer_b200/csrc/host_codec.cpp.  Pure host code: no CUDA, no allocation,
 * no global state.  Counts are element counts.  Every check (null/alignment, byte-range
 * overflow, pairwise overlap of the three buffers, finite inputs, rounding mode) happens before
 * the first output byte is written, so a rejected call leaves the outputs untouched.
 */
#ifndef TINYINFER_HOST_CODEC_H
#define TINYINFER_HOST_CODEC_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
enum ti_host_status { TI_HOST_OK = 0, TI_HOST_INVALID = 1, TI_HOST_INTERNAL = 2 };

/* reference backend/host_codec.cpp:57 -- always 1. */
int ti_host_codec_abi_version(void);

/* f16_bits is an [elements/columns, columns] matrix of IEEE binary16 bit patterns; columns are
 * output channels.  scales[c] = fp32(max|column c| / 127.0) (1.0 for an all-zero column) and
 * q = clip(round_half_even(double(w) / double(scale)), -127, 127).
 * reference backend/host_codec.cpp:58-85 == llm/quantization.py:27-42. */
int ti_host_quantize_f16(const uint16_t* f16_bits, size_t elements, size_t columns,
                         int8_t* q, size_t q_elements, float* scales, size_t scale_elements);

/* f16 = round_to_nearest_even(fp32(q) * scales[column]).  Rejects q == -128, scales that are
 * not finite and positive, and products whose magnitude reaches 65520.
 * reference backend/host_codec.cpp:86-103 == llm/quantization.py:45-56. */
int ti_host_dequantize_i8(const int8_t* q, size_t elements, size_t columns,
                          const float* scales, size_t scale_elements,
                          uint16_t* f16_bits, size_t output_elements);
#ifdef __cplusplus
}
#endif
#endif
