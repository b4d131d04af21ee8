// Host quantisation codec (ti_host_* ABI v1, include/tinyinfer_host_codec.h).
//
// Bit-exact with the reference codec (backend/host_codec.cpp:58-103) and with the pure-Python
// specification (llm/quantization.py:27-56):
//   scale[c] = fp32( double(max_r |w[r,c]|) / 127.0 ),  1.0f when the column is all zero
//   q[r,c]   = clip( round_half_even( double(w[r,c]) / double(scale[c]) ), -127, 127 )
//   deq[r,c] = fp16_rn( fp32(q[r,c]) * scale[c] )
// The passes walk the matrix row by row (the layout is row-major with the output channel as
// the fast axis), keeping the per-column running maximum in the caller's scale array; that is
// safe for failure atomicity because, once every input is known to be finite binary16, every
// scale is finite and positive (2^-24/127 <= scale <= 65504/127).
#include "tinyinfer_host_codec.h"

#include <cfenv>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>

namespace {

static_assert(std::numeric_limits<float>::is_iec559 && sizeof(float) == 4, "IEEE binary32 required");

inline float widen(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16, mag = h & 0x7fffu;
  uint32_t bits;
  if (mag >= 0x0400u) bits = sign | ((mag << 13) + 0x38000000u);       // normal (inf/nan never reach here)
  else {                                                                // zero / subnormal: value = mag * 2^-24
    float f = float(mag) * 5.9604644775390625e-08f;
    std::memcpy(&bits, &f, 4);
    bits |= sign;
  }
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

// Round-to-nearest-even narrowing of a finite float whose magnitude is below 65520.
inline uint16_t narrow(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  const uint16_t sign = uint16_t((bits >> 16) & 0x8000u);
  const uint32_t mag = bits & 0x7fffffffu;
  const int e = int(mag >> 23) - 127;
  if (e < -25) return sign;
  uint32_t keep, rest, half_way;
  uint32_t base;
  if (e < -14) {                       // lands in the binary16 subnormal range
    const uint32_t sig = (mag & 0x7fffffu) | 0x800000u;
    const unsigned shift = unsigned(-e - 1);
    keep = sig >> shift; rest = sig & ((1u << shift) - 1u); half_way = 1u << (shift - 1);
    base = keep;
  } else {
    keep = (mag & 0x7fffffu) >> 13; rest = mag & 0x1fffu; half_way = 0x1000u;
    base = (uint32_t(e + 15) << 10) + keep;
  }
  base += (rest > half_way || (rest == half_way && (base & 1u))) ? 1u : 0u;
  return uint16_t(sign | base);
}

inline bool finite_half(uint16_t h) { return (h & 0x7c00u) != 0x7c00u; }

struct Range { uintptr_t lo, hi; };
inline bool range_of(const void* p, size_t count, size_t width, Range& r) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if (!p || a % width != 0 || count > SIZE_MAX / width) return false;
  const size_t bytes = count * width;
  if (bytes > UINTPTR_MAX - a) return false;
  r = {a, a + bytes};
  return true;
}
inline bool apart(Range a, Range b) { return a.hi <= b.lo || b.hi <= a.lo; }
inline bool rectangular(size_t elements, size_t columns) {
  return elements && columns && elements % columns == 0 &&
         elements <= size_t(std::numeric_limits<int64_t>::max()) / sizeof(float);
}

inline int nearest_even(double v) {
  const double lo = std::floor(v), frac = v - lo;
  int r = int(lo);
  if (frac > 0.5 || (frac == 0.5 && (r & 1))) ++r;
  return r;
}

}  // namespace

extern "C" int ti_host_codec_abi_version(void) { return 1; }

extern "C" int ti_host_quantize_f16(const uint16_t* w, size_t elements, size_t columns,
                                    int8_t* q, size_t q_elements, float* scales, size_t scale_elements) {
  Range rw{}, rq{}, rs{};
  if (!rectangular(elements, columns) || q_elements != elements || scale_elements != columns ||
      std::fegetround() != FE_TONEAREST || !range_of(w, elements, 2, rw) || !range_of(q, elements, 1, rq) ||
      !range_of(scales, columns, 4, rs) || !apart(rw, rq) || !apart(rw, rs) || !apart(rq, rs))
    return TI_HOST_INVALID;
  for (size_t i = 0; i < elements; ++i)
    if (!finite_half(w[i])) return TI_HOST_INVALID;
  // From here on nothing can fail: outputs may be written.
  for (size_t c = 0; c < columns; ++c) scales[c] = 0.f;
  for (size_t base = 0; base < elements; base += columns)
    for (size_t c = 0; c < columns; ++c) {
      const float a = std::fabs(widen(w[base + c]));
      if (a > scales[c]) scales[c] = a;
    }
  for (size_t c = 0; c < columns; ++c) scales[c] = scales[c] != 0.f ? float(double(scales[c]) / 127.0) : 1.0f;
  for (size_t base = 0; base < elements; base += columns)
    for (size_t c = 0; c < columns; ++c) {
      const int v = nearest_even(double(widen(w[base + c])) / double(scales[c]));
      q[base + c] = int8_t(v < -127 ? -127 : v > 127 ? 127 : v);
    }
  return TI_HOST_OK;
}

extern "C" int ti_host_dequantize_i8(const int8_t* q, size_t elements, size_t columns,
                                     const float* scales, size_t scale_elements,
                                     uint16_t* out, size_t output_elements) {
  Range rq{}, rs{}, ro{};
  if (!rectangular(elements, columns) || scale_elements != columns || output_elements != elements ||
      std::fegetround() != FE_TONEAREST || !range_of(q, elements, 1, rq) || !range_of(scales, columns, 4, rs) ||
      !range_of(out, elements, 2, ro) || !apart(rq, rs) || !apart(rq, ro) || !apart(rs, ro))
    return TI_HOST_INVALID;
  for (size_t c = 0; c < columns; ++c)
    if (!std::isfinite(scales[c]) || scales[c] <= 0.f) return TI_HOST_INVALID;
  for (size_t base = 0; base < elements; base += columns)
    for (size_t c = 0; c < columns; ++c) {
      if (q[base + c] == -128) return TI_HOST_INVALID;
      const float v = float(q[base + c]) * scales[c];
      if (!std::isfinite(v) || std::fabs(v) >= 65520.0f) return TI_HOST_INVALID;   // would round to infinity
    }
  for (size_t base = 0; base < elements; base += columns)
    for (size_t c = 0; c < columns; ++c) out[base + c] = narrow(float(q[base + c]) * scales[c]);
  return TI_HOST_OK;
}
