// Host-side exact narrowing of JSON literals (doubles) to the element type an
// op declares, so that constants enter the kernels already rounded once, the
// way a typed constant tensor holds them
// (akg-mlir/lib/Target/MindsporeDialect/TranslateToMindsporeDialect.cpp:1320-1329).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace akgb {

// IEEE binary16 bits of `v`, round-to-nearest-even, single rounding.
inline uint16_t f64_to_f16_bits(double v) {
  uint16_t sign = std::signbit(v) ? 0x8000 : 0;
  if (std::isnan(v)) return 0x7e00;
  double a = std::fabs(v);
  if (std::isinf(a)) return sign | 0x7c00;
  if (a == 0.0) return sign;
  int e;
  double fr = std::frexp(a, &e);  // a = fr * 2^e, fr in [0.5, 1)
  int exp16 = e - 1 + 15;
  if (exp16 <= 0) {  // subnormal range: spacing 2^-24
    double q = std::nearbyint(std::ldexp(a, 24));
    return sign | (uint16_t)q;  // q == 1024 lands on the smallest normal, as it should
  }
  double q = std::nearbyint(std::ldexp(fr, 11));  // [1024, 2048]
  unsigned mi = (unsigned)q;
  if (mi == 2048) {
    mi = 1024;
    ++exp16;
  }
  if (exp16 >= 31) return sign | 0x7c00;
  return sign | (uint16_t)((exp16 << 10) | (mi - 1024));
}

inline double f16_bits_to_f64(uint16_t b) {
  int e = (b >> 10) & 0x1f;
  int m = b & 0x3ff;
  double v;
  if (e == 31) v = m ? NAN : INFINITY;
  else if (e == 0) v = std::ldexp((double)m, -24);
  else v = std::ldexp((double)(m | 0x400), e - 25);
  return (b & 0x8000) ? -v : v;
}

inline float round_f64_to_f16(double v) { return (float)f16_bits_to_f64(f64_to_f16_bits(v)); }

// bfloat16 via one rounding from double: round the f64 to 8 significant bits.
inline float round_f64_to_bf16(double v) {
  if (std::isnan(v) || std::isinf(v) || v == 0.0) return (float)v;
  int e;
  double fr = std::frexp(std::fabs(v), &e);
  double q = std::nearbyint(std::ldexp(fr, 8));
  double r = std::ldexp(q, e - 8);
  return (float)(std::signbit(v) ? -r : r);
}

}  // namespace akgb
