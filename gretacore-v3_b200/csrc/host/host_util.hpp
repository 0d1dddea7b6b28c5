// Small host-side helpers shared by the C++ layer.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>

#include "greta_cuda.h"

namespace gcore::host {

// IEEE fp16 <-> fp32, round-to-nearest-even.
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u, ax = x & 0x7FFFFFFFu;
  if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0u));
  if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
  if (ax < 0x33000001u) return (uint16_t)sign;
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
  int shift = e < -14 ? 13 + (-14 - e) : 13;
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  uint32_t res = e < -14 ? q : (((uint32_t)(e + 15) << 10) + (q - 0x400u));
  return (uint16_t)(sign | res);
}
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu, out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign;
    } else {
      int e = 1;
      while (!(mant & 0x400u)) {
        mant <<= 1;
        --e;
      }
      out = sign | ((uint32_t)(e + 112) << 23) | ((mant & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    out = sign | 0x7F800000u | (mant << 13);
  } else {
    out = sign | ((exp + 112u) << 23) | (mant << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

inline std::string cuda_error(const char *what) { return std::string(what) + ": " + greta_cuda_last_error(); }
inline bool fail(std::string *err, const std::string &msg) {
  if (err) *err = msg;
  return false;
}

}  // namespace gcore::host
