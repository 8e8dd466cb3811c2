// Software fp16 / bf16 <-> fp32 conversion (round to nearest even) for host-side
// oracles and the CPU emulator; no CUDA headers involved.
#pragma once

#include <cstdint>
#include <cstring>

#include "types.h"

namespace b200ipc {

inline uint32_t f32_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float bits_f32(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline float half_to_float(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return bits_f32(sign);
    // subnormal: normalise
    int e = -1;
    do {
      ++e;
      man <<= 1;
    } while ((man & 0x400u) == 0);
    man &= 0x3ffu;
    return bits_f32(sign | (uint32_t(127 - 15 - e) << 23) | (man << 13));
  }
  if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
  return bits_f32(sign | ((exp + 112) << 23) | (man << 13));
}

inline uint16_t float_to_half(float f) {
  const uint32_t x = f32_bits(f);
  const uint16_t sign = uint16_t((x >> 16) & 0x8000u);
  const uint32_t abs = x & 0x7fffffffu;
  if (abs >= 0x7f800000u) return uint16_t(sign | 0x7c00u | (abs > 0x7f800000u ? 0x200u : 0));  // inf / nan
  if (abs >= 0x477ff000u) return uint16_t(sign | 0x7c00u);                                     // rounds to inf
  if (abs < 0x33000001u) return sign;                                                          // rounds to zero
  int exp = int(abs >> 23) - 127;
  uint32_t man = (abs & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) {  // subnormal result
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = uint32_t(exp + 15) << 10;
    man &= 0x7fffffu;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  return uint16_t(sign | (base + q));
}

inline float bf16_to_float(uint16_t b) { return bits_f32(uint32_t(b) << 16); }
inline uint16_t float_to_bf16(float f) {
  uint32_t x = f32_bits(f);
  if ((x & 0x7fffffffu) > 0x7f800000u) return uint16_t((x >> 16) | 0x40u);  // nan
  x += 0x7fffu + ((x >> 16) & 1u);
  return uint16_t(x >> 16);
}

inline float to_float(DType t, uint16_t v) { return t == DType::F16 ? half_to_float(v) : bf16_to_float(v); }
inline uint16_t from_float(DType t, float f) { return t == DType::F16 ? float_to_half(f) : float_to_bf16(f); }

}  // namespace b200ipc
