// bf16 <-> fp32 conversions shared by the CPU backend's translation units.
#pragma once
#include <cstdint>
#include <cstring>

namespace b200cpu {

using bf16_t = uint16_t;

static inline float bf16_to_f32(bf16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
static inline bf16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40);   // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                            // nearest even
  return (bf16_t)(u >> 16);
}
// Value after one rounding to bf16 (the oracle rounds intermediate tensors the same way).
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

static inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {                                  // subnormal: renormalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);                    // overflow -> inf
  if (x < 0x33000000u) return (uint16_t)sign;                                 // underflow -> 0
  int exp = (int)(x >> 23) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (exp <= 0) {                                                             // subnormal half
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t r = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)exp << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
  return (uint16_t)(sign | r);
}

}  // namespace b200cpu
