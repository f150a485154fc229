// Number-format encoders shared by the quantisation producers and the fused-chain interpreter:
// fp8 e4m3 (saturating), fp4 e2m1 (nearest, ties to the even code, saturating at 6), and the byte
// offset of one NVFP4 block scale in the 128 x 4 chunk layout that block-scaled MMAs read.
#pragma once
#include <cuda_fp8.h>

#include <cstdint>

namespace b200 {

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __nv_fp8_e4m3 t;
  t.__x = b;
  return (float)t;
}
__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t float_to_e2m1(float v) {
  // round to nearest representable magnitude (ties to even code), saturate at 6
  const float a = fabsf(v);
  uint32_t code;
  if (a <= 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a <= 5.0f) code = 6;
  else code = 7;
  return code | (v < 0.f ? 8u : 0u);
}

// Scale of row t, 16-wide group gidx, of a [T, K] operand: [T/128][K/64][32 rows][4 row-groups][4 k].
__device__ __forceinline__ size_t nvfp4_sf_chunk_offset(long t, int gidx, int K) {
  const long rb = t / 128, r = t % 128;
  return ((size_t)rb * (K / 64) + gidx / 4) * 512 + (size_t)(r % 32) * 16 + (size_t)(r / 32) * 4 + gidx % 4;
}

}  // namespace b200
