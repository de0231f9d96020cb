// 8-bit moment codes of the block-wise AdamW kernels, written to keep the special-function unit
// (square roots, reciprocals AND int <-> float conversions all issue there, at a quarter of the
// FMA rate) out of the way: the kernels are bound by that unit, not by memory, when every element
// costs nine such operations.
//
//   first moment  m: signed code q in [-127, 127], |m| = (|q| / 127)^2 * absmax
//   second moment v: unsigned code q in [0, 255],   v  = (q / 255)^4 * absmax
//
// Decoding converts the code with the 2^23 trick (bits 0x4B000000 | q are the float 2^23 + q) and
// multiplies; encoding rounds with the 1.5 * 2^23 trick. Both stay on the integer / FMA pipes. The
// update shares one square root between Adam's denominator and the fourth-root code of v:
// sqrt(v) feeds sqrt(v / bc2) = sqrt(v) * rsqrt(bc2) and sqrt(sqrt(v * iv)) = sqrt(sqrt(v) * sqrt(iv)).
// Four special-function operations per element remain: sqrt(v), the reciprocal of the denominator,
// and one square root per code.
#pragma once
#include <stdint.h>

namespace eri {

__device__ __forceinline__ float u8_to_float(uint32_t q) {   // q in [0, 255], exact
  return __uint_as_float(0x4B000000u | q) - 8388608.f;
}
__device__ __forceinline__ uint32_t round_to_u32(float x) {  // x in [0, 2^22): round to nearest even
  return __float_as_uint(x + 12582912.f) & 0x3FFFFFu;
}
__device__ __forceinline__ float decode_m(int8_t q, float absmax) {
  const uint32_t mag = (uint32_t)(q < 0 ? -q : q);
  const float a = u8_to_float(mag) * (1.f / 127.f);
  const float v = a * a * absmax;
  return __uint_as_float(__float_as_uint(v) | (((uint32_t)(uint8_t)q & 0x80u) << 24));
}
__device__ __forceinline__ float decode_v(uint8_t q, float absmax) {
  float a = u8_to_float(q) * (1.f / 255.f);
  a = a * a;
  return a * a * absmax;
}
// |m| * inv_absmax in [0, 1] -> signed code
__device__ __forceinline__ int8_t encode_m(float m, float inv_absmax) {
  const float a = sqrtf(fminf(fabsf(m) * inv_absmax, 1.f));
  const int q = (int)round_to_u32(a * 127.f);
  return (int8_t)(m < 0.f ? -q : q);
}
// sqrt_v = sqrt(v) (already computed for the update), sqrt_inv = sqrt(1 / absmax) of the block
__device__ __forceinline__ uint8_t encode_v_from_sqrt(float sqrt_v, float sqrt_inv) {
  const float a = sqrtf(fminf(sqrt_v * sqrt_inv, 1.f));
  uint32_t q = round_to_u32(a * 255.f);
  if (q == 0u && sqrt_v > 0.f) q = 1u;  // a positive second moment never collapses to zero
  return (uint8_t)q;
}

}  // namespace eri
