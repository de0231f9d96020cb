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

// ---------------------------------------------------------------------------------------------
// The same step on packed fp32 pairs, with about half the instructions per element. A code byte
// becomes a float with ONE byte permute (the byte lands in the mantissa of 2^23; a signed code is
// first biased by 128 with one XOR per four codes); signed codes are written by adding 1.5 * 2^23 to
// the signed value (the low mantissa byte is then the two's complement code); the floor "a positive
// second moment never codes as zero" is a clamp instead of a compare and select; one hash serves the
// stochastic rounding of two elements. Used by the optimizer kernel and by the fused data-parallel
// step. Needs f32x2 and its helpers (ptx.cuh) before this header.

__device__ __forceinline__ uint32_t adam8_prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ float adam8_rcp(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t adam8_hash(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

struct Adam8Consts {
  f32x2 b1, c1, b2, c2, rb, eps, moff, voff, magic, k127, k255, big;
  float inv_bc1;
};

// gs: the factor on the gradient (loss scale, clip coefficient, 1 / world)
__device__ __forceinline__ void adam8_consts(Adam8Consts& k, float beta1, float beta2, float eps, float bc1,
                                             float bc2, float gs) {
  const float c1 = (1.f - beta1) * gs, c2 = (1.f - beta2) * gs * gs, rb = rsqrtf(bc2);
  k.b1 = f2_pack(beta1, beta1); k.c1 = f2_pack(c1, c1); k.b2 = f2_pack(beta2, beta2); k.c2 = f2_pack(c2, c2);
  k.rb = f2_pack(rb, rb); k.eps = f2_pack(eps, eps);
  k.moff = f2_pack(-8388736.f, -8388736.f); k.voff = f2_pack(-8388608.f, -8388608.f);
  k.magic = f2_pack(12582912.f, 12582912.f); k.k127 = f2_pack(127.f, 127.f); k.k255 = f2_pack(255.f, 255.f);
  k.big = f2_pack(1e30f, 1e30f);
  k.inv_bc1 = 1.f / bc1;
}

// One lane's eight elements: g2 the gradients as four fp32 pairs, pw the eight bf16 parameters,
// mraw / vraw their codes, ma / va the block's maxima. Out: the new moments m2, sqrt(v) sv2 (shared by
// Adam's denominator and the code of v), the new parameters p2, and this lane's maxima.
__device__ __forceinline__ void adam8_update8(const Adam8Consts& k, const f32x2 (&g2)[4], uint4 pw, uint2 mraw,
                                              uint2 vraw, float ma, float va, float lr, float weight_decay,
                                              f32x2 (&m2)[4], f32x2 (&sv2)[4], f32x2 (&p2)[4], float& mmax,
                                              float& vmax) {
  const float decay = 1.f - lr * weight_decay, nlr = -lr * k.inv_bc1;
  const f32x2 kDecay = f2_pack(decay, decay), kNlr = f2_pack(nlr, nlr);
  const float cm = ma * (1.f / (127.f * 127.f));
  const float cv = va * (1.f / (255.f * 255.f * 255.f * 255.f));
  const f32x2 kCm = f2_pack(cm, cm), kCv = f2_pack(cv, cv);
  const uint32_t pws[4] = {pw.x, pw.y, pw.z, pw.w};
  const uint32_t mxs[2] = {mraw.x ^ 0x80808080u, mraw.y ^ 0x80808080u}, vws[2] = {vraw.x, vraw.y};
  mmax = 0.f;
  vmax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t mw = mxs[i >> 1], vw = vws[i >> 1];
    const uint32_t s0 = 0x7650u | (uint32_t)((2 * i) & 3), s1 = s0 + 1u;
    // signed code q: byte (q + 128) in the mantissa of 2^23, minus (2^23 + 128)
    const f32x2 q =
        f2_add(f2_pack_bits(adam8_prmt(mw, 0x4B000000u, s0), adam8_prmt(mw, 0x4B000000u, s1)), k.moff);
    f32x2 m = f2_mul(f2_mul(q, q & 0x7fffffff7fffffffull), kCm);        // q * |q| * absmax / 127^2
    const f32x2 u =
        f2_add(f2_pack_bits(adam8_prmt(vw, 0x4B000000u, s0), adam8_prmt(vw, 0x4B000000u, s1)), k.voff);
    const f32x2 u2 = f2_mul(u, u);
    f32x2 v = f2_mul(f2_mul(u2, kCv), u2);                              // q^4 * absmax / 255^4
    const f32x2 p = f2_pack_bits(pws[i] << 16, pws[i] & 0xffff0000u);
    m = f2_fma(g2[i], k.c1, f2_mul(m, k.b1));
    v = f2_fma(f2_mul(g2[i], g2[i]), k.c2, f2_mul(v, k.b2));
    float m0, m1, v0, v1;
    f2_unpack(m, m0, m1);
    f2_unpack(v, v0, v1);
    mmax = fmaxf(mmax, fmaxf(fabsf(m0), fabsf(m1)));
    vmax = fmaxf(vmax, fmaxf(v0, v1));
    const f32x2 sv = f2_pack(sqrtf(v0), sqrtf(v1));
    float d0, d1;
    f2_unpack(f2_fma(sv, k.rb, k.eps), d0, d1);
    const f32x2 t = f2_mul(m, f2_pack(adam8_rcp(d0), adam8_rcp(d1)));
    p2[i] = f2_fma(t, kNlr, f2_mul(p, kDecay));
    m2[i] = m;
    sv2[i] = sv;
  }
}

// mmax / vmax: the block's maxima (after the warp reduction). idx0: the global index of the lane's first
// element (the stochastic rounding of elements idx0 + 2i and idx0 + 2i + 1 shares one hash).
__device__ __forceinline__ void adam8_encode8(const f32x2 (&m2)[4], const f32x2 (&sv2)[4], const f32x2 (&p2)[4],
                                              float mmax, float vmax, bool stochastic, uint32_t seed,
                                              uint32_t idx0, uint2& mo, uint2& vo, uint4& po) {
  constexpr float kXmin = (0.51f / 255.f) * (0.51f / 255.f);   // sqrt(kXmin) * 255 rounds to code 1
  const float im = mmax > 0.f ? 1.f / mmax : 0.f, siv = vmax > 0.f ? rsqrtf(vmax) : 0.f;
  const f32x2 kIm = f2_pack(im, im), kSiv = f2_pack(siv, siv);
  const f32x2 kMagic = f2_pack(12582912.f, 12582912.f), k127 = f2_pack(127.f, 127.f),
              k255 = f2_pack(255.f, 255.f), kBig = f2_pack(1e30f, 1e30f);
  uint32_t mz[8], vz[8], pz[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float x0, x1, y0, y1, l0, l1, mm0, mm1;
    f2_unpack(m2[i], mm0, mm1);
    f2_unpack(f2_mul(m2[i], kIm), x0, x1);
    f2_unpack(f2_mul(f2_pack(sqrtf(fminf(fabsf(x0), 1.f)), sqrtf(fminf(fabsf(x1), 1.f))), k127), y0, y1);
    // the sign of m on the magnitude code, then + 1.5 * 2^23: the low byte is the int8 code
    const f32x2 z = f2_add(f2_pack_bits(__float_as_uint(y0) | (__float_as_uint(mm0) & 0x80000000u),
                                        __float_as_uint(y1) | (__float_as_uint(mm1) & 0x80000000u)),
                           kMagic);
    f2_unpack(z, y0, y1);
    mz[2 * i] = __float_as_uint(y0);
    mz[2 * i + 1] = __float_as_uint(y1);
    const f32x2 xv = f2_mul(sv2[i], kSiv);
    f2_unpack(xv, x0, x1);
    f2_unpack(f2_mul(xv, kBig), l0, l1);
    x0 = fmaxf(fminf(x0, 1.f), fminf(l0, kXmin));   // a positive second moment never codes as zero
    x1 = fmaxf(fminf(x1, 1.f), fminf(l1, kXmin));
    f2_unpack(f2_fma(f2_pack(sqrtf(x0), sqrtf(x1)), k255, kMagic), y0, y1);
    vz[2 * i] = __float_as_uint(y0);
    vz[2 * i + 1] = __float_as_uint(y1);
    if (stochastic) {
      float q0, q1;
      f2_unpack(p2[i], q0, q1);
      const uint32_t r = adam8_hash(seed ^ ((idx0 + 2u * i) * 0x9E3779B9u));
      const int b0 = (int)__float_as_uint(q0), b1 = (int)__float_as_uint(q1);
      // a NaN (0x7fffffff) would wrap: keep the unrounded bits whenever the sum is not larger
      const int n0 = max(b0, (int)((uint32_t)b0 + (r & 0xffffu))), n1 = max(b1, (int)((uint32_t)b1 + (r >> 16)));
      pz[i] = adam8_prmt((uint32_t)n0, (uint32_t)n1, 0x7632u);
    } else {
      pz[i] = f2_to_bf162(p2[i]);
    }
  }
  mo.x = adam8_prmt(adam8_prmt(mz[0], mz[1], 0x0040u), adam8_prmt(mz[2], mz[3], 0x0040u), 0x5410u);
  mo.y = adam8_prmt(adam8_prmt(mz[4], mz[5], 0x0040u), adam8_prmt(mz[6], mz[7], 0x0040u), 0x5410u);
  vo.x = adam8_prmt(adam8_prmt(vz[0], vz[1], 0x0040u), adam8_prmt(vz[2], vz[3], 0x0040u), 0x5410u);
  vo.y = adam8_prmt(adam8_prmt(vz[4], vz[5], 0x0040u), adam8_prmt(vz[6], vz[7], 0x0040u), 0x5410u);
  po = make_uint4(pz[0], pz[1], pz[2], pz[3]);
}

}  // namespace eri
