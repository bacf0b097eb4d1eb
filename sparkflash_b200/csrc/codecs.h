// Number formats used by the DeepSeek-V4.1-Flash checkpoint and KV caches, written once for
// host and device. Every function is bit-defined (no libm, no hardware converts) so the C++
// oracle, the Python tests and the CUDA kernels agree on every code.
//
//   E4M3 (fn)  : 1-4-3, bias 7, no inf, NaN = 0x7f/0xff, max 448, round-to-nearest-even, saturating.
//   E2M1       : 1-2-1, values {0, .5, 1, 1.5, 2, 3, 4, 6}, round-to-nearest-even, saturating.
//   UE8M0      : 8-bit unsigned exponent, value 2^(code-127); code 255 is NaN.
//
// Scale rules (reference behaviour: kernels/m4_activation_quant_sm121.cuh,
// docs/architecture/01-csa2-attention.md section 8):
//   * FP8 activation, group of 32: amax floored at 1e-4, scale = smallest power of two >= amax/448.
//   * MXFP4 (indexer q/k), group of 32: amax floored at 6*2^-126, scale = 2^ceil(log2(amax/6)).
//   * NVFP4-style KV, group of 16: amax floored at 6*2^-9, scale = e4m3(amax/6) (not a power of two).
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define SFB_HD __host__ __device__ __forceinline__
#else
#define SFB_HD inline
#endif

namespace sfb {

SFB_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
SFB_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f; memcpy(&f, &u, 4); return f;
#endif
}

// ---- bf16 -------------------------------------------------------------------------------------
SFB_HD uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
SFB_HD float bf16_bits_to_f32(uint16_t b) { return bits_f32(((uint32_t)b) << 16); }
SFB_HD float round_bf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

// ---- UE8M0 ------------------------------------------------------------------------------------
SFB_HD float ue8m0_to_f32(uint8_t c) {
  if (c == 0) return bits_f32(0x00400000u);  // 2^-127 (a subnormal float)
  return bits_f32(((uint32_t)c) << 23);
}
// Smallest power of two >= x (x > 0, finite), as a UE8M0 code.
SFB_HD uint8_t ue8m0_ceil(float x) {
  uint32_t b = f32_bits(x);
  int e = (int)((b >> 23) & 0xffu);
  uint32_t man = b & 0x7fffffu;
  if (e == 0) return (uint8_t)(man > 0x400000u ? 1 : 0);  // subnormal input
  int code = e + (man != 0u ? 1 : 0);
  if (code > 254) code = 254;
  return (uint8_t)code;
}
SFB_HD uint8_t act_scale_code_fp8(float amax) {
  float a = amax > 1.0e-4f ? amax : 1.0e-4f;
  return ue8m0_ceil(a * (1.0f / 448.0f));
}
SFB_HD uint8_t act_scale_code_fp4(float amax) {
  const float floor_v = 7.052966e-38f;  // 6 * 2^-126
  float a = amax > floor_v ? amax : floor_v;
  return ue8m0_ceil(a * (1.0f / 6.0f));
}

// ---- E4M3 -------------------------------------------------------------------------------------
SFB_HD float e4m3_to_f32(uint8_t v) {
  uint32_t sign = ((uint32_t)(v & 0x80u)) << 24;
  uint32_t e = (v >> 3) & 0xfu, m = v & 7u;
  if (e == 0xfu && m == 7u) return bits_f32(sign | 0x7fc00000u);
  if (e == 0) {  // subnormal: m * 2^-9
    float f = (float)m * 0.001953125f;
    return bits_f32(f32_bits(f) | sign);
  }
  return bits_f32(sign | ((e + 120u) << 23) | (m << 20));
}
SFB_HD uint8_t f32_to_e4m3(float f) {
  uint32_t u = f32_bits(f);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu);  // NaN
  if (a >= 0x43e80000u) return (uint8_t)(sign | 0x7eu); // >= 464 saturates to 448 (and inf)
  if (a < 0x3c800000u) {                                // |f| < 2^-6: subnormal grid of 2^-9
    float af = bits_f32(a);
    // round-to-nearest-even onto multiples of 2^-9 via the magic-number trick
    float r = af * 512.0f;
    float magic = 8388608.0f;  // 2^23
    float q = (r + magic) - magic;
    uint32_t m = (uint32_t)q;  // 0..8
    return (uint8_t)(sign | m);  // m == 8 lands on the smallest normal 0x08
  }
  // normal: keep 3 mantissa bits, RNE on the 20 dropped bits
  uint32_t lsb = (a >> 20) & 1u;
  a += 0x7ffffu + lsb;
  uint32_t e = (a >> 23) - 120u, m = (a >> 20) & 7u;
  uint32_t code = (e << 3) | m;
  if (code > 0x7eu) code = 0x7eu;
  return (uint8_t)(sign | code);
}

// ---- E2M1 -------------------------------------------------------------------------------------
SFB_HD float e2m1_to_f32(uint8_t v) {
  const float tab[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float f = tab[v & 7u];
  return (v & 8u) ? -f : f;
}
SFB_HD uint8_t f32_to_e2m1(float f) {
  uint8_t sign = (f32_bits(f) >> 28) & 8u;
  float a = f < 0 ? -f : f;
  uint8_t c;
  // midpoints, ties to the code with an even mantissa bit
  if (!(a == a)) c = 7;
  else if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return (uint8_t)(sign | c);
}

// ---- Scale-factor addressing ---------------------------------------------------------------------
// Per-row, per-32-K UE8M0 scales are stored in the order tcgen05 block-scaled MMA consumes them:
// atoms of 128 rows x 4 k-blocks = 512 bytes; inside an atom byte (r%32)*16 + ((r%128)/32)*4 + kb%4.
// Atoms are laid out row-atom-major: atom (ra, ka) at ((ra * ceil(KB/4)) + ka) * 512.
SFB_HD int64_t sf_offset(int64_t row, int64_t kb, int64_t kblocks) {
  int64_t katoms = (kblocks + 3) >> 2;
  int64_t atom = (row >> 7) * katoms + (kb >> 2);
  int64_t r = row & 127;
  return atom * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3);
}
SFB_HD int64_t sf_bytes(int64_t rows, int64_t kblocks) {
  return ((rows + 127) >> 7) * ((kblocks + 3) >> 2) * 512;
}

}  // namespace sfb
