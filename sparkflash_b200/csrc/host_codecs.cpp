// Host-side bulk codecs: the C ABI the Python layer and the converter use to quantise and
// dequantise tensors with exactly the same bit rules as the device kernels (codecs.h).
// Reference behaviour: crates/sparkflash-weights/src/quant*, crates/sparkflash-kernels/src/m4_quant.rs.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include <vector>

#include "codecs.h"

using namespace sfb;

extern "C" {

// ---- scalar probes (golden-table tests) ---------------------------------------------------------
uint8_t sfb_f32_to_e4m3(float f) { return f32_to_e4m3(f); }
float sfb_e4m3_to_f32(uint8_t c) { return e4m3_to_f32(c); }
uint8_t sfb_f32_to_e2m1(float f) { return f32_to_e2m1(f); }
float sfb_e2m1_to_f32(uint8_t c) { return e2m1_to_f32(c); }
float sfb_ue8m0_to_f32(uint8_t c) { return ue8m0_to_f32(c); }
uint8_t sfb_ue8m0_ceil(float x) { return ue8m0_ceil(x); }
uint8_t sfb_act_scale_code_fp8(float amax) { return act_scale_code_fp8(amax); }
uint8_t sfb_act_scale_code_fp4(float amax) { return act_scale_code_fp4(amax); }
uint16_t sfb_f32_to_bf16(float f) { return f32_to_bf16_bits(f); }
int64_t sfb_sf_offset(int64_t row, int64_t kb, int64_t kblocks) { return sf_offset(row, kb, kblocks); }
int64_t sfb_sf_bytes(int64_t rows, int64_t kblocks) { return sf_bytes(rows, kblocks); }

// ---- FP8 activation quant: rows x k (k % 32 == 0); scales row-major [rows, k/32] -----------------
void sfb_act_quant_fp8(const float* x, int64_t rows, int64_t k, uint8_t* q, uint8_t* sc) {
  const int64_t kb = k / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < kb; ++b) {
      const float* p = x + r * k + b * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) { float a = fabsf(p[i]); if (a > amax) amax = a; }
      uint8_t code = act_scale_code_fp8(amax);
      float inv = 1.0f / ue8m0_to_f32(code);
      sc[r * kb + b] = code;
      for (int i = 0; i < 32; ++i) q[r * k + b * 32 + i] = f32_to_e4m3(p[i] * inv);
    }
}

void sfb_act_dequant_fp8(const uint8_t* q, const uint8_t* sc, int64_t rows, int64_t k, float* x) {
  const int64_t kb = k / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < k; ++i)
      x[r * k + i] = e4m3_to_f32(q[r * k + i]) * ue8m0_to_f32(sc[r * kb + i / 32]);
}

// ---- MXFP4 activation quant (indexer q/k): packed two per byte, low nibble = even element --------
void sfb_act_quant_fp4(const float* x, int64_t rows, int64_t k, uint8_t* q, uint8_t* sc) {
  const int64_t kb = k / 32;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < kb; ++b) {
      const float* p = x + r * k + b * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) { float a = fabsf(p[i]); if (a > amax) amax = a; }
      uint8_t code = act_scale_code_fp4(amax);
      float inv = 1.0f / ue8m0_to_f32(code);
      sc[r * kb + b] = code;
      for (int i = 0; i < 32; i += 2) {
        uint8_t lo = f32_to_e2m1(p[i] * inv), hi = f32_to_e2m1(p[i + 1] * inv);
        q[(r * k + b * 32 + i) / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
}

// ---- NVFP4-style KV quant: group 16, E4M3 scale = e4m3(max(amax, 6*2^-9)/6) ----------------------
void sfb_kv_quant_fp4(const float* x, int64_t rows, int64_t k, uint8_t* q, uint8_t* sc) {
  const int64_t g = k / 16;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t b = 0; b < g; ++b) {
      const float* p = x + r * k + b * 16;
      float amax = 0.f;
      for (int i = 0; i < 16; ++i) { float a = fabsf(p[i]); if (a > amax) amax = a; }
      const float fl = 6.0f * 0.001953125f;
      if (amax < fl) amax = fl;
      uint8_t code = f32_to_e4m3(amax / 6.0f);
      float s = e4m3_to_f32(code);
      sc[r * g + b] = code;
      for (int i = 0; i < 16; i += 2) {
        uint8_t lo = f32_to_e2m1(p[i] / s), hi = f32_to_e2m1(p[i + 1] / s);
        q[(r * k + b * 16 + i) / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
}
void sfb_kv_dequant_fp4(const uint8_t* q, const uint8_t* sc, int64_t rows, int64_t k, float* x) {
  const int64_t g = k / 16;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < k; ++i) {
      uint8_t byte = q[(r * k + i) / 2];
      uint8_t nib = (i & 1) ? (byte >> 4) : (byte & 15);
      x[r * k + i] = e2m1_to_f32(nib) * e4m3_to_f32(sc[r * g + i / 16]);
    }
}

// ---- Checkpoint weight grid: scale = 2^(floor(log2 amax) - emax) ---------------------------------
static uint8_t weight_scale_code(float amax, int emax) {
  if (!(amax > 0.f)) return 127 - 20;
  int e = (int)((f32_bits(amax) >> 23) & 0xff) - 127;
  int code = e - emax + 127;
  if (code < 0) code = 0;
  if (code > 254) code = 254;
  return (uint8_t)code;
}

// FP8 weight with 32x32 block scales (checkpoint layout): w [out, in] -> q [out, in], s [ceil(out/32), in/32].
void sfb_weight_quant_fp8_block32(const float* w, int64_t out, int64_t in, uint8_t* q, uint8_t* s) {
  const int64_t ob = (out + 31) / 32, ib = in / 32;
  for (int64_t bo = 0; bo < ob; ++bo)
    for (int64_t bi = 0; bi < ib; ++bi) {
      float amax = 0.f;
      for (int64_t r = bo * 32; r < bo * 32 + 32 && r < out; ++r)
        for (int64_t c = bi * 32; c < bi * 32 + 32; ++c) { float a = fabsf(w[r * in + c]); if (a > amax) amax = a; }
      uint8_t code = weight_scale_code(amax, 8);
      float inv = 1.0f / ue8m0_to_f32(code);
      s[bo * ib + bi] = code;
      for (int64_t r = bo * 32; r < bo * 32 + 32 && r < out; ++r)
        for (int64_t c = bi * 32; c < bi * 32 + 32; ++c) q[r * in + c] = f32_to_e4m3(w[r * in + c] * inv);
    }
}

// FP4 expert weight with per-row, per-32-K scales: w [out, in] -> q [out, in/2], s [out, in/32].
void sfb_weight_quant_fp4_row32(const float* w, int64_t out, int64_t in, uint8_t* q, uint8_t* s) {
  const int64_t ib = in / 32;
  for (int64_t r = 0; r < out; ++r)
    for (int64_t bi = 0; bi < ib; ++bi) {
      const float* p = w + r * in + bi * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) { float a = fabsf(p[i]); if (a > amax) amax = a; }
      uint8_t code = weight_scale_code(amax, 2);
      float inv = 1.0f / ue8m0_to_f32(code);
      s[r * ib + bi] = code;
      for (int i = 0; i < 32; i += 2) {
        uint8_t lo = f32_to_e2m1(p[i] * inv), hi = f32_to_e2m1(p[i + 1] * inv);
        q[(r * in + bi * 32 + i) / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
}

// Expand checkpoint scales to the prepared per-row swizzled layout (see sf_offset).
// block_rows = 32 for 32x32-block FP8 weights, 1 for per-row FP4 scales.
void sfb_scales_to_prepared(const uint8_t* s, int64_t out, int64_t kblocks, int64_t block_rows,
                            uint8_t* dst /* sf_bytes(out, kblocks), pre-filled with 127 */) {
  for (int64_t r = 0; r < out; ++r)
    for (int64_t kb = 0; kb < kblocks; ++kb)
      dst[sf_offset(r, kb, kblocks)] = s[(r / block_rows) * kblocks + kb];
}

}  // extern "C"
