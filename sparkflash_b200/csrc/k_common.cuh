// Device helpers shared by every kernel file: hardware format converts, warp/block reductions,
// activation quantisation of one 32-group held by a warp, bounded waits and the status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "codecs.h"
#include "launch.cuh"

#define SFB_CHECK_LAUNCH() (int)cudaGetLastError()

namespace sfb {

// ---- status word -------------------------------------------------------------------------------------
// Kernels that wait on a flag or detect a bad index never trap: they record a code here and return.
enum StatusCode : int { ST_OK = 0, ST_TIMEOUT = 1, ST_BOUNDS = 2, ST_BAD_ARG = 3 };
struct Status {
  int code;      // first non-zero StatusCode recorded
  int where;     // kernel-defined site id
  int detail0;   // e.g. peer rank / index
  int detail1;   // e.g. expected epoch
};
__device__ __forceinline__ void status_set(Status* st, int code, int where, int d0, int d1) {
  if (st && atomicCAS(&st->code, 0, code) == 0) {
    st->where = where; st->detail0 = d0; st->detail1 = d1;
  }
}

// ---- converts -------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 cvt_e4m3x2(uint16_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
__device__ __forceinline__ float2 cvt_e2m1x2(uint8_t v) {
  uint32_t h2;
  uint16_t w = v;
  asm("{.reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t;}" : "=r"(h2) : "h"(w));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// 16 E4M3 codes (one uint4) -> 16 floats
__device__ __forceinline__ void decode16_e4m3(const uint4& v, float* f) {
  const uint16_t* p = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
  for (int i = 0; i < 8; ++i) { float2 t = cvt_e4m3x2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
// 32 E2M1 codes (one uint4) -> 32 floats
__device__ __forceinline__ void decode32_e2m1(const uint4& v, float* f) {
  const uint8_t* p = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
  for (int i = 0; i < 16; ++i) { float2 t = cvt_e2m1x2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
// ---- integer-pipe decodes ------------------------------------------------------------------------------------
// Format converts run on a narrow pipe; hot loops instead build fp32 bit patterns with shifts and
// masks.  The result is the true value times a fixed power of two (2^-120 for E4M3, 2^-126 for
// E2M1; subnormal codes land on fp32 subnormals, which FMA handles exactly), and the caller folds
// the inverse power into the block scale it multiplies by anyway.
#define SFB_E4M3_RAW_EXP 120
#define SFB_E2M1_RAW_EXP 126
__device__ __forceinline__ void decode4_e4m3_raw(uint32_t w, float* f) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = w << (24 - 8 * j);  // byte j in the top byte
    f[j] = __uint_as_float((t & 0x80000000u) | ((t & 0x7f000000u) >> 4));
  }
}
__device__ __forceinline__ void decode16_e4m3_raw(const uint4& v, float* f) {
  decode4_e4m3_raw(v.x, f); decode4_e4m3_raw(v.y, f + 4); decode4_e4m3_raw(v.z, f + 8); decode4_e4m3_raw(v.w, f + 12);
}
__device__ __forceinline__ void decode8_e2m1_raw(uint32_t w, float* f) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t t = w << (28 - 4 * j);  // nibble j in the top nibble
    f[j] = __uint_as_float((t & 0x80000000u) | ((t & 0x70000000u) >> 6));
  }
}
__device__ __forceinline__ void decode32_e2m1_raw(const uint4& v, float* f) {
  decode8_e2m1_raw(v.x, f); decode8_e2m1_raw(v.y, f + 8); decode8_e2m1_raw(v.z, f + 16); decode8_e2m1_raw(v.w, f + 24);
}
// block scale 2^(code-127) times 2^extra, as one float (code + extra stays below 255 for any
// weight or cache scale the model produces; saturates otherwise)
__device__ __forceinline__ float ue8m0_shifted(uint8_t code, int extra) {
  int e = (int)code + extra;
  e = e > 254 ? 254 : (e < 1 ? 1 : e);
  return __uint_as_float((uint32_t)e << 23);
}

__device__ __forceinline__ float bf16_to_f(__nv_bfloat16 b) { return __bfloat162float(b); }
__device__ __forceinline__ float bfr(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ uint8_t enc_e4m3(float f) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(f));
  return (uint8_t)(r & 0xff);
}
__device__ __forceinline__ uint16_t enc_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ uint4 ldg_nc(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// ---- one thread of a warp ----------------------------------------------------------------------------------
// One lane of a converged warp.  Unlike a test of the lane index, the election tells the compiler that exactly one thread
// runs the guarded code, so the operands of the TMA / tcgen05 instructions in it can stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// ---- reductions -------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `sh` must hold 32 floats; result broadcast to all threads. Deterministic order.
__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += sh[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float t = sh[0];
  for (int i = 1; i < nw; ++i) t = fmaxf(t, sh[i]);
  return t;
}

// ---- quantise one 32-group held one-element-per-lane by a full warp ---------------------------------------
// Returns the E4M3 code of this lane's element; *scale_code is the group's UE8M0 code (all lanes).
__device__ __forceinline__ uint8_t warp_quant_fp8(float v, uint8_t* scale_code) {
  float amax = warp_max(fabsf(v));    // (a single redux.max over the bit patterns measured slower than the five shuffles here)
  uint8_t sc = act_scale_code_fp8(amax);
  *scale_code = sc;
  float inv = bits_f32(((uint32_t)(254 - sc)) << 23);  // 2^-(sc-127); sc in [~100, 254)
  return enc_e4m3(v * inv);
}

// ---- time-bounded spin ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= want (wrap-safe signed compare) or the budget runs out. Returns true on success.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, uint64_t budget_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (int it = 0; it < (1 << 28); ++it) {
    if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((it & 63) == 63 && globaltimer_ns() - t0 > budget_ns) return false;
    __nanosleep(20);
  }
  return false;
}

// Shared-memory activation rows are padded by 4 floats per 32 so that lanes reading consecutive
// 16-byte-chunk-aligned slices with 128-bit loads do not collide on banks.
__host__ __device__ __forceinline__ int sm_pad(int k) { return k + ((k >> 5) << 2); }

// Dequantise `count16` chunks of 16 FP8 codes (+ one UE8M0 scale per 32) into padded shared memory.
// src codes are 16-byte aligned; dst index space is sm_pad().
__device__ __forceinline__ void stage_fp8_to_smem(const uint8_t* q, const uint8_t* sc, int count16,
                                                  float* dst, int nthreads) {
  for (int i = threadIdx.x; i < count16; i += nthreads) {
    const uint4 v = *reinterpret_cast<const uint4*>(q + (size_t)i * 16);
    const float s = ue8m0_to_f32(sc[i >> 1]);
    float f[16];
    decode16_e4m3(v, f);
    float4* o = reinterpret_cast<float4*>(dst + sm_pad(i * 16));
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = make_float4(f[4 * j] * s, f[4 * j + 1] * s, f[4 * j + 2] * s, f[4 * j + 3] * s);
  }
}

// splitmix64: the sampler's stateless noise and the synthetic-weight generator
__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

}  // namespace sfb
