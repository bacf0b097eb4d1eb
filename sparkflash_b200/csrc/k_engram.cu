// Engram on the device: gather + dequantise the hashed rows of this rank's shard, and the gated residual write.
// Reference behaviour: docs/architecture/04-engram.md sections 6-7; crates/sparkflash-deepseek-forward/src/
// tp4_forward/spec.rs:134-265 (lookup wired into the step), kernels: opt_rows engram gate.
//   rows out of this rank's range contribute zeros (the ranks' partial lookups are then summed)
//   gate = sigmoid(copysign(sqrt(max(|dot|, 1e-6)), dot)),  dot = sum(h * w * key) * rstd_h * rstd_key * dim^-0.5
//   h[c] += gate[c] * value   for each of the hc copies;  a masked (image) token keeps h exactly
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "k_common.cuh"

namespace sfb {

// grid (n, cols): one block per (token, hash column); 64 threads x 4 values
__global__ void engram_gather_kernel(const uint8_t* __restrict__ shard, int64_t first_row, int64_t n_rows, int stride,
                                     const int64_t* __restrict__ ids, int cols, int width, __nv_bfloat16* __restrict__ out) {
  const int tok = blockIdx.x, col = blockIdx.y;
  const int64_t id = ids[(size_t)tok * cols + col] - first_row;
  __nv_bfloat16* dst = out + ((size_t)tok * cols + col) * width;
  const bool mine = id >= 0 && id < n_rows;
  for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (mine) {
      const uint8_t* row = shard + (size_t)id * stride;
      const uint32_t q = *reinterpret_cast<const uint32_t*>(row + i);
      const float sc = ue8m0_to_f32(row[width + i / 32]);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = e4m3_to_f32((uint8_t)(q >> (8 * j))) * sc;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[i + j] = __float2bfloat16(v[j]);
  }
}

// grid (n, hc), 256 threads.  kv: [n, (hc+1)*d] bf16 (keys of the hc copies then the value); h: [n, hc, d] f32
__global__ void engram_gate_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ kv, const float* __restrict__ w,
                                   const uint8_t* __restrict__ token_mask, int hc, int d, float eps) {
  const int tok = blockIdx.x, c = blockIdx.y;
  float* hp = h + ((size_t)tok * hc + c) * d;
  const __nv_bfloat16* key = kv + (size_t)tok * (hc + 1) * d + (size_t)c * d;
  const __nv_bfloat16* val = kv + (size_t)tok * (hc + 1) * d + (size_t)hc * d;
  const float* wp = w + (size_t)c * d;
  float sh = 0.f, sk = 0.f, dot = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float a = hp[i], k = __bfloat162float(key[i]);
    sh += a * a; sk += k * k; dot += a * wp[i] * k;
  }
  __shared__ float red[3][32];
  sh = block_sum(sh, red[0]); sk = block_sum(sk, red[1]); dot = block_sum(dot, red[2]);
  const float rstd = rsqrtf(sh / d + eps) * rsqrtf(sk / d + eps);
  dot = dot * rstd * rsqrtf((float)d);
  float g = sqrtf(fmaxf(fabsf(dot), 1e-6f));
  g = 1.f / (1.f + __expf(-copysignf(g, dot)));
  if (token_mask && token_mask[tok] == 0) g = 0.f;
  if (g == 0.f) return;
  for (int i = threadIdx.x; i < d; i += blockDim.x) hp[i] += g * __bfloat162float(val[i]);
}


// the same gate on a bf16 residual stream (the serving engine keeps h in bf16): read fp32, write bf16-rounded
__global__ void __launch_bounds__(256) engram_gate_bf16_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ kv,
                                                              const float* __restrict__ w, const uint8_t* __restrict__ token_mask, int hc,
                                                              int d, float eps) {
  const int tok = blockIdx.x, c = blockIdx.y;
  __nv_bfloat16* hp = h + ((size_t)tok * hc + c) * d;
  const __nv_bfloat16* key = kv + (size_t)tok * (hc + 1) * d + (size_t)c * d;
  const __nv_bfloat16* val = kv + (size_t)tok * (hc + 1) * d + (size_t)hc * d;
  const float* wp = w + (size_t)c * d;
  float sh = 0.f, sk = 0.f, dot = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float a = __bfloat162float(hp[i]), k = __bfloat162float(key[i]);
    sh += a * a; sk += k * k; dot += a * wp[i] * k;
  }
  __shared__ float red[3][32];
  sh = block_sum(sh, red[0]); sk = block_sum(sk, red[1]); dot = block_sum(dot, red[2]);
  const float rstd = rsqrtf(sh / d + eps) * rsqrtf(sk / d + eps);
  dot = dot * rstd * rsqrtf((float)d);
  float g = sqrtf(fmaxf(fabsf(dot), 1e-6f));
  g = 1.f / (1.f + __expf(-copysignf(g, dot)));
  if (token_mask && token_mask[tok] != 0) g = 0.f;       // engine convention: mask = 1 on image rows (dead for the memory)
  if (g == 0.f) return;
  for (int i = threadIdx.x; i < d; i += blockDim.x) hp[i] = __float2bfloat16_rn(__bfloat162float(hp[i]) + g * __bfloat162float(val[i]));
}

}  // namespace sfb

extern "C" {

int sfb_engram_gather(const void* shard, long long first_row, long long n_rows, int stride, const void* ids, int n, int cols,
                      int width, void* out, void* stream) {
  if (width % 4 || stride % 4) return 1;
  sfb::engram_gather_kernel<<<dim3(n, cols), 64, 0, (cudaStream_t)stream>>>((const uint8_t*)shard, first_row, n_rows, stride,
                                                                           (const int64_t*)ids, cols, width, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}
int sfb_engram_gate_bf16(void* h, const void* kv, const void* w, const void* image_mask, int n, int hc, int d, float eps, void* stream) {
  sfb::engram_gate_bf16_kernel<<<dim3(n, hc), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)h, (const __nv_bfloat16*)kv, (const float*)w,
                                                                             (const uint8_t*)image_mask, hc, d, eps);
  return (int)cudaGetLastError();
}
int sfb_engram_gate(void* h, const void* kv, const void* w, const void* token_mask, int n, int hc, int d, float eps, void* stream) {
  sfb::engram_gate_kernel<<<dim3(n, hc), 256, 0, (cudaStream_t)stream>>>((float*)h, (const __nv_bfloat16*)kv, (const float*)w,
                                                                        (const uint8_t*)token_mask, hc, d, eps);
  return (int)cudaGetLastError();
}

}  // extern "C"
