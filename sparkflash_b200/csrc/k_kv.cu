// KV-side kernels of the CSA2 attention: q_norm + FP8 quant of the low-rank query, kv_norm + RoPE +
// FP8 window append, and the compressor (softmax pooling over `ratio` positions, norm, index key,
// RoPE at the compressed position, FP4 append).  All caches are position-addressed (slot =
// position % ring, entry = position / ratio), so rejecting speculative rows is a pointer move.
//
// Reference behaviour: kernels/opt_rows_sm121.cu kv:921 (kv_norm+rope+quant+append via a row table),
// kernels/opt_misc_sm121.cu rows_group_pool:663 / rows_group_keys:695 / rows_group_append:726,
// kernels/kv_path_sm121.cu, kernels/compressed_append_sm121.cu; docs/architecture/01-csa2-attention.md:124-188.
#include "k_common.cuh"

namespace sfb {

__device__ __forceinline__ void rope_pair(float& a, float& b, float2 cs, bool inverse) {
  float cf = cs.x, sf = cs.y;
  if (inverse) sf = -sf;
  float na = a * cf - b * sf, nb = a * sf + b * cf;
  a = na; b = nb;
}

struct QkvPostArgs {
  const __nv_bfloat16* raw;   // [n, q + hd]: wq_a output then wkv output
  const float* q_norm_w;      // [q]
  const float* kv_norm_w;     // [hd]
  const float2* rope;         // [n, rope_stride]: (cos, sin) of the row's position, this layer's variant
  int rope_stride;
  const int* row_lane;        // [n]
  const int* row_pos;         // [n]
  uint8_t* qr_q;              // [n, q] e4m3
  uint8_t* qr_s;              // [n, q/32]
  uint8_t* qr_atom;           // optional scale atoms (rows = tokens) for the tensor-core arm
  __nv_bfloat16* qr_b;        // optional [n, q] bf16 (tests)
  uint8_t* win_q;             // [lanes, ring, hd] e4m3
  uint8_t* win_s;             // [lanes, ring, hd/32]
  int64_t win_lane_stride_q, win_lane_stride_s;
  int n, q, hd, rd, ring;
  float eps;
};

// one block per row, 256 threads
__global__ void __launch_bounds__(256) qkv_post_kernel(QkvPostArgs a) {
  __shared__ float sh[32];
  extern __shared__ float buf[];  // max(q, hd) floats
  const int row = blockIdx.x;
  const __nv_bfloat16* raw = a.raw + (size_t)row * (a.q + a.hd);
  float ss = 0.f, rs;
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.y == 0) {
  // ---- q_norm + quant ----
  for (int i = threadIdx.x; i < a.q; i += 256) { float v = bf16_to_f(raw[i]); buf[i] = v; ss += v * v; }
  ss = block_sum(ss, sh);
  rs = rsqrtf(ss / (float)a.q + a.eps);
  for (int i0 = (threadIdx.x >> 5) * 32; i0 < a.q; i0 += 256) {
    const int i = i0 + (threadIdx.x & 31);
    float v = bfr(buf[i] * rs * a.q_norm_w[i]);
    if (a.qr_b) a.qr_b[(size_t)row * a.q + i] = __float2bfloat16_rn(v);
    uint8_t sc;
    uint8_t qv = warp_quant_fp8(v, &sc);
    a.qr_q[(size_t)row * a.q + i] = qv;
    if ((threadIdx.x & 31) == 0) {
      a.qr_s[(size_t)row * (a.q / 32) + i / 32] = sc;
      if (a.qr_atom) a.qr_atom[sf_offset(row, i / 32, a.q / 32)] = sc;
    }
  }
  return;
  }
  // ---- kv_norm + rope + fp8 + window append ----
  const int pos = a.row_pos[row], lane_id = a.row_lane[row];
  ss = 0.f;
  for (int i = threadIdx.x; i < a.hd; i += 256) { float v = bf16_to_f(raw[a.q + i]); buf[i] = v; ss += v * v; }
  ss = block_sum(ss, sh);
  rs = rsqrtf(ss / (float)a.hd + a.eps);
  for (int i = threadIdx.x; i < a.hd; i += 256) buf[i] = bfr(buf[i] * rs * a.kv_norm_w[i]);
  __syncthreads();
  const int r0 = a.hd - a.rd;
  for (int p = threadIdx.x; p < a.rd / 2; p += 256) {
    float x = buf[r0 + 2 * p], y = buf[r0 + 2 * p + 1];
    rope_pair(x, y, a.rope[(size_t)row * a.rope_stride + p], false);
    buf[r0 + 2 * p] = bfr(x); buf[r0 + 2 * p + 1] = bfr(y);
  }
  __syncthreads();
  const int slot = pos % a.ring;
  uint8_t* wq = a.win_q + (size_t)lane_id * a.win_lane_stride_q + (size_t)slot * a.hd;
  uint8_t* ws = a.win_s + (size_t)lane_id * a.win_lane_stride_s + (size_t)slot * (a.hd / 32);
  for (int i0 = (threadIdx.x >> 5) * 32; i0 < a.hd; i0 += 256) {
    const int i = i0 + (threadIdx.x & 31);
    uint8_t sc;
    uint8_t qv = warp_quant_fp8(buf[i], &sc);
    wq[i] = qv;
    if ((threadIdx.x & 31) == 0) ws[i / 32] = sc;
  }
}

struct CompressArgs {
  const float* raw;          // [n, raw_stride]: compressor wkv out [hd], then wgate out [hd] when ratio > 1
  int64_t raw_stride;
  const float* norm_w;       // [hd]
  const __nv_bfloat16* wk;   // [idh, hd] indexer key projection
  const float* k_norm_w;     // [idh]
  const float2* rope;        // [n, rope_stride]: (cos, sin) at the compressed position of the row
  int rope_stride;
  const int* row_lane;
  const int* row_pos;
  float* cin;                // [lanes, cring, 2*hd] pending (kv, score) per position (ratio > 1)
  int64_t cin_lane_stride;
  int cring;
  uint8_t* ckv_q;            // [lanes, max_entries, hd/2] packed e2m1
  uint8_t* ckv_s;            // [lanes, max_entries, hd/16] e4m3 scales
  uint8_t* ik_q;             // [lanes, max_entries, idh/2]
  uint8_t* ik_s;             // [lanes, max_entries, idh/32] ue8m0
  int64_t ckv_lane_q, ckv_lane_s, ik_lane_q, ik_lane_s;  // lane strides in bytes
  int max_entries;
  int n, hd, idh, rd, ratio;
  float eps;
  Status* status;
};

// one block per row, 256 threads. dynamic smem: (2*hd + idh) floats
__global__ void __launch_bounds__(256) compress_append_kernel(CompressArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  extern __shared__ float buf[];
  float* lat = buf;            // [hd]
  float* rot = buf + a.hd;     // [hd]
  float* key = buf + 2 * a.hd; // [idh]
  const int row = blockIdx.x;
  const int pos = a.row_pos[row], L = a.row_lane[row];
  const float* raw = a.raw + (size_t)row * a.raw_stride;
  const int hd = a.hd, ratio = a.ratio;
  if (ratio > 1) {
    float* ring = a.cin + (size_t)L * a.cin_lane_stride + (size_t)(pos % a.cring) * 2 * hd;
    for (int i = threadIdx.x; i < 2 * hd; i += 256) ring[i] = raw[i];
    if ((pos + 1) % ratio) return;
    // pool the group pos+1-ratio .. pos; rows of this launch are read from `raw`, older ones from the ring
    for (int i = threadIdx.x; i < hd; i += 256) {
      float mx = -INFINITY;
      for (int t = 0; t < ratio; ++t) {
        const int back = ratio - 1 - t;  // position pos-back
        const int prow = row - back;
        const float* src = (prow >= 0 && a.row_lane[prow] == L && a.row_pos[prow] == pos - back)
                               ? a.raw + (size_t)prow * a.raw_stride
                               : a.cin + (size_t)L * a.cin_lane_stride + (size_t)((pos - back) % a.cring) * 2 * hd;
        mx = fmaxf(mx, src[hd + i]);
      }
      float den = 0.f, num = 0.f;
      for (int t = 0; t < ratio; ++t) {
        const int back = ratio - 1 - t;
        const int prow = row - back;
        const float* src = (prow >= 0 && a.row_lane[prow] == L && a.row_pos[prow] == pos - back)
                               ? a.raw + (size_t)prow * a.raw_stride
                               : a.cin + (size_t)L * a.cin_lane_stride + (size_t)((pos - back) % a.cring) * 2 * hd;
        float e = expf(src[hd + i] - mx);
        den += e; num += e * src[i];
      }
      lat[i] = bfr(num / den);
    }
  } else {
    for (int i = threadIdx.x; i < hd; i += 256) lat[i] = bfr(raw[i]);
  }
  __syncthreads();
  float ss = 0.f;
  for (int i = threadIdx.x; i < hd; i += 256) ss += lat[i] * lat[i];
  ss = block_sum(ss, sh);
  float rs = rsqrtf(ss / (float)hd + a.eps);
  for (int i = threadIdx.x; i < hd; i += 256) lat[i] = bfr(lat[i] * rs * a.norm_w[i]);
  __syncthreads();
  const int j = pos / ratio;
  if (j >= a.max_entries) { status_set(a.status, ST_BOUNDS, 2, j, a.max_entries); return; }
  // ---- index key: k_norm(wk . latent), rope, MXFP4 ----
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int o = warp; o < a.idh; o += 8) {
    const __nv_bfloat16* wr = a.wk + (size_t)o * hd;
    float s = 0.f;
    for (int i = lane; i < hd; i += 32) s = fmaf(bf16_to_f(wr[i]), lat[i], s);
    s = warp_sum(s);
    if (lane == 0) key[o] = bfr(s);
  }
  __syncthreads();
  ss = 0.f;
  for (int i = threadIdx.x; i < a.idh; i += 256) ss += key[i] * key[i];
  ss = block_sum(ss, sh);
  rs = rsqrtf(ss / (float)a.idh + a.eps);
  for (int i = threadIdx.x; i < a.idh; i += 256) key[i] = bfr(key[i] * rs * a.k_norm_w[i]);
  for (int i = threadIdx.x; i < hd; i += 256) rot[i] = lat[i];
  __syncthreads();
  for (int p = threadIdx.x; p < a.rd / 2; p += 256) {
    {
      const int r0 = a.idh - a.rd;
      float x = key[r0 + 2 * p], y = key[r0 + 2 * p + 1];
      rope_pair(x, y, a.rope[(size_t)row * a.rope_stride + p], false);
      key[r0 + 2 * p] = bfr(x); key[r0 + 2 * p + 1] = bfr(y);
    }
    {
      const int r0 = hd - a.rd;
      float x = rot[r0 + 2 * p], y = rot[r0 + 2 * p + 1];
      rope_pair(x, y, a.rope[(size_t)row * a.rope_stride + p], false);
      rot[r0 + 2 * p] = bfr(x); rot[r0 + 2 * p + 1] = bfr(y);
    }
  }
  __syncthreads();
  // MXFP4 index key: groups of 32, one per warp iteration
  uint8_t* ikq = a.ik_q + (size_t)L * a.ik_lane_q + (size_t)j * (a.idh / 2);
  uint8_t* iks = a.ik_s + (size_t)L * a.ik_lane_s + (size_t)j * (a.idh / 32);
  for (int g = warp; g < a.idh / 32; g += 8) {
    float v = key[g * 32 + lane];
    float amax = warp_max(fabsf(v));
    uint8_t sc = act_scale_code_fp4(amax);
    uint8_t c = f32_to_e2m1(v / ue8m0_to_f32(sc));
    uint8_t hi = (uint8_t)__shfl_down_sync(0xffffffffu, (int)c, 1);
    if ((lane & 1) == 0) ikq[g * 16 + lane / 2] = (uint8_t)(c | (hi << 4));
    if (lane == 0) iks[g] = sc;
  }
  // NVFP4-style KV: groups of 16 (half-warps), E4M3 scale
  uint8_t* cq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)j * (hd / 2);
  uint8_t* cs = a.ckv_s + (size_t)L * a.ckv_lane_s + (size_t)j * (hd / 16);
  for (int g = warp; g < hd / 32; g += 8) {
    float v = rot[g * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 6.0f * 0.001953125f);
    uint8_t sc = f32_to_e4m3(amax / 6.0f);
    float s = e4m3_to_f32(sc);
    uint8_t c = f32_to_e2m1(v / s);
    uint8_t hi = (uint8_t)__shfl_down_sync(0xffffffffu, (int)c, 1);
    if ((lane & 1) == 0) cq[g * 16 + lane / 2] = (uint8_t)(c | (hi << 4));
    if ((lane & 15) == 0) cs[g * 2 + lane / 16] = sc;
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_qkv_post(const void* raw, const float* q_norm_w, const float* kv_norm_w, const void* rope, int rope_stride,
                 const int* row_lane, const int* row_pos, void* qr_q, void* qr_s, void* qr_atom, void* qr_b, void* win_q,
                 void* win_s, int64_t win_lane_stride_q, int64_t win_lane_stride_s, int n, int q, int hd,
                 int rd, int ring, float eps, cudaStream_t stream) {
  if (q % 32 || hd % 32 || rd % 2) return (int)cudaErrorInvalidValue;
  QkvPostArgs a{(const __nv_bfloat16*)raw, q_norm_w, kv_norm_w, (const float2*)rope, rope_stride, row_lane, row_pos,
                (uint8_t*)qr_q, (uint8_t*)qr_s, (uint8_t*)qr_atom, (__nv_bfloat16*)qr_b, (uint8_t*)win_q, (uint8_t*)win_s,
                win_lane_stride_q, win_lane_stride_s, n, q, hd, rd, ring, eps};
  const size_t smem = sizeof(float) * (size_t)(q > hd ? q : hd);
  return (int)sfb_launch(qkv_post_kernel, dim3(n, 2), dim3(256), smem, stream, a);
}

int sfb_compress_append(const float* raw, int64_t raw_stride, const float* norm_w, const void* wk,
                        const float* k_norm_w, const void* rope, int rope_stride, const int* row_lane,
                        const int* row_pos, float* cin, int64_t cin_lane_stride, int cring, void* ckv_q,
                        void* ckv_s, void* ik_q, void* ik_s, int64_t ckv_lane_q, int64_t ckv_lane_s,
                        int64_t ik_lane_q, int64_t ik_lane_s, int max_entries, int n, int hd, int idh,
                        int rd, int ratio, float eps, void* status, cudaStream_t stream) {
  if (hd % 32 || idh % 32) return (int)cudaErrorInvalidValue;
  CompressArgs a{raw, raw_stride, norm_w, (const __nv_bfloat16*)wk, k_norm_w, (const float2*)rope, rope_stride,
                 row_lane, row_pos,
                 cin, cin_lane_stride, cring, (uint8_t*)ckv_q, (uint8_t*)ckv_s, (uint8_t*)ik_q,
                 (uint8_t*)ik_s, ckv_lane_q, ckv_lane_s, ik_lane_q, ik_lane_s, max_entries, n, hd, idh, rd,
                 ratio, eps, (Status*)status};
  const size_t smem = sizeof(float) * (size_t)(2 * hd + idh);
  return (int)sfb_launch(compress_append_kernel, dim3(n), dim3(256), smem, stream, a);
}

}  // extern "C"
