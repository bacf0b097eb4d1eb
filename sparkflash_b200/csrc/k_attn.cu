// CSA2 sparse-MLA attention for the rows step: every (row, head) attends the causal window
// (FP8 ring, one UE8M0 scale per 32) followed by the selected compressed entries (FP4 with an E4M3
// scale per 16) of the layer that owns the compressed cache.  One latent KV row serves as key and
// value for all heads.  Online softmax; the per-head sink enters the denominator only; the query
// RoPE is applied on load and the inverse RoPE on the output's rope slice.
//
// Reference behaviour: kernels/opt_attn_sm121.cu:96 (opt_flash_mla_csa2_seq), kernels/opt_rows_sm121.cu
// attn:1097, kernels/flash_mla_csa2_common_sm121.cuh; docs/architecture/01-csa2-attention.md:98-104,212-229.
#include "k_common.cuh"

namespace sfb {

struct AttnArgs {
  const __nv_bfloat16* q;   // [n, q_stride]; head h at h*hd
  int64_t q_stride;
  const double* inv_freq;   // [rd/2]
  const int* row_lane;
  const int* row_pos;
  const uint8_t* win_q;     // [lanes, ring, hd]
  const uint8_t* win_s;     // [lanes, ring, hd/32]
  int64_t win_lane_q, win_lane_s;
  const uint8_t* ckv_q;     // [lanes, max_entries, hd/2] (null when the layer has no compressed path)
  const uint8_t* ckv_s;     // [lanes, max_entries, hd/16]
  int64_t ckv_lane_q, ckv_lane_s;
  const int* sel;           // [n, K] ascending ids, -1 padded
  const int* sel_count;     // [n]
  int K;
  const float* sink;        // [heads]
  __nv_bfloat16* out;       // [n, heads*hd]
  int n, heads, rd, window, ring;
  float scale;
};

template <int HD>
__global__ void __launch_bounds__(256) attn_rows_kernel(AttnArgs a) {
  constexpr int EPL = HD / 32;  // elements per lane
  __shared__ float qs[HD];
  __shared__ float m_w[8], l_w[8];
  __shared__ float acc_w[8][HD];
  const int head = blockIdx.x, row = blockIdx.y;
  const int pos = a.row_pos[row], L = a.row_lane[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // ---- load q, rope its last rd dims ----
  const __nv_bfloat16* qp = a.q + (size_t)row * a.q_stride + (size_t)head * HD;
  for (int i = threadIdx.x; i < HD; i += 256) qs[i] = bf16_to_f(qp[i]);
  __syncthreads();
  const int r0 = HD - a.rd;
  for (int p = threadIdx.x; p < a.rd / 2; p += 256) {
    double s, c;
    sincos((double)pos * a.inv_freq[p], &s, &c);
    float x = qs[r0 + 2 * p], y = qs[r0 + 2 * p + 1];
    qs[r0 + 2 * p] = bfr(x * (float)c - y * (float)s);
    qs[r0 + 2 * p + 1] = bfr(x * (float)s + y * (float)c);
  }
  __syncthreads();
  float ql[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) ql[j] = qs[lane * EPL + j];

  const int w_first = pos - a.window + 1 > 0 ? pos - a.window + 1 : 0;
  const int n_win = pos - w_first + 1;
  const int n_sel = a.ckv_q ? a.sel_count[row] : 0;
  const int total = n_win + n_sel;
  float m = -1e30f, l = 0.f, acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;

  for (int e = warp; e < total; e += 8) {
    float kv[EPL];
    if (e < n_win) {
      const int slot = (w_first + e) % a.ring;
      const uint8_t* kq = a.win_q + (size_t)L * a.win_lane_q + (size_t)slot * HD + lane * EPL;
      float sc = ue8m0_to_f32(a.win_s[(size_t)L * a.win_lane_s + (size_t)slot * (HD / 32) + (lane * EPL) / 32]);
      if (EPL == 16) {
        uint4 v = *reinterpret_cast<const uint4*>(kq);
        decode16_e4m3_raw(v, kv);  // values carry a fixed 2^-120; undo it in two exact steps
#pragma unroll
        for (int j = 0; j < EPL; ++j) kv[j] *= 1.152921504606847e18f;  // 2^60
        sc *= 1.152921504606847e18f;
      } else {
#pragma unroll
        for (int j = 0; j < EPL; j += 2) {
          float2 t = cvt_e4m3x2(*reinterpret_cast<const uint16_t*>(kq + j));
          kv[j] = t.x; kv[j + 1] = t.y;
        }
      }
#pragma unroll
      for (int j = 0; j < EPL; ++j) kv[j] *= sc;
    } else {
      const int id = a.sel[(size_t)row * a.K + (e - n_win)];
      const uint8_t* kq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)id * (HD / 2) + lane * (EPL / 2);
      float sc = e4m3_to_f32(a.ckv_s[(size_t)L * a.ckv_lane_s + (size_t)id * (HD / 16) + (lane * EPL) / 16]);
      if (EPL == 16) {
        uint2 v = *reinterpret_cast<const uint2*>(kq);
        decode8_e2m1_raw(v.x, kv); decode8_e2m1_raw(v.y, kv + 8);  // fixed 2^-126
#pragma unroll
        for (int j = 0; j < EPL; ++j) kv[j] *= 9.223372036854776e18f;  // 2^63
        sc *= 9.223372036854776e18f;
      } else {
#pragma unroll
        for (int j = 0; j < EPL / 2; ++j) { float2 t = cvt_e2m1x2(kq[j]); kv[2 * j] = t.x; kv[2 * j + 1] = t.y; }
      }
#pragma unroll
      for (int j = 0; j < EPL; ++j) kv[j] *= sc;
    }
    float d = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) d = fmaf(ql[j], kv[j], d);
    d = warp_sum(d) * a.scale;
    const float mn = fmaxf(m, d);
    const float corr = expf(m - mn), p = expf(d - mn);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc[j] = acc[j] * corr + p * kv[j];
    m = mn;
  }
  // ---- merge the 8 warps ----
  if (lane == 0) { m_w[warp] = m; l_w[warp] = l; }
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc_w[warp][lane * EPL + j] = acc[j];
  __syncthreads();
  float mt = m_w[0];
  for (int w = 1; w < 8; ++w) mt = fmaxf(mt, m_w[w]);
  float den = expf(a.sink[head] - mt);
  for (int w = 0; w < 8; ++w) den += l_w[w] * expf(m_w[w] - mt);
  for (int i = threadIdx.x; i < HD; i += 256) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += acc_w[w][i] * expf(m_w[w] - mt);
    qs[i] = bfr(s / den);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < a.rd / 2; p += 256) {
    double s, c;
    sincos((double)pos * a.inv_freq[p], &s, &c);
    float x = qs[r0 + 2 * p], y = qs[r0 + 2 * p + 1];
    qs[r0 + 2 * p] = bfr(x * (float)c + y * (float)s);
    qs[r0 + 2 * p + 1] = bfr(-x * (float)s + y * (float)c);
  }
  __syncthreads();
  __nv_bfloat16* op = a.out + ((size_t)row * a.heads + head) * HD;
  for (int i = threadIdx.x; i < HD; i += 256) op[i] = __float2bfloat16_rn(qs[i]);
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_attn_rows(const void* q, int64_t q_stride, const double* inv_freq, const int* row_lane,
                  const int* row_pos, const void* win_q, const void* win_s, int64_t win_lane_q,
                  int64_t win_lane_s, const void* ckv_q, const void* ckv_s, int64_t ckv_lane_q,
                  int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink,
                  void* out, int n, int heads, int hd, int rd, int window, int ring, float scale,
                  cudaStream_t stream) {
  AttnArgs a{(const __nv_bfloat16*)q, q_stride, inv_freq, row_lane, row_pos, (const uint8_t*)win_q,
             (const uint8_t*)win_s, win_lane_q, win_lane_s, (const uint8_t*)ckv_q, (const uint8_t*)ckv_s,
             ckv_lane_q, ckv_lane_s, sel, sel_count, K, sink, (__nv_bfloat16*)out, n, heads, rd, window, ring,
             scale};
  dim3 grid(heads, n);
  if (hd == 512) attn_rows_kernel<512><<<grid, 256, 0, stream>>>(a);
  else if (hd == 64) attn_rows_kernel<64><<<grid, 256, 0, stream>>>(a);
  else if (hd == 128) attn_rows_kernel<128><<<grid, 256, 0, stream>>>(a);
  else return (int)cudaErrorInvalidValue;
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
