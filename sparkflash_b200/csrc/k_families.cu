// Kernels of the other model families: gated delta-net / KDA linear attention (recurrent state per head), the
// short causal depthwise convolution with carried history, and soft-capping.
// Reference behaviour: kernels/qwen4_exp_sm121.cu (gdn_conv, kda_decay, gdn_recur), kernels/qwen4_scan_sm121.cu
// (gdn_scan / kda_scan), kernels/inkling_conv_sm121.cu (short_conv, conv_history_copy/restore),
// kernels/inkling_softcap_sm121.cuh, kernels/inkling_epilogue_sm121.cu (softcapped_swiglu, logit_softcap).
//
// Delta rule for one head with state S [dk, dv] (fp32, resident in HBM, touched once per token):
//     S <- diag(a) S            a = scalar decay (GDN) or one decay per key channel (KDA)
//     r  = v - S^T k            what the memory does not already say about k
//     S <- S + b * k r^T        b = write strength
//     o  = S^T q
// Rows of one sequence are applied in order inside one block, so a chunk of T rows gives the bits of T single steps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "k_common.cuh"

namespace sfb {

struct DeltaArgs {
  const float* q;      // [T, H, dk]
  const float* k;      // [T, H, dk]   (already normalised by the caller's recipe)
  const float* v;      // [T, H, dv]
  const float* a;      // [T, H] (GDN) or [T, H, dk] (KDA): decay in (0, 1]
  const float* b;      // [T, H]
  float* S;            // [lanes, H, dk, dv]
  float* o;            // [T, H, dv]
  const int* row_lane; // [T] lane of each row; rows of one lane are consecutive and in order
  int T, H, dk, dv, per_channel;
};

// grid (H, lanes_in_step): block handles one (head, lane): every row of that lane in order.  Thread j owns column j of S.
__global__ void __launch_bounds__(256) delta_rule_kernel(DeltaArgs p, const int* lane_ids, int n_lanes) {
  const int h = blockIdx.x, lane = lane_ids[blockIdx.y];
  extern __shared__ float sm[];          // k [dk], q [dk], a [dk]
  float* ks = sm; float* qs = sm + p.dk; float* as = sm + 2 * p.dk;
  float* S = p.S + ((size_t)lane * p.H + h) * p.dk * p.dv;
  for (int t = 0; t < p.T; ++t) {
    if (p.row_lane[t] != lane) continue;
    for (int i = threadIdx.x; i < p.dk; i += blockDim.x) {
      ks[i] = p.k[((size_t)t * p.H + h) * p.dk + i];
      qs[i] = p.q[((size_t)t * p.H + h) * p.dk + i];
      as[i] = p.per_channel ? p.a[((size_t)t * p.H + h) * p.dk + i] : p.a[(size_t)t * p.H + h];
    }
    __syncthreads();
    const float beta = p.b[(size_t)t * p.H + h];
    for (int j = threadIdx.x; j < p.dv; j += blockDim.x) {
      float mem = 0.f;
      for (int i = 0; i < p.dk; ++i) {            // decay, then read the memory along k
        const float s = S[(size_t)i * p.dv + j] * as[i];
        S[(size_t)i * p.dv + j] = s;
        mem += s * ks[i];
      }
      const float r = (p.v[((size_t)t * p.H + h) * p.dv + j] - mem) * beta;
      float out = 0.f;
      for (int i = 0; i < p.dk; ++i) {
        const float s = S[(size_t)i * p.dv + j] + ks[i] * r;
        S[(size_t)i * p.dv + j] = s;
        out += s * qs[i];
      }
      p.o[((size_t)t * p.H + h) * p.dv + j] = out;
    }
    __syncthreads();
  }
}

// Short causal depthwise convolution (width W <= 8) with history: y[t, c] = sum_j w[c, j] * x[t - (W-1) + j, c]; rows before
// the chunk come from hist[lane, c, 0..W-2] (oldest first), which is updated to the chunk's last W-1 rows.
struct ConvArgs {
  const __nv_bfloat16* x;   // [T, C]
  const float* w;           // [C, W]
  float* hist;              // [lanes, C, W-1]
  __nv_bfloat16* y;         // [T, C]
  const int* row_lane;      // [T]; rows of one lane consecutive and in order
  int T, C, W, silu;
};

__global__ void __launch_bounds__(256) short_conv_kernel(ConvArgs p, const int* lane_ids) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = lane_ids[blockIdx.y];
  if (c >= p.C) return;
  float win[8];
  const int Wm = p.W - 1;
  for (int j = 0; j < Wm; ++j) win[j] = p.hist[((size_t)lane * p.C + c) * Wm + j];
  float wc[8];
  for (int j = 0; j < p.W; ++j) wc[j] = p.w[(size_t)c * p.W + j];
  for (int t = 0; t < p.T; ++t) {
    if (p.row_lane[t] != lane) continue;
    const float xt = __bfloat162float(p.x[(size_t)t * p.C + c]);
    float acc = wc[Wm] * xt;
    for (int j = 0; j < Wm; ++j) acc += wc[j] * win[j];
    for (int j = 0; j + 1 < Wm; ++j) win[j] = win[j + 1];
    if (Wm > 0) win[Wm - 1] = xt;
    if (p.silu) acc = acc / (1.f + __expf(-acc));
    p.y[(size_t)t * p.C + c] = __float2bfloat16_rn(acc);
  }
  for (int j = 0; j < Wm; ++j) p.hist[((size_t)lane * p.C + c) * Wm + j] = win[j];
}

// y = cap * tanh(x / cap), in place on fp32 logits; and the soft-capped SwiGLU: silu(softcap(g)) * u
__global__ void softcap_kernel(float* x, int64_t n, float cap) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}
__global__ void softcapped_swiglu_kernel(const __nv_bfloat16* g, const __nv_bfloat16* u, __nv_bfloat16* y, int64_t n, float cap) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float gc = cap * tanhf(__bfloat162float(g[i]) / cap);
    y[i] = __float2bfloat16_rn(gc / (1.f + __expf(-gc)) * __bfloat162float(u[i]));
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_delta_rule(const void* q, const void* k, const void* v, const void* a, const void* b, void* S, void* o, const void* row_lane,
                   const void* lane_ids, int n_lanes, int T, int H, int dk, int dv, int per_channel, cudaStream_t stream) {
  if (dk > 1024 || n_lanes < 1) return (int)cudaErrorInvalidValue;
  DeltaArgs p{(const float*)q, (const float*)k, (const float*)v, (const float*)a, (const float*)b, (float*)S, (float*)o,
              (const int*)row_lane, T, H, dk, dv, per_channel};
  delta_rule_kernel<<<dim3(H, n_lanes), dv < 256 ? ((dv + 31) / 32 * 32) : 256, 3 * dk * sizeof(float), stream>>>(p, (const int*)lane_ids, n_lanes);
  return SFB_CHECK_LAUNCH();
}
int sfb_short_conv(const void* x, const void* w, void* hist, void* y, const void* row_lane, const void* lane_ids, int n_lanes, int T, int C,
                   int W, int silu, cudaStream_t stream) {
  if (W < 1 || W > 8) return (int)cudaErrorInvalidValue;
  ConvArgs p{(const __nv_bfloat16*)x, (const float*)w, (float*)hist, (__nv_bfloat16*)y, (const int*)row_lane, T, C, W, silu};
  short_conv_kernel<<<dim3((C + 255) / 256, n_lanes), 256, 0, stream>>>(p, (const int*)lane_ids);
  return SFB_CHECK_LAUNCH();
}
int sfb_softcap(void* x, long long n, float cap, cudaStream_t stream) {
  softcap_kernel<<<148 * 4, 256, 0, stream>>>((float*)x, n, cap);
  return SFB_CHECK_LAUNCH();
}
int sfb_softcapped_swiglu(const void* g, const void* u, void* y, long long n, float cap, cudaStream_t stream) {
  softcapped_swiglu_kernel<<<148 * 4, 256, 0, stream>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)y, n, cap);
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
