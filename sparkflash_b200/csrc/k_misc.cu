// Embedding gather, stateless Gumbel-max sampling, taps for the drafter and synthetic weight fill.
//
// Reference behaviour: kernels/opt_rows_sm121.cu embed_own:2564 / argmax_fold:1810 / argmax_pick:1834,
// kernels/opt_sample_sm121.cuh (noise keyed on seed, position, token id),
// crates/sparkflash-model-deepseek-v41/src/synthetic.rs (weights from a hash of name and seed).
#include <cooperative_groups.h>

#include "k_common.cuh"

namespace sfb {

// h[row, c, :] = embed[token[row], :] for every hc copy
__global__ void embed_kernel(const __nv_bfloat16* embed, const int* tokens, __nv_bfloat16* h, int n, int hc,
                             int d, int vocab, Status* st) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  int tok = tokens[row];
  if (tok < 0 || tok >= vocab) { if (threadIdx.x == 0 && blockIdx.x == 0) status_set(st, ST_BOUNDS, 3, tok, vocab); tok = 0; }
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (col >= d) return;
  const uint4 v = *reinterpret_cast<const uint4*>(embed + (size_t)tok * d + col);
  for (int c = 0; c < hc; ++c) *reinterpret_cast<uint4*>(h + ((size_t)row * hc + c) * d + col) = v;
}

// rows flagged in `mask` take their input embedding from `override` (image tokens: the vision tower's output or
// one of the learned delimiter vectors) instead of the embedding table
__global__ void embed_override_kernel(const __nv_bfloat16* override_rows, const uint8_t* mask, __nv_bfloat16* h, int hc, int d) {
  const int row = blockIdx.y;
  if (!mask[row]) return;
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (col >= d) return;
  const uint4 v = *reinterpret_cast<const uint4*>(override_rows + (size_t)row * d + col);
  for (int c = 0; c < hc; ++c) *reinterpret_cast<uint4*>(h + ((size_t)row * hc + c) * d + col) = v;
}

// Markov head of the draft block: logits[row, v] += dot(head[v, :], embed[prev, :]) with prev read from device memory
// (the token sampled for the previous block position), one warp per vocabulary entry.
__global__ void __launch_bounds__(256) markov_bias_kernel(float* logits, const __nv_bfloat16* head, const __nv_bfloat16* embed,
                                                         const int* prev, int vl, int r, int vocab) {
  const int v = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (v >= vl) return;
  int p = *prev;
  if (p < 0 || p >= vocab) p = 0;
  float s = 0.f;
  for (int i = lane; i < r; i += 32) s += bf16_to_f(head[(size_t)v * r + i]) * bf16_to_f(embed[(size_t)p * r + i]);
  s = warp_sum(s);
  if (lane == 0) logits[v] += s;
}

// tap[row, :] = bf16(mean over copies of h[row, c, :])
__global__ void tap_mean_kernel(const __nv_bfloat16* h, __nv_bfloat16* tap, int64_t tap_stride, int hc, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= d) return;
  float s = 0.f;
  for (int c = 0; c < hc; ++c) s += bf16_to_f(h[((size_t)row * hc + c) * d + col]);
  tap[(size_t)row * tap_stride + col] = __float2bfloat16_rn(s / (float)hc);
}

// rope[row, v, p] = (cos, sin)(angle) with angle = ((pos / ratio_v) * ratio_v) * inv_freq_v[p], evaluated in
// double once per step; every layer's kernels read this table instead of calling sincos themselves.
struct RopeTableArgs {
  const double* inv_freq[4];
  int ratio[4];
  int V, half;
  const int* row_pos;
  float2* out;  // [n, V, half]
};
__global__ void rope_table_kernel(RopeTableArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int pos = a.row_pos[row];
  for (int i = threadIdx.x; i < a.V * a.half; i += blockDim.x) {
    const int v = i / a.half, p = i - v * a.half;
    const int pp = (pos / a.ratio[v]) * a.ratio[v];
    double s, c;
    sincos((double)pp * a.inv_freq[v][p], &s, &c);
    a.out[((size_t)row * a.V + v) * a.half + p] = make_float2((float)c, (float)s);
  }
}

// L2 prefetch of a weight range: decode kernels are short and latency-bound, so the next kernel's weights are
// pulled into L2 on a side stream while the current one runs (reference: kernels/prefetch_sm121.cuh:44,
// opt_rows prefetch_l2:2508 - the same instruction, there issued under the all-reduce).
__global__ void prefetch_l2_kernel(const uint8_t* p, size_t bytes) {
  const size_t off = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2048;
  if (off >= bytes) return;
  size_t sz = bytes - off < 2048 ? bytes - off : 2048;
  sz &= ~(size_t)15;
  if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"((uint32_t)sz) : "memory");
}
// the same for the experts a row selected: expert e occupies [base + e*stride, +bytes)
__global__ void prefetch_experts_kernel(const uint8_t* base, size_t stride, size_t bytes, const int* ids, int k) {
  const int e = ids[blockIdx.y];  // blockIdx.y indexes (row, slot) pairs: ids is [rows*k] flattened
  const size_t off = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2048;
  if (off >= bytes) return;
  size_t sz = bytes - off < 2048 ? bytes - off : 2048;
  sz &= ~(size_t)15;
  if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + (size_t)e * stride + off), "r"((uint32_t)sz) : "memory");
}

__device__ __forceinline__ float gumbel(uint64_t base, int id) {
  const uint64_t h = splitmix64(base ^ ((uint64_t)id * 0x9E3779B97F4A7C15ull));
  const double u = ((double)(h >> 40) + 0.5) * (1.0 / 16777216.0);
  return (float)(-log(-log(u)));
}

struct SampleArgs {
  const float* logits;    // [n, V] this rank's vocabulary slice
  int64_t stride;
  const int* row_pos;     // sampling position = row_pos + 1 (the position the new token will occupy)
  const float* temperature;  // [n]
  const uint64_t* seed;      // [n]
  const uint8_t* mask;    // optional [n, mask_stride] allowed-token bytes (constrained decoding), 0 = banned
  int64_t mask_stride;
  float* best_val;        // [n]
  int* best_id;           // [n] global token id
  int V, vocab_offset;
};

constexpr int SAMPLE_CLUSTER = 8;   // CTAs per row: each scans an eighth of the vocabulary slice, CTA 0 merges through DSMEM

__global__ void __cluster_dims__(SAMPLE_CLUSTER, 1, 1) __launch_bounds__(1024) sample_kernel(SampleArgs a) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cv[SAMPLE_CLUSTER];
  __shared__ int ci[SAMPLE_CLUSTER];
  const int row = blockIdx.y, part = blockIdx.x;   // part == rank in the cluster
  const float T = a.temperature[row];
  const bool greedy = T < 1e-5f;
  const uint64_t base = splitmix64(a.seed[row] ^ splitmix64((uint64_t)(a.row_pos[row] + 1)));
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  // (value, lowest id) is a total order, so the winner does not depend on how the slice is cut
  for (int i = part * 1024 + threadIdx.x; i < a.V; i += 1024 * SAMPLE_CLUSTER) {
    const int id = a.vocab_offset + i;
    if (a.mask && a.mask[(size_t)row * a.mask_stride + id] == 0) continue;
    float v = a.logits[(size_t)row * a.stride + i];
    if (!greedy) v = v / T + gumbel(base, id);
    if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 32; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    *cluster.map_shared_rank(&cv[part], 0) = bv;
    *cluster.map_shared_rank(&ci[part], 0) = bi;
  }
  cluster.sync();
  if (part == 0 && threadIdx.x == 0) {
    bv = cv[0]; bi = ci[0];
    for (int p = 1; p < SAMPLE_CLUSTER; ++p)
      if (cv[p] > bv || (cv[p] == bv && ci[p] < bi)) { bv = cv[p]; bi = ci[p]; }
    a.best_val[row] = bv;
    a.best_id[row] = bi;
  }
}

// Fold W ranks' (value, id) winners: larger value wins, ties to the lower id.  vals / ids are [W, stride].
// With flags the kernel first waits (bounded) until every rank's winners have arrived.
struct FoldBestArgs {
  const float* vals;
  const int* ids;
  int W, n, stride;
  int* out_tokens;
  const uint32_t* flags[8];
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  uint64_t wait_ns;
  Status* status;
};
__global__ void sample_fold_kernel(FoldBestArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  if (a.flags[0] != nullptr) {
    const uint32_t want = *a.epoch_ptr + a.epoch_add;
    if (threadIdx.x < a.W && !wait_flag_ge(a.flags[threadIdx.x], want, a.wait_ns))
      status_set(a.status, ST_TIMEOUT, 4, threadIdx.x, (int)want);
    __syncthreads();
  }
  for (int row = threadIdx.x; row < a.n; row += blockDim.x) {
    float bv = a.vals[row];
    int bi = a.ids[row];
    for (int r = 1; r < a.W; ++r) {
      const float v = a.vals[(size_t)r * a.stride + row];
      const int id = a.ids[(size_t)r * a.stride + row];
      if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; }
    }
    a.out_tokens[row] = bi;
  }
}

// ---- synthetic weights: bytes from a hash of (tensor seed, element index) ----------------------------------
// fp8: E4M3 codes of ~N(0, sigma) values pre-divided by the block scale 2^(scale_code-127).
__global__ void synth_fp8_kernel(uint8_t* q, int64_t count, uint64_t seed, float sigma_over_scale) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i * 4 >= count) return;
  uint64_t h = splitmix64(seed ^ (uint64_t)i);
  // four values per hash: each from the sum of four 4-bit uniforms (approximately normal)
  uint32_t packed = 0;
  for (int j = 0; j < 4; ++j) {
    uint32_t bits = (uint32_t)(h >> (16 * j)) & 0xffffu;
    float s = (float)((bits & 15) + ((bits >> 4) & 15) + ((bits >> 8) & 15) + ((bits >> 12) & 15)) - 30.f;
    float v = s * (1.f / 9.2195f) * sigma_over_scale;  // var of the sum = 4 * (255/12) = 85 -> std 9.2195
    packed |= (uint32_t)enc_e4m3(v) << (8 * j);
  }
  if (i * 4 + 3 < count) *reinterpret_cast<uint32_t*>(q + i * 4) = packed;
  else for (int j = 0; i * 4 + j < count; ++j) q[i * 4 + j] = (uint8_t)(packed >> (8 * j));
}

// fp4: packed E2M1 codes of ~N(0, sigma)/scale values, 8 per 32-bit word
__global__ void synth_fp4_kernel(uint32_t* q, int64_t words, uint64_t seed, float sigma_over_scale) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= words) return;
  uint64_t h0 = splitmix64(seed ^ (uint64_t)(2 * i)), h1 = splitmix64(seed ^ (uint64_t)(2 * i + 1));
  uint32_t packed = 0;
  for (int j = 0; j < 8; ++j) {
    uint32_t bits = (uint32_t)((j < 4 ? h0 : h1) >> (16 * (j & 3))) & 0xffffu;
    float s = (float)((bits & 15) + ((bits >> 4) & 15) + ((bits >> 8) & 15) + ((bits >> 12) & 15)) - 30.f;
    float v = s * (1.f / 9.2195f) * sigma_over_scale;
    packed |= (uint32_t)f32_to_e2m1(v) << (4 * j);
  }
  q[i] = packed;
}

__global__ void synth_bf16_kernel(__nv_bfloat16* w, int64_t count, uint64_t seed, float sigma, float mean) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  uint64_t h = splitmix64(seed ^ (uint64_t)i);
  uint32_t bits = (uint32_t)h;
  float s = 0.f;
  for (int j = 0; j < 8; ++j) s += (float)((bits >> (4 * j)) & 15);
  w[i] = __float2bfloat16_rn(mean + (s - 60.f) * (1.f / 13.038f) * sigma);  // std of sum of 8 = 13.038
}

__global__ void synth_f32_kernel(float* w, int64_t count, uint64_t seed, float sigma, float mean) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  uint64_t h = splitmix64(seed ^ (uint64_t)i);
  uint32_t bits = (uint32_t)h;
  float s = 0.f;
  for (int j = 0; j < 8; ++j) s += (float)((bits >> (4 * j)) & 15);
  w[i] = mean + (s - 60.f) * (1.f / 13.038f) * sigma;
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_embed(const void* embed, const int* tokens, void* h, int n, int hc, int d, int vocab, void* status,
              cudaStream_t stream) {
  if (d % 8) return (int)cudaErrorInvalidValue;
  embed_kernel<<<dim3((d / 8 + 127) / 128, n), 128, 0, stream>>>((const __nv_bfloat16*)embed, tokens,
                                                               (__nv_bfloat16*)h, n, hc, d, vocab, (Status*)status);
  return SFB_CHECK_LAUNCH();
}

int sfb_markov_bias(void* logits_row, const void* head, const void* embed, const int* prev, int vl, int r, int vocab, cudaStream_t stream) {
  markov_bias_kernel<<<(vl + 7) / 8, 256, 0, stream>>>((float*)logits_row, (const __nv_bfloat16*)head, (const __nv_bfloat16*)embed, prev, vl, r, vocab);
  return SFB_CHECK_LAUNCH();
}

int sfb_embed_override(const void* override_rows, const void* mask, void* h, int n, int hc, int d, cudaStream_t stream) {
  if (d % 8) return (int)cudaErrorInvalidValue;
  embed_override_kernel<<<dim3((d / 8 + 127) / 128, n), 128, 0, stream>>>((const __nv_bfloat16*)override_rows, (const uint8_t*)mask,
                                                                        (__nv_bfloat16*)h, hc, d);
  return SFB_CHECK_LAUNCH();
}

// variants: V <= 4 (inv_freq device pointer, ratio) pairs
int sfb_rope_table(const double* const* inv_freq, const int* ratio, int V, int half, const int* row_pos, void* out,
                   int n, cudaStream_t stream) {
  if (V < 1 || V > 4) return (int)cudaErrorInvalidValue;
  RopeTableArgs a{};
  for (int v = 0; v < V; ++v) { a.inv_freq[v] = inv_freq[v]; a.ratio[v] = ratio[v] > 0 ? ratio[v] : 1; }
  a.V = V; a.half = half; a.row_pos = row_pos; a.out = (float2*)out;
  return (int)sfb_launch(rope_table_kernel, dim3(n), dim3(128), 0, stream, a);
}

int sfb_prefetch_l2(const void* p, int64_t bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  const int64_t threads = (bytes + 2047) / 2048;
  prefetch_l2_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, stream>>>((const uint8_t*)p, (size_t)bytes);
  return SFB_CHECK_LAUNCH();
}

int sfb_prefetch_experts(const void* base, int64_t stride, int64_t bytes, const int* ids, int n_ids, cudaStream_t stream) {
  if (bytes <= 0 || n_ids <= 0) return 0;
  const int64_t threads = (bytes + 2047) / 2048;
  prefetch_experts_kernel<<<dim3((unsigned)((threads + 127) / 128), n_ids), 128, 0, stream>>>(
      (const uint8_t*)base, (size_t)stride, (size_t)bytes, ids, 0);
  return SFB_CHECK_LAUNCH();
}

int sfb_tap_mean(const void* h, void* tap, int64_t tap_stride, int n, int hc, int d, cudaStream_t stream) {
  return (int)sfb_launch(tap_mean_kernel, dim3((d + 255) / 256, n), dim3(256), 0, stream, (const __nv_bfloat16*)h,
                         (__nv_bfloat16*)tap, tap_stride, hc, d);
}

int sfb_sample(const float* logits, int64_t stride, const int* row_pos, const float* temperature,
               const void* seed, const void* mask, int64_t mask_stride, float* best_val, int* best_id, int n,
               int V, int vocab_offset, cudaStream_t stream) {
  SampleArgs a{logits, stride, row_pos, temperature, (const uint64_t*)seed, (const uint8_t*)mask, mask_stride,
               best_val, best_id, V, vocab_offset};
  return (int)sfb_launch(sample_kernel, dim3(SAMPLE_CLUSTER, n), dim3(1024), 0, stream, a);
}

int sfb_sample_fold(const void* vals, const void* ids, int W, int n, int stride, int* out_tokens,
                    const void* const* flag_ptrs, const void* epoch_ptr, uint32_t epoch_add, uint64_t wait_ns,
                    void* status, cudaStream_t stream) {
  if (W < 1 || W > 8) return (int)cudaErrorInvalidValue;
  FoldBestArgs a{};
  a.vals = (const float*)vals; a.ids = (const int*)ids; a.W = W; a.n = n; a.stride = stride; a.out_tokens = out_tokens;
  for (int r = 0; r < 8; ++r) a.flags[r] = (flag_ptrs && r < W) ? (const uint32_t*)flag_ptrs[r] : nullptr;
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns ? wait_ns : 2000000000ull;
  a.status = (Status*)status;
  return (int)sfb_launch(sample_fold_kernel, dim3(1), dim3(64), 0, stream, a);
}

// kind: 0 fp8 bytes, 1 fp4 bytes (count = bytes), 2 bf16 elements, 3 f32 elements
int sfb_synth_fill(int kind, void* dst, int64_t count, uint64_t seed, float sigma, float mean,
                   cudaStream_t stream) {
  const int T = 256;
  if (kind == 0) {
    int64_t thr = (count + 3) / 4;
    synth_fp8_kernel<<<(unsigned)((thr + T - 1) / T), T, 0, stream>>>((uint8_t*)dst, count, seed, sigma);
  } else if (kind == 1) {
    if (count % 4) return (int)cudaErrorInvalidValue;
    int64_t words = count / 4;
    synth_fp4_kernel<<<(unsigned)((words + T - 1) / T), T, 0, stream>>>((uint32_t*)dst, words, seed, sigma);
  } else if (kind == 2) {
    synth_bf16_kernel<<<(unsigned)((count + T - 1) / T), T, 0, stream>>>((__nv_bfloat16*)dst, count, seed, sigma, mean);
  } else if (kind == 3) {
    synth_f32_kernel<<<(unsigned)((count + T - 1) / T), T, 0, stream>>>((float*)dst, count, seed, sigma, mean);
  } else return (int)cudaErrorInvalidValue;
  return SFB_CHECK_LAUNCH();
}

int sfb_device_info(int* sm_count, int* cc_major, int* cc_minor, int64_t* total_mem) {
  cudaDeviceProp p;
  int dev = 0;
  int e = (int)cudaGetDevice(&dev);
  if (e) return e;
  e = (int)cudaGetDeviceProperties(&p, dev);
  if (e) return e;
  *sm_count = p.multiProcessorCount; *cc_major = p.major; *cc_minor = p.minor; *total_mem = (int64_t)p.totalGlobalMem;
  return 0;
}

}  // extern "C"
