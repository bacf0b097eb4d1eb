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
  const float2* rope;       // [n, rope_stride]: (cos, sin) of the row's position
  int rope_stride;
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
  uint8_t* out_q;           // optional two-term FP8 copy for the tensor-core arm: rows [0,n) hi, [n,2n) lo
  uint8_t* out_atom;        // its scale atoms (rows = hi rows then lo rows)
  float* scratch;           // [n, head_groups, splits, 8, hd + 2] partial (acc, m, l) per split
  unsigned int* tickets;    // [n, head_groups], zero between launches
  int n, heads, rd, window, ring, splits;
  float scale;
};

constexpr int AT_HPB = 8;  // heads per block = warps per block

// grid (head_groups, splits, n), block 256.  A block stages its share of the row's KV entries in shared
// memory once (decoded to fp32) and every warp runs one head over them; the block that finishes a
// (row, head group) last merges the splits in split order.
template <int HD>
__global__ void __launch_bounds__(256) attn_rows_kernel(AttnArgs a) {
  constexpr int EPL = HD / 32;          // elements per lane
  constexpr int TPE = HD / 32;          // threads that decode one entry (32 elements each)
  constexpr int SUB = 256 / TPE;        // entries staged per pass
  extern __shared__ float smem[];
  float* qs = smem;                     // [8][HD]
  float* kvs = smem + AT_HPB * HD;      // [SUB][HD]
  __shared__ int is_last;
  const int hg = blockIdx.x, sp = blockIdx.y, row = blockIdx.z;
  const int pos = a.row_pos[row], L = a.row_lane[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = hg * AT_HPB + warp;
  const bool head_ok = head < a.heads;
  const int r0 = HD - a.rd;
  // ---- queries of the group's heads, rope on the last rd dims ----
  for (int i = threadIdx.x; i < AT_HPB * HD; i += 256) {
    const int hh = hg * AT_HPB + i / HD;
    qs[i] = hh < a.heads ? bf16_to_f(a.q[(size_t)row * a.q_stride + (size_t)hh * HD + (i % HD)]) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < AT_HPB * (a.rd / 2); i += 256) {
    const int hh = i / (a.rd / 2), p = i % (a.rd / 2);
    const float2 c2 = a.rope[(size_t)row * a.rope_stride + p];
    float* qq = qs + hh * HD + r0 + 2 * p;
    const float x = qq[0], y = qq[1];
    qq[0] = bfr(x * c2.x - y * c2.y);
    qq[1] = bfr(x * c2.y + y * c2.x);
  }
  __syncthreads();
  float ql[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) ql[j] = qs[warp * HD + lane * EPL + j];

  const int w_first = pos - a.window + 1 > 0 ? pos - a.window + 1 : 0;
  const int n_win = pos - w_first + 1;
  const int n_sel = a.ckv_q ? a.sel_count[row] : 0;
  const int total = n_win + n_sel;
  const int e_lo = (int)((int64_t)total * sp / a.splits), e_hi = (int)((int64_t)total * (sp + 1) / a.splits);
  float m = -1e30f, l = 0.f, acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;

  for (int base = e_lo; base < e_hi; base += SUB) {
    const int cnt = e_hi - base < SUB ? e_hi - base : SUB;
    {  // stage: thread t decodes 32 elements of entry t / TPE
      const int el = threadIdx.x / TPE, part = threadIdx.x % TPE;
      if (el < cnt) {
        const int e = base + el;
        float f[32];
        if (e < n_win) {
          const int slot = (w_first + e) % a.ring;
          const uint8_t* kq = a.win_q + (size_t)L * a.win_lane_q + (size_t)slot * HD + part * 32;
          const float sc = ue8m0_to_f32(a.win_s[(size_t)L * a.win_lane_s + (size_t)slot * (HD / 32) + part]) *
                           1.152921504606847e18f;  // 2^60: half of the raw decode's 2^-120
          const uint4 v0 = *reinterpret_cast<const uint4*>(kq), v1 = *reinterpret_cast<const uint4*>(kq + 16);
          decode16_e4m3_raw(v0, f); decode16_e4m3_raw(v1, f + 16);
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = (f[j] * 1.152921504606847e18f) * sc;
        } else {
          const int id = a.sel[(size_t)row * a.K + (e - n_win)];
          const uint8_t* kq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)id * (HD / 2) + part * 16;
          const uint8_t* ks = a.ckv_s + (size_t)L * a.ckv_lane_s + (size_t)id * (HD / 16) + part * 2;
          const float s0 = e4m3_to_f32(ks[0]) * 9.223372036854776e18f, s1 = e4m3_to_f32(ks[1]) * 9.223372036854776e18f;
          const uint4 v = *reinterpret_cast<const uint4*>(kq);
          decode32_e2m1_raw(v, f);
#pragma unroll
          for (int j = 0; j < 16; ++j) f[j] = (f[j] * 9.223372036854776e18f) * s0;     // 2^63 twice = 2^126
#pragma unroll
          for (int j = 16; j < 32; ++j) f[j] = (f[j] * 9.223372036854776e18f) * s1;
        }
        float4* dst = reinterpret_cast<float4*>(kvs + el * HD + part * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
      }
    }
    __syncthreads();
    if (head_ok) {
      for (int j0 = 0; j0 < cnt; ++j0) {
        const float* kp = kvs + j0 * HD + lane * EPL;
        float kv[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) kv[j] = kp[j];
        float d = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) d = fmaf(ql[j], kv[j], d);
        d = warp_sum(d) * a.scale;
        const float mn = fmaxf(m, d);
        const float corr = __expf(m - mn), p = __expf(d - mn);
        l = l * corr + p;
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[j] = acc[j] * corr + p * kv[j];
        m = mn;
      }
    }
    __syncthreads();
  }
  // ---- partial of this split ----
  const size_t rec = HD + 2;
  float* mine = a.scratch + ((((size_t)row * gridDim.x + hg) * a.splits + sp) * AT_HPB + warp) * rec;
#pragma unroll
  for (int j = 0; j < EPL; ++j) mine[lane * EPL + j] = acc[j];
  if (lane == 0) { mine[HD] = m; mine[HD + 1] = l; }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* t = a.tickets + (size_t)row * gridDim.x + hg;
    const unsigned int prev = atomicAdd(t, 1u);
    is_last = prev == (unsigned int)a.splits - 1;
    if (is_last) *t = 0;
  }
  __syncthreads();
  if (!is_last || !head_ok) return;
  __threadfence();
  // ---- merge the splits in split order, sink, normalise, inverse rope, write ----
  const float* base_rec = a.scratch + ((((size_t)row * gridDim.x + hg) * a.splits) * AT_HPB + warp) * rec;
  float mt = -1e30f;
  for (int s2 = 0; s2 < a.splits; ++s2) mt = fmaxf(mt, __ldcg(base_rec + (size_t)s2 * AT_HPB * rec + HD));
  float den = __expf(a.sink[head] - mt);
  float o[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) o[j] = 0.f;
  for (int s2 = 0; s2 < a.splits; ++s2) {
    const float* r = base_rec + (size_t)s2 * AT_HPB * rec;
    const float wgt = __expf(__ldcg(r + HD) - mt);
    den += __ldcg(r + HD + 1) * wgt;
#pragma unroll
    for (int j = 0; j < EPL; ++j) o[j] += __ldcg(r + lane * EPL + j) * wgt;
  }
#pragma unroll
  for (int j = 0; j < EPL; ++j) o[j] = bfr(o[j] / den);
  // inverse rope: pairs live inside one lane's chunk (EPL is even)
#pragma unroll
  for (int j = 0; j < EPL; j += 2) {
    const int e = lane * EPL + j;
    if (e >= r0) {
      const int p = (e - r0) >> 1;
      const float2 c2 = a.rope[(size_t)row * a.rope_stride + p];
      const float x = o[j], y = o[j + 1];
      o[j] = bfr(x * c2.x + y * c2.y);
      o[j + 1] = bfr(-x * c2.y + y * c2.x);
    }
  }
  __nv_bfloat16* op = a.out + ((size_t)row * a.heads + head) * HD + lane * EPL;
#pragma unroll
  for (int j = 0; j < EPL; ++j) op[j] = __float2bfloat16_rn(o[j]);
  if (a.out_q) {
    // per-32 groups = 32/EPL consecutive lanes
    constexpr int LPG = 32 / EPL;
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) amax = fmaxf(amax, fabsf(o[j]));
#pragma unroll
    for (int ofs = 1; ofs < LPG; ofs <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, ofs));
    const uint8_t sc = act_scale_code_fp8(amax);
    const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
    const size_t Wd = (size_t)a.heads * HD;
    const size_t c = (size_t)head * HD + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const uint8_t hi = enc_e4m3(o[j] * inv);
      const uint8_t lo = enc_e4m3((o[j] * inv - e4m3_to_f32(hi)) * 16.f);
      a.out_q[(size_t)row * Wd + c + j] = hi;
      a.out_q[(size_t)(a.n + row) * Wd + c + j] = lo;
    }
    if ((lane % LPG) == 0) {
      const int KB = a.heads * HD / 32;
      const int kb = head * (HD / 32) + lane / LPG;
      a.out_atom[sf_offset(row, kb, KB)] = sc;
      a.out_atom[sf_offset(a.n + row, kb, KB)] = sc >= 4 ? (uint8_t)(sc - 4) : (uint8_t)0;
    }
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_attn_groups(int heads) { return (heads + AT_HPB - 1) / AT_HPB; }
int sfb_attn_scratch_floats(int n, int heads, int hd, int splits) {
  return n * sfb_attn_groups(heads) * splits * AT_HPB * (hd + 2);
}

int sfb_attn_rows(const void* q, int64_t q_stride, const void* rope, int rope_stride, const int* row_lane,
                  const int* row_pos, const void* win_q, const void* win_s, int64_t win_lane_q,
                  int64_t win_lane_s, const void* ckv_q, const void* ckv_s, int64_t ckv_lane_q,
                  int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink,
                  void* out, void* out_q, void* out_atom, float* scratch, unsigned int* tickets, int splits, int n,
                  int heads, int hd, int rd, int window, int ring, float scale, cudaStream_t stream) {
  if (splits < 1 || !scratch || !tickets || (hd / 32) % 2) return (int)cudaErrorInvalidValue;
  AttnArgs a{(const __nv_bfloat16*)q, q_stride, (const float2*)rope, rope_stride, row_lane, row_pos, (const uint8_t*)win_q,
             (const uint8_t*)win_s, win_lane_q, win_lane_s, (const uint8_t*)ckv_q, (const uint8_t*)ckv_s,
             ckv_lane_q, ckv_lane_s, sel, sel_count, K, sink, (__nv_bfloat16*)out, (uint8_t*)out_q, (uint8_t*)out_atom,
             scratch, tickets, n, heads, rd, window, ring, splits, scale};
  dim3 grid(sfb_attn_groups(heads), splits, n);
  const size_t smem = sizeof(float) * (size_t)(AT_HPB * hd + 8192);
#define SFB_AT(HDV)                                                                                         \
  {                                                                                                         \
    static bool done = false;                                                                               \
    if (!done) {                                                                                            \
      cudaFuncSetAttribute(attn_rows_kernel<HDV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      done = true;                                                                                          \
    }                                                                                                       \
    attn_rows_kernel<HDV><<<grid, 256, smem, stream>>>(a);                                                  \
  }
  if (hd == 512) SFB_AT(512) else if (hd == 64) SFB_AT(64) else if (hd == 128) SFB_AT(128)
  else return (int)cudaErrorInvalidValue;
#undef SFB_AT
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
