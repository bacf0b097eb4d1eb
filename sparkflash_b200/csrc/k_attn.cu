// CSA2 sparse-MLA attention for the rows step: every (row, head) attends the causal window
// (FP8 ring, one UE8M0 scale per 32) followed by the selected compressed entries (FP4 with an E4M3
// scale per 16) of the layer that owns the compressed cache.  One latent KV row serves as key and
// value for all heads.  Online softmax; the per-head sink enters the denominator only; the query
// RoPE is applied on load and the inverse RoPE on the output's rope slice.
//
// Reference behaviour: kernels/opt_attn_sm121.cu:96 (opt_flash_mla_csa2_seq), kernels/opt_rows_sm121.cu
// attn:1097, kernels/flash_mla_csa2_common_sm121.cuh; docs/architecture/01-csa2-attention.md:98-104,212-229.
#include <cooperative_groups.h>

#include "k_common.cuh"

namespace cg = cooperative_groups;

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
  int n, heads, rd, window, ring;
  float scale;
  // optional explicit window per row: positions [win_lo[row], win_hi[row]] of the ring instead of the causal window that
  // ends at the row's own position (draft blocks attend their whole block: no causal mask inside it)
  const int* win_lo;
  const int* win_hi;
};

constexpr int AT_HPB = 4;       // heads per block = warps per block
constexpr int AT_THREADS = AT_HPB * 32;
constexpr int AT_SPLITS = 8;    // CTAs of one cluster share a (row, head group); each takes 1/8 of the entries

// grid (AT_SPLITS, head_groups, n) in clusters of AT_SPLITS.  A CTA stages its share of the row's KV
// entries in shared memory once (decoded to fp32) and every warp runs one head over them; the partial
// (max, sum, accumulator) of every head stays in shared memory, and after a cluster barrier CTA rank h
// merges head h across the eight CTAs in rank order through distributed shared memory - no global
// scratch, no atomics.  The split count is fixed, so a row's bits do not depend on the batch.
template <int HD>
__global__ void __cluster_dims__(AT_SPLITS, 1, 1) __launch_bounds__(AT_THREADS) attn_rows_kernel(AttnArgs a) {
  constexpr int EPL = HD / 32;          // elements per lane
  constexpr int TPE = HD / 32;          // threads that decode one entry (32 elements each)
  constexpr int SUB = AT_THREADS / TPE; // entries staged per pass
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ float smem[];
  float* qs = smem;                        // [HPB][HD]
  float* kvs = smem + AT_HPB * HD;         // [SUB][HD]
  float* part = kvs + SUB * HD;            // [HPB][HD + 2]: acc | m | l
  const int sp = blockIdx.x, hg = blockIdx.y, row = blockIdx.z;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = a.row_pos[row], L = a.row_lane[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = hg * AT_HPB + warp;
  const bool head_ok = head < a.heads;
  const int r0 = HD - a.rd;
  // ---- queries of the group's heads, rope on the last rd dims ----
  for (int i = threadIdx.x; i < AT_HPB * HD; i += AT_THREADS) {
    const int hh = hg * AT_HPB + i / HD;
    qs[i] = hh < a.heads ? bf16_to_f(a.q[(size_t)row * a.q_stride + (size_t)hh * HD + (i % HD)]) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < AT_HPB * (a.rd / 2); i += AT_THREADS) {
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

  const int w_first = a.win_lo ? a.win_lo[row] : (pos - a.window + 1 > 0 ? pos - a.window + 1 : 0);
  const int n_win = (a.win_hi ? a.win_hi[row] : pos) - w_first + 1;
  const int n_sel = a.ckv_q ? a.sel_count[row] : 0;
  const int total = n_win + n_sel;
  const int e_lo = (int)((int64_t)total * sp / AT_SPLITS), e_hi = (int)((int64_t)total * (sp + 1) / AT_SPLITS);
  float m = -1e30f, l = 0.f, acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;

  // Shared-memory layout of a staged entry: element (lane, j) of the lane-chunked row sits at word j*32 + lane,
  // so that a warp reading "its j-th element" touches 32 different banks.
  const int el = threadIdx.x / TPE, prt = threadIdx.x % TPE;
  uint4 raw0, raw1;
  float rs0 = 0.f, rs1 = 0.f;
  int rkind = 0;  // 0 none, 1 window (fp8), 2 compressed (fp4)
  auto fetch = [&](int base) {
    rkind = 0;
    const int e = base + el;
    if (e < e_hi) {
      if (e < n_win) {
        const int slot = (w_first + e) % a.ring;
        const uint8_t* kq = a.win_q + (size_t)L * a.win_lane_q + (size_t)slot * HD + prt * 32;
        rs0 = ue8m0_to_f32(a.win_s[(size_t)L * a.win_lane_s + (size_t)slot * (HD / 32) + prt]) * 1.152921504606847e18f;
        raw0 = *reinterpret_cast<const uint4*>(kq);
        raw1 = *reinterpret_cast<const uint4*>(kq + 16);
        rkind = 1;
      } else {
        const int id = a.sel[(size_t)row * a.K + (e - n_win)];
        const uint8_t* kq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)id * (HD / 2) + prt * 16;
        const uint8_t* ks = a.ckv_s + (size_t)L * a.ckv_lane_s + (size_t)id * (HD / 16) + prt * 2;
        rs0 = e4m3_to_f32(ks[0]) * 9.223372036854776e18f;
        rs1 = e4m3_to_f32(ks[1]) * 9.223372036854776e18f;
        raw0 = *reinterpret_cast<const uint4*>(kq);
        rkind = 2;
      }
    }
  };
  fetch(e_lo);
  for (int base = e_lo; base < e_hi; base += SUB) {
    const int cnt = e_hi - base < SUB ? e_hi - base : SUB;
    if (rkind) {  // decode the prefetched registers into shared memory
      float f[32];
      if (rkind == 1) {
        decode16_e4m3_raw(raw0, f); decode16_e4m3_raw(raw1, f + 16);   // fixed 2^-120, undone in two exact steps
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = (f[j] * 1.152921504606847e18f) * rs0;
      } else {
        decode32_e2m1_raw(raw0, f);                                      // fixed 2^-126
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = (f[j] * 9.223372036854776e18f) * rs0;
#pragma unroll
        for (int j = 16; j < 32; ++j) f[j] = (f[j] * 9.223372036854776e18f) * rs1;
      }
      float* dst = kvs + el * HD;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int e = prt * 32 + j;                 // element of the row
        dst[(e % EPL) * 32 + e / EPL] = f[j];
      }
    }
    __syncthreads();
    fetch(base + SUB);   // next pass's global loads fly while this pass is consumed
    if (head_ok) {
      for (int j0 = 0; j0 < cnt; j0 += 4) {
        float d[4];
        float kv[4][EPL];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float* kp = kvs + (j0 + u) * HD + lane;
          d[u] = 0.f;
          if (j0 + u < cnt) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) { kv[u][j] = kp[j * 32]; d[u] = fmaf(ql[j], kv[u][j], d[u]); }
          } else {
#pragma unroll
            for (int j = 0; j < EPL; ++j) kv[u][j] = 0.f;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
          for (int u = 0; u < 4; ++u) d[u] += __shfl_xor_sync(0xffffffffu, d[u], o);
        }
        float mn = m;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          d[u] = j0 + u < cnt ? d[u] * a.scale : -INFINITY;
          mn = fmaxf(mn, d[u]);
        }
        const float corr = __expf(m - mn);
        float pu[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) pu[u] = __expf(d[u] - mn);
        l = l * corr + ((pu[0] + pu[1]) + (pu[2] + pu[3]));
#pragma unroll
        for (int j = 0; j < EPL; ++j)
          acc[j] = acc[j] * corr + ((pu[0] * kv[0][j] + pu[1] * kv[1][j]) + (pu[2] * kv[2][j] + pu[3] * kv[3][j]));
        m = mn;
      }
    }
    __syncthreads();
  }
  // ---- partial of this CTA, visible to the cluster ----
  float* mine = part + warp * (HD + 2);
#pragma unroll
  for (int j = 0; j < EPL; ++j) mine[j * 32 + lane] = acc[j];
  if (lane == 0) { mine[HD] = m; mine[HD + 1] = l; }
  cluster.sync();
  // ---- CTA rank h (< HPB) merges head h over the eight CTAs in rank order (one warp) ----
  if (sp < AT_HPB && warp == 0 && hg * AT_HPB + sp < a.heads) {
    const int mh = sp;                        // head slot merged by this CTA
    const int ghead = hg * AT_HPB + mh;
    float mt = -1e30f;
    for (int r = 0; r < AT_SPLITS; ++r) mt = fmaxf(mt, cluster.map_shared_rank(part, r)[mh * (HD + 2) + HD]);
    float den = __expf(a.sink[ghead] - mt);
    float o[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) o[j] = 0.f;
    for (int r = 0; r < AT_SPLITS; ++r) {
      const float* rp = cluster.map_shared_rank(part, r) + mh * (HD + 2);
      const float wgt = __expf(rp[HD] - mt);
      den += rp[HD + 1] * wgt;
#pragma unroll
      for (int j = 0; j < EPL; ++j) o[j] += rp[j * 32 + lane] * wgt;
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) o[j] = bfr(o[j] / den);
    // inverse rope: pairs live inside one lane's chunk (EPL is even)
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      const int e = lane * EPL + j;
      if (e >= r0) {
        const float2 c2 = a.rope[(size_t)row * a.rope_stride + ((e - r0) >> 1)];
        const float x = o[j], y = o[j + 1];
        o[j] = bfr(x * c2.x + y * c2.y);
        o[j + 1] = bfr(-x * c2.y + y * c2.x);
      }
    }
    __nv_bfloat16* op = a.out + ((size_t)row * a.heads + ghead) * HD + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) op[j] = __float2bfloat16_rn(o[j]);
    if (a.out_q) {
      constexpr int LPG = 32 / EPL;  // lanes per 32-group
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) amax = fmaxf(amax, fabsf(o[j]));
#pragma unroll
      for (int ofs = 1; ofs < LPG; ofs <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, ofs));
      const uint8_t sc = act_scale_code_fp8(amax);
      const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
      const size_t Wd = (size_t)a.heads * HD;
      const size_t c = (size_t)ghead * HD + lane * EPL;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const uint8_t hi = enc_e4m3(o[j] * inv);
        const uint8_t lo = enc_e4m3((o[j] * inv - e4m3_to_f32(hi)) * 16.f);
        a.out_q[(size_t)row * Wd + c + j] = hi;
        a.out_q[(size_t)(a.n + row) * Wd + c + j] = lo;
      }
      if ((lane % LPG) == 0) {
        const int KB = a.heads * HD / 32;
        const int kb = ghead * (HD / 32) + lane / LPG;
        a.out_atom[sf_offset(row, kb, KB)] = sc;
        a.out_atom[sf_offset(a.n + row, kb, KB)] = sc >= 4 ? (uint8_t)(sc - 4) : (uint8_t)0;
      }
    }
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_attn_rows_range(const void* q, int64_t q_stride, const void* rope, int rope_stride, const int* row_lane,
                        const int* row_pos, const void* win_q, const void* win_s, int64_t win_lane_q,
                        int64_t win_lane_s, const void* ckv_q, const void* ckv_s, int64_t ckv_lane_q,
                        int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink,
                        void* out, void* out_q, void* out_atom, int n, int heads, int hd, int rd, int window, int ring,
                        float scale, const int* win_lo, const int* win_hi, cudaStream_t stream);

int sfb_attn_rows(const void* q, int64_t q_stride, const void* rope, int rope_stride, const int* row_lane,
                  const int* row_pos, const void* win_q, const void* win_s, int64_t win_lane_q,
                  int64_t win_lane_s, const void* ckv_q, const void* ckv_s, int64_t ckv_lane_q,
                  int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink,
                  void* out, void* out_q, void* out_atom, int n, int heads, int hd, int rd, int window, int ring,
                  float scale, cudaStream_t stream) {
  return sfb_attn_rows_range(q, q_stride, rope, rope_stride, row_lane, row_pos, win_q, win_s, win_lane_q, win_lane_s, ckv_q, ckv_s,
                             ckv_lane_q, ckv_lane_s, sel, sel_count, K, sink, out, out_q, out_atom, n, heads, hd, rd, window, ring,
                             scale, nullptr, nullptr, stream);
}

int sfb_attn_rows_range(const void* q, int64_t q_stride, const void* rope, int rope_stride, const int* row_lane,
                        const int* row_pos, const void* win_q, const void* win_s, int64_t win_lane_q,
                        int64_t win_lane_s, const void* ckv_q, const void* ckv_s, int64_t ckv_lane_q,
                        int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink,
                        void* out, void* out_q, void* out_atom, int n, int heads, int hd, int rd, int window, int ring,
                        float scale, const int* win_lo, const int* win_hi, cudaStream_t stream) {
  if ((hd / 32) % 2) return (int)cudaErrorInvalidValue;
  AttnArgs a{(const __nv_bfloat16*)q, q_stride, (const float2*)rope, rope_stride, row_lane, row_pos, (const uint8_t*)win_q,
             (const uint8_t*)win_s, win_lane_q, win_lane_s, (const uint8_t*)ckv_q, (const uint8_t*)ckv_s,
             ckv_lane_q, ckv_lane_s, sel, sel_count, K, sink, (__nv_bfloat16*)out, (uint8_t*)out_q, (uint8_t*)out_atom,
             n, heads, rd, window, ring, scale, win_lo, win_hi};
  dim3 grid(AT_SPLITS, (heads + AT_HPB - 1) / AT_HPB, n);
  const size_t smem = sizeof(float) * (size_t)(AT_HPB * hd + AT_THREADS * 32 + AT_HPB * (hd + 2));
  cudaError_t launch_rc = cudaSuccess;
#define SFB_AT(HDV)                                                                                         \
  {                                                                                                         \
    static bool done = false;                                                                               \
    if (!done) {                                                                                            \
      cudaFuncSetAttribute(attn_rows_kernel<HDV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      done = true;                                                                                          \
    }                                                                                                       \
    launch_rc = sfb_launch(attn_rows_kernel<HDV>, grid, dim3(AT_THREADS), smem, stream, a);                \
  }
  if (hd == 512) SFB_AT(512) else if (hd == 64) SFB_AT(64) else if (hd == 128) SFB_AT(128)
  else return (int)cudaErrorInvalidValue;
#undef SFB_AT
  return (int)launch_rc;
}

}  // extern "C"
