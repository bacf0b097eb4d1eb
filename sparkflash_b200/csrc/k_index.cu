// CSA2 indexer: MXFP4 query/key index scores, HSI candidate blocks and the top-k select.
//
//   score[t] = sum_h relu(q_h . k_t) * w_h      over compressed entries t < compress_len(row)
//   top-k by value, ties to the lowest index, -inf never selected, ids returned ascending.
//
// Reference behaviour: kernels/opt_select_sm121.cu (opt_select_scores:563, _rows:610, opt_ref_select:101,
// opt_select_fast:484 - radix select up to 2M positions), kernels/select_body_sm121.cuh,
// kernels/opt_mma_sm121.cu:1066 (index scores on tensor cores), docs/architecture/01-csa2-attention.md:152-208,
// crates/sparkflash-kernels/tests/ref_select_rules.rs (tie rule).
#include "k_common.cuh"

namespace sfb {

__device__ __forceinline__ void rope_pair_f(float& a, float& b, float2 cs) {
  float cf = cs.x, sf = cs.y;
  float na = a * cf - b * sf, nb = a * sf + b * cf;
  a = na; b = nb;
}

// ---- query side: rope + MXFP4 round trip of the indexer query, and the head weights -----------------------
struct IndexQArgs {
  const __nv_bfloat16* qraw;  // [n, q_stride], indexer part starts at q_off: [inh, idh]
  int64_t q_stride, q_off;
  const float* wraw;          // [n, w_stride] weights_proj output (fp32) at w_off: [inh]
  int64_t w_stride, w_off;
  const float2* rope;         // [n, rope_stride]
  int rope_stride;
  const int* row_pos;
  float* qi;                  // [n, idh, inh]  (transposed: element-major, head-minor)
  float* wt;                  // [n, inh]
  int n, inh, idh, rd;
  float wscale;
};

// grid (n, IQ_SPLIT), block 256; one warp per (head, 32-group), the items dealt round-robin over the row's CTAs
__global__ void __launch_bounds__(256) index_q_kernel(IndexQArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gph = a.idh / 32;
  for (int item = warp + 8 * blockIdx.y; item < a.inh * gph; item += 8 * gridDim.y) {
    const int h = item / gph, g = item % gph;
    const int e = g * 32 + lane;
    float v = bf16_to_f(a.qraw[(size_t)row * a.q_stride + a.q_off + (size_t)h * a.idh + e]);
    const int r0 = a.idh - a.rd;
    if (e >= r0) {
      const int p = (e - r0) >> 1;
      float other = __shfl_xor_sync(0xffffffffu, v, 1);
      float x = (e & 1) ? other : v, y = (e & 1) ? v : other;
      rope_pair_f(x, y, a.rope[(size_t)row * a.rope_stride + p]);
      v = (e & 1) ? y : x;
    } else {
      (void)__shfl_xor_sync(0xffffffffu, v, 1);
    }
    v = bfr(v);
    float amax = warp_max(fabsf(v));
    uint8_t sc = act_scale_code_fp4(amax);
    float s = ue8m0_to_f32(sc);
    float dq = e2m1_to_f32(f32_to_e2m1(v / s)) * s;
    a.qi[((size_t)row * a.idh + e) * a.inh + h] = dq;
  }
  if (blockIdx.y != 0) return;
  for (int h = threadIdx.x; h < a.inh; h += 256)
    a.wt[(size_t)row * a.inh + h] = bfr(a.wraw[(size_t)row * a.w_stride + a.w_off + h]) * a.wscale;
}

// ---- scores --------------------------------------------------------------------------------------------------
struct IndexScoreArgs {
  const float* qi;        // [n, idh, inh]
  const float* wt;        // [n, inh]
  const uint8_t* ik_q;    // [lanes, max_entries, idh/2]
  const uint8_t* ik_s;    // [lanes, max_entries, idh/32]
  int64_t ik_lane_q, ik_lane_s;
  const int* row_lane;
  const int* row_pos;
  const uint8_t* cand;    // optional [n, cand_stride] block flags (1 = in pool)
  int64_t cand_stride;
  int cand_block;
  float* scores;          // [n, score_stride]
  int64_t score_stride;
  int n, inh, idh, ratio, max_len;
};

constexpr int IS_ENT_PER_BLOCK = 64;

// grid (ceil(max_len/64), n), block 256: each warp scores 8 entries
__global__ void __launch_bounds__(256) index_scores_kernel(IndexScoreArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* q = sm;                         // [idh * inh]
  float* kbuf = sm + a.idh * a.inh;      // [8 warps][idh]
  const int row = blockIdx.y;
  const int clen = (a.row_pos[row] + 1) / a.ratio;
  const int e0 = blockIdx.x * IS_ENT_PER_BLOCK;
  if (e0 >= clen) return;  // the select and the block maxima only read entries below compress_len
  for (int i = threadIdx.x; i < a.idh * a.inh; i += 256) q[i] = a.qi[(size_t)row * a.idh * a.inh + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = a.row_lane[row];
  float* kw = kbuf + warp * a.idh;
  for (int t = warp; t < IS_ENT_PER_BLOCK; t += 8) {
    const int ent = e0 + t;
    if (ent >= a.max_len) break;
    float score = -INFINITY;
    bool live = ent < clen;
    if (live && a.cand) live = a.cand[(size_t)row * a.cand_stride + ent / a.cand_block] != 0;
    if (live) {
      const uint8_t* kq = a.ik_q + (size_t)L * a.ik_lane_q + (size_t)ent * (a.idh / 2);
      const uint8_t* ks = a.ik_s + (size_t)L * a.ik_lane_s + (size_t)ent * (a.idh / 32);
      for (int b = lane; b < a.idh / 2; b += 32) {
        float2 v = cvt_e2m1x2(kq[b]);
        float s = ue8m0_to_f32(ks[(2 * b) / 32]);
        kw[2 * b] = v.x * s; kw[2 * b + 1] = v.y * s;
      }
      __syncwarp();
      float part = 0.f;
      for (int h = lane; h < a.inh; h += 32) {
        float dsum = 0.f;
        for (int i = 0; i < a.idh; ++i) dsum = fmaf(q[i * a.inh + h], kw[i], dsum);
        part += fmaxf(dsum, 0.f) * a.wt[(size_t)row * a.inh + h];
      }
      score = warp_sum(part);
      __syncwarp();
    }
    if (lane == 0) a.scores[(size_t)row * a.score_stride + ent] = score;
  }
}

// ---- HSI block maxima ---------------------------------------------------------------------------------------
// bscore[row, b] = max over the block's entries (< clen); the newest block is pinned to +inf.
__global__ void hsi_blockmax_kernel(const float* scores, int64_t score_stride, const int* row_pos, int ratio,
                                    int bs, float* bscore, int64_t b_stride, int max_blocks) {
  const int row = blockIdx.y;
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= max_blocks) return;
  const int clen = (row_pos[row] + 1) / ratio;
  const int nb = (clen + bs - 1) / bs;
  float m = -INFINITY;
  if (b < nb) {
    for (int i = 0; i < bs; ++i) {
      const int e = b * bs + i;
      if (e < clen) m = fmaxf(m, scores[(size_t)row * score_stride + e]);
    }
    if (b == nb - 1) m = INFINITY;
  }
  bscore[(size_t)row * b_stride + b] = m;
}

// flags[row, b] = 1 for each selected block id
__global__ void hsi_mark_kernel(const int* ids, int K, uint8_t* flags, int64_t f_stride, int max_blocks) {
  const int row = blockIdx.y;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < max_blocks; b += gridDim.x * blockDim.x)
    flags[(size_t)row * f_stride + b] = 0;
}
__global__ void hsi_mark2_kernel(const int* ids, int K, uint8_t* flags, int64_t f_stride) {
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < K) {
    const int id = ids[(size_t)row * K + i];
    if (id >= 0) flags[(size_t)row * f_stride + id] = 1;
  }
}

// ---- top-k select --------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float -> larger key
}

struct SelectArgs {
  const float* scores;   // [n, stride]
  int64_t stride;
  const int* row_pos;    // length per row = (row_pos+1)/ratio / len_div (rounded up), capped by max_len
  int ratio, len_div, max_len;
  int K;
  int* ids;              // [n, K] ascending, -1 padded
  int* count;            // [n]
};

constexpr int SEL_THREADS = 1024;

// One block selects the top K of `len` elements: 4 radix passes of 8 bits, then an ordered compaction.  Element i is
// sc[i] (IND = false; the id written is base + i) or sc[list[i]] with `list` ascending (IND = true; the id written is
// list[i]), so "ties go to the lowest index" holds in both forms.
template <bool IND>
__device__ __forceinline__ void select_run(const float* sc, const int* list, int len, int base, int K, int* out, int* count_out) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_total;
  __shared__ uint32_t wsum[32];
  struct { int K; } a{K};
  const uint32_t NEG_INF_KEY = order_key(-INFINITY);
  auto at = [&](int i) -> float { return IND ? sc[list[i]] : sc[i]; };
  // count finite candidates (key > key(-inf))
  if (threadIdx.x == 0) s_total = 0;
  __syncthreads();
  uint32_t cnt = 0;
  for (int i = threadIdx.x; i < len; i += SEL_THREADS) cnt += order_key(at(i)) > NEG_INF_KEY;
  cnt = (uint32_t)__reduce_add_sync(0xffffffffu, cnt);
  if ((threadIdx.x & 31) == 0 && cnt) atomicAdd(&s_total, cnt);
  __syncthreads();
  const uint32_t total = s_total;
  const uint32_t k = min((uint32_t)a.K, total);
  uint32_t thr_key = 0, need_eq = 0;  // take every key > thr_key and the first need_eq with key == thr_key
  if (k > 0 && k < total) {
    uint32_t prefix = 0, need = k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = threadIdx.x; i < 256; i += SEL_THREADS) hist[i] = 0;
      __syncthreads();
      // histogram of the pass's byte: the lanes of a warp that hit the same bin add once (scores cluster in a few bins of the
      // top bytes, and one shared-memory atomic per lane serialised them)
      for (int i0 = 0; i0 < len; i0 += SEL_THREADS) {
        const int i = i0 + threadIdx.x;
        uint32_t bin = 256u + (threadIdx.x & 31);      // no bin: a value of its own, matched by no other lane
        if (i < len) {
          const uint32_t key = order_key(at(i));
          if (key > NEG_INF_KEY && (key & mask) == prefix) bin = (key >> shift) & 255u;
        }
        const uint32_t same = __match_any_sync(0xffffffffu, bin);
        if (bin < 256u && (threadIdx.x & 31) == (uint32_t)(__ffs(same) - 1)) atomicAdd(&hist[bin], (uint32_t)__popc(same));
      }
      __syncthreads();
      // the bin in which the count from the top reaches `need`: the largest b with sum(hist[b..255]) >= need (bin 0 when only
      // the whole histogram does).  One warp: lane l owns bins 8l..8l+7, a shuffle scan gives the count above them.
      if (threadIdx.x < 32) {
        const int l = threadIdx.x;
        uint32_t h[8], own = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { h[j] = hist[8 * l + j]; own += h[j]; }
        uint32_t incl = own;                        // own bins and every bin above them
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t v = __shfl_down_sync(0xffffffffu, incl, o);
          if (l + o < 32) incl += v;
        }
        const uint32_t above = incl - own;
        if (above < need && (incl >= need || l == 0)) {      // exactly one lane: the crossing lies in its bins
          uint32_t acc = above;
          int j = 7;
          for (; j > 0; --j) {
            if (acc + h[j] >= need) break;
            acc += h[j];
          }
          if (l > 0 || acc + h[j] >= need || j == 0) {
            s_prefix = prefix | ((uint32_t)(8 * l + j) << shift);
            s_need = need - acc;
          }
        }
      }
      __syncthreads();
      prefix = s_prefix; need = s_need;
      __syncthreads();
    }
    thr_key = prefix; need_eq = need;
  } else if (k > 0) {  // k == total: take every finite entry
    thr_key = NEG_INF_KEY; need_eq = 0;
  }
  // ordered compaction: chunks of SEL_THREADS in index order
  __shared__ uint32_t s_base_gt, s_base_eq;
  if (threadIdx.x == 0) { s_base_gt = 0; s_base_eq = 0; }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c0 = 0; c0 < len && k > 0; c0 += SEL_THREADS) {
    const int i = c0 + threadIdx.x;
    uint32_t key = i < len ? order_key(at(i)) : 0u;
    const bool gt = i < len && key > thr_key;
    const bool eq = i < len && key == thr_key && need_eq > 0 && key > NEG_INF_KEY;
    // eq entries are admitted in index order until need_eq is used up, so rank them first
    const uint32_t eq_ballot = __ballot_sync(0xffffffffu, eq);
    const uint32_t eq_rank_w = __popc(eq_ballot & ((1u << lane) - 1));
    if (lane == 0) wsum[warp] = __popc(eq_ballot);
    __syncthreads();
    uint32_t eq_before = s_base_eq;
    for (int w = 0; w < warp; ++w) eq_before += wsum[w];
    uint32_t eq_chunk = 0;
    for (int w = 0; w < SEL_THREADS / 32; ++w) eq_chunk += wsum[w];
    const bool take = gt || (eq && (eq_before + eq_rank_w) < need_eq);
    __syncthreads();
    const uint32_t tk_ballot = __ballot_sync(0xffffffffu, take);
    const uint32_t tk_rank_w = __popc(tk_ballot & ((1u << lane) - 1));
    if (lane == 0) wsum[warp] = __popc(tk_ballot);
    __syncthreads();
    uint32_t before = s_base_gt;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    uint32_t chunk = 0;
    for (int w = 0; w < SEL_THREADS / 32; ++w) chunk += wsum[w];
    if (take && before + tk_rank_w < (uint32_t)a.K) out[before + tk_rank_w] = IND ? list[i] : base + i;
    __syncthreads();
    if (threadIdx.x == 0) { s_base_gt += chunk; s_base_eq += eq_chunk; }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < a.K; i += SEL_THREADS)
    if ((uint32_t)i >= k) out[i] = -1;
  if (threadIdx.x == 0) *count_out = (int)k;
  __syncthreads();
}

__device__ __forceinline__ int select_len(const SelectArgs& a, int row) {
  int len = (a.row_pos[row] + 1) / a.ratio;
  len = (len + a.len_div - 1) / a.len_div;
  return len > a.max_len ? a.max_len : len;
}

// one block per row
__global__ void __launch_bounds__(SEL_THREADS) select_topk_kernel(SelectArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  select_run<false>(a.scores + (size_t)row * a.stride, nullptr, select_len(a, row), 0, a.K, a.ids + (size_t)row * a.K, a.count + row);
}

// Long rows, stage 1: grid (chunks, rows); block (c, row) selects the top K of its chunk of the row into
// tmp_ids[row, c, :] (ascending ids) and tmp_cnt[row, c].  The top K of the row is a subset of the union of the chunks'
// top K (with the same order on (value, index)), which stage 2 selects from.
__global__ void __launch_bounds__(SEL_THREADS) select_chunks_kernel(SelectArgs a, int chunk, int* tmp_ids, int* tmp_cnt) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x, row = blockIdx.y, nch = gridDim.x;
  const int len = select_len(a, row), base = c * chunk;
  int lc = len - base;
  lc = lc < 0 ? 0 : (lc > chunk ? chunk : lc);
  select_run<false>(a.scores + (size_t)row * a.stride + base, nullptr, lc, base, a.K, tmp_ids + ((size_t)row * nch + c) * a.K,
                    tmp_cnt + (size_t)row * nch + c);
}

// stage 2: one block per row gathers the chunks' winners (ascending by construction) and selects among them
__global__ void __launch_bounds__(SEL_THREADS) select_merge_kernel(SelectArgs a, int nch, const int* tmp_ids, const int* tmp_cnt, int* tmp_list) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int off[257];
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    int o = 0;
    for (int c = 0; c < nch; ++c) { off[c] = o; o += tmp_cnt[(size_t)row * nch + c]; }
    off[nch] = o;
  }
  __syncthreads();
  int* list = tmp_list + (size_t)row * nch * a.K;
  for (int c = 0; c < nch; ++c) {
    const int cnt = off[c + 1] - off[c];
    for (int i = threadIdx.x; i < cnt; i += SEL_THREADS) list[off[c] + i] = tmp_ids[((size_t)row * nch + c) * a.K + i];
  }
  __syncthreads();
  select_run<true>(a.scores + (size_t)row * a.stride, list, off[nch], 0, a.K, a.ids + (size_t)row * a.K, a.count + row);
}


}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_index_q(const void* qraw, int64_t q_stride, int64_t q_off, const float* wraw, int64_t w_stride,
                int64_t w_off, const void* rope, int rope_stride, const int* row_pos, float* qi, float* wt, int n,
                int inh, int idh, int rd, float wscale, cudaStream_t stream) {
  if (idh % 32) return (int)cudaErrorInvalidValue;
  IndexQArgs a{(const __nv_bfloat16*)qraw, q_stride, q_off, wraw, w_stride, w_off, (const float2*)rope, rope_stride,
               row_pos, qi, wt,
               n, inh, idh, rd, wscale};
  return (int)sfb_launch(index_q_kernel, dim3(n, n <= 16 ? 4 : 1), dim3(256), 0, stream, a);
}

int sfb_index_scores(const float* qi, const float* wt, const void* ik_q, const void* ik_s, int64_t ik_lane_q,
                     int64_t ik_lane_s, const int* row_lane, const int* row_pos, const void* cand,
                     int64_t cand_stride, int cand_block, float* scores, int64_t score_stride, int n, int inh,
                     int idh, int ratio, int max_len, cudaStream_t stream) {
  if (max_len <= 0) return 0;
  IndexScoreArgs a{qi, wt, (const uint8_t*)ik_q, (const uint8_t*)ik_s, ik_lane_q, ik_lane_s, row_lane, row_pos,
                   (const uint8_t*)cand, cand_stride, cand_block, scores, score_stride, n, inh, idh, ratio,
                   max_len};
  const size_t smem = sizeof(float) * (size_t)(idh * inh + 8 * idh);
  if (smem > 48 * 1024) {
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(index_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); done = true; }
  }
  dim3 grid((max_len + IS_ENT_PER_BLOCK - 1) / IS_ENT_PER_BLOCK, n);
  return (int)sfb_launch(index_scores_kernel, grid, dim3(256), smem, stream, a);
}

int sfb_hsi_blockmax(const float* scores, int64_t score_stride, const int* row_pos, int ratio, int bs,
                     float* bscore, int64_t b_stride, int max_blocks, int n, cudaStream_t stream) {
  if (max_blocks <= 0) return 0;
  hsi_blockmax_kernel<<<dim3((max_blocks + 255) / 256, n), 256, 0, stream>>>(scores, score_stride, row_pos, ratio,
                                                                          bs, bscore, b_stride, max_blocks);
  return SFB_CHECK_LAUNCH();
}

int sfb_hsi_mark(const int* ids, int K, void* flags, int64_t f_stride, int max_blocks, int n,
                 cudaStream_t stream) {
  if (max_blocks <= 0) return 0;
  int gb = (max_blocks + 255) / 256;
  if (gb > 1024) gb = 1024;
  hsi_mark_kernel<<<dim3(gb, n), 256, 0, stream>>>(ids, K, (uint8_t*)flags, f_stride, max_blocks);
  hsi_mark2_kernel<<<dim3((K + 255) / 256, n), 256, 0, stream>>>(ids, K, (uint8_t*)flags, f_stride);
  return SFB_CHECK_LAUNCH();
}

// Long rows: the row cut into `chunk`-sized pieces selected by separate blocks, then merged.  tmp_ids [n, chunks, K],
// tmp_cnt [n, chunks], tmp_list [n, chunks * K] are caller-provided int32 scratch; chunks = ceil(max_len / chunk) <= 256.
int sfb_select_topk_long(const float* scores, int64_t stride, const int* row_pos, int ratio, int len_div, int max_len, int K,
                         int* ids, int* count, int n, int chunk, int* tmp_ids, int* tmp_cnt, int* tmp_list, cudaStream_t stream) {
  const int nch = (max_len + chunk - 1) / chunk;
  if (chunk < 1 || nch < 1 || nch > 256) return (int)cudaErrorInvalidValue;
  SelectArgs a{scores, stride, row_pos, ratio, len_div, max_len, K, ids, count};
  cudaError_t e = sfb_launch(select_chunks_kernel, dim3(nch, n), dim3(SEL_THREADS), 0, stream, a, chunk, tmp_ids, tmp_cnt);
  if (e != cudaSuccess) return (int)e;
  return (int)sfb_launch(select_merge_kernel, dim3(n), dim3(SEL_THREADS), 0, stream, a, nch, (const int*)tmp_ids, (const int*)tmp_cnt,
                         tmp_list);
}

// length of row = ceil(((row_pos+1)/ratio) / len_div), capped at max_len
int sfb_select_topk(const float* scores, int64_t stride, const int* row_pos, int ratio, int len_div,
                    int max_len, int K, int* ids, int* count, int n, cudaStream_t stream) {
  SelectArgs a{scores, stride, row_pos, ratio, len_div, max_len, K, ids, count};
  return (int)sfb_launch(select_topk_kernel, dim3(n), dim3(SEL_THREADS), 0, stream, a);
}

}  // extern "C"
