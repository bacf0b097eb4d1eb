// mHC seam kernels: the only place the residual stream is read and written.
//
// One seam sits between two sublayers and is split in two launches:
//
//  * seam_fold (critical path): finishes the previous sublayer - folds the W per-rank partial outputs in
//    rank order (the reduce half of the all-reduce; the partials sit in this GPU's memory, pushed there
//    by the producers), applies hc_post with that sublayer's post/comb coefficients, writes the new
//    residual copies - and prepares the next one: collapse with the previous seam's `pre` (single-pass
//    mHC shift rule), RMSNorm, bf16 + per-32 FP8 activations.  One thread-block cluster per row; the
//    row's sum of squares is combined through distributed shared memory in CTA-rank order.
//  * seam_coef (off the critical path, runs beside the sublayer's GEMMs): predictor dots over the
//    flattened hc*d row of the *new* residual, sigmoid / softmax / Sinkhorn -> (pre, post, comb) that
//    the next seam consumes.
//
// Reference behaviour: kernels/opt_seams_sm121.cu (opt_mhc_seam:122, opt_mhc_post:261),
// kernels/opt_rows_sm121.cu (mhc_seam:395, mhc_partials:566, mhc_tail:578, mhc_post:861),
// docs/architecture/02-mhc.md:40-181.
#include <cooperative_groups.h>

#include "k_common.cuh"

namespace cg = cooperative_groups;

namespace sfb {

constexpr int MAX_HC = 4;
constexpr int MAX_MIX = 24;
constexpr int FOLD_CLUSTER = 8;
constexpr int FOLD_THREADS = 320;
constexpr int FOLD_MAX_IT = 4;     // columns per thread: d <= 8 * 320 * 4
constexpr int COEF_COLS = 32;      // columns per block in seam_coef
constexpr int COEF_THREADS = 256;  // 8 predictor parts x 32 columns (one warp per part)
constexpr int COEF_PARTS = 8;
constexpr int MAX_MQ = 3;

// coefficient record per row: pre[hc] | post[hc] | comb[hc*hc]
__host__ __device__ inline int coef_stride(int hc) { return 2 * hc + hc * hc; }

struct FoldArgs {
  __nv_bfloat16* h;              // [n, hc, d] residual copies, updated in place
  const __nv_bfloat16* y[8];     // W partial sublayer outputs [n, d] (unused when !has_post)
  const uint32_t* flags[8];      // optional arrival flags (one per producer rank), may be null
  const uint32_t* epoch_ptr;     // device step counter (may be null: epoch_add alone)
  uint32_t epoch_add;            // flags must reach *epoch_ptr + epoch_add
  int W;
  int has_post;
  const float* coef_prev;        // [n, COEF] coefficients of the finished sublayer (post, comb)
  const float* a_pre;            // [n, a_stride] collapse coefficients (pre of the previous seam)
  int a_stride;
  __nv_bfloat16* ysum;           // optional [n, d]: folded sublayer output (tests)
  const float* norm_w;           // [d]
  __nv_bfloat16* xn;             // [n, d] normalised bf16 (may be null)
  uint8_t* xq;                   // [n, d] e4m3 (may be null)
  uint8_t* xs;                   // [n, d/32] ue8m0, row-major
  float* hss;                    // optional [n]: sum of squares of the row's new residual copies (all hc*d values), for the
                                 //   many-row coefficient path
  uint8_t* xs_atom;              // optional scale atoms for the tensor-core arm (see atom_mode)
  int atom_mode;                 // 0: rows of one atom set = tokens; 1: one atom set per token, token at row 0
  Status* status;
  uint64_t wait_ns;              // time limit of the flag wait
  int n, hc, d;
  float norm_eps;
};

__global__ void __cluster_dims__(FOLD_CLUSTER, 1, 1) __launch_bounds__(FOLD_THREADS) seam_fold_kernel(FoldArgs a) {
  cg::cluster_group cluster = cg::this_cluster();
  const int row = blockIdx.y;
  const int rank = blockIdx.x;  // == cluster rank
  const int hc = a.hc, d = a.d;
  const int cpc = d / FOLD_CLUSTER;            // columns of this CTA (multiple of 32)
  const int c_lo = rank * cpc;
  __shared__ float part_ss, part_hss;
  __shared__ float sh[32];
  pdl_launch_dependents();
  pdl_wait();
  float hsq = 0.f;

  if (a.has_post && a.flags[0] != nullptr) {
    const uint32_t want = (a.epoch_ptr ? *a.epoch_ptr : 0u) + a.epoch_add;
    if (threadIdx.x < a.W && !wait_flag_ge(a.flags[threadIdx.x], want, a.wait_ns))
      status_set(a.status, ST_TIMEOUT, 1, threadIdx.x, (int)want);
    __syncthreads();
  }
  float post[MAX_HC], comb[MAX_HC * MAX_HC], ap[MAX_HC];
#pragma unroll
  for (int c = 0; c < MAX_HC; ++c) {
    ap[c] = c < hc ? a.a_pre[(size_t)row * a.a_stride + c] : 0.f;
    post[c] = 0.f;
  }
  if (a.has_post) {
    const float* cp = a.coef_prev + (size_t)row * coef_stride(hc);
#pragma unroll
    for (int c = 0; c < MAX_HC; ++c)
      if (c < hc) post[c] = cp[hc + c];
#pragma unroll
    for (int i = 0; i < MAX_HC * MAX_HC; ++i)
      if (i < hc * hc) comb[i] = cp[2 * hc + i];
  }
  float xh[FOLD_MAX_IT];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < FOLD_MAX_IT; ++it) {
    xh[it] = 0.f;
    const int lc = it * FOLD_THREADS + threadIdx.x;
    if (lc < cpc) {
      const int col = c_lo + lc;
      __nv_bfloat16* hp = a.h + (size_t)row * hc * d + col;
      float x[MAX_HC];
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c) x[c] = c < hc ? bf16_to_f(hp[(size_t)c * d]) : 0.f;
      if (a.has_post) {
        float y = 0.f;
        for (int r = 0; r < a.W; ++r) y += bf16_to_f(a.y[r][(size_t)row * d + col]);
        y = bfr(y);
        if (a.ysum) a.ysum[(size_t)row * d + col] = __float2bfloat16_rn(y);
        float nx[MAX_HC];
#pragma unroll
        for (int k = 0; k < MAX_HC; ++k) {
          float v = post[k] * y;
#pragma unroll
          for (int j = 0; j < MAX_HC; ++j)
            if (j < hc && k < hc) v += comb[j * hc + k] * x[j];
          nx[k] = bfr(v);
        }
#pragma unroll
        for (int c = 0; c < MAX_HC; ++c) {
          if (c < hc) { x[c] = nx[c]; hp[(size_t)c * d] = __float2bfloat16_rn(nx[c]); }
        }
      }
      float v = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c)
        if (c < hc) { v += ap[c] * x[c]; hsq += x[c] * x[c]; }
      v = bfr(v);
      xh[it] = v;
      ss += v * v;
    }
  }
  ss = block_sum(ss, sh);
  if (a.hss) hsq = block_sum(hsq, sh);
  if (threadIdx.x == 0) { part_ss = ss; part_hss = hsq; }
  cluster.sync();
  float total = 0.f;
  for (int r = 0; r < FOLD_CLUSTER; ++r) total += *cluster.map_shared_rank(&part_ss, r);
  if (a.hss && rank == 0 && threadIdx.x == 0) {
    float t2 = 0.f;
    for (int r = 0; r < FOLD_CLUSTER; ++r) t2 += *cluster.map_shared_rank(&part_hss, r);
    a.hss[row] = t2;
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
  const float rsx = rsqrtf(total / (float)d + a.norm_eps);
  const int KB = d / 32;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int it = 0; it < FOLD_MAX_IT; ++it) {
    const int lc = it * FOLD_THREADS + threadIdx.x;
    // whole warps are in or out of range (cpc and FOLD_THREADS are multiples of 32)
    if (lc - lane < cpc) {
      const int col = c_lo + lc;
      const float v = bfr(xh[it] * rsx * a.norm_w[col]);
      if (a.xn) a.xn[(size_t)row * d + col] = __float2bfloat16_rn(v);
      if (a.xq) {
        uint8_t sc;
        const uint8_t qv = warp_quant_fp8(v, &sc);
        a.xq[(size_t)row * d + col] = qv;
        if (lane == 0) {
          a.xs[(size_t)row * KB + col / 32] = sc;
          if (a.xs_atom) {
            if (a.atom_mode == 0) a.xs_atom[sf_offset(row, col / 32, KB)] = sc;
            else a.xs_atom[(size_t)row * sf_bytes(1, KB) + sf_offset(0, col / 32, KB)] = sc;
          }
        }
      }
    }
  }
}

// Many-row variant of seam_fold: one block per row, no cluster.  A thread owns groups of four consecutive columns, eight
// lanes share a 32-column scale group; the row sums go through one block reduction.  Same arithmetic per element as the
// cluster kernel (the sums of squares are added in a different order, so the normalised values may differ in the last bit).
constexpr int FOLDR_THREADS = 256;
constexpr int FOLDR_MAX_IT = 8;      // d <= 256 * 4 * 8

__global__ void __launch_bounds__(FOLDR_THREADS) seam_fold_rows_kernel(FoldArgs a) {
  const int row = blockIdx.x;
  const int hc = a.hc, d = a.d;
  __shared__ float sh[32];
  pdl_launch_dependents();
  pdl_wait();
  if (a.has_post && a.flags[0] != nullptr) {
    const uint32_t want = (a.epoch_ptr ? *a.epoch_ptr : 0u) + a.epoch_add;
    if (threadIdx.x < a.W && !wait_flag_ge(a.flags[threadIdx.x], want, a.wait_ns))
      status_set(a.status, ST_TIMEOUT, 2, threadIdx.x, (int)want);
    __syncthreads();
  }
  float post[MAX_HC], comb[MAX_HC * MAX_HC], ap[MAX_HC];
#pragma unroll
  for (int c = 0; c < MAX_HC; ++c) {
    ap[c] = c < hc ? a.a_pre[(size_t)row * a.a_stride + c] : 0.f;
    post[c] = 0.f;
  }
  if (a.has_post) {
    const float* cp = a.coef_prev + (size_t)row * coef_stride(hc);
#pragma unroll
    for (int c = 0; c < MAX_HC; ++c)
      if (c < hc) post[c] = cp[hc + c];
#pragma unroll
    for (int i = 0; i < MAX_HC * MAX_HC; ++i)
      if (i < hc * hc) comb[i] = cp[2 * hc + i];
  }
  float xh[FOLDR_MAX_IT][4];
  float ss = 0.f, hsq = 0.f;
#pragma unroll
  for (int it = 0; it < FOLDR_MAX_IT; ++it) {
    const int col = (it * FOLDR_THREADS + threadIdx.x) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) xh[it][e] = 0.f;
    if (col < d) {
      float x[MAX_HC][4];
      __nv_bfloat16* hp = a.h + (size_t)row * hc * d + col;
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c) {
        if (c < hc) {
          const uint2 u = *reinterpret_cast<const uint2*>(hp + (size_t)c * d);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
          x[c][0] = f0.x; x[c][1] = f0.y; x[c][2] = f1.x; x[c][3] = f1.y;
        } else {
          x[c][0] = x[c][1] = x[c][2] = x[c][3] = 0.f;
        }
      }
      if (a.has_post) {
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < a.W; ++r) {
          const uint2 u = *reinterpret_cast<const uint2*>(a.y[r] + (size_t)row * d + col);
          const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          const float2 f0 = __bfloat1622float2(y2[0]), f1 = __bfloat1622float2(y2[1]);
          y[0] += f0.x; y[1] += f0.y; y[2] += f1.x; y[3] += f1.y;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = bfr(y[e]);
        if (a.ysum) {
          __nv_bfloat16* yo = a.ysum + (size_t)row * d + col;
#pragma unroll
          for (int e = 0; e < 4; ++e) yo[e] = __float2bfloat16_rn(y[e]);
        }
        float nx[MAX_HC][4];
#pragma unroll
        for (int k = 0; k < MAX_HC; ++k) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = post[k] * y[e];
#pragma unroll
            for (int j = 0; j < MAX_HC; ++j)
              if (j < hc && k < hc) v += comb[j * hc + k] * x[j][e];
            nx[k][e] = bfr(v);
          }
        }
#pragma unroll
        for (int c = 0; c < MAX_HC; ++c) {
          if (c < hc) {
            __nv_bfloat162 o2[2] = {__floats2bfloat162_rn(nx[c][0], nx[c][1]), __floats2bfloat162_rn(nx[c][2], nx[c][3])};
            *reinterpret_cast<uint2*>(hp + (size_t)c * d) = *reinterpret_cast<uint2*>(o2);
#pragma unroll
            for (int e = 0; e < 4; ++e) x[c][e] = nx[c][e];
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = 0.f;
#pragma unroll
        for (int c = 0; c < MAX_HC; ++c)
          if (c < hc) { v += ap[c] * x[c][e]; hsq += x[c][e] * x[c][e]; }
        v = bfr(v);
        xh[it][e] = v;
        ss += v * v;
      }
    }
  }
  ss = block_sum(ss, sh);
  if (a.hss) {
    hsq = block_sum(hsq, sh);
    if (threadIdx.x == 0) a.hss[row] = hsq;
  }
  const float rsx = rsqrtf(ss / (float)d + a.norm_eps);
  const int KB = d / 32;
#pragma unroll
  for (int it = 0; it < FOLDR_MAX_IT; ++it) {
    const int col = (it * FOLDR_THREADS + threadIdx.x) * 4;
    // whole warps are in or out of range (d is a multiple of 128)
    if (col - (int)(threadIdx.x & 31) * 4 < d) {
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        v[e] = col < d ? bfr(xh[it][e] * rsx * a.norm_w[col + e]) : 0.f;
        amax = fmaxf(amax, fabsf(v[e]));
      }
      if (a.xn && col < d) {
        __nv_bfloat162 o2[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
        *reinterpret_cast<uint2*>(a.xn + (size_t)row * d + col) = *reinterpret_cast<uint2*>(o2);
      }
      if (a.xq) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        if (col < d) {
          const uint8_t sc = act_scale_code_fp8(amax);
          const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
          uint32_t q4 = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) q4 |= (uint32_t)enc_e4m3(v[e] * inv) << (8 * e);
          *reinterpret_cast<uint32_t*>(a.xq + (size_t)row * d + col) = q4;
          if ((threadIdx.x & 7) == 0) {
            a.xs[(size_t)row * KB + col / 32] = sc;
            if (a.xs_atom) {
              if (a.atom_mode == 0) a.xs_atom[sf_offset(row, col / 32, KB)] = sc;
              else a.xs_atom[(size_t)row * sf_bytes(1, KB) + sf_offset(0, col / 32, KB)] = sc;
            }
          }
        }
      }
    }
  }
}

struct CoefArgs {
  const __nv_bfloat16* h;        // [n, hc, d] (already folded)
  const float* fn;               // [mix, hc*d]
  const float* hc_scale;         // [3]
  const float* hc_base;          // [mix]
  float* partials;               // [n, nblk, 1 + mix]
  unsigned int* tickets;         // [n], zero between launches
  float* coef;                   // [n, coef_stride]
  int n, hc, d, mix, iters;
  float norm_eps, hc_eps;
  int rb;                        // rows per block
};

__global__ void __launch_bounds__(COEF_THREADS) seam_coef_kernel(CoefArgs a) {
  // a block owns 32 columns of the flattened row for `rb` consecutive rows: its slice of the predictor matrix is loaded
  // once and stays in registers while the rows stream through (many-row steps would otherwise re-read it per row)
  const int lcol = threadIdx.x & (COEF_COLS - 1);
  const int part = threadIdx.x / COEF_COLS;  // = warp
  const int col = blockIdx.x * COEF_COLS + lcol;
  const int hc = a.hc, d = a.d, lane = threadIdx.x & 31;
  __shared__ float red[COEF_PARTS][MAX_MQ + 1];
  __shared__ float tot[1 + MAX_MIX];
  __shared__ int is_last;
  const bool live = col < d;
  const int mq = (a.mix + COEF_PARTS - 1) / COEF_PARTS;
  float fv[MAX_MQ][MAX_HC];
#pragma unroll
  for (int i = 0; i < MAX_MQ; ++i) {
    const int m = part * mq + i;
#pragma unroll
    for (int c = 0; c < MAX_HC; ++c)
      fv[i][c] = (i < mq && m < a.mix && live && c < hc) ? a.fn[((size_t)m * hc + c) * d + col] : 0.f;
  }
  const int row_end = min(a.n, (int)(blockIdx.y + 1) * a.rb);
  for (int row = blockIdx.y * a.rb; row < row_end; ++row) {
    float x[MAX_HC];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_HC; ++c) {
      x[c] = (live && c < hc) ? bf16_to_f(a.h[((size_t)row * hc + c) * d + col]) : 0.f;
      ss += x[c] * x[c];
    }
    float dots[MAX_MQ];
#pragma unroll
    for (int i = 0; i < MAX_MQ; ++i) {
      dots[i] = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c)
        if (c < hc) dots[i] += fv[i][c] * x[c];
    }
#pragma unroll
    for (int i = 0; i < MAX_MQ; ++i) dots[i] = warp_sum(dots[i]);
    ss = warp_sum(ss);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < MAX_MQ; ++i) red[part][i] = dots[i];
      red[part][MAX_MQ] = ss;
    }
    __syncthreads();
    const int nv = 1 + a.mix;
    float* out = a.partials + ((size_t)row * gridDim.x + blockIdx.x) * nv;
    if (threadIdx.x < a.mix) out[1 + threadIdx.x] = red[threadIdx.x / mq][threadIdx.x % mq];
    if (threadIdx.x == 32) out[0] = red[0][MAX_MQ];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned int prev = atomicAdd(&a.tickets[row], 1u);
      is_last = prev == gridDim.x - 1;
      if (is_last) a.tickets[row] = 0;
    }
    __syncthreads();
    if (!is_last) continue;
    __threadfence();
    {  // totals in a fixed order (independent of which block runs the tail)
      const int w = threadIdx.x >> 5;
      for (int v = w; v < nv; v += 8) {
        const float* p = a.partials + (size_t)row * gridDim.x * nv + v;
        float s = 0.f;
        for (int b = lane; b < (int)gridDim.x; b += 32) s += __ldcg(p + (size_t)b * nv);
        s = warp_sum(s);
        if (lane == 0) tot[v] = s;
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // lanes 0..hc*hc-1 own comb[j][k]; lanes < hc also own pre/post
      const float rs = rsqrtf(tot[0] / (float)(hc * d) + a.norm_eps);
      float* cp = a.coef + (size_t)row * coef_stride(hc);
      if (lane < hc) {
        float m0 = tot[1 + lane] * rs, m1 = tot[1 + hc + lane] * rs;
        cp[lane] = 1.f / (1.f + expf(-(m0 * a.hc_scale[0] + a.hc_base[lane]))) + a.hc_eps;
        cp[hc + lane] = 2.f / (1.f + expf(-(m1 * a.hc_scale[1] + a.hc_base[hc + lane])));
      }
      const int nel = hc * hc;
      const bool on = lane < nel;
      float v = on ? tot[1 + 2 * hc + lane] * rs * a.hc_scale[2] + a.hc_base[2 * hc + lane] : -1e30f;
      float mx = v;
      for (int o = 1; o < hc; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float e = on ? expf(v - mx) : 0.f;
      float rsum = e;
      for (int o = 1; o < hc; o <<= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
      float c = e / rsum + a.hc_eps;
      float csum = c;
      for (int o = hc; o < nel; o <<= 1) csum += __shfl_xor_sync(0xffffffffu, csum, o);
      c = c / (csum + a.hc_eps);
      for (int it = 1; it < a.iters; ++it) {
        float r2 = c;
        for (int o = 1; o < hc; o <<= 1) r2 += __shfl_xor_sync(0xffffffffu, r2, o);
        c = c / (r2 + a.hc_eps);
        float c2 = c;
        for (int o = hc; o < nel; o <<= 1) c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        c = c / (c2 + a.hc_eps);
      }
      if (on) cp[2 * hc + lane] = c;
    }
    __syncthreads();   // the tail's shared totals are not overwritten while a lane still reads them
  }
}

// Many-row coefficient path, last step: the predictor dots come from a bf16 tensor-core GEMM of the flattened residual
// rows against the predictor matrix split in two bf16 terms (rows 0..mix-1 = high parts, mix..2*mix-1 = low parts), the
// sum of squares from seam_fold.  One warp per row adds the two terms and runs the sigmoid / softmax / Sinkhorn tail.
struct CoefFinishArgs {
  const float* acc;              // [n, acc_stride]: column m = high-term dot of mix m, column mix + m = low-term dot
  int acc_stride;
  const float* hss;              // [n]
  const float* hc_scale;
  const float* hc_base;
  float* coef;                   // [n, coef_stride]
  int n, hc, d, mix, iters;
  float norm_eps, hc_eps;
};

__global__ void __launch_bounds__(128) seam_coef_finish_kernel(CoefFinishArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= a.n) return;
  const int hc = a.hc;
  const float* ac = a.acc + (size_t)row * a.acc_stride;
  auto tot = [&](int m) { return ac[m] + ac[a.mix + m]; };
  const float rs = rsqrtf(a.hss[row] / (float)(hc * a.d) + a.norm_eps);
  float* cp = a.coef + (size_t)row * coef_stride(hc);
  if (lane < hc) {
    const float m0 = tot(lane) * rs, m1 = tot(hc + lane) * rs;
    cp[lane] = 1.f / (1.f + expf(-(m0 * a.hc_scale[0] + a.hc_base[lane]))) + a.hc_eps;
    cp[hc + lane] = 2.f / (1.f + expf(-(m1 * a.hc_scale[1] + a.hc_base[hc + lane])));
  }
  const int nel = hc * hc;
  const bool on = lane < nel;
  float v = on ? tot(2 * hc + lane) * rs * a.hc_scale[2] + a.hc_base[2 * hc + lane] : -1e30f;
  float mx = v;
  for (int o = 1; o < hc; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float e = on ? expf(v - mx) : 0.f;
  float rsum = e;
  for (int o = 1; o < hc; o <<= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
  float c = e / rsum + a.hc_eps;
  float csum = c;
  for (int o = hc; o < nel; o <<= 1) csum += __shfl_xor_sync(0xffffffffu, csum, o);
  c = c / (csum + a.hc_eps);
  for (int it = 1; it < a.iters; ++it) {
    float r2 = c;
    for (int o = 1; o < hc; o <<= 1) r2 += __shfl_xor_sync(0xffffffffu, r2, o);
    c = c / (r2 + a.hc_eps);
    float c2 = c;
    for (int o = hc; o < nel; o <<= 1) c2 += __shfl_xor_sync(0xffffffffu, c2, o);
    c = c / (c2 + a.hc_eps);
  }
  if (on) cp[2 * hc + lane] = c;
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_seam_nblk(int d) { return (d + COEF_COLS - 1) / COEF_COLS; }
int sfb_coef_stride(int hc) { return coef_stride(hc); }

// Critical-path half of a seam. y_ptrs / flag_ptrs: host arrays of W device pointers (flag_ptrs may be null).
int sfb_seam_fold(void* h, const void* const* y_ptrs, const void* const* flag_ptrs, const void* epoch_ptr,
                  uint32_t epoch_add, uint64_t wait_ns, int W,
                  int has_post, const float* coef_prev, const float* a_pre, int a_stride, void* ysum,
                  const float* norm_w, void* xn, void* xq, void* xs, void* xs_atom, int atom_mode, void* status,
                  int n, int hc, int d, float norm_eps, float* hss, cudaStream_t stream) {
  if (hc > MAX_HC || W > 8 || (hc & (hc - 1)) || d % (32 * FOLD_CLUSTER) || d > FOLD_CLUSTER * FOLD_THREADS * FOLD_MAX_IT)
    return (int)cudaErrorInvalidValue;
  FoldArgs a{};
  a.h = (__nv_bfloat16*)h;
  for (int r = 0; r < 8; ++r) {
    a.y[r] = (has_post && r < W) ? (const __nv_bfloat16*)y_ptrs[r] : nullptr;
    a.flags[r] = (has_post && flag_ptrs && r < W) ? (const uint32_t*)flag_ptrs[r] : nullptr;
  }
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns ? wait_ns : 2000000000ull; a.W = W; a.has_post = has_post; a.coef_prev = coef_prev; a.a_pre = a_pre; a.a_stride = a_stride;
  a.ysum = (__nv_bfloat16*)ysum; a.norm_w = norm_w; a.xn = (__nv_bfloat16*)xn; a.xq = (uint8_t*)xq;
  a.xs = (uint8_t*)xs; a.xs_atom = (uint8_t*)xs_atom; a.atom_mode = atom_mode; a.status = (Status*)status;
  a.n = n; a.hc = hc; a.d = d; a.norm_eps = norm_eps; a.hss = hss;
  if (n > 128 && d % 128 == 0 && d <= FOLDR_THREADS * 4 * FOLDR_MAX_IT)       // many rows: one block per row
    return (int)sfb_launch(seam_fold_rows_kernel, dim3(n), dim3(FOLDR_THREADS), 0, stream, a);
  return (int)sfb_launch(seam_fold_kernel, dim3(FOLD_CLUSTER, n), dim3(FOLD_THREADS), 0, stream, a);
}

// Coefficient half: reads the folded residual, writes (pre, post, comb) for the next seam.
int sfb_seam_coef(const void* h, const float* fn, const float* hc_scale, const float* hc_base, float* partials,
                  unsigned int* tickets, float* coef_out, int n, int hc, int d, int iters, float norm_eps,
                  float hc_eps, cudaStream_t stream) {
  if (hc > MAX_HC || (hc & (hc - 1)) || !tickets) return (int)cudaErrorInvalidValue;
  const int rb = n <= 32 ? 1 : (n <= 256 ? 4 : 16);
  CoefArgs a{(const __nv_bfloat16*)h, fn, hc_scale, hc_base, partials, tickets, coef_out, n, hc, d, (2 + hc) * hc,
             iters, norm_eps, hc_eps, rb};
  seam_coef_kernel<<<dim3(sfb_seam_nblk(d), (n + rb - 1) / rb), COEF_THREADS, 0, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

int sfb_seam_coef_finish(const float* acc, int acc_stride, const float* hss, const float* hc_scale, const float* hc_base,
                         float* coef_out, int n, int hc, int d, int iters, float norm_eps, float hc_eps, cudaStream_t stream) {
  if (hc > MAX_HC || (hc & (hc - 1)) || hc * hc > 32) return (int)cudaErrorInvalidValue;
  CoefFinishArgs a{acc, acc_stride, hss, hc_scale, hc_base, coef_out, n, hc, d, (2 + hc) * hc, iters, norm_eps, hc_eps};
  return (int)sfb_launch(seam_coef_finish_kernel, dim3((n + 3) / 4), dim3(128), 0, stream, a);
}

}  // extern "C"
