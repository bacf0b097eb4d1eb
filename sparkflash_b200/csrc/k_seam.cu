// mHC seam kernels: the only place the residual stream is read and written.
//
// One seam sits between two sublayers.  It (1) finishes the previous sublayer: folds the W
// per-rank partial outputs in rank order (this is the reduce half of the all-reduce; the partials
// sit in this GPU's memory, pushed there by the producers), applies hc_post with that sublayer's
// post/comb coefficients and writes the new residual copies; (2) prepares the next sublayer:
// collapses the copies with the *previous* seam's `pre` coefficients (single-pass mHC shift
// rule), and accumulates the statistics the next coefficients need (predictor dots over the
// flattened hc*d row, sum of squares); a second small kernel finalises the coefficients (sigmoid /
// softmax / Sinkhorn), applies RMSNorm and emits the bf16 and per-32 FP8 activations.
//
// Reference behaviour: kernels/opt_seams_sm121.cu (opt_mhc_seam:122, opt_mhc_post:261),
// kernels/opt_rows_sm121.cu (mhc_seam:395, mhc_partials:566, mhc_tail:578, mhc_post:861),
// docs/architecture/02-mhc.md:40-181.
#include "k_common.cuh"

namespace sfb {

constexpr int SEAM_COLS = 64;     // columns per block in pass A
constexpr int SEAM_THREADS = 256; // 4 dot-parts x 64 columns
constexpr int MAX_HC = 4;
constexpr int MAX_MIX = 24;

struct SeamArgs {
  __nv_bfloat16* h;              // [n, hc, d] residual copies, updated in place
  const __nv_bfloat16* y[8];     // W partial sublayer outputs [n, d] (unused when !has_post)
  const uint32_t* flags[8];      // optional arrival flags (one per producer rank), may be null
  uint32_t epoch;                // value the flags must reach
  int W;
  int has_post;
  const float* coef_prev;        // [n, COEF] coefficients of the finished sublayer (post, comb)
  const float* a_pre;            // [n, a_stride] collapse coefficients (pre of the previous seam)
  int a_stride;
  const float* fn;               // [mix, hc*d] predictor, null for the final seam
  __nv_bfloat16* xhat;           // [n, d] collapsed rows (bf16)
  float* partials;               // [n, nblk, 2 + mix]
  __nv_bfloat16* ysum;           // optional [n, d]: folded sublayer output (taps / tests)
  Status* status;
  int n, hc, d, mix;
};

// coefficient record per row: pre[hc] | post[hc] | comb[hc*hc]
__host__ __device__ inline int coef_stride(int hc) { return 2 * hc + hc * hc; }

__global__ void __launch_bounds__(SEAM_THREADS) seam_a_kernel(SeamArgs a) {
  const int row = blockIdx.y;
  const int colb = blockIdx.x * SEAM_COLS;
  const int lcol = threadIdx.x & (SEAM_COLS - 1);
  const int part = threadIdx.x / SEAM_COLS;  // 0..3
  const int col = colb + lcol;
  const int hc = a.hc, d = a.d;
  __shared__ float red[8][MAX_MIX / 4 + 2];

  if (a.has_post && a.flags[0] != nullptr && threadIdx.x < a.W) {
    if (!wait_flag_ge(a.flags[threadIdx.x], a.epoch, 2000000000ull))
      status_set(a.status, ST_TIMEOUT, 1, threadIdx.x, (int)a.epoch);
  }
  if (a.has_post && a.flags[0] != nullptr) __syncthreads();

  float x[MAX_HC];
  float xh = 0.f, ss = 0.f;
  const bool live = col < d;
#pragma unroll
  for (int c = 0; c < MAX_HC; ++c)
    x[c] = (live && c < hc) ? bf16_to_f(a.h[((size_t)row * hc + c) * d + col]) : 0.f;
  __syncthreads();  // every part has read the old copies before part 0 overwrites them
  if (live) {
    __nv_bfloat16* hp = a.h + (size_t)row * hc * d + col;
    if (a.has_post) {
      float y = 0.f;
      for (int r = 0; r < a.W; ++r) y += bf16_to_f(a.y[r][(size_t)row * d + col]);
      y = bfr(y);
      if (a.ysum && part == 0) a.ysum[(size_t)row * d + col] = __float2bfloat16_rn(y);
      const float* cp = a.coef_prev + (size_t)row * coef_stride(hc);
      const float* post = cp + hc;
      const float* comb = cp + 2 * hc;
      float nx[MAX_HC];
#pragma unroll
      for (int k = 0; k < MAX_HC; ++k) {
        if (k < hc) {
          float v = post[k] * y;
          for (int j = 0; j < hc; ++j) v += comb[j * hc + k] * x[j];
          nx[k] = bfr(v);
        } else nx[k] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c) {
        x[c] = nx[c];
        if (c < hc && part == 0) hp[(size_t)c * d] = __float2bfloat16_rn(nx[c]);
      }
    }
    const float* ap = a.a_pre + (size_t)row * a.a_stride;
#pragma unroll
    for (int c = 0; c < MAX_HC; ++c)
      if (c < hc) { xh += ap[c] * x[c]; ss += x[c] * x[c]; }
    xh = bfr(xh);
    if (part == 0) a.xhat[(size_t)row * d + col] = __float2bfloat16_rn(xh);
  }
  // predictor dots: this thread covers mixes part*mq .. part*mq+mq-1
  const int mq = (a.mix + 3) / 4;
  float dots[MAX_MIX / 4];
#pragma unroll
  for (int i = 0; i < MAX_MIX / 4; ++i) {
    dots[i] = 0.f;
    const int m = part * mq + i;
    if (a.fn && i < mq && m < a.mix && live) {
      const float* f = a.fn + (size_t)m * hc * d + col;
#pragma unroll
      for (int c = 0; c < MAX_HC; ++c)
        if (c < hc) dots[i] += f[(size_t)c * d] * x[c];
    }
  }
  // reduce over the 64 columns: two warps per part
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < MAX_MIX / 4; ++i) dots[i] = warp_sum(dots[i]);
  float xh2 = warp_sum(xh * xh);
  ss = warp_sum(ss);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < MAX_MIX / 4; ++i) red[w][i] = dots[i];
    red[w][MAX_MIX / 4] = ss;
    red[w][MAX_MIX / 4 + 1] = xh2;
  }
  __syncthreads();
  float* out = a.partials + ((size_t)row * gridDim.x + blockIdx.x) * (2 + a.mix);
  if (threadIdx.x < a.mix) {
    const int m = threadIdx.x, p = m / mq, i = m % mq;
    out[2 + m] = red[2 * p][i] + red[2 * p + 1][i];
  }
  if (threadIdx.x == 32) out[0] = red[0][MAX_MIX / 4] + red[1][MAX_MIX / 4];          // sum x^2 (flat)
  if (threadIdx.x == 33) out[1] = red[0][MAX_MIX / 4 + 1] + red[1][MAX_MIX / 4 + 1];  // sum xhat^2
}

struct SeamBArgs {
  const float* partials;   // [n, nblk, 2+mix]
  int nblk;
  const __nv_bfloat16* xhat;  // [n, d]
  const float* norm_w;        // [d]
  const float* hc_scale;      // [3]
  const float* hc_base;       // [mix]
  float* coef;                // [n, coef_stride] out (null for the final seam)
  __nv_bfloat16* xn;          // [n, d] normalised bf16 (may be null)
  uint8_t* xq;                // [n, d] e4m3 (may be null)
  uint8_t* xs;                // [n, d/32] ue8m0, row-major
  uint8_t* xs_atom;           // optional scale atoms for the tensor-core arm (see atom_mode)
  int atom_mode;              // 0: rows of one atom set = tokens; 1: one atom set per token, token at row 0
  int n, hc, d, mix, iters;
  float norm_eps, hc_eps;
};

__global__ void __launch_bounds__(256) seam_b_kernel(SeamBArgs a) {
  const int row = blockIdx.y;
  __shared__ float tot[2 + MAX_MIX];
  const int nv = 2 + a.mix;
  {
    // 8 warps x 32 lanes: warp w sums values v = w, w+8, .. ; lanes stride the blocks, then a fixed
    // shuffle tree - the order depends only on nblk, never on the row count.
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int v = w; v < nv; v += 8) {
      const float* p = a.partials + (size_t)row * a.nblk * nv + v;
      float s = 0.f;
      for (int b = lane; b < a.nblk; b += 32) s += p[(size_t)b * nv];
      s = warp_sum(s);
      if (lane == 0) tot[v] = s;
    }
  }
  __syncthreads();
  const int hc = a.hc, d = a.d;
  if (blockIdx.x == 0 && a.coef != nullptr && threadIdx.x < 32) {
    // coefficients: lanes 0..hc*hc-1 own comb[j][k]; lanes < hc also own pre/post
    const int lane = threadIdx.x;
    const float rs = rsqrtf(tot[0] / (float)(hc * d) + a.norm_eps);
    float* cp = a.coef + (size_t)row * coef_stride(hc);
    if (lane < hc) {
      float m0 = tot[2 + lane] * rs, m1 = tot[2 + hc + lane] * rs;
      cp[lane] = 1.f / (1.f + expf(-(m0 * a.hc_scale[0] + a.hc_base[lane]))) + a.hc_eps;
      cp[hc + lane] = 2.f / (1.f + expf(-(m1 * a.hc_scale[1] + a.hc_base[hc + lane])));
    }
    // comb: hc x hc matrix, element (j,k) on lane j*hc+k  (hc is 1, 2 or 4)
    const int nel = hc * hc;
    const bool on = lane < nel;
    float v = on ? tot[2 + 2 * hc + lane] * rs * a.hc_scale[2] + a.hc_base[2 * hc + lane] : -1e30f;
    // row softmax over k (lanes with the same j are contiguous groups of hc)
    float mx = v;
    for (int o = 1; o < hc; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float e = on ? expf(v - mx) : 0.f;
    float rsum = e;
    for (int o = 1; o < hc; o <<= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, o);
    float c = e / rsum + a.hc_eps;
    // column pass
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
  // RMSNorm + quant of this block's 256 columns (one 32-group per warp)
  const int col = blockIdx.x * 256 + threadIdx.x;
  const float rsx = rsqrtf(tot[1] / (float)d + a.norm_eps);
  float v = 0.f;
  if (col < d) {
    v = bfr(bf16_to_f(a.xhat[(size_t)row * d + col]) * rsx * a.norm_w[col]);
    if (a.xn) a.xn[(size_t)row * d + col] = __float2bfloat16_rn(v);
  }
  if (a.xq) {
    uint8_t sc;
    uint8_t q = warp_quant_fp8(v, &sc);
    if (col < d) {
      a.xq[(size_t)row * d + col] = q;
      if ((threadIdx.x & 31) == 0) {
        a.xs[(size_t)row * (d / 32) + col / 32] = sc;
        if (a.xs_atom) {
          const int kb = col / 32, KB = d / 32;
          if (a.atom_mode == 0) a.xs_atom[sf_offset(row, kb, KB)] = sc;
          else a.xs_atom[(size_t)row * sf_bytes(1, KB) + sf_offset(0, kb, KB)] = sc;
        }
      }
    }
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_seam_nblk(int d) { return (d + SEAM_COLS - 1) / SEAM_COLS; }
int sfb_coef_stride(int hc) { return coef_stride(hc); }

// y_ptrs / flag_ptrs: host arrays of W device pointers (flag_ptrs may be null).
int sfb_seam(void* h, const void* const* y_ptrs, const void* const* flag_ptrs, uint32_t epoch, int W,
             int has_post, const float* coef_prev, const float* a_pre, int a_stride, const float* fn,
             void* xhat, float* partials, void* ysum, const float* norm_w, const float* hc_scale,
             const float* hc_base, float* coef_out, void* xn, void* xq, void* xs, void* xs_atom, int atom_mode,
             void* status, int n, int hc, int d, int iters, float norm_eps, float hc_eps, cudaStream_t stream) {
  if (hc > MAX_HC || W > 8 || (hc & (hc - 1))) return (int)cudaErrorInvalidValue;
  SeamArgs a{};
  a.h = (__nv_bfloat16*)h;
  for (int r = 0; r < 8; ++r) {
    a.y[r] = (has_post && r < W) ? (const __nv_bfloat16*)y_ptrs[r] : nullptr;
    a.flags[r] = (has_post && flag_ptrs && r < W) ? (const uint32_t*)flag_ptrs[r] : nullptr;
  }
  a.epoch = epoch; a.W = W; a.has_post = has_post; a.coef_prev = coef_prev; a.a_pre = a_pre;
  a.a_stride = a_stride; a.fn = fn; a.xhat = (__nv_bfloat16*)xhat; a.partials = partials;
  a.ysum = (__nv_bfloat16*)ysum; a.status = (Status*)status; a.n = n; a.hc = hc; a.d = d;
  a.mix = (2 + hc) * hc;
  const int nblk = sfb_seam_nblk(d);
  seam_a_kernel<<<dim3(nblk, n), SEAM_THREADS, 0, stream>>>(a);
  SeamBArgs b{};
  b.partials = partials; b.nblk = nblk; b.xhat = (const __nv_bfloat16*)xhat; b.norm_w = norm_w;
  b.hc_scale = hc_scale; b.hc_base = hc_base; b.coef = fn ? coef_out : nullptr;
  b.xn = (__nv_bfloat16*)xn; b.xq = (uint8_t*)xq; b.xs = (uint8_t*)xs; b.xs_atom = (uint8_t*)xs_atom;
  b.atom_mode = atom_mode; b.n = n; b.hc = hc; b.d = d;
  b.mix = a.mix; b.iters = iters; b.norm_eps = norm_eps; b.hc_eps = hc_eps;
  seam_b_kernel<<<dim3((d + 255) / 256, n), 256, 0, stream>>>(b);
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
