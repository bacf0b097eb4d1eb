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

// The fold's sums are written with explicit multiply-add intrinsics: the compiler may contract `a * b + c * d` either way
// round, and the three fold kernels (cluster, rows, rows through bulk copies) must produce the same bits for a row.
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
  int rs_rows;                   // > 0: the partials were reduced by a two-shot exchange - row t has ONE part, in y[t / rs_rows] at
                                 //      row rs_rows + t % rs_rows (the W flags are still waited for); many-row kernels only
};

// HC > 0 fixes the number of residual copies at compile time (the coefficient arrays then live in registers; indexed with a
// run-time hc they sat in local memory and the fold of a row took three times as long); HC = 0 reads it from the arguments.
template <int HC>
__global__ void __cluster_dims__(FOLD_CLUSTER, 1, 1) __launch_bounds__(FOLD_THREADS) seam_fold_kernel(FoldArgs a) {
  cg::cluster_group cluster = cg::this_cluster();
  const int row = blockIdx.y;
  const int rank = blockIdx.x;  // == cluster rank
  const int hc = HC > 0 ? HC : a.hc, d = a.d;
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
          float v = __fmul_rn(post[k], y);
#pragma unroll
          for (int j = 0; j < MAX_HC; ++j)
            if (j < hc && k < hc) v = __fmaf_rn(comb[j * hc + k], x[j], v);
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
        if (c < hc) { v = __fmaf_rn(ap[c], x[c], v); hsq = __fmaf_rn(x[c], x[c], hsq); }
      v = bfr(v);
      xh[it] = v;
      ss = __fmaf_rn(v, v, ss);
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

template <int HC>
__global__ void __launch_bounds__(FOLDR_THREADS) seam_fold_rows_kernel(FoldArgs a) {
  const int row = blockIdx.x;
  const int hc = HC > 0 ? HC : a.hc, d = a.d;
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
        const int nparts = a.rs_rows > 0 ? 1 : a.W;
        for (int r = 0; r < nparts; ++r) {
          const __nv_bfloat16* yr = a.rs_rows > 0 ? a.y[row / a.rs_rows] + (size_t)(a.rs_rows + row % a.rs_rows) * d : a.y[r] + (size_t)row * d;
          const uint2 u = *reinterpret_cast<const uint2*>(yr + col);
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
            float v = __fmul_rn(post[k], y[e]);
#pragma unroll
            for (int j = 0; j < MAX_HC; ++j)
              if (j < hc && k < hc) v = __fmaf_rn(comb[j * hc + k], x[j][e], v);
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
          if (c < hc) { v = __fmaf_rn(ap[c], x[c][e], v); hsq = __fmaf_rn(x[c][e], x[c][e], hsq); }
        v = bfr(v);
        xh[it][e] = v;
        ss = __fmaf_rn(v, v, ss);
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

// Many-row seam with the row moved by bulk copies: the row's residual copies (hc x d bf16, contiguous) and the W partial
// outputs arrive in shared memory as one asynchronous copy each, the fold and the normalisation run from there, and the new
// residual, the folded output, the normalised row, its FP8 codes and scale bytes leave as one bulk copy each.  With 8-byte
// loads per thread and the in-place stores between them the register version kept too few bytes in flight (a third of the
// copy bandwidth).  Same arithmetic, in the same order, as seam_fold_rows_kernel: the outputs are bit-identical.
__device__ __forceinline__ uint32_t fold_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool fold_mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {      // bounded: several hundred milliseconds
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(fold_smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void fold_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(fold_smem_u32(dst)), "l"(src), "r"(bytes), "r"(fold_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fold_bulk_store(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(fold_smem_u32(src_smem)), "r"(bytes) : "memory");
}

// phase marks of the bulk-copy fold (measurement builds): eight %globaltimer words per row of the last launch -
// entry, dependencies met, row landed, fold done, sums done, outputs staged, copies read
#ifdef SFB_KERNEL_MARKS
__device__ unsigned long long g_fold_marks[4096 * 8];
#define FOLD_MARK(slot) do { if (threadIdx.x == 0 && blockIdx.x < 4096) g_fold_marks[blockIdx.x * 8 + (slot)] = globaltimer_ns(); } while (0)
#else
#define FOLD_MARK(slot) do { } while (0)
#endif

template <int HC>
__global__ void __launch_bounds__(FOLDR_THREADS) seam_fold_rows_bulk_kernel(FoldArgs a) {
  extern __shared__ __align__(128) uint8_t fold_sm[];
  FOLD_MARK(0);
  const int row = blockIdx.x;
  const int hc = HC > 0 ? HC : a.hc, d = a.d;
  const int W = a.has_post ? (a.rs_rows > 0 ? 1 : a.W) : 0;      // parts of the row in shared memory
  const int KB = d / 32;
  __nv_bfloat16* sh_h = reinterpret_cast<__nv_bfloat16*>(fold_sm);
  __nv_bfloat16* sh_y = sh_h + (size_t)hc * d;
  __nv_bfloat16* sh_xn = sh_y + (size_t)W * d;
  uint8_t* sh_xq = reinterpret_cast<uint8_t*>(sh_xn + d);
  uint8_t* sh_xs = sh_xq + d;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sh_xs + ((KB + 15) & ~15));
  __shared__ float sh[32];
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(fold_smem_u32(bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  pdl_wait();
  if (a.has_post && a.flags[0] != nullptr) {
    const uint32_t want = (a.epoch_ptr ? *a.epoch_ptr : 0u) + a.epoch_add;
    if (threadIdx.x < a.W && !wait_flag_ge(a.flags[threadIdx.x], want, a.wait_ns))
      status_set(a.status, ST_TIMEOUT, 2, threadIdx.x, (int)want);
  }
  __syncthreads();
  FOLD_MARK(1);
  if (threadIdx.x < 32 && elect_one()) {
    asm volatile("fence.proxy.async;" ::: "memory");      // the partials were published to the generic proxy; the copies read them
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fold_smem_u32(bar)), "r"((uint32_t)((hc + W) * d * 2)) : "memory");
    fold_bulk_load(sh_h, a.h + (size_t)row * hc * d, (uint32_t)(hc * d * 2), bar);
    if (a.rs_rows > 0 && W) fold_bulk_load(sh_y, a.y[row / a.rs_rows] + (size_t)(a.rs_rows + row % a.rs_rows) * d, (uint32_t)(d * 2), bar);
    else for (int r = 0; r < W; ++r) fold_bulk_load(sh_y + (size_t)r * d, a.y[r] + (size_t)row * d, (uint32_t)(d * 2), bar);
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
  const bool landed = __syncthreads_and(fold_mbar_wait(bar, 0) ? 1 : 0) != 0;
  if (!landed) {
    if (threadIdx.x == 0) status_set(a.status, ST_TIMEOUT, 3, row, 0);
    return;
  }
  FOLD_MARK(2);
  float xh[FOLDR_MAX_IT][4];
  float ss = 0.f, hsq = 0.f;
#pragma unroll
  for (int it = 0; it < FOLDR_MAX_IT; ++it) {
    const int col = (it * FOLDR_THREADS + threadIdx.x) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) xh[it][e] = 0.f;
    if (col < d) {
      float x[MAX_HC][4];
      __nv_bfloat16* hp = sh_h + col;
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
        for (int r = 0; r < W; ++r) {
          const uint2 u = *reinterpret_cast<const uint2*>(sh_y + (size_t)r * d + col);
          const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          const float2 f0 = __bfloat1622float2(y2[0]), f1 = __bfloat1622float2(y2[1]);
          y[0] += f0.x; y[1] += f0.y; y[2] += f1.x; y[3] += f1.y;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = bfr(y[e]);
        if (a.ysum) {      // into the first partial's place: this thread alone reads and writes these four columns
          __nv_bfloat162 o2[2] = {__floats2bfloat162_rn(y[0], y[1]), __floats2bfloat162_rn(y[2], y[3])};
          *reinterpret_cast<uint2*>(sh_y + col) = *reinterpret_cast<uint2*>(o2);
        }
        float nx[MAX_HC][4];
#pragma unroll
        for (int k = 0; k < MAX_HC; ++k) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = __fmul_rn(post[k], y[e]);
#pragma unroll
            for (int j = 0; j < MAX_HC; ++j)
              if (j < hc && k < hc) v = __fmaf_rn(comb[j * hc + k], x[j][e], v);
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
          if (c < hc) { v = __fmaf_rn(ap[c], x[c][e], v); hsq = __fmaf_rn(x[c][e], x[c][e], hsq); }
        v = bfr(v);
        xh[it][e] = v;
        ss = __fmaf_rn(v, v, ss);
      }
    }
  }
  FOLD_MARK(3);
  ss = block_sum(ss, sh);
  if (a.hss) {
    hsq = block_sum(hsq, sh);
    if (threadIdx.x == 0) a.hss[row] = hsq;
  }
  FOLD_MARK(4);
  const float rsx = rsqrtf(ss / (float)d + a.norm_eps);
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
        *reinterpret_cast<uint2*>(sh_xn + col) = *reinterpret_cast<uint2*>(o2);
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
          *reinterpret_cast<uint32_t*>(sh_xq + col) = q4;
          if ((threadIdx.x & 7) == 0) {
            sh_xs[col / 32] = sc;
            if (a.xs_atom) {
              if (a.atom_mode == 0) a.xs_atom[sf_offset(row, col / 32, KB)] = sc;
              else a.xs_atom[(size_t)row * sf_bytes(1, KB) + sf_offset(0, col / 32, KB)] = sc;
            }
          }
        }
      }
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  FOLD_MARK(5);
  if (threadIdx.x < 32 && elect_one()) {
    if (a.has_post) {
      fold_bulk_store(a.h + (size_t)row * hc * d, sh_h, (uint32_t)(hc * d * 2));
      if (a.ysum) fold_bulk_store(a.ysum + (size_t)row * d, sh_y, (uint32_t)(d * 2));
    }
    if (a.xn) fold_bulk_store(a.xn + (size_t)row * d, sh_xn, (uint32_t)(d * 2));
    if (a.xq) {
      fold_bulk_store(a.xq + (size_t)row * d, sh_xq, (uint32_t)d);
      fold_bulk_store(a.xs + (size_t)row * KB, sh_xs, (uint32_t)KB);
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the block may leave once its shared memory has been read
  }
  __syncwarp();
  FOLD_MARK(6);
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

// copies the phase marks of the last bulk-copy fold (rows x 8 words) to host memory; -1 when the library has none
int sfb_seam_read_marks(unsigned long long* dst, int rows) {
#ifdef SFB_KERNEL_MARKS
  return (int)cudaMemcpyFromSymbol(dst, g_fold_marks, (size_t)(rows < 4096 ? rows : 4096) * 8 * sizeof(unsigned long long));
#else
  (void)dst; (void)rows;
  return -1;
#endif
}
static int g_seam_tune = 0;      // 1: the many-row fold never takes the bulk-copy kernel (measurements, equality tests)
int sfb_seam_tune(int v) { g_seam_tune = v; return 0; }
int sfb_seam_nblk(int d) { return (d + COEF_COLS - 1) / COEF_COLS; }
int sfb_coef_stride(int hc) { return coef_stride(hc); }

// Critical-path half of a seam. y_ptrs / flag_ptrs: host arrays of W device pointers (flag_ptrs may be null).
int sfb_seam_fold(void* h, const void* const* y_ptrs, const void* const* flag_ptrs, const void* epoch_ptr,
                  uint32_t epoch_add, uint64_t wait_ns, int W,
                  int has_post, const float* coef_prev, const float* a_pre, int a_stride, void* ysum,
                  const float* norm_w, void* xn, void* xq, void* xs, void* xs_atom, int atom_mode, void* status,
                  int n, int hc, int d, float norm_eps, float* hss, int rs_rows, cudaStream_t stream) {
  if (hc > MAX_HC || W > 8 || (hc & (hc - 1)) || d % (32 * FOLD_CLUSTER) || d > FOLD_CLUSTER * FOLD_THREADS * FOLD_MAX_IT)
    return (int)cudaErrorInvalidValue;
  if (rs_rows > 0 && (!has_post || n <= 128 || d % 128 || (int64_t)rs_rows * W < n)) return (int)cudaErrorInvalidValue;
  FoldArgs a{};
  a.h = (__nv_bfloat16*)h;
  for (int r = 0; r < 8; ++r) {
    a.y[r] = (has_post && r < W) ? (const __nv_bfloat16*)y_ptrs[r] : nullptr;
    a.flags[r] = (has_post && flag_ptrs && r < W) ? (const uint32_t*)flag_ptrs[r] : nullptr;
  }
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns ? wait_ns : 2000000000ull; a.W = W; a.has_post = has_post; a.coef_prev = coef_prev; a.a_pre = a_pre; a.a_stride = a_stride;
  a.ysum = (__nv_bfloat16*)ysum; a.norm_w = norm_w; a.xn = (__nv_bfloat16*)xn; a.xq = (uint8_t*)xq;
  a.xs = (uint8_t*)xs; a.xs_atom = (uint8_t*)xs_atom; a.atom_mode = atom_mode; a.status = (Status*)status;
  a.n = n; a.hc = hc; a.d = d; a.norm_eps = norm_eps; a.hss = hss; a.rs_rows = rs_rows;
  if (n > 128 && d % 128 == 0 && d <= FOLDR_THREADS * 4 * FOLDR_MAX_IT) {     // many rows: one block per row
    // rows through bulk copies when every row of every buffer starts on a 16-byte boundary and a row's buffers fit in
    // shared memory (g_seam_tune: 1 = never)
    const int Wp = has_post ? (rs_rows > 0 ? 1 : W) : 0;      // parts of a row held in shared memory
    const size_t smem = (size_t)(hc + Wp + 1) * d * 2 + d + ((d / 32 + 15) & ~15) + 16;
    uintptr_t bits = (uintptr_t)h | (uintptr_t)ysum | (uintptr_t)xn | (uintptr_t)xq | (uintptr_t)xs;
    for (int r = 0; r < (has_post ? W : 0); ++r) bits |= (uintptr_t)y_ptrs[r];
    if (g_seam_tune != 1 && d % 512 == 0 && (bits & 15) == 0 && smem <= 200 * 1024 && (xq == nullptr || xs != nullptr)) {
      static bool attr = false;
      if (!attr) {
        cudaError_t rc = cudaFuncSetAttribute(seam_fold_rows_bulk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
        if (rc == cudaSuccess) rc = cudaFuncSetAttribute(seam_fold_rows_bulk_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
        if (rc != cudaSuccess) return (int)rc;
        attr = true;
      }
      if (hc == 4) return (int)sfb_launch(seam_fold_rows_bulk_kernel<4>, dim3(n), dim3(FOLDR_THREADS), smem, stream, a);
      return (int)sfb_launch(seam_fold_rows_bulk_kernel<0>, dim3(n), dim3(FOLDR_THREADS), smem, stream, a);
    }
    if (hc == 4) return (int)sfb_launch(seam_fold_rows_kernel<4>, dim3(n), dim3(FOLDR_THREADS), 0, stream, a);
    return (int)sfb_launch(seam_fold_rows_kernel<0>, dim3(n), dim3(FOLDR_THREADS), 0, stream, a);
  }
  if (hc == 4) return (int)sfb_launch(seam_fold_kernel<4>, dim3(FOLD_CLUSTER, n), dim3(FOLD_THREADS), 0, stream, a);
  return (int)sfb_launch(seam_fold_kernel<0>, dim3(FOLD_CLUSTER, n), dim3(FOLD_THREADS), 0, stream, a);
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
