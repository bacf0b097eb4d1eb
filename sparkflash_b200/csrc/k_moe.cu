// MoE for the rows step (exact CUDA-core arm): router, gate/up with clamp-SwiGLU + FP8 re-quant,
// and down projection with the top-k + shared-expert sum.  Routed experts are W4A8 (MXFP4 weights,
// per-32 FP8 activations); the shared expert is W8A8 and rides along as slot `top_k`.
//
// Each rank holds an intermediate-width slice of every expert (tensor-parallel experts) or whole
// experts (expert-parallel); the kernels only see `inter` = the local width and per-expert base
// pointers.
//
// Reference behaviour: kernels/opt_router_sm121.cu:219-221, kernels/opt_moe_sm121.cu:225-227 (gate/up),
// :348-349 (down + combine), kernels/swiglu_quant_sm121.cuh; docs/architecture/03-moe.md:25-163.
#include "k_common.cuh"

namespace sfb {

// ---- router ----------------------------------------------------------------------------------------------
struct RouterArgs {
  const float* dots;      // [nsplit, n, E] raw gate logits (fp32), split-K slices added in index order
  int nsplit;
  int64_t split_stride;
  const float* bias;      // [E]
  const float* bias_vl;   // [E] (image rows) or null
  const uint8_t* is_image;  // [n] or null
  int* ids;               // [n, k] ascending expert ids
  float* wts;             // [n, k]
  int n, E, k;
  float route_scale;
};

__global__ void __launch_bounds__(128) router_topk_kernel(RouterArgs a) {
  extern __shared__ float sm[];
  float* s = sm;            // [E] scores
  float* key = sm + a.E;    // [E] selection keys
  __shared__ float rv[4];
  __shared__ int ri[4];
  __shared__ int pick[16];
  const int row = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const float* bias = (a.is_image && a.bias_vl && a.is_image[row]) ? a.bias_vl : a.bias;
  for (int e = threadIdx.x; e < a.E; e += 128) {
    float x = 0.f;
    for (int z = 0; z < a.nsplit; ++z) x += a.dots[(size_t)z * a.split_stride + (size_t)row * a.E + e];
    float sp = x > 20.f ? x : log1pf(expf(x));
    float v = sqrtf(sp);
    s[e] = v;
    key[e] = v + bias[e];
  }
  __syncthreads();
  for (int t = 0; t < a.k; ++t) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = threadIdx.x; e < a.E; e += 128) {
      float v = key[e];
      if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { rv[threadIdx.x >> 5] = bv; ri[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 4; ++w)
        if (rv[w] > bv || (rv[w] == bv && ri[w] < bi)) { bv = rv[w]; bi = ri[w]; }
      pick[t] = bi;
      key[bi] = -INFINITY;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    for (int i = 1; i < a.k; ++i) {  // ascending ids
      int v = pick[i], j = i - 1;
      while (j >= 0 && pick[j] > v) { pick[j + 1] = pick[j]; --j; }
      pick[j + 1] = v;
    }
    float sum = 0.f;
    for (int i = 0; i < a.k; ++i) sum += s[pick[i]];
    for (int i = 0; i < a.k; ++i) {
      a.ids[(size_t)row * a.k + i] = pick[i];
      a.wts[(size_t)row * a.k + i] = s[pick[i]] / (sum + 1e-20f) * a.route_scale;
    }
  }
}

// ---- gate / up ---------------------------------------------------------------------------------------------
struct GateUpArgs {
  const uint8_t* xq;      // [n, d] e4m3
  const uint8_t* xs;      // [n, d/32]
  const int* ids;         // [n, k]
  const float* wts;       // [n, k]
  const uint8_t* w13;     // routed: [E, 2, inter, d/2] packed e2m1
  const uint8_t* w13_sf;  // routed: [E, 2, inter, d/32] row-major scales
  const uint8_t* s13;     // shared: [2, inter, d] e4m3 (null when there is no shared expert)
  const uint8_t* s13_sf;  // shared: [2, inter, d/32]
  uint8_t* act_q;         // [n, k+1, inter] e4m3
  uint8_t* act_s;         // [n, k+1, inter/32]
  int n, k, d, inter;
  float limit;
};

// NR weight rows against one activation row; all NR loads of a chunk step are issued before use.
template <int FP4, int NR>
__device__ __forceinline__ void dot_rows(const uint8_t* const* wrow, const uint8_t* const* sf, const int64_t* sf_row,
                                         int KB, const float* x, int K, int lane, float* out) {
  constexpr int EPC = FP4 ? 32 : 16;
  constexpr int U = 2;
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) acc[i] = 0.f;
  const int chunks = K / EPC;
  for (int cb = lane; cb < chunks; cb += 32 * U) {
    uint4 wv[U][NR];
    float sc[U][NR];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = cb + 32 * u;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        if (c < chunks) {
          wv[u][i] = ldg_nc(wrow[i] + (size_t)c * 16);
          sc[u][i] = ue8m0_shifted(__ldg(sf[i] + sf_row[i] * KB + ((c * EPC) >> 5)),
                                   FP4 ? SFB_E2M1_RAW_EXP : SFB_E4M3_RAW_EXP);
        } else { wv[u][i] = make_uint4(0, 0, 0, 0); sc[u][i] = 0.f; }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = cb + 32 * u;
      if (c >= chunks) break;
      const float4* xp = reinterpret_cast<const float4*>(x + sm_pad(c * EPC));
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        float f[EPC];
        if (FP4) decode32_e2m1_raw(wv[u][i], f); else decode16_e4m3_raw(wv[u][i], f);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < EPC / 4; ++j) {
          float4 xv = xp[j];
          s = fmaf(f[4 * j], xv.x, s); s = fmaf(f[4 * j + 1], xv.y, s);
          s = fmaf(f[4 * j + 2], xv.z, s); s = fmaf(f[4 * j + 3], xv.w, s);
        }
        acc[i] = fmaf(s, sc[u][i], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NR; ++i) out[i] = warp_sum(acc[i]);
}

// grid (inter/32, k+1, n), block 256; dynamic smem d floats
__global__ void __launch_bounds__(256) moe_gate_up_kernel(GateUpArgs a) {
  extern __shared__ float xsm[];
  __shared__ float gu[2][32];
  const int row = blockIdx.z, slot = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = a.d, KB = d / 32;
  stage_fp8_to_smem(a.xq + (size_t)row * d, a.xs + (size_t)row * KB, d / 16, xsm, 256);
  __syncthreads();
  const bool shared_slot = slot == a.k;
  float weight = 1.f;
  const uint8_t *w1, *w3, *sf1, *sf3;
  const int64_t sfb = (int64_t)a.inter * KB;  // row-major scales per matrix
  if (shared_slot) {
    w1 = a.s13; w3 = a.s13 + (size_t)a.inter * d;
    sf1 = a.s13_sf; sf3 = a.s13_sf + sfb;
  } else {
    const int e = a.ids[(size_t)row * a.k + slot];
    weight = a.wts[(size_t)row * a.k + slot];
    const size_t per = (size_t)a.inter * (d / 2);
    w1 = a.w13 + (size_t)e * 2 * per; w3 = w1 + per;
    sf1 = a.w13_sf + (size_t)e * 2 * sfb; sf3 = sf1 + sfb;
  }
  // 64 dot products (32 gate + 32 up) per column tile: each warp takes 4 output columns, gate and up
  // rows together
  for (int ob = blockIdx.x * 32; ob < a.inter; ob += gridDim.x * 32) {
    const int oc = warp * 4;  // columns oc..oc+3 of this block's 32
    const uint8_t* wr[8];
    const uint8_t* sfp[8];
    int64_t sfr[8];
    const size_t rb = shared_slot ? (size_t)d : (size_t)(d / 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int which = i >> 2, o = ob + oc + (i & 3);
      wr[i] = (which ? w3 : w1) + (size_t)o * rb;
      sfp[i] = which ? sf3 : sf1;
      sfr[i] = o;
    }
    float v[8];
    if (shared_slot) dot_rows<0, 8>(wr, sfp, sfr, KB, xsm, d, lane, v);
    else dot_rows<1, 8>(wr, sfp, sfr, KB, xsm, d, lane, v);
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) gu[i >> 2][oc + (i & 3)] = bfr(v[i]);
    }
  __syncthreads();
  if (warp == 0) {
    float g = fminf(gu[0][lane], a.limit);
    float u = fminf(fmaxf(gu[1][lane], -a.limit), a.limit);
    float v = bfr(g / (1.f + expf(-g)) * u * weight);
    uint8_t sc;
    uint8_t q = warp_quant_fp8(v, &sc);
    const size_t base = ((size_t)row * (a.k + 1) + slot) * a.inter;
    a.act_q[base + ob + lane] = q;
    if (lane == 0) a.act_s[base / 32 + ob / 32] = sc;
  }
  __syncthreads();
  }
}

// ---- down + combine -------------------------------------------------------------------------------------------
struct DownArgs {
  const uint8_t* act_q;   // [n, k+1, inter]
  const uint8_t* act_s;   // [n, k+1, inter/32]
  const int* ids;         // [n, k]
  const uint8_t* w2;      // routed: [E, d, inter/2]
  const uint8_t* w2_sf;   // routed: [E, d, inter/32]
  const uint8_t* s2;      // shared: [d, inter] e4m3
  const uint8_t* s2_sf;   // shared: [d, inter/32]
  __nv_bfloat16* out;     // [n, d] this rank's partial
  int n, k, d, inter, has_shared;
};

constexpr int DN_COLS = 16;  // output columns per block (2 per warp)

// grid (d/16, n), block 256; dynamic smem (k+1)*inter floats
__global__ void __launch_bounds__(256) moe_down_kernel(DownArgs a) {
  extern __shared__ float asm_[];
  const int row = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int inter = a.inter, KB = inter / 32, slots = a.k + a.has_shared;
  {
    const size_t o = (size_t)row * (a.k + 1) * inter;
    stage_fp8_to_smem(a.act_q + o, a.act_s + o / 32, slots * inter / 16, asm_, 256);
  }
  __syncthreads();
  const int64_t sfb = (int64_t)a.d * KB;  // row-major scales per expert
  const int c4 = inter / 32, c8 = inter / 16;      // chunks per routed / shared slot
  const int items = a.k * c4 + (a.has_shared ? c8 : 0);
  for (int cb = blockIdx.x * DN_COLS; cb < a.d; cb += gridDim.x * DN_COLS) {
    const int col0 = cb + warp * 2;
    constexpr int U = 2;
    float acc[2] = {0.f, 0.f};
    for (int ib = lane; ib < items; ib += 32 * U) {
      uint4 wv[U][2];
      float sc[U][2];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = ib + 32 * u;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int col = col0 + cc;
          if (it < items && col < a.d) {
            if (it < a.k * c4) {
              const int slot = it / c4, c = it - slot * c4;
              const int e = a.ids[(size_t)row * a.k + slot];
              wv[u][cc] = ldg_nc(a.w2 + ((size_t)e * a.d + col) * (inter / 2) + (size_t)c * 16);
              sc[u][cc] = ue8m0_shifted(__ldg(a.w2_sf + (size_t)e * sfb + (size_t)col * KB + c), SFB_E2M1_RAW_EXP);
            } else {
              const int c = it - a.k * c4;
              wv[u][cc] = ldg_nc(a.s2 + (size_t)col * inter + (size_t)c * 16);
              sc[u][cc] = ue8m0_shifted(__ldg(a.s2_sf + (size_t)col * KB + (c >> 1)), SFB_E4M3_RAW_EXP);
            }
          } else { wv[u][cc] = make_uint4(0, 0, 0, 0); sc[u][cc] = 0.f; }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int it = ib + 32 * u;
        if (it >= items) break;
        if (it < a.k * c4) {
          const int slot = it / c4, c = it - slot * c4;
          const float4* x = reinterpret_cast<const float4*>(asm_ + sm_pad(slot * inter + c * 32));
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            float f[32];
            decode32_e2m1_raw(wv[u][cc], f);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 xv = x[j];
              s = fmaf(f[4 * j], xv.x, s); s = fmaf(f[4 * j + 1], xv.y, s);
              s = fmaf(f[4 * j + 2], xv.z, s); s = fmaf(f[4 * j + 3], xv.w, s);
            }
            acc[cc] = fmaf(s, sc[u][cc], acc[cc]);
          }
        } else {
          const int c = it - a.k * c4;
          const float4* x = reinterpret_cast<const float4*>(asm_ + sm_pad(a.k * inter + c * 16));
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            float f[16];
            decode16_e4m3_raw(wv[u][cc], f);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float4 xv = x[j];
              s = fmaf(f[4 * j], xv.x, s); s = fmaf(f[4 * j + 1], xv.y, s);
              s = fmaf(f[4 * j + 2], xv.z, s); s = fmaf(f[4 * j + 3], xv.w, s);
            }
            acc[cc] = fmaf(s, sc[u][cc], acc[cc]);
          }
        }
      }
    }
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const float v = warp_sum(acc[cc]);
      if (lane == 0 && col0 + cc < a.d) a.out[(size_t)row * a.d + col0 + cc] = __float2bfloat16_rn(v);
    }
  }
}


// ---- grouped MoE plan: the (token, expert) pairs of a step sorted by expert, cut into segments of up to 16 pairs ----------
// Every expert's weights are then read once per segment instead of once per pair, and the shared expert once per 16 tokens.
// Reference behaviour: the MoE grouping / dedup plan built once per stage call (crates/sparkflash-kernels/src/moe_routed_device.rs:
// 1568-2063; DECISIONS D102).  The arithmetic per pair is unchanged: one accumulator column per pair, summed per token in slot order.
struct MoePlanArgs {
  const int* ids;        // [n, k] expert id (local; < 0 = not on this rank)
  const float* wts;      // [n, k]
  int n, k, E, shared, S;          // S = segments launched (fixed per row count)
  int seg;                         // pair slots per segment (16, or 64 for many-row steps)
  int* seg_expert;       // [S]  -1 unused, -2 shared expert
  int* seg_count;        // [S]
  float* seg_weight;     // [S*16]
  int* seg_token;        // [S*16] token of the pair slot, -1 unused
  int* pair_pos;         // [n, k+1] pair slot of (token, slot), -1 = skipped
};

__global__ void __launch_bounds__(512) moe_plan_kernel(MoePlanArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int plan_sm[];     // cnt[E] | base[E + 1] | fill[E]
  int* cnt = plan_sm; int* base = plan_sm + a.E; int* fill = plan_sm + 2 * a.E + 1;
  const int P = a.n * a.k;
  for (int i = threadIdx.x; i < a.E; i += blockDim.x) { cnt[i] = 0; fill[i] = 0; }
  for (int i = threadIdx.x; i < a.S; i += blockDim.x) { a.seg_expert[i] = -1; a.seg_count[i] = 0; }
  for (int i = threadIdx.x; i < a.S * a.seg; i += blockDim.x) { a.seg_token[i] = -1; a.seg_weight[i] = 0.f; }
  for (int i = threadIdx.x; i < a.n * (a.k + 1); i += blockDim.x) a.pair_pos[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) { const int e = a.ids[p]; if (e >= 0 && e < a.E) atomicAdd(&cnt[e], 1); }
  __syncthreads();
  if (threadIdx.x == 0) {
    int b = 0;
    for (int e = 0; e < a.E; ++e) { base[e] = b; b += (cnt[e] + a.seg - 1) / a.seg; }
    base[a.E] = b;                     // first segment of the shared expert
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x)
    for (int sgi = 0, c = cnt[e]; c > 0; ++sgi, c -= a.seg)
      if (base[e] + sgi < a.S) { a.seg_expert[base[e] + sgi] = e; a.seg_count[base[e] + sgi] = c < a.seg ? c : a.seg; }
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = a.ids[p];
    if (e < 0 || e >= a.E) continue;
    int r = 0;
    if (P <= 1024) {                    // rank among the earlier pairs of the same expert: the order inside a segment is the pair order
      for (int q = 0; q < p; ++q) r += a.ids[q] == e;
    } else {
      // many pairs: take the next free place of the expert instead of counting the earlier pairs.  A pair is its own
      // accumulator column wherever it sits, so the place changes no result
      r = cnt[e] - 1 - atomicAdd(&fill[e], 1);
    }
    const int seg = base[e] + r / a.seg, slot = seg * a.seg + (r % a.seg);
    if (seg < a.S) {
      a.seg_token[slot] = p / a.k; a.seg_weight[slot] = a.wts[p];
      a.pair_pos[(p / a.k) * (a.k + 1) + p % a.k] = slot;
    }
  }
  if (a.shared) {
    for (int t = threadIdx.x; t < a.n; t += blockDim.x) {
      const int seg = base[a.E] + t / a.seg, slot = seg * a.seg + (t % a.seg);
      if (seg < a.S) { a.seg_token[slot] = t; a.seg_weight[slot] = 1.f; a.pair_pos[t * (a.k + 1) + a.k] = slot; }
    }
    for (int sgi = threadIdx.x; sgi * a.seg < a.n; sgi += blockDim.x)
      if (base[a.E] + sgi < a.S) { a.seg_expert[base[a.E] + sgi] = -2; a.seg_count[base[a.E] + sgi] = a.n - sgi * a.seg < a.seg ? a.n - sgi * a.seg : a.seg; }
  }
}

// one block per pair slot: the token's FP8 row and its scales (as row j of the segment's atom set)
__global__ void __launch_bounds__(128) moe_permute_kernel(const uint8_t* xq, const uint8_t* xs, const int* seg_token, uint8_t* xperm,
                                                         uint8_t* seg_atoms, int d, int atom_set_bytes, int seg_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.x, tok = seg_token[slot];
  if (tok < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)tok * d);
  uint4* dst = reinterpret_cast<uint4*>(xperm + (size_t)slot * d);
  for (int i = threadIdx.x; i < d / 16; i += blockDim.x) dst[i] = src[i];
  const int KB = d / 32, seg = slot / seg_size, j = slot % seg_size;
  for (int kb = threadIdx.x; kb < KB; kb += blockDim.x) seg_atoms[(size_t)seg * atom_set_bytes + sf_offset(j, kb, KB)] = xs[(size_t)tok * KB + kb];
}

// y[t, :] = bf16( sum over the token's pair slots, in slot order, of ypair[slot, :] )
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* ypair, const int* pair_pos, __nv_bfloat16* y, int k1, int d, int64_t y_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= d) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sl = 0; sl < k1; ++sl) {
    const int pos = pair_pos[t * k1 + sl];
    if (pos < 0) continue;
    const float4 v = *reinterpret_cast<const float4*>(ypair + (size_t)pos * d + c);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  __nv_bfloat16* o = y + (size_t)t * y_stride + c;
  o[0] = __float2bfloat16_rn(acc.x); o[1] = __float2bfloat16_rn(acc.y); o[2] = __float2bfloat16_rn(acc.z); o[3] = __float2bfloat16_rn(acc.w);
}

// expert parallelism: global expert ids -> this rank's local ids, -1 for experts held elsewhere (the grouped GEMMs skip them)
__global__ void expert_remap_kernel(int* ids, int n, int lo, int count) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { const int e = ids[i] - lo; ids[i] = (e >= 0 && e < count) ? e : -1; }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_router_topk(const float* dots, int nsplit, int64_t split_stride, const float* bias, const float* bias_vl, const void* is_image, int* ids,
                    float* wts, int n, int E, int k, float route_scale, cudaStream_t stream) {
  if (k > 16) return (int)cudaErrorInvalidValue;
  RouterArgs a{dots, nsplit < 1 ? 1 : nsplit, split_stride, bias, bias_vl, (const uint8_t*)is_image, ids, wts, n, E, k, route_scale};
  return (int)sfb_launch(router_topk_kernel, dim3(n), dim3(128), sizeof(float) * 2 * E, stream, a);
}

int sfb_moe_gate_up(const void* xq, const void* xs, const int* ids, const float* wts, const void* w13,
                    const void* w13_sf, const void* s13, const void* s13_sf, void* act_q, void* act_s, int n,
                    int k, int d, int inter, float limit, cudaStream_t stream) {
  if (inter % 32 || d % 32) return (int)cudaErrorInvalidValue;
  GateUpArgs a{(const uint8_t*)xq, (const uint8_t*)xs, ids, wts, (const uint8_t*)w13, (const uint8_t*)w13_sf,
               (const uint8_t*)s13, (const uint8_t*)s13_sf, (uint8_t*)act_q, (uint8_t*)act_s, n, k, d, inter, limit};
  const int slots = k + (s13 ? 1 : 0);
  int gx = inter / 32;
  const int cap = (148 * 3 + slots * n - 1) / (slots * n);  // ~3 resident blocks per SM in total
  if (gx > cap) gx = cap > 0 ? cap : 1;
  moe_gate_up_kernel<<<dim3(gx, slots, n), 256, sizeof(float) * sm_pad(d), stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

int sfb_moe_down(const void* act_q, const void* act_s, const int* ids, const void* w2, const void* w2_sf,
                 const void* s2, const void* s2_sf, void* out, int n, int k, int d, int inter,
                 cudaStream_t stream) {
  DownArgs a{(const uint8_t*)act_q, (const uint8_t*)act_s, ids, (const uint8_t*)w2, (const uint8_t*)w2_sf,
             (const uint8_t*)s2, (const uint8_t*)s2_sf, (__nv_bfloat16*)out, n, k, d, inter, s2 ? 1 : 0};
  const size_t smem = sizeof(float) * (size_t)sm_pad((k + 1) * inter);
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); done = true; }
  if (smem > 160 * 1024) return (int)cudaErrorInvalidValue;
  int gx = (d + DN_COLS - 1) / DN_COLS;
  const int cap = (148 * 2 + n - 1) / n;
  if (gx > cap) gx = cap > 0 ? cap : 1;
  moe_down_kernel<<<dim3(gx, n), 256, smem, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"

extern "C" int sfb_expert_remap(void* ids, int n, int lo, int count, cudaStream_t stream) {
  return (int)sfb::sfb_launch(sfb::expert_remap_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, (int*)ids, n, lo, count);
}

extern "C" int sfb_moe_plan(const void* ids, const void* wts, int n, int k, int E, int shared, int S, int seg, void* seg_expert, void* seg_count,
                            void* seg_weight, void* seg_token, void* pair_pos, cudaStream_t stream) {
  if (E > 4096 || (seg != 16 && seg != 64)) return (int)cudaErrorInvalidValue;
  sfb::MoePlanArgs a{(const int*)ids, (const float*)wts, n, k, E, shared, S, seg, (int*)seg_expert, (int*)seg_count, (float*)seg_weight,
                     (int*)seg_token, (int*)pair_pos};
  return (int)sfb::sfb_launch(sfb::moe_plan_kernel, dim3(1), dim3(512), (size_t)(3 * E + 1) * sizeof(int), stream, a);
}
extern "C" int sfb_moe_permute(const void* xq, const void* xs, const void* seg_token, void* xperm, void* seg_atoms, int slots, int d,
                               int atom_set_bytes, int seg_size, cudaStream_t stream) {
  if (d % 32 || seg_size < 1) return (int)cudaErrorInvalidValue;
  return (int)sfb::sfb_launch(sfb::moe_permute_kernel, dim3(slots), dim3(128), 0, stream, (const uint8_t*)xq, (const uint8_t*)xs,
                              (const int*)seg_token, (uint8_t*)xperm, (uint8_t*)seg_atoms, d, atom_set_bytes, seg_size);
}
extern "C" int sfb_moe_combine(const void* ypair, const void* pair_pos, void* y, int n, int k1, int d, int64_t y_stride, cudaStream_t stream) {
  if (d % 4) return (int)cudaErrorInvalidValue;
  return (int)sfb::sfb_launch(sfb::moe_combine_kernel, dim3((d / 4 + 255) / 256, n), dim3(256), 0, stream, (const float*)ypair,
                              (const int*)pair_pos, (__nv_bfloat16*)y, k1, d, y_stride);
}
