// CUDA-core skinny GEMM ("GEMV") family: y[n, N] = x[n, K] * W[N, K]^T for a handful of rows.
//
// This is the exact arm of every projection: fp32 accumulation in a fixed order that does not
// depend on how many rows share the launch (row i's bits are the same for n = 1 and n = 64), which
// is the batch-invariance the rows step relies on.  The tensor-core arm (k_umma_*.cu) covers the
// same shapes with tcgen05; this file is also the fallback for shapes it does not take.
//
// Weight formats: MXFP8 (E4M3, one UE8M0 scale per row per 32 K) and MXFP4 (packed E2M1, same
// scales), here with the scales row-major [rows, K/32]; plain bf16.
// Activations: per-32 FP8 (codes + row-major scales) or bf16.
//
// Reference behaviour: kernels/opt_gemv_sm121.cu:418-435,732-740 (decode MXFP8 GEMV, rows variants),
// kernels/b12x_bf16a_mxfp8w_dense_sm121.cu (bf16 activations on FP8 weights), kernels/q4e_gemv_sm121.cuh.
#include "k_common.cuh"

namespace sfb {

constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = 8;
constexpr int GV_RPW = 2;                    // output rows per warp, loaded together
constexpr int GV_ROWS = GV_WARPS * GV_RPW;   // output rows per block
__host__ __device__ constexpr int gv_rpw(int wf, int r) { return (wf == 2 && r >= 4) ? 4 : GV_RPW; }

struct GemvArgs {
  const uint8_t* w;        // payload, row-major [groups*N, row_bytes]
  const uint8_t* sf;       // row-major scales [groups*N, K/32] (null for bf16 weights); consecutive lanes read
                           // consecutive bytes, unlike the 128x4-atom order the tensor-core arm consumes
  int64_t row_bytes;
  int N;                   // output rows per group
  int K;                   // reduction length per group
  int KB;                  // K/32
  int groups;              // blockIdx.y; group g reads activation columns [g*K, (g+1)*K)
  int n;                   // activation rows
  // activations
  const uint8_t* xq;       // fp8 codes [n, x_stride] or null
  const uint8_t* xs;       // scales [n, x_stride/32]
  const __nv_bfloat16* xb; // bf16 [n, x_stride] or null
  const float* xf;         // fp32 [n, x_stride] or null
  int64_t x_stride;        // elements per activation row
  int x_quant;             // quantise bf16/fp32 activations per 32 to FP8 while loading (W8A8 semantics)
  // outputs [n, out_stride], column = group*N + row
  __nv_bfloat16* out_b;
  float* out_f;
  int64_t out_stride;
  // split-K (blockIdx.z): slice z covers chunks [z*chunks/ksplit, (z+1)*chunks/ksplit) and writes its fp32
  // partial to out_f + z*split_stride; the consumer adds the slices in index order
  int ksplit;
  int64_t split_stride;
  // blockIdx.x = row_group * tile_blocks + tile_block: each row group takes every row_groups-th set of R activation
  // rows, so many-row launches spread over the machine instead of looping in one wave (same sums per row either way)
  int tile_blocks;
  int row_groups;
};

template <int R>
__device__ __forceinline__ void load_x(const GemvArgs& a, int r0, int kcol0, float* xs_sm) {
  // xs_sm[r][sm_pad(k)] for r < R, k < K (zero rows past n)
  const int KP = sm_pad(a.K);
  if (a.xq) {
    const int c16 = a.K / 16;
    for (int i = threadIdx.x; i < R * c16; i += GV_THREADS) {
      const int r = i / c16, c = i - r * c16, row = r0 + r;
      float f[16];
      float s = 0.f;
      if (row < a.n) {
        const uint4 v = *reinterpret_cast<const uint4*>(a.xq + (int64_t)row * a.x_stride + kcol0 + c * 16);
        s = ue8m0_to_f32(a.xs[(int64_t)row * (a.x_stride / 32) + (kcol0 + c * 16) / 32]);
        decode16_e4m3(v, f);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = 0.f;
      }
      float4* o = reinterpret_cast<float4*>(xs_sm + r * KP + sm_pad(c * 16));
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = make_float4(f[4 * j] * s, f[4 * j + 1] * s, f[4 * j + 2] * s, f[4 * j + 3] * s);
    }
  } else if (a.xb) {
    const int c8 = a.K / 8, total = R * c8;
    for (int base = 0; base < total; base += GV_THREADS) {  // uniform trip count: shuffles below
      const int i = base + threadIdx.x;
      const bool on = i < total;
      const int r = on ? i / c8 : 0, c = on ? i - r * c8 : 0, row = r0 + r;
      float f[8];
      if (on && row < a.n) {
        const uint4 v = *reinterpret_cast<const uint4*>(a.xb + (int64_t)row * a.x_stride + kcol0 + c * 8);
        const uint32_t* p = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { f[2 * j] = __uint_as_float(p[j] << 16); f[2 * j + 1] = __uint_as_float(p[j] & 0xffff0000u); }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.f;
      }
      if (a.x_quant) {  // per-32 FP8 round trip: 4 neighbouring lanes hold one aligned group
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint8_t sc = act_scale_code_fp8(amax);
        const float inv = bits_f32(((uint32_t)(254 - sc)) << 23), s = ue8m0_to_f32(sc);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 t = cvt_e4m3x2(enc_e4m3x2(f[2 * j] * inv, f[2 * j + 1] * inv));
          f[2 * j] = t.x * s; f[2 * j + 1] = t.y * s;
        }
      }
      if (on) {
        float4* o = reinterpret_cast<float4*>(xs_sm + r * KP + sm_pad(c * 8));
        o[0] = make_float4(f[0], f[1], f[2], f[3]);
        o[1] = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < R * a.K; idx += GV_THREADS) {
      const int r = idx / a.K, k = idx - r * a.K, row = r0 + r;
      xs_sm[r * KP + sm_pad(k)] = row < a.n ? a.xf[(int64_t)row * a.x_stride + kcol0 + k] : 0.f;
    }
  }
}

// WF: 0 = fp8 weights, 1 = fp4 weights, 2 = bf16 weights
template <int WF, int R>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(GemvArgs a) {
  extern __shared__ float xs_sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int EPC = WF == 0 ? 16 : (WF == 1 ? 32 : 8);  // elements per 16-byte chunk
  // output rows per warp: many-row bf16 launches (head, router, auxiliary projections) take four, so that one read of an
  // activation chunk from shared memory feeds four weight rows; a row's sum is the same either way
  constexpr int RPW = gv_rpw(WF, R);
  constexpr int ROWS = GV_WARPS * RPW;
  const int chunks = a.K / EPC;
  const int c_lo = (int)((int64_t)chunks * blockIdx.z / a.ksplit), c_hi = (int)((int64_t)chunks * (blockIdx.z + 1) / a.ksplit);

  const int tile_block = blockIdx.x % a.tile_blocks, row_group = blockIdx.x / a.tile_blocks;
  for (int r0 = row_group * R; r0 < a.n; r0 += R * a.row_groups) {
    __syncthreads();
    load_x<R>(a, r0, g * a.K, xs_sm);
    __syncthreads();
   for (int tile = tile_block; tile * ROWS < a.N; tile += a.tile_blocks) {
    const int row0 = tile * ROWS + warp * RPW;
    float acc[RPW][R];
#pragma unroll
    for (int i = 0; i < RPW; ++i)
#pragma unroll
      for (int r = 0; r < R; ++r) acc[i][r] = 0.f;

    if (row0 < a.N) {
      const int64_t grow0 = (int64_t)g * a.N + row0;
      constexpr int U = RPW == 4 ? 2 : 4;  // chunks in flight per row per lane
      for (int cb = c_lo + lane; cb < c_hi; cb += 32 * U) {
        uint4 wv[U][RPW];
        float sc[U][RPW];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = cb + 32 * u;
#pragma unroll
          for (int i = 0; i < RPW; ++i) {
            const bool ok = row0 + i < a.N && c < c_hi;
            const int64_t gr = row0 + i < a.N ? grow0 + i : grow0;
            if (ok) {
              wv[u][i] = ldg_nc(a.w + gr * a.row_bytes + (int64_t)c * 16);
              sc[u][i] = WF == 2 ? 1.f
                                 : ue8m0_shifted(__ldg(a.sf + gr * a.KB + ((c * EPC) >> 5)),
                                                 WF == 0 ? SFB_E4M3_RAW_EXP : SFB_E2M1_RAW_EXP);
            } else {
              wv[u][i] = make_uint4(0, 0, 0, 0);
              sc[u][i] = 0.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = cb + 32 * u;
          if (c >= c_hi) break;
          // decode this chunk of every weight row first, then read each activation row's chunk from shared memory once
          // and use it for all of them (the shared-memory reads, not the FMAs, bound many-row launches)
          float f[RPW][EPC];
#pragma unroll
          for (int i = 0; i < RPW; ++i) {
            if (WF == 0) decode16_e4m3_raw(wv[u][i], f[i]);
            else if (WF == 1) decode32_e2m1_raw(wv[u][i], f[i]);
            else {
              const uint32_t* p = reinterpret_cast<const uint32_t*>(&wv[u][i]);
#pragma unroll
              for (int j = 0; j < 4; ++j) { f[i][2 * j] = __uint_as_float(p[j] << 16); f[i][2 * j + 1] = __uint_as_float(p[j] & 0xffff0000u); }
            }
          }
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const float4* xp = reinterpret_cast<const float4*>(xs_sm + r * sm_pad(a.K) + sm_pad(c * EPC));
            float s[RPW];
#pragma unroll
            for (int i = 0; i < RPW; ++i) s[i] = 0.f;
#pragma unroll
            for (int j = 0; j < EPC / 4; ++j) {
              const float4 xv = xp[j];
#pragma unroll
              for (int i = 0; i < RPW; ++i) {
                s[i] = fmaf(f[i][4 * j], xv.x, s[i]); s[i] = fmaf(f[i][4 * j + 1], xv.y, s[i]);
                s[i] = fmaf(f[i][4 * j + 2], xv.z, s[i]); s[i] = fmaf(f[i][4 * j + 3], xv.w, s[i]);
              }
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) acc[i][r] = fmaf(s[i], sc[u][i], acc[i][r]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float v = warp_sum(acc[i][r]);
        const int orow = row0 + i, arow = r0 + r;
        if (lane == 0 && orow < a.N && arow < a.n) {
          const int64_t o = (int64_t)arow * a.out_stride + (int64_t)g * a.N + orow;
          if (a.out_b) a.out_b[o] = __float2bfloat16_rn(v);
          if (a.out_f) a.out_f[o + (int64_t)blockIdx.z * a.split_stride] = v;
        }
      }
   }
  }
}

template <int WF>
static int launch_gemv(GemvArgs a, cudaStream_t stream) {
  const int64_t smem1 = (int64_t)sm_pad(a.K) * 4;
  int R = 1;
  if (a.n >= 4 && smem1 * 4 <= 96 * 1024) R = 4;
  else if (a.n >= 2 && smem1 * 2 <= 96 * 1024) R = 2;
  if (smem1 > 96 * 1024) return (int)cudaErrorInvalidValue;
  const int rows_per_block = GV_WARPS * gv_rpw(WF, R);
  int tiles = (a.N + rows_per_block - 1) / rows_per_block;
  const int cap = (148 * 4 + a.groups - 1) / a.groups;  // a few resident blocks per SM; each loops over row tiles
  a.tile_blocks = tiles < cap ? tiles : cap;
  const int passes = (a.n + R - 1) / R;
  const int room = cap * 2 / (a.tile_blocks * a.ksplit);          // row groups while the grid stays within a couple of waves
  a.row_groups = passes < room ? passes : (room < 1 ? 1 : room);
  dim3 grid(a.tile_blocks * a.row_groups, a.groups, a.ksplit);
  const size_t smem = (size_t)smem1 * R;
  cudaError_t launch_rc = cudaSuccess;
#define SFB_GV(RR)                                                                                   \
  {                                                                                                  \
    static bool attr_done = false;                                                                   \
    if (!attr_done) {                                                                                \
      cudaFuncSetAttribute(gemv_kernel<WF, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
      attr_done = true;                                                                              \
    }                                                                                                \
    launch_rc = sfb_launch(gemv_kernel<WF, RR>, grid, dim3(GV_THREADS), smem, stream, a);             \
  }
  if (R == 4) SFB_GV(4) else if (R == 2) SFB_GV(2) else SFB_GV(1)
#undef SFB_GV
  return (int)launch_rc;
}

}  // namespace sfb

using namespace sfb;

extern "C" {

// wfmt: 0 fp8, 1 fp4, 2 bf16.  Exactly one of xq / xb / xf is non-null; one or both outputs.
int sfb_gemv(int wfmt, const void* w, const void* sf, int64_t row_bytes, int N, int K, int groups, int n,
             const void* xq, const void* xs, const void* xb, const void* xf, int64_t x_stride, int x_quant,
             void* out_b, void* out_f, int64_t out_stride, int ksplit, int64_t split_stride, cudaStream_t stream) {
  const int epc = wfmt == 0 ? 16 : (wfmt == 1 ? 32 : 8);
  if (K % 32 || K % epc || n <= 0 || (wfmt != 2 && sf == nullptr)) return (int)cudaErrorInvalidValue;
  GemvArgs a{};
  a.w = (const uint8_t*)w; a.sf = (const uint8_t*)sf; a.row_bytes = row_bytes; a.N = N; a.K = K;
  a.KB = K / 32; a.groups = groups; a.n = n; a.xq = (const uint8_t*)xq; a.xs = (const uint8_t*)xs;
  a.xb = (const __nv_bfloat16*)xb; a.xf = (const float*)xf; a.x_stride = x_stride; a.x_quant = x_quant;
  a.out_b = (__nv_bfloat16*)out_b; a.out_f = (float*)out_f; a.out_stride = out_stride;
  a.ksplit = ksplit < 1 ? 1 : ksplit; a.split_stride = split_stride;
  if (a.ksplit > 1 && (out_b || !out_f)) return (int)cudaErrorInvalidValue;
  if (wfmt == 0) return launch_gemv<0>(a, stream);
  if (wfmt == 1) return launch_gemv<1>(a, stream);
  return launch_gemv<2>(a, stream);
}

}  // extern "C"
