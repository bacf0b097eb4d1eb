// Activation quantisers that feed the tensor-core arm: bf16 rows -> per-32 FP8 codes with row-major
// scales and scale atoms; optionally as a two-term split (value = hi + lo, the second term carrying
// the residual at 1/16 of the block scale) so that a bf16 activation goes through the FP8 tensor
// path with bf16-level accuracy (used where the model multiplies bf16 activations, e.g. wo_a).
//
// Reference behaviour: kernels/swiglu_mxfp8_quant_sm121.cu (mxfp8_quantize_activations:47),
// kernels/m4_activation_quant_sm121.cuh (scale rule).
#include "k_common.cuh"

namespace sfb {

struct QuantArgs {
  const __nv_bfloat16* x;   // [n, K]
  uint8_t* q;               // [rows_out, K]: rows 0..n-1 = hi; rows split_off.. = lo when split
  uint8_t* s;               // optional row-major scales [rows_out, K/32]
  uint8_t* atom;            // optional atoms (rows = output rows)
  int n, K, split, split_off;
  uint32_t* epoch;          // optional step counter of a fused collective, advanced by `epoch_add` by one thread of the launch
  uint32_t epoch_add;       // (saves the one-thread launch that did nothing else)
};

// grid (K/256 rounded up, n), block 256: one 32-group per warp
__global__ void __launch_bounds__(256) quant_rows_kernel(QuantArgs a) {
  if (a.epoch && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *a.epoch += a.epoch_add;
  const int row = blockIdx.y;
  const int col = blockIdx.x * 256 + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const int KB = a.K / 32;
  float v = col < a.K ? bf16_to_f(a.x[(size_t)row * a.K + col]) : 0.f;
  const float amax = warp_max(fabsf(v));
  const uint8_t sc = act_scale_code_fp8(amax);
  const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
  const uint8_t hi = enc_e4m3(v * inv);
  if (col < a.K) {
    a.q[(size_t)row * a.K + col] = hi;
    if (lane == 0) {
      if (a.s) a.s[(size_t)row * KB + col / 32] = sc;
      if (a.atom) a.atom[sf_offset(row, col / 32, KB)] = sc;
    }
  }
  if (a.split) {
    const float r = v * inv - e4m3_to_f32(hi);   // exact in fp32
    const uint8_t lo = enc_e4m3(r * 16.f);
    const uint8_t sc_lo = sc >= 4 ? (uint8_t)(sc - 4) : (uint8_t)0;
    const int orow = a.split_off + row;
    if (col < a.K) {
      a.q[(size_t)orow * a.K + col] = lo;
      if (lane == 0) {
        if (a.s) a.s[(size_t)orow * KB + col / 32] = sc_lo;
        if (a.atom) a.atom[sf_offset(orow, col / 32, KB)] = sc_lo;
      }
    }
  }
}


// Bulk variant (many rows): a thread owns 8 consecutive columns (one 16-byte load, one 8-byte store), four lanes
// share a 32-column scale group.  grid (ceil(K / 1024), n), block 128.
__global__ void __launch_bounds__(128) quant_rows_vec_kernel(QuantArgs a) {
  if (a.epoch && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *a.epoch += a.epoch_add;
  const int row = blockIdx.y;
  const int col = (blockIdx.x * 128 + threadIdx.x) * 8;
  const int KB = a.K / 32;
  float v[8];
  float amax = 0.f;
  if (col < a.K) {
    const uint4 u = *reinterpret_cast<const uint4*>(a.x + (size_t)row * a.K + col);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (col >= a.K) return;
  const uint8_t sc = act_scale_code_fp8(amax);
  const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
  uint2 q;
  uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
  for (int j = 0; j < 8; ++j) qb[j] = enc_e4m3(v[j] * inv);
  *reinterpret_cast<uint2*>(a.q + (size_t)row * a.K + col) = q;
  if ((threadIdx.x & 3) == 0) {
    if (a.s) a.s[(size_t)row * KB + col / 32] = sc;
    if (a.atom) a.atom[sf_offset(row, col / 32, KB)] = sc;
  }
}

}  // namespace sfb

using namespace sfb;

static int quant_rows_launch(const QuantArgs& a, cudaStream_t stream);

extern "C" int sfb_quant_rows(const void* x, void* q, void* s, void* atom, int n, int K, int split, int split_off,
                              cudaStream_t stream) {
  if (K % 32) return (int)cudaErrorInvalidValue;
  QuantArgs a{(const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)s, (uint8_t*)atom, n, K, split, split_off, nullptr, 0u};
  return quant_rows_launch(a, stream);
}

// The same, and *epoch += epoch_add inside the launch (the fused collectives count their steps on the device).
extern "C" int sfb_quant_rows_bump(const void* x, void* q, void* s, void* atom, int n, int K, void* epoch, uint32_t epoch_add,
                                   cudaStream_t stream) {
  if (K % 32 || !epoch) return (int)cudaErrorInvalidValue;
  QuantArgs a{(const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)s, (uint8_t*)atom, n, K, 0, 0, (uint32_t*)epoch, epoch_add};
  return quant_rows_launch(a, stream);
}

static int quant_rows_launch(const QuantArgs& a, cudaStream_t stream) {
  const int n = a.n, K = a.K, split = a.split;
  if (!split && n >= 32) {      // same arithmetic, wider accesses
    quant_rows_vec_kernel<<<dim3((K + 1023) / 1024, n), 128, 0, stream>>>(a);
    return SFB_CHECK_LAUNCH();
  }
  quant_rows_kernel<<<dim3((K + 255) / 256, n), 256, 0, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}
