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
};

// grid (K/256 rounded up, n), block 256: one 32-group per warp
__global__ void __launch_bounds__(256) quant_rows_kernel(QuantArgs a) {
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

}  // namespace sfb

using namespace sfb;

extern "C" int sfb_quant_rows(const void* x, void* q, void* s, void* atom, int n, int K, int split, int split_off,
                              cudaStream_t stream) {
  if (K % 32) return (int)cudaErrorInvalidValue;
  QuantArgs a{(const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)s, (uint8_t*)atom, n, K, split, split_off};
  quant_rows_kernel<<<dim3((K + 255) / 256, n), 256, 0, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}
