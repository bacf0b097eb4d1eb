// CSA2 sparse-MLA attention on tcgen05 for steps of many rows (prompt chunks, wide verify steps).
//
// One CTA = one row x one group of NH heads.  The row's keys (the causal window from the FP8 ring, then the
// selected compressed FP4 entries) are decoded once into a bf16 tile of 128 keys x 512 dims in shared memory,
// laid out as eight slabs of [128 keys x 64 dims] with the 128-byte swizzle.  The one latent row is key and
// value for every head, so the same tile feeds both contractions:
//
//   S^T[key, head] = K[key, :] . Q[head, :]      A = key tile, K-major (dims contiguous);  B = Q, K-major
//   O^T[dim, head] += V^T[dim, key] P^T[key, head]   A = the same tile read MN-major (dims are M);  B = P, K-major
//
// Both run as tcgen05.mma kind::f16 (bf16 in, fp32 accumulators in TMEM): S^T is 128 lanes (keys) x NH columns,
// O^T is four 128-dim tiles x NH columns.  FP8 x 2^k and FP4 x E4M3 products are exact in bf16, so QK^T sees the
// cache's exact values; P is rounded to bf16 for the second contraction (the CUDA-core rows kernel keeps it in
// fp32: this kernel is a tolerance arm, not a bit-exact one).  Softmax is online over tiles of 128 keys: the
// score tile goes TMEM -> registers -> shared memory (transposed), threads then own heads, and the running
// accumulator in TMEM is rescaled per column when a head's maximum moves.  The sink enters the denominator only.
// Query RoPE on load, inverse RoPE on the output's rope slice, optional two-term FP8 copy for the wo_a GEMM.
//
// No cluster, no multicast; every mbarrier wait is bounded and reports through the status word.
//
// Reference behaviour replaced: kernels/opt_mma_sm121.cu:1243 (opt_bulk_attn: one block per row, heads as the MMA M),
// kernels/flash_mla_csa2_common_sm121.cuh; docs/architecture/01-csa2-attention.md:98-104,212-229.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "k_common.cuh"

namespace sfb {

namespace atc {

constexpr int HD = 512;            // latent width
constexpr int KT = 128;            // keys per tile
constexpr int SLABS = HD / 64;     // 64 bf16 = one 128-byte swizzle row
constexpr int SLAB_BYTES = KT * 128;
constexpr int THREADS = 256;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// shared -> global bulk copy; the commit waits only until the copy has read its shared-memory source
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store_commit_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 version bit set), 128-byte swizzle.
//   K-major operand:  rows of 128 bytes, 8-row groups `sbo` bytes apart (lbo unused).
//   MN-major operand: 64 contiguous MN elements per 128-byte row, one row per k; 8-k groups `sbo` bytes apart,
//                     64-element MN blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}
// kind::f16, bf16 operands, fp32 accumulator; a_mn: A operand is MN-major
__device__ __forceinline__ uint32_t make_idesc(int M, int N, int a_mn) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)((N >> 3) & 63) << 17;
  d |= (uint32_t)((M >> 4) & 31) << 24;
  return d;
}
// byte offset of 16-byte chunk `c16` (0..7) of row `r` inside a 128-byte-swizzled slab
__device__ __forceinline__ uint32_t swz(int r, int c16) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c16 ^ (r & 7)) << 4)); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

}  // namespace atc

struct AttnTcArgs {
  const __nv_bfloat16* q;   // [n, q_stride]; head h at h*512
  int64_t q_stride;
  const float2* rope;       // [n, rope_stride]: (cos, sin) of the row's position
  int rope_stride;
  const int* row_lane;
  const int* row_pos;
  const uint8_t* win_q;     // [lanes, ring, 512]
  const uint8_t* win_s;     // [lanes, ring, 16]
  int64_t win_lane_q, win_lane_s;
  const uint8_t* ckv_q;     // [lanes, max_entries, 256] (null: window only)
  const uint8_t* ckv_s;     // [lanes, max_entries, 32]
  int64_t ckv_lane_q, ckv_lane_s;
  const int* sel;           // [n, K] ascending ids, -1 padded
  const int* sel_count;     // [n]
  int K;
  const float* sink;        // [heads]
  __nv_bfloat16* out;       // [n, heads*512]
  uint8_t* out_q;           // optional two-term FP8 copy in blocks of 2*pair_block rows: hi rows then lo rows of each block
  uint8_t* out_atom;        // its scale atoms (128 rows per atom block)
  int pair_block;           // rows per block of the two-term copy (64), or 0: hi rows [0,n), lo rows [n,2n) as the rows kernel
  int n, heads, rd, window, ring;
  float scale;
  const int* win_lo;        // optional explicit inclusive window range per row
  const int* win_hi;
  Status* status;
  unsigned long long* marks;  // optional phase marks (builds with -DSFB_KERNEL_MARKS): sixteen %globaltimer words per CTA
  int marks_cap;
};

}  // namespace sfb

namespace sfb {

using namespace atc;

// slots: 0 entry, 1 set-up done, 2 queries staged, 3 first tile decoded, 4 its scores done, 5 its softmax done, 6 its value
// MMAs done, 7 exit, 8 epilogue starts (last tile done), 9 outputs staged, 10 copies issued, 11 / 12 thread 0 done with the
// bf16 pass / every thread done with it
#ifdef SFB_KERNEL_MARKS
#define SFB_ATTN_MARKS_ON 1
__device__ __forceinline__ void at_mark(const AttnTcArgs& a, int slot) {
  if (a.marks && threadIdx.x == 0) {
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    if (cta < a.marks_cap) a.marks[(size_t)cta * 16 + slot] = globaltimer_ns();
  }
}
#else
#define SFB_ATTN_MARKS_ON 0
__device__ __forceinline__ void at_mark(const AttnTcArgs&, int) {}
#endif

// ---- cache codes -> bf16 by bit placement ----------------------------------------------------------------------
// An E4M3 byte shifted into a bf16 (sign to bit 15, the seven exponent|mantissa bits to bits 4..10) is the code's value
// times 2^-120, subnormal codes included (they land on bf16 subnormals); an E2M1 nibble placed the same way (sign to bit
// 15, three bits to 6..8) is its value times 2^-126.  Two exact bf16 multiplications by powers of two (the second one
// carrying the block scale) undo the factor; every intermediate is representable, so the result is the exact product.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_raw(uint32_t two_bytes_in_high_halves) {
  // input: byte a in bits 8..15, byte b in bits 24..31
  const uint32_t t = two_bytes_in_high_halves;
  return (t & 0x80008000u) | ((t >> 4) & 0x07f007f0u);
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf16x2_splat(float f) {
  __nv_bfloat162 r = __float2bfloat162_rn(f);
  return *reinterpret_cast<uint32_t*>(&r);
}
// 16 E4M3 codes (one uint4) with one power-of-two scale -> two uint4 of bf16; m1, m2: splatted bf16 multipliers
__device__ __forceinline__ void fp8x16_to_bf16(const uint4& v, uint32_t m1, uint32_t m2, uint4& o0, uint4& o1) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t r[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = __byte_perm(w[i], 0u, 0x1404);   // bytes: [0, b0, 0, b1] -> b0 in bits 8..15, b1 in bits 24..31
    const uint32_t hi = __byte_perm(w[i], 0u, 0x3424);   // b2, b3
    r[2 * i] = bf16x2_mul(bf16x2_mul(e4m3x2_to_bf16x2_raw(lo), m1), m2);
    r[2 * i + 1] = bf16x2_mul(bf16x2_mul(e4m3x2_to_bf16x2_raw(hi), m1), m2);
  }
  o0 = make_uint4(r[0], r[1], r[2], r[3]);
  o1 = make_uint4(r[4], r[5], r[6], r[7]);
}
// 8 E2M1 codes (one 32-bit word, element i in nibble i) -> one uint4 of bf16
__device__ __forceinline__ uint4 fp4x8_to_bf16(uint32_t w, uint32_t m1, uint32_t m2) {
  uint32_t r[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = (w >> (8 * i)) & 0xffu;
    const uint32_t lanes = (x & 0xfu) | ((x & 0xf0u) << 12);          // nibble 0 in bits 0..3, nibble 1 in bits 16..19
    const uint32_t raw = ((lanes & 0x00080008u) << 12) | ((lanes & 0x00070007u) << 6);
    r[i] = bf16x2_mul(bf16x2_mul(raw, m1), m2);
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

template <int NH>
struct AttnTcSmem {
  alignas(1024) uint8_t kv[SLABS * SLAB_BYTES];   // 128 keys x 512 dims bf16, eight swizzled slabs
  alignas(1024) uint8_t q[SLABS * NH * 128];      // NH heads x 512 dims bf16
  alignas(1024) uint8_t p[2 * NH * 128];          // NH heads x 128 keys bf16 (two slabs of 64 keys)
  float sbuf[(NH < 32 ? NH : 32)][KT + 1];        // scores of the tile, head-major: 32 heads per softmax pass
  alignas(8) float red[THREADS];                  // per (key part, head) partial max / sum; outside the softmax: the row's rope table
  float fac[NH];                                  // per-head rescale of the running accumulator; 1/denominator at the end
  alignas(8) uint64_t bar;                        // score MMAs done (two issuing threads)
  alignas(8) uint64_t bar_pv;                     // value MMAs done (four issuing threads)
  uint32_t tmem_base;
};

// grid (head groups, rows), 256 threads = two halves of four warps.  Half h of thread pair (key slot = tid % 128) decodes
// dims [256 h, 256 h + 256) of its key; in TMEM accesses warp w and warp w + 4 share lanes 32 (w % 4).. and split the
// columns (score tile) or the 128-dim output tiles (half h owns tiles 2h, 2h + 1).  For the softmax a thread owns head
// tid % NH over the key part tid / NH.
template <int NH>
__global__ void __launch_bounds__(THREADS, 1) attn_tc_kernel(AttnTcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = AttnTcSmem<NH>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  // scores: two partial accumulators (latent dims 0..255 and 256..511, one issuing thread each, added when they are read);
  // output: four 128-dim tiles (one issuing thread each).  A thread issues one tcgen05 operation per ~80 cycles whatever its
  // size, and with 32-column MMAs that paced the tile.
  constexpr uint32_t TMEM_COLS = NH * 6 <= 128 ? 128 : (NH * 6 <= 256 ? 256 : 512);
  // the softmax runs over SH heads at a time (all of them up to 32; two passes for a 64-head group, which halves the
  // conversions of the key tiles per row against two 32-head CTAs)
  constexpr int SH = NH < 32 ? NH : 32;
  constexpr int NPASS = NH / SH;
  constexpr int PARTS = THREADS / SH;      // key parts per head in the softmax
  constexpr int KPP = KT / PARTS;          // keys per part
  constexpr int CH = SH / 2;               // score columns per half and pass
  constexpr float LOG2E = 1.4426950408889634f;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = tid >> 7, key_slot = tid & 127;
  const int hg = blockIdx.x, row = blockIdx.y;

  at_mark(a, 0);
  if (tid == 0) {
    mbar_init(&S.bar, 2);
    mbar_init(&S.bar_pv, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  at_mark(a, 1);
  const uint32_t tmem = S.tmem_base;
  const uint32_t t_s = tmem, t_o = tmem + 2 * NH;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

  const int pos = a.row_pos[row], L = a.row_lane[row];
  const int r0 = HD - a.rd;
  // (cos, sin) of the row's position for the rd / 2 roped pairs, kept in the softmax scratch while no softmax runs: for the
  // queries before the first tile's scores, again for the outputs after the last tile (rd <= THREADS)
  float2* rope_tab = reinterpret_cast<float2*>(S.red);
  if (tid < (a.rd >> 1)) rope_tab[tid] = a.rope[(size_t)row * a.rope_stride + tid];      // visible after the first barrier below
  // ---- queries of the group's heads: asynchronous 16-byte copies into the swizzled K-major tile; they land while the
  // first key tile is decoded, and the rope of the last rd dims is applied in place after that ----
  for (int idx = tid; idx < NH * 64; idx += THREADS) {
    const int hh = idx >> 6, c = idx & 63;          // head in group, 8-dim chunk
    const int ghead = hg * NH + hh;
    uint8_t* dst = S.q + (c >> 3) * (NH * 128) + swz(hh, c & 7);
    if (ghead < a.heads) cp_async16(smem_u32(dst), a.q + (size_t)row * a.q_stride + (size_t)ghead * HD + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  at_mark(a, 2);
  const int w_first = a.win_lo ? a.win_lo[row] : (pos - a.window + 1 > 0 ? pos - a.window + 1 : 0);
  const int n_win = (a.win_hi ? a.win_hi[row] : pos) - w_first + 1;
  const int n_sel = a.ckv_q ? a.sel_count[row] : 0;
  const int total = n_win + n_sel;
  const int tiles = (total + KT - 1) / KT;
  const int my_head = tid % SH, my_part = tid / SH;
  float m_run[NPASS], l_run[NPASS];        // identical in every thread that shares my_head
#pragma unroll
  for (int ps = 0; ps < NPASS; ++ps) { m_run[ps] = -1e30f; l_run[ps] = 0.f; }
  uint32_t parity = 0;
  bool ok = true;
  const float sl2 = a.scale * LOG2E;
  const uint32_t M60 = bf16x2_splat(1.152921504606847e18f);      // 2^60
  const uint32_t M100 = bf16x2_splat(1.2676506002282294e30f);    // 2^100

  // the FP4 codes and scales of the NEXT tile's compressed entry are requested while the current tile is multiplied and
  // normalised, so that the gather's trip to L2 / HBM is not on the tile's critical path
  uint4 nraw[8], nsc4;
  bool have_next = false;
#pragma unroll 1
  for (int tile = 0; tile < tiles && ok; ++tile) {
    // ---- decode dims [256 half, +256) of key slot `key_slot` into the bf16 tile ----
    {
      const int e = tile * KT + key_slot;
      uint8_t* rowp = S.kv;
      if (e < n_win) {
        const int slot = (w_first + e) % a.ring;
        const uint8_t* kq = a.win_q + (size_t)L * a.win_lane_q + (size_t)slot * HD + half * 256;
        const uint8_t* ks = a.win_s + (size_t)L * a.win_lane_s + (size_t)slot * (HD / 32) + half * 8;
        const uint2 sc2 = *reinterpret_cast<const uint2*>(ks);
        const uint8_t* scb = reinterpret_cast<const uint8_t*>(&sc2);
#pragma unroll 1
        for (int b = 0; b < 2; ++b) {          // two batches of eight 16-byte loads in flight
          uint4 raw[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) raw[i] = *reinterpret_cast<const uint4*>(kq + (b * 8 + i) * 16);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            // block scale 2^(code - 127) times the 2^60 left over from the raw placement (2^-120 = 2^-60 2^-60)
            const uint32_t m2 = bf16x2_splat(ue8m0_shifted(scb[(b * 8 + i) >> 1], 60));
            uint4 o0, o1;
            fp8x16_to_bf16(raw[i], M60, m2, o0, o1);
            const int c = half * 32 + (b * 8 + i) * 2;
            *reinterpret_cast<uint4*>(rowp + (c >> 3) * SLAB_BYTES + swz(key_slot, c & 7)) = o0;
            *reinterpret_cast<uint4*>(rowp + ((c + 1) >> 3) * SLAB_BYTES + swz(key_slot, (c + 1) & 7)) = o1;
          }
        }
      } else if (e < total) {
        uint4 raw[8], sc4;
        if (have_next) {
#pragma unroll
          for (int i = 0; i < 8; ++i) raw[i] = nraw[i];
          sc4 = nsc4;
        } else {
          const int id = a.sel[(size_t)row * a.K + (e - n_win)];
          const uint8_t* kq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)id * (HD / 2) + half * 128;
          const uint8_t* ks = a.ckv_s + (size_t)L * a.ckv_lane_s + (size_t)id * (HD / 16) + half * 16;
#pragma unroll
          for (int i = 0; i < 8; ++i) raw[i] = *reinterpret_cast<const uint4*>(kq + i * 16);
          sc4 = *reinterpret_cast<const uint4*>(ks);
        }
        const uint8_t* scb = reinterpret_cast<const uint8_t*>(&sc4);
#pragma unroll
        for (int i = 0; i < 8; ++i) {          // 32 codes per uint4, two E4M3 scales
          const uint32_t w4[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // E4M3 scale (exact in bf16) times the 2^26 left over: 2^-126 = 2^-100 2^-26
            const uint32_t m2 = bf16x2_splat(e4m3_to_f32(scb[2 * i + (j >> 1)]) * 67108864.f);
            const int c = half * 32 + i * 4 + j;
            *reinterpret_cast<uint4*>(rowp + (c >> 3) * SLAB_BYTES + swz(key_slot, c & 7)) = fp4x8_to_bf16(w4[j], M100, m2);
          }
        }
      } else {
        // past the row's last key: zeros, so that the value contraction adds 0 x 0 and never meets stale bits
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 4
        for (int c = half * 32; c < half * 32 + 32; ++c) *reinterpret_cast<uint4*>(rowp + (c >> 3) * SLAB_BYTES + swz(key_slot, c & 7)) = z;
      }
    }
    {
      const int en = (tile + 1) * KT + key_slot;      // this thread's entry of the next tile
      have_next = en >= n_win && en < total;
      if (have_next) {
        const int id = a.sel[(size_t)row * a.K + (en - n_win)];
        const uint8_t* kq = a.ckv_q + (size_t)L * a.ckv_lane_q + (size_t)id * (HD / 2) + half * 128;
        const uint8_t* ks = a.ckv_s + (size_t)L * a.ckv_lane_s + (size_t)id * (HD / 16) + half * 16;
#pragma unroll
        for (int i = 0; i < 8; ++i) nraw[i] = *reinterpret_cast<const uint4*>(kq + i * 16);
        nsc4 = *reinterpret_cast<const uint4*>(ks);
      }
    }
    if (tile == 0) {
      // the queries have landed: rope on dims [r0, 512) of every head, in place (one 8-dim chunk per thread and turn)
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      const int rc = a.rd >> 3;                     // roped chunks per head
      for (int idx = tid; idx < NH * rc; idx += THREADS) {
        const int hh = idx / rc, c = (r0 >> 3) + idx % rc;
        if (hg * NH + hh >= a.heads) continue;
        uint4* qp = reinterpret_cast<uint4*>(S.q + (c >> 3) * (NH * 128) + swz(hh, c & 7));
        uint4 v = *qp;
        __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 c2 = rope_tab[((c * 8 - r0) >> 1) + j];
          const float x = __bfloat162float(pr[j].x), y = __bfloat162float(pr[j].y);
          pr[j] = __floats2bfloat162_rn(x * c2.x - y * c2.y, x * c2.y + y * c2.x);
        }
        *qp = v;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (tile == 0) at_mark(a, 3);
    // ---- S^T = K Q^T ----
    if (warp < 2 && elect_one()) {      // warp 0: slabs 0..3 into S0, warp 1: slabs 4..7 into S1
      tc_fence_after();
      const uint32_t idesc = make_idesc(128, NH, 0);
      const uint32_t kvb = smem_u32(S.kv), qb = smem_u32(S.q);
      const int s0 = warp * (SLABS / 2);
#pragma unroll 1
      for (int s = s0; s < s0 + SLABS / 2; ++s) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_f16(t_s + warp * NH, make_desc(kvb + s * SLAB_BYTES + kk * 32, 1024, 16), make_desc(qb + s * (NH * 128) + kk * 32, 1024, 16),
                     idesc, ((s - s0) | kk) ? 1u : 0u);
      }
      tc_commit(&S.bar);
    }
    ok = mbar_wait(&S.bar, parity);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) break;
    tc_fence_after();
    if (tile == 0) at_mark(a, 4);
    // ---- scores: TMEM (lane = key) -> shared memory, head-major; each half takes half of the pass's head columns ----
    int any_rescale = 0;
#pragma unroll 1
    for (int ps = 0; ps < NPASS; ++ps) {
      {
        const bool valid = tile * KT + key_slot < total;
        if constexpr (CH == 16) {
          uint32_t v[16], v1[16];
          tc_ld16(t_s + lane_base + ps * SH + half * CH, v);
          tc_ld16(t_s + NH + lane_base + ps * SH + half * CH, v1);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            S.sbuf[half * CH + j][key_slot] = valid ? (__uint_as_float(v[j]) + __uint_as_float(v1[j])) * sl2 : -INFINITY;
        } else {
          uint32_t v[8], v1[8];
          tc_ld8(t_s + lane_base + ps * SH + half * CH, v);
          tc_ld8(t_s + NH + lane_base + ps * SH + half * CH, v1);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            S.sbuf[half * CH + j][key_slot] = valid ? (__uint_as_float(v[j]) + __uint_as_float(v1[j])) * sl2 : -INFINITY;
        }
      }
      __syncthreads();
      // ---- online softmax: thread = (head of the pass, key part) ----
      float mloc = -INFINITY;
      const float* srow = &S.sbuf[my_head][my_part * KPP];
#pragma unroll
      for (int i = 0; i < KPP; ++i) mloc = fmaxf(mloc, srow[i]);
      S.red[my_part * SH + my_head] = mloc;
      __syncthreads();
      float m_new = m_run[ps];
#pragma unroll
      for (int pp = 0; pp < PARTS; ++pp) m_new = fmaxf(m_new, S.red[pp * SH + my_head]);
      // the reference exponent moves only when the maximum grew by more than 2^8: probabilities up to 256 are as exact in
      // bf16 as probabilities up to 1, numerator and denominator use the same reference, and the running output then
      // rarely needs rescaling (a read-modify-write of the whole TMEM accumulator per tile)
      if (m_new - m_run[ps] <= 8.f) m_new = m_run[ps];
      const float corr = exp2f(m_run[ps] - m_new);
      if (corr != 1.f) any_rescale = 1;
      __syncthreads();                 // everyone has read the maxima before the sums overwrite them
      float lsum = 0.f;
      const int gh = ps * SH + my_head;            // head inside the CTA's group
#pragma unroll
      for (int i = 0; i < KPP; i += 2) {
        const float p0 = exp2f(srow[i] - m_new), p1 = exp2f(srow[i + 1] - m_new);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        lsum += __bfloat162float(pb.x) + __bfloat162float(pb.y);      // the denominator sums what the value contraction multiplies
        const int key = my_part * KPP + i;
        *reinterpret_cast<__nv_bfloat162*>(S.p + (key >> 6) * (NH * 128) + swz(gh, (key & 63) >> 3) + (key & 7) * 2) = pb;
      }
      S.red[my_part * SH + my_head] = lsum;
      if (my_part == 0) S.fac[gh] = corr;
      __syncthreads();
      float lt = 0.f;
#pragma unroll
      for (int pp = 0; pp < PARTS; ++pp) lt += S.red[pp * SH + my_head];
      l_run[ps] = l_run[ps] * corr + lt;
      m_run[ps] = m_new;
      if (NPASS > 1) __syncthreads();    // the next pass overwrites sbuf and red
    }
    // ---- rescale the running O^T (lane = dim, column = head): half h owns the 128-dim tiles 2h and 2h + 1 ----
    any_rescale = __syncthreads_or(any_rescale);      // CTA-uniform: did any head's reference exponent move?
    if (tile == 0) at_mark(a, 5);
    if (tile > 0 && any_rescale) {
#pragma unroll 1
      for (int jj = 0; jj < 2; ++jj) {
        const int j = half * 2 + jj;
#pragma unroll 1
        for (int c0 = 0; c0 < NH; c0 += 16) {
          uint32_t v[16];
          tc_ld16(t_o + lane_base + j * NH + c0, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * S.fac[c0 + i]);
          tc_st16(t_o + lane_base + j * NH + c0, v);
        }
      }
      tc_wait_st();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    // ---- O^T += V^T P^T ----
    if (warp < 4 && elect_one()) {      // warp j issues the 128-dim output tile j
      tc_fence_after();
      const uint32_t idesc = make_idesc(128, NH, 1);
      const uint32_t kvb = smem_u32(S.kv), pb = smem_u32(S.p);
      const int j = warp;
#pragma unroll
      for (int t8 = 0; t8 < KT / 16; ++t8)
        tc_mma_f16(t_o + j * NH, make_desc(kvb + (2 * j) * SLAB_BYTES + t8 * 2048, 1024, SLAB_BYTES),
                   make_desc(pb + (t8 >> 2) * (NH * 128) + (t8 & 3) * 32, 1024, 16), idesc, (tile > 0 || t8 > 0) ? 1u : 0u);
      tc_commit(&S.bar_pv);
    }
    ok = mbar_wait(&S.bar_pv, parity);
    parity ^= 1;
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc_fence_after();
    if (tile == 0) at_mark(a, 6);
  }
  at_mark(a, 8);

  // ---- epilogue: O^T / denominator (sink in the denominator only), inverse rope, bf16 (+ two-term FP8 copy) ----
  if (ok) {
    if (tid < (a.rd >> 1)) rope_tab[tid] = a.rope[(size_t)row * a.rope_stride + tid];      // the last softmax is done with the scratch
    if (my_part == 0) {
#pragma unroll
      for (int ps = 0; ps < NPASS; ++ps) {
        const int ghead = hg * NH + ps * SH + my_head;
        const float sk = ghead < a.heads ? a.sink[ghead] : 0.f;
        S.fac[ps * SH + my_head] = 1.f / (l_run[ps] + exp2f(sk * LOG2E - m_run[ps]));
      }
    }
    __syncthreads();
    const size_t Wd = (size_t)a.heads * HD;
    int row_hi = row, row_lo = a.n + row;
    if (a.pair_block > 0) {
      row_hi = (row / a.pair_block) * 2 * a.pair_block + row % a.pair_block;
      row_lo = row_hi + a.pair_block;
    }
    const int KB = a.heads * (HD / 32);
    // The row's outputs are collected in the (now idle) KV tile buffer - bf16 [NH][512], the two FP8 terms [NH][512] each and
    // their scale bytes - and leave the SM as three bulk copies plus one 4-byte word of scales per thread: the head groups
    // are contiguous in every output.  (Element stores from inside the column loop dominated the kernel.)
    __nv_bfloat16* st_o = reinterpret_cast<__nv_bfloat16*>(S.kv);
    uint8_t* st_hi = S.kv + NH * HD * 2;
    uint8_t* st_lo = st_hi + NH * HD;
    // scale codes of the hi term [NH * 16] and of the lo term: in the query buffer, which nothing reads any more (for a
    // 64-head group the three staged outputs fill the KV buffer exactly)
    uint8_t* st_sh = S.q;
    uint8_t* st_sl = st_sh + NH * (HD / 32);
    // pass 1: TMEM (lane = dim, column = head) -> bf16 [head][dim] in shared memory
#pragma unroll 1
    for (int jj = 0; jj < 2; ++jj) {
      const int j = half * 2 + jj;
      const int dim = j * 128 + (warp & 3) * 32 + lane;
      // every 16-head chunk of the tile is requested before the one wait: a load's round trip (several hundred cycles) was
      // paid once per chunk
      constexpr int NCH = NH / 16;
      uint32_t v[NCH][16];
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) tc_ld16(t_o + lane_base + j * NH + ch * 16, v[ch]);
      tc_wait_ld();
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        const int c0 = ch * 16;
#pragma unroll
        for (int i = 0; i < 16; ++i) st_o[(c0 + i) * HD + dim] = __float2bfloat16_rn(__uint_as_float(v[ch][i]) * S.fac[c0 + i]);
      }
    }
    // pass 2: inverse rope on the last rd dims and the two-term FP8 copy, both from the staged bf16 rows: sixteen consecutive dims of one head per thread and turn
    // (two neighbouring lanes share a 32-dim scale block), packed conversions, 16-byte stores.  (Quantising straight
    // from the TMEM layout - one dim per lane, one warp reduction per head - took 55 % of the CTA's life.)
    at_mark(a, 11);
    {
      __syncthreads();
      at_mark(a, 12);
      const int seg0 = r0 >> 4;                     // first 16-dim segment that carries rope (rd is a multiple of 32)
      for (int sgm = tid; sgm < NH * 32; sgm += THREADS) {
        const int hh = sgm >> 5, seg = sgm & 31;
        if (!a.out_q && seg < seg0) continue;
        uint4* src = reinterpret_cast<uint4*>(st_o + hh * HD + seg * 16);
        const uint4 a0 = src[0], a1 = src[1];
        uint32_t w[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        if (seg >= seg0) {
          // inverse rope on the segment's eight (even, odd) pairs, one word each; written back for the bf16 output
          const float2* rt = &rope_tab[(seg * 16 - r0) >> 1];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float x = __uint_as_float(w[k] << 16), y = __uint_as_float(w[k] & 0xffff0000u);
            const float2 c2 = rt[k];
            w[k] = pack_bf16(__fmaf_rn(x, c2.x, __fmul_rn(y, c2.y)), __fmaf_rn(y, c2.x, -__fmul_rn(x, c2.y)));
          }
          src[0] = make_uint4(w[0], w[1], w[2], w[3]);
          src[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
        if (!a.out_q) continue;
        float o[16];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          o[2 * k] = __uint_as_float(w[k] << 16);
          o[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
          amax = fmaxf(amax, fmaxf(fabsf(o[2 * k]), fabsf(o[2 * k + 1])));      // fmaxf drops a NaN operand: it counts as 0
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        const uint8_t sc = act_scale_code_fp8(amax);
        const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float x0 = o[2 * k] * inv, x1 = o[2 * k + 1] * inv;
          const uint16_t h2 = enc_e4m3x2(x0, x1);
          uint32_t hf;
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hf) : "h"(h2));
          const float2 dq = __half22float2(*reinterpret_cast<const __half2*>(&hf));
          const uint16_t l2 = enc_e4m3x2((x0 - dq.x) * 16.f, (x1 - dq.y) * 16.f);
          if (k & 1) { hw[k >> 1] |= (uint32_t)h2 << 16; lw[k >> 1] |= (uint32_t)l2 << 16; }
          else { hw[k >> 1] = h2; lw[k >> 1] = l2; }
        }
        *reinterpret_cast<uint4*>(st_hi + hh * HD + seg * 16) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4*>(st_lo + hh * HD + seg * 16) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        if (!(tid & 1)) {
          st_sh[hh * (HD / 32) + (seg >> 1)] = sc;
          st_sl[hh * (HD / 32) + (seg >> 1)] = sc >= 4 ? (uint8_t)(sc - 4) : (uint8_t)0;
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    at_mark(a, 9);
    const int head0 = hg * NH;
    const int nvalid = a.heads - head0 < NH ? a.heads - head0 : NH;        // heads of this group that exist
    if (nvalid > 0) {
      if (tid == 0) {
        bulk_store(a.out + ((size_t)row * a.heads + head0) * HD, smem_u32(st_o), (uint32_t)nvalid * HD * 2);
        bulk_store_commit_wait_read();
      } else if (tid == 32 && a.out_q) {
        bulk_store(a.out_q + (size_t)row_hi * Wd + (size_t)head0 * HD, smem_u32(st_hi), (uint32_t)nvalid * HD);
        bulk_store_commit_wait_read();
      } else if (tid == 64 && a.out_q) {
        bulk_store(a.out_q + (size_t)row_lo * Wd + (size_t)head0 * HD, smem_u32(st_lo), (uint32_t)nvalid * HD);
        bulk_store_commit_wait_read();
      }
      if (a.out_q) {
        // scale bytes: four k-blocks (one k-atom) of a row are four consecutive bytes of the atom layout
        for (int wd = tid; wd < nvalid * (HD / 128); wd += THREADS) {
          const int kb = head0 * (HD / 32) + wd * 4;
          *reinterpret_cast<uint32_t*>(a.out_atom + sf_offset(row_hi, kb, KB)) = reinterpret_cast<const uint32_t*>(st_sh)[wd];
          *reinterpret_cast<uint32_t*>(a.out_atom + sf_offset(row_lo, kb, KB)) = reinterpret_cast<const uint32_t*>(st_sl)[wd];
        }
      }
    }
  } else if (tid == 0) {
    status_set(a.status, ST_TIMEOUT, 50, blockIdx.x, blockIdx.y);
  }
  at_mark(a, 10);
  tc_fence_before();
  __syncthreads();
  at_mark(a, 7);
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace sfb

using namespace sfb;

extern "C" {

// Phase marks of the NEXT sfb_attn_tc launch of this thread (measurement builds only).
static thread_local unsigned long long* g_attn_marks = nullptr;
static thread_local int g_attn_marks_cap = 0;
int sfb_attn_set_marks(void* buf, int cap_ctas) {
  if (buf && !SFB_ATTN_MARKS_ON) return (int)cudaErrorNotSupported;
  g_attn_marks = (unsigned long long*)buf; g_attn_marks_cap = buf ? cap_ctas : 0;
  return 0;
}

// Same arguments as sfb_attn_rows_range plus the layout of the two-term copy (pair_block) and the status word.
// hd must be 512; rd a multiple of 32.  Heads are processed in groups of 64 (16 or 32 when the rank holds at most that many).
int sfb_attn_tc(const void* q, int64_t q_stride, const void* rope, int rope_stride, const int* row_lane, const int* row_pos,
                const void* win_q, const void* win_s, int64_t win_lane_q, int64_t win_lane_s, const void* ckv_q, const void* ckv_s,
                int64_t ckv_lane_q, int64_t ckv_lane_s, const int* sel, const int* sel_count, int K, const float* sink, void* out,
                void* out_q, void* out_atom, int pair_block, int n, int heads, int hd, int rd, int window, int ring, float scale,
                const int* win_lo, const int* win_hi, void* status, cudaStream_t stream) {
  if (hd != atc::HD || rd % 32 || rd > 256 || n < 1 || heads < 1 || (q_stride % 8)) return (int)cudaErrorInvalidValue;
  AttnTcArgs a{};
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride; a.rope = (const float2*)rope; a.rope_stride = rope_stride;
  a.row_lane = row_lane; a.row_pos = row_pos; a.win_q = (const uint8_t*)win_q; a.win_s = (const uint8_t*)win_s;
  a.win_lane_q = win_lane_q; a.win_lane_s = win_lane_s; a.ckv_q = (const uint8_t*)ckv_q; a.ckv_s = (const uint8_t*)ckv_s;
  a.ckv_lane_q = ckv_lane_q; a.ckv_lane_s = ckv_lane_s; a.sel = sel; a.sel_count = sel_count; a.K = K; a.sink = sink;
  a.out = (__nv_bfloat16*)out; a.out_q = (uint8_t*)out_q; a.out_atom = (uint8_t*)out_atom; a.pair_block = pair_block;
  a.n = n; a.heads = heads; a.rd = rd; a.window = window; a.ring = ring; a.scale = scale; a.win_lo = win_lo; a.win_hi = win_hi;
  a.status = (Status*)status;
  a.marks = g_attn_marks; a.marks_cap = g_attn_marks_cap;
  g_attn_marks = nullptr; g_attn_marks_cap = 0;
  cudaError_t rc;
  if (heads <= 16) {
    const size_t smem = sizeof(AttnTcSmem<16>) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(attn_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    rc = sfb_launch(attn_tc_kernel<16>, dim3(1, n), dim3(atc::THREADS), smem, stream, a);
  } else if (heads <= 32) {
    const size_t smem = sizeof(AttnTcSmem<32>) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(attn_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    rc = sfb_launch(attn_tc_kernel<32>, dim3(1, n), dim3(atc::THREADS), smem, stream, a);
  } else {       // 64 heads per CTA: a row's key tiles are converted once for all of them
    const size_t smem = sizeof(AttnTcSmem<64>) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(attn_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    rc = sfb_launch(attn_tc_kernel<64>, dim3((heads + 63) / 64, n), dim3(atc::THREADS), smem, stream, a);
  }
  return (int)rc;
}

}  // extern "C"
