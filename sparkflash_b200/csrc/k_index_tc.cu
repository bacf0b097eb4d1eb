// CSA2 indexer scores on tcgen05: score[row, t] = sum_h relu(q[row, h, :] . k[t, :]) * w[row, h]
//
// Keys (MXFP4, 128 dims, one UE8M0 scale per 32) are the M = 128 operand of one block-scaled MMA step
// (kind::mxf8f6f4 with E2M1 on both sides, K = 128 = four K = 32 instructions); the queries of one or four rows
// (32 heads each, MXFP4) are the N = 32 / 128 operand.  A CTA takes one tile of 128 cache entries: TMA unpacks the
// packed FP4 codes into 8-bit containers, the entry scales (stored [entry][4]) are permuted into the 128 x 4 atom
// order in shared memory, and the epilogue reads the 128 x N accumulator from TMEM with the entry as the lane: each
// thread applies relu, the head weights and the head sum for its entry and writes one score per row.  Entries at or
// past the row's compressed length, or outside the candidate blocks, get -inf.
//
// The products are those of the CUDA-core kernel (exact FP4 x FP4 with power-of-two scales); the fp32 sum over the
// 128 dims runs in the tensor core's order.
//
// Reference behaviour replaced: kernels/opt_mma_sm121.cu:1066 (opt_mma_index_scores on mxf4nvf4 mma.sync),
// kernels/opt_select_sm121.cu:563-885; docs/architecture/01-csa2-attention.md:152-188.
#include <cuda.h>

#include "k_common.cuh"

namespace sfb {
namespace itc {

constexpr int THREADS = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void tc_mma_bs(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t lbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7) << 61;
  return d;
}
// kind::mxf8f6f4.block_scale: operand formats at bits 7-9 / 10-12 (E2M1 = 5), N/8 at 17-22, UE8M0 scales (bit 23), M/16 at 24-28
__device__ __forceinline__ uint32_t make_idesc(int a_fmt, int b_fmt, int M, int N) {
  uint32_t d = 0;
  d |= (uint32_t)(a_fmt & 7) << 7;
  d |= (uint32_t)(b_fmt & 7) << 10;
  d |= (uint32_t)((N >> 3) & 63) << 17;
  d |= 1u << 23;
  d |= (uint32_t)((M >> 4) & 31) << 24;
  return d;
}

}  // namespace itc

// ---- query side: rope, MXFP4 codes (packed) and scale atoms, head weights -----------------------------------------
struct IndexQ4Args {
  const __nv_bfloat16* qraw;  // [n, q_stride], indexer part at q_off: [32 heads, 128]
  int64_t q_stride, q_off;
  const float* wraw;          // [n, w_stride] weights_proj output at w_off: [32]
  int64_t w_stride, w_off;
  const float2* rope;
  int rope_stride;
  uint8_t* q4;                // [n * 32, 64] packed E2M1 (element 2i in the low nibble)
  uint8_t* q_atoms;           // rows_per_group * 32 query rows per 512-byte atom: group g at g * 512
  float* wt;                  // [n, 32]
  int n, rd, rows_per_group;
  float wscale;
};

// grid (n), block 256: warp w takes heads w, w + 8, ..; a lane owns four consecutive dims of the 128
__global__ void __launch_bounds__(256) index_q4_kernel(IndexQ4Args a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int INH = 32, IDH = 128;
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = IDH - a.rd;
  for (int h = warp; h < INH; h += 8) {
    const __nv_bfloat16* src = a.qraw + (size_t)row * a.q_stride + a.q_off + (size_t)h * IDH + lane * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = bf16_to_f(src[j]);
    const int e = lane * 4;
    if (e >= r0) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const float2 c2 = a.rope[(size_t)row * a.rope_stride + ((e + j - r0) >> 1)];
        const float x = v[j], y = v[j + 1];
        v[j] = x * c2.x - y * c2.y; v[j + 1] = x * c2.y + y * c2.x;
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = bfr(v[j]); amax = fmaxf(amax, fabsf(v[j])); }
    // one scale per 32 dims = 8 lanes
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const uint8_t sc = act_scale_code_fp4(amax);
    const float s = ue8m0_to_f32(sc);
    uint32_t codes = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) codes |= (uint32_t)f32_to_e2m1(v[j] / s) << (4 * j);
    *reinterpret_cast<uint16_t*>(a.q4 + ((size_t)row * INH + h) * (IDH / 2) + lane * 2) = (uint16_t)codes;
    if ((lane & 7) == 0) {
      const int g = row / a.rows_per_group, r = (row % a.rows_per_group) * INH + h;
      a.q_atoms[(size_t)g * 512 + sf_offset(r, lane >> 3, 4)] = sc;
    }
  }
  if (threadIdx.x < INH) a.wt[(size_t)row * INH + threadIdx.x] = bfr(a.wraw[(size_t)row * a.w_stride + a.w_off + threadIdx.x]) * a.wscale;
}

struct IndexTcArgs {
  const uint8_t* ik_s;      // [lanes, max_entries, 4] entry scales (UE8M0), row-major
  int64_t ik_lane_s;
  int64_t lane_rows;        // rows of one lane in the key tensor map (= max_entries)
  const uint8_t* q_atoms;   // one 512-byte atom per row group
  const float* wt;          // [n, 32]
  const int* row_lane;
  const int* row_pos;
  const uint8_t* cand;      // optional [n, cand_stride] block flags
  int64_t cand_stride;
  int cand_block;
  float* scores;            // [n, score_stride]
  int64_t score_stride;
  int n, ratio, max_len;
  Status* status;
};

template <int NP>
struct IndexTcSmem {
  alignas(1024) uint8_t a[128 * 128];     // key tile: 128 entries x 128 one-byte containers
  alignas(1024) uint8_t b[NP * 128];      // query rows
  alignas(128) uint8_t sfa[512];
  alignas(128) uint8_t sfb[512];
  float wt[NP];
  alignas(8) uint64_t full, done;
  uint32_t tmem_base;
};

// grid (entry tiles, row groups); NP = 32 (one row) or 128 (four consecutive rows of one lane)
template <int NP>
__global__ void __launch_bounds__(itc::THREADS) index_scores_tc_kernel(const __grid_constant__ CUtensorMap tmapK,
                                                                       const __grid_constant__ CUtensorMap tmapQ, IndexTcArgs a) {
  using namespace itc;
  extern __shared__ uint8_t smem_raw[];
  using Smem = IndexTcSmem<NP>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int RPG = NP / 32;
  constexpr uint32_t TMEM_COLS = NP + 8 <= 64 ? 64 : 256;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = blockIdx.x * 128, row0 = blockIdx.y * RPG;
  if (tid == 0) {
    mbar_init(&S.full, 1); mbar_init(&S.done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) { tmem_alloc(&S.tmem_base, TMEM_COLS); tmem_relinquish(); }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem = S.tmem_base;
  const uint32_t t_acc = tmem, t_sfa = tmem + NP, t_sfb = tmem + NP + 4;
  const int L = a.row_lane[row0];
  // longest compressed length among the group's rows: tiles wholly past it only write -inf
  int clen_max = 0;
#pragma unroll
  for (int r = 0; r < RPG; ++r)
    if (row0 + r < a.n) clen_max = max(clen_max, (a.row_pos[row0 + r] + 1) / a.ratio);
  const bool work = e0 < clen_max;
  bool ok = true;
  if (work) {
    if (warp == 0 && elect_one()) {
      mbar_expect_tx(&S.full, 128 * 64 + NP * 64 + 512);
      tma_load_2d(S.a, &tmapK, 0, (int)(L * a.lane_rows) + e0, &S.full);
      tma_load_2d(S.b, &tmapQ, 0, row0 * 32, &S.full);
      bulk_load(S.sfb, a.q_atoms + (size_t)blockIdx.y * 512, 512, &S.full);
    }
    {  // entry scales [entry][4] -> atom order: the word of entry r goes to word (r % 32) * 4 + r / 32
      const int ent = e0 + tid;
      uint32_t wv = 0x7f7f7f7fu;
      if (ent < a.max_len) wv = *reinterpret_cast<const uint32_t*>(a.ik_s + (size_t)L * a.ik_lane_s + (size_t)ent * 4);
      reinterpret_cast<uint32_t*>(S.sfa)[(tid & 31) * 4 + (tid >> 5)] = wv;
    }
    if (tid < NP) {
      const int r = row0 + tid / 32;
      S.wt[tid] = r < a.n ? a.wt[(size_t)r * 32 + (tid & 31)] : 0.f;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 0 && elect_one()) {
      ok = mbar_wait(&S.full, 0);
      tc_fence_after();
      tc_cp_sf(t_sfa, make_desc(smem_u32(S.sfa), 128, 0, 0));
      tc_cp_sf(t_sfb, make_desc(smem_u32(S.sfb), 128, 0, 0));
      const uint32_t idesc = make_idesc(5, 5, 128, NP);
      const uint32_t a_addr = smem_u32(S.a), b_addr = smem_u32(S.b);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        tc_mma_bs(t_acc, make_desc(a_addr + kk * 32, 1024, 16, 2), make_desc(b_addr + kk * 32, 1024, 16, 2),
                  idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4), t_sfa, t_sfb, kk > 0 ? 1u : 0u);
      tc_commit(&S.done);     // arrives even after a failed wait, so nobody hangs below
    }
    const bool got = mbar_wait(&S.done, 0);
    ok = __syncthreads_and((ok && got) ? 1 : 0) != 0;
    tc_fence_after();
  }
  // ---- epilogue: thread = entry ----
  const int ent = e0 + tid;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll
  for (int r = 0; r < RPG; ++r) {
    float score = 0.f;
    if (work) {
#pragma unroll
      for (int c0 = 0; c0 < 32; c0 += 16) {
        uint32_t v[16];
        tc_ld16(t_acc + lane_base + r * 32 + c0, v);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) score += fmaxf(__uint_as_float(v[j]), 0.f) * S.wt[r * 32 + c0 + j];
      }
    }
    const int row = row0 + r;
    if (row < a.n && ent < a.max_len) {
      const int clen = (a.row_pos[row] + 1) / a.ratio;
      bool live = ent < clen && ok;
      if (live && a.cand) live = a.cand[(size_t)row * a.cand_stride + ent / a.cand_block] != 0;
      a.scores[(size_t)row * a.score_stride + ent] = live ? score : -INFINITY;
    }
  }
  if (!ok && tid == 0) status_set(a.status, ST_TIMEOUT, 60, blockIdx.x, blockIdx.y);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace sfb

using namespace sfb;

extern "C" {

// Query side for the tensor-core scores: packed MXFP4 codes [n*32, 64], scale atoms (one 512-byte atom per group of
// rows_per_group rows: 1 or 4) and head weights.  32 index heads of 128 dims.
int sfb_index_q4(const void* qraw, int64_t q_stride, int64_t q_off, const float* wraw, int64_t w_stride, int64_t w_off,
                 const void* rope, int rope_stride, void* q4, void* q_atoms, float* wt, int n, int inh, int idh, int rd,
                 int rows_per_group, float wscale, cudaStream_t stream) {
  if (inh != 32 || idh != 128 || (rows_per_group != 1 && rows_per_group != 4) || rd % 4) return (int)cudaErrorInvalidValue;
  IndexQ4Args a{(const __nv_bfloat16*)qraw, q_stride, q_off, wraw, w_stride, w_off, (const float2*)rope, rope_stride,
                (uint8_t*)q4, (uint8_t*)q_atoms, wt, n, rd, rows_per_group, wscale};
  return (int)sfb_launch(index_q4_kernel, dim3(n), dim3(256), 0, stream, a);
}

// tmapK: FP4 map over the lanes' index keys viewed as [lanes * max_entries, 128] (box 128 rows); tmapQ: FP4 map over q4
// [n*32, 128] with a box of 32 * rows_per_group rows.  With rows_per_group = 4 the rows of a group must share a lane
// (consecutive positions of one sequence).
int sfb_index_scores_tc(const void* tmapK, const void* tmapQ, const void* ik_s, int64_t ik_lane_s, int64_t lane_rows,
                        const void* q_atoms, const float* wt, const int* row_lane, const int* row_pos, const void* cand,
                        int64_t cand_stride, int cand_block, float* scores, int64_t score_stride, int n, int ratio, int max_len,
                        int rows_per_group, void* status, cudaStream_t stream) {
  if (max_len <= 0) return 0;
  if (rows_per_group != 1 && rows_per_group != 4) return (int)cudaErrorInvalidValue;
  IndexTcArgs a{(const uint8_t*)ik_s, ik_lane_s, lane_rows, (const uint8_t*)q_atoms, wt, row_lane, row_pos, (const uint8_t*)cand,
                cand_stride, cand_block, scores, score_stride, n, ratio, max_len, (Status*)status};
  const dim3 grid((max_len + 127) / 128, (n + rows_per_group - 1) / rows_per_group);
  const CUtensorMap* mk = (const CUtensorMap*)tmapK;
  const CUtensorMap* mq = (const CUtensorMap*)tmapQ;
  if (rows_per_group == 1) {
    const size_t smem = sizeof(IndexTcSmem<32>) + 1024;
    return (int)sfb_launch(index_scores_tc_kernel<32>, grid, dim3(itc::THREADS), smem, stream, *mk, *mq, a);
  }
  const size_t smem = sizeof(IndexTcSmem<128>) + 1024;
  return (int)sfb_launch(index_scores_tc_kernel<128>, grid, dim3(itc::THREADS), smem, stream, *mk, *mq, a);
}

}  // extern "C"
