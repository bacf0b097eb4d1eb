// Tensor-core arm: block-scaled MXFP8 / MXFP4 (W4A8) skinny GEMM on tcgen05 with TMEM accumulators.
//
//   out[token, col] = sum_k  W[col, k] * X[token, k]        W: E4M3 or E2M1 + UE8M0/32,  X: E4M3 + UE8M0/32
//
// "Swap-AB": the weight rows are the M = 128 operand of `tcgen05.mma.kind::mxf8f6f4.block_scale`
// and the (few) token rows are N = 16..128, so one CTA streams a 128-row weight tile through the
// whole reduction at full TMA rate no matter how few tokens there are, and every token is an
// independent accumulator column (row i's result does not depend on which other tokens share the
// launch).  FP4 weights stay packed in HBM; TMA unpacks them into 8-bit containers on the way into
// shared memory (16U4_ALIGN16B), and the tensor core widens them - the model's W4A8 arithmetic.
//
// Roles inside a CTA of 192 threads: warp 0 = TMA producer (one elected lane), warp 1 = TMEM
// allocator + MMA issuer (one elected lane), warps 2..5 = epilogue (each owns the 32 TMEM lanes
// its warp id selects).  Stages are handed over with mbarriers; every wait is bounded and reports
// through the status word instead of spinning forever.  No cluster launch, no multicast.
//
// Split-K (for shapes with few weight tiles) writes fp32 partials to a scratch buffer; the CTA
// that arrives last at the tile's ticket adds the splits in index order, so the result does not
// depend on arrival order.
//
// Reference behaviour replaced: kernels/opt_gemv_sm121.cu:967-969 (decode GEMV on warp-level
// block-scaled MMA), kernels/opt_mma_sm121.cu (128x128 bulk GEMMs), kernels/opt_moe_sm121.cu.
#include <cuda.h>
#include <stdio.h>

#include "k_common.cuh"
#include "sfb_noalloc.h"

namespace sfb {

constexpr int UM_THREADS = 192;
constexpr int UM_BK = 128;        // K elements (= bytes in shared memory) per stage
// pipeline depth per kernel flavour: as many bytes in flight per SM as shared memory allows
constexpr int UM_STAGES_DENSE = 4;    // 16 KiB weights + <= 2 KiB tokens + 1 KiB scales per stage (NP <= 32)
constexpr int UM_STAGES_WIDE = 4;     // NP = 64 / 128
constexpr int UM_STAGES_GATEUP = 6;   // two weight tiles per stage
constexpr int UM_A_BYTES = 128 * UM_BK;  // 16 KiB
constexpr uint32_t UM_SPIN_LIMIT = 1u << 22;

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
// Bounded wait: false after UM_SPIN_LIMIT polls (several hundred milliseconds).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < UM_SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);      // a poll suspends the thread for a while by itself; sleeping early delayed every hand-over
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
// shared -> global bulk copy (works for peer memory too); completion is tracked by the thread's bulk group
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store_commit_wait() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// commit and wait only until the copies have READ their shared-memory source (the CTA may then reuse or leave it; the
// global writes complete on their own before the grid counts as finished)
__device__ __forceinline__ void bulk_store_commit_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
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
__device__ __forceinline__ void tc_mma_bs(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                          uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// bf16 x bf16 -> fp32, operands from shared memory (no block scales)
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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major shared-memory matrix descriptor. SWIZZLE_128B: rows of 128 bytes, 8-row groups 1024 bytes
// apart (SBO); no swizzle (scale-factor atoms): 8 rows x 16 bytes per core matrix, 128 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t sbo_bytes, uint32_t lbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;              // descriptor version for sm_100
  d |= (uint64_t)(layout & 7) << 61;   // 2 = SWIZZLE_128B, 0 = none
  return d;
}

// instruction descriptor for kind::mxf8f6f4.block_scale (see the bit layout in the file header of
// the CUTLASS sm100 descriptor definitions): formats E4M3 = 0, E2M1 = 5; UE8M0 scales.
__host__ __device__ inline uint32_t make_idesc(int a_fmt, int b_fmt, int M, int N) {
  uint32_t d = 0;
  d |= (uint32_t)(a_fmt & 7) << 7;
  d |= (uint32_t)(b_fmt & 7) << 10;
  d |= (uint32_t)((N >> 3) & 63) << 17;
  d |= 1u << 23;                       // scale format UE8M0
  d |= (uint32_t)((M >> 4) & 31) << 24;
  return d;
}

// instruction descriptor for kind::f16 with bf16 operands and an fp32 accumulator: accumulator format F32 = 1 at bits 4-5,
// operand formats BF16 = 1 at bits 7-9 / 10-12, both operands K-major (bits 15, 16 clear), N/8 at 17-22, M/16 at 24-28.
// a_mn != 0 marks the A operand as MN-major (bit 15).
__host__ __device__ inline uint32_t make_idesc_bf16(int M, int N, int a_mn = 0) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)((N >> 3) & 63) << 17;
  d |= (uint32_t)((M >> 4) & 31) << 24;
  return d;
}

enum UmmaMode : int { UM_DENSE = 0, UM_DOWN = 2, UM_DOWN_GROUPED = 3 };

struct UmmaArgs {
  // A (weights): rows x K through tmapA (tmapA2 = the shared expert in MoE modes); scale atoms
  // (128 rows x 4 k-blocks, 512 bytes each), atom (ra, ka) at ((ra * katoms_a) + ka) * 512
  const uint8_t* sfa;
  const uint8_t* sfa2;
  int katoms_a;
  // B (activations): token rows x K_total through tmapB; scale atoms likewise
  const uint8_t* sfb;
  int katoms_b;
  int n;                      // valid token rows (dense); number of tokens = gridDim.z (MoE)
  int K;                      // reduction length per item
  int a_fp4;                  // format of tmapA (tmapA2 is always FP8)
  int bf16;                   // dense mode: both operands are bf16 (K counts bytes: two per element), no block scales
  int mode;
  // dense / grouped
  int N;                      // output columns per group
  int groups;                 // group g: A rows g*N.., B k-offset g*K, out column g*N..
  int pair;                   // > 0: out[t] = acc[t] + acc[t + pair] (two-term activations)
  // split-K (dense) or slot accumulation (down)
  int splits;
  float* scratch;             // [splits, tiles_total, 128, NP] fp32
  unsigned int* tickets;      // [tiles_total], zero before the launch; reset by the last CTA
  // outputs [rows, out_stride]
  __nv_bfloat16* out_b;
  float* out_f;
  int64_t out_stride;
  // fused collective (producer half): the bf16 output also goes to the same offset of every rank's slot buffer
  // with plain peer stores, and when the last tile of the kernel is done an arrival flag is raised on every rank
  __nv_bfloat16* peer_out[8];
  uint32_t* peer_flag[8];
  int n_peers;                // 0 = off
  const uint32_t* epoch_ptr;  // flag value = *epoch_ptr + epoch_add
  uint32_t epoch_add;
  unsigned int* done_counter; // zero between launches
  // bulk shapes and the other fused collectives (dense mode, template flag BULK)
  int tok_tiles;              // > 1: blockIdx.z = group * tok_tiles + token tile (NP must be 128)
  const CUtensorMap* b_maps;  // all-gather -> GEMM: activations sharded along K over the ranks; map r covers k in
  int b_k_per_map;            //   [r * b_k_per_map, (r+1) * b_k_per_map) and may point into rank r's memory
  const uint8_t* sfb_maps[8]; //   scale atoms of each shard (katoms = b_k_per_map / 128 per row block)
  const uint32_t* gflag[8];   // optional arrival flag per map (null = that shard is already there): the producer warp waits
  const uint32_t* gepoch_ptr; //   (bounded) for flag >= *gepoch_ptr + gepoch_add before the first load from that map, so the
  uint32_t gepoch_add;        //   GEMM starts on the shards that have arrived while the others are still in flight
  uint64_t gwait_ns;
  int force_bulk;             // entry point for bulk shapes: always the staged-epilogue instantiation
  int rs_rows;                // GEMM -> reduce-scatter: token row t goes only to rank t / rs_rows, at row t % rs_rows
  int defer_reduce;           // split-K partials are left in scratch for splitk_reduce_kernel (many-row dense launches)
  uint8_t* out_q;             // optional: the bf16-rounded output re-quantised per 32 columns (E4M3)
  uint8_t* out_q_atom;        //           and its scale atoms (rows = tokens, kb = out_stride/32)
  // MoE
  const int* ids;             // [n_tok, top_k] expert ids
  const float* wts;           // [n_tok, top_k]
  int top_k, slots;           // slots = top_k + (shared ? 1 : 0)
  int inter;                  // stored local intermediate width (multiple of 128)
  int d;                      // model width
  uint8_t* act_q;             // gate_up out: [n_tok, slots, inter]
  uint8_t* act_s;             //              [n_tok, slots, inter/32] row-major
  uint8_t* act_sf;            //              one atom set per (token, slot), the row at atom row 0
  float limit;
  // grouped MoE (rows of a step sorted by expert; one CTA column = one segment of up to 16 (token, expert) pairs)
  const int* seg_expert;      // [segments] local expert id, -2 = the shared expert, -1 = unused segment
  const int* seg_count;       // [segments] pairs in the segment (1..16)
  const float* seg_weight;    // [segments * 16] routing weight of every pair slot
  unsigned long long* marks;  // optional phase marks: sixteen %globaltimer words per CTA (see um_mark), for the first marks_cap CTAs
  int marks_cap;
  int swap_xy;                // grouped modes: blockIdx.x = segment, blockIdx.y = column tile (CTAs that run together work on
                              // different segments, so one activation tile is not fetched by every SM at the same moment)
  Status* status;
};

// Phase marks inside a kernel (sixteen words per CTA; 8 = the epilogue's first accumulator read is in registers): slot 0 entry, 1 set-up done (barriers, TMEM), 2 producer about to issue its first load,
// 3 first stage landed, 4 last MMA issued, 5 accumulator complete (epilogue starts), 6 epilogue done (stores issued and
// waited for), 7 exit.  One word per slot and CTA, written by one thread of the role that reaches the point.
// Compiled in only with -DSFB_KERNEL_MARKS (SFB_KERNEL_MARKS=1 at build time): with the marks present but unarmed a decode
// step measured 3.5 % slower, so the shipped kernels carry none.
#ifdef SFB_KERNEL_MARKS
#define SFB_MARKS_ON 1
__device__ __forceinline__ void um_mark(const UmmaArgs& a, int slot) {
  if (a.marks) {
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (cta < a.marks_cap) a.marks[(size_t)cta * 16 + slot] = globaltimer_ns();
  }
}
#else
#define SFB_MARKS_ON 0
__device__ __forceinline__ void um_mark(const UmmaArgs&, int) {}
#endif

template <int NP, int NA, int ST>  // token columns; weight tiles per stage (2 for gate|up); stages
struct UmmaSmem {
  alignas(1024) uint8_t a[ST][NA][UM_A_BYTES];
  alignas(1024) uint8_t b[ST][NP * UM_BK];
  alignas(128) uint8_t sfa[ST][NA][512];
  alignas(128) uint8_t sfb[ST][512];
  alignas(8) uint64_t full[ST];
  alignas(8) uint64_t empty[ST];
  alignas(8) uint64_t sfready[ST][2];     // gate/up kernel: the stage's scale factors are in TMEM (one barrier per accumulator)
  alignas(8) uint64_t acc_full;
  uint32_t tmem_base;
  int last_flag;
  int fail;
};

// what one CTA multiplies
struct UmmaWork {
  const CUtensorMap* ma;
  int a_fp4;
  int a_row0;                 // first weight row of the tile in `ma`
  const uint8_t* sfa;         // atom of k-step 0 for this tile (512 bytes per k-step)
  int b_x0, b_row0;           // B coordinates of k-step 0
  const uint8_t* sfb;         // atom of k-step 0
  int ks0, nks;
  int split, splits, tile_id, tiles_total;
  int out_row0, n_valid, col0, col_limit;
};

// STO > 0 overrides the pipeline depth (and asks for three CTAs per SM): launches of many short-K CTAs, where a CTA's
// prologue and epilogue are as long as its weight stream and only more resident CTAs keep the stream busy
template <int NP, bool BULK, int STO = 0>
__global__ void __launch_bounds__(UM_THREADS, STO ? 3 : 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapA2,
                 const __grid_constant__ CUtensorMap tmapB, UmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // bulk tiles of 128 tokens run two CTAs per SM (3 stages = 99 KiB each): one CTA's epilogue hides behind the other's mainloop
  constexpr int UM_STAGES = STO ? STO : (NP <= 32 ? UM_STAGES_DENSE : ((BULK && NP == 128) ? 3 : UM_STAGES_WIDE));
  using Smem = UmmaSmem<NP, 1, UM_STAGES>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = NP + 16 <= 32 ? 32 : (NP + 16 <= 64 ? 64 : (NP + 16 <= 128 ? 128 : 256));

  if (threadIdx.x == 0) {
    um_mark(a, 0);
    for (int s = 0; s < UM_STAGES; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    mbar_init(&S.acc_full, 1);
    S.fail = 0;
    S.last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) um_mark(a, 1);
  UmmaWork w;
  int tok_tile = 0;
  bool skip = false;
  int pre = 0;   // stages whose weight tile was requested before the dependency wait
  if (a.mode == UM_DENSE) {
    const int tile = blockIdx.x;
    int g = blockIdx.z;
    if (BULK) { tok_tile = blockIdx.z % a.tok_tiles; g = blockIdx.z / a.tok_tiles; }
    const int ksteps = (a.K + UM_BK - 1) / UM_BK;
    w.ma = &tmapA; w.a_fp4 = a.a_fp4;
    w.a_row0 = g * a.N + tile * 128;
    w.ks0 = (int)((int64_t)ksteps * blockIdx.y / a.splits);
    w.nks = (int)((int64_t)ksteps * (blockIdx.y + 1) / a.splits) - w.ks0;
    w.sfa = a.sfa + ((size_t)(w.a_row0 >> 7) * a.katoms_a + w.ks0) * 512;
    w.b_x0 = g * a.K + w.ks0 * UM_BK; w.b_row0 = 0;
    w.sfb = a.sfb + ((size_t)(g * ksteps + w.ks0)) * 512;
    w.split = blockIdx.y; w.splits = a.splits;
    w.tile_id = blockIdx.z * gridDim.x + tile; w.tiles_total = gridDim.x * gridDim.z;
    w.out_row0 = 0; w.n_valid = a.n; w.col0 = w.a_row0; w.col_limit = (g + 1) * a.N;
    if (BULK) {
      w.b_row0 = tok_tile * NP; w.out_row0 = tok_tile * NP;
      w.n_valid = min(NP, a.n - tok_tile * NP);
      w.sfb = a.sfb + ((size_t)((tok_tile * NP) >> 7) * a.katoms_b + g * ksteps + w.ks0) * 512;
      if (a.pair > 0) {   // two-term activations in blocks: tile = `pair` hi rows then `pair` lo rows; a.n counts logical rows
        w.out_row0 = tok_tile * a.pair;
        w.n_valid = min(a.pair, a.n - tok_tile * a.pair);
      }
    }
    // dense weights and their scales do not depend on the previous kernel: request the first stages' weight tiles now, so
    // that their fetch overlaps the predecessor's tail; the activation tiles follow after the wait
    if (warp == 0) {
      pre = w.nks < UM_STAGES ? w.nks : UM_STAGES;      // in every lane: whichever lane is elected below and later knows it
      if (elect_one()) {
        const uint32_t stage_tx = (w.a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + (a.bf16 ? 0 : 1024);
        for (int i = 0; i < pre; ++i) {
          mbar_expect_tx(&S.full[i], stage_tx);
          tma_load_2d(S.a[i][0], w.ma, (w.ks0 + i) * UM_BK, w.a_row0, &S.full[i]);
          if (!a.bf16) bulk_load(S.sfa[i][0], w.sfa + (size_t)i * 512, 512, &S.full[i]);
        }
      }
    }
  }
  pdl_wait();   // operands written by the previous kernel (activations, expert ids) are read below
  if (a.mode == UM_DENSE) {
  } else if (a.mode == UM_DOWN_GROUPED) {   // x = column tile of d, y = segment: W2_e times the segment's activation rows
    const int tile = a.swap_xy ? blockIdx.y : blockIdx.x, seg = a.swap_xy ? blockIdx.x : blockIdx.y;
    const int n_tiles = a.swap_xy ? gridDim.y : gridDim.x;
    const int ksteps = (a.inter + UM_BK - 1) / UM_BK;
    int e = a.seg_expert[seg];
    if (e == -1) { skip = true; e = 0; }
    if (e >= 0) {
      w.ma = &tmapA; w.a_fp4 = a.a_fp4;
      w.a_row0 = e * a.d + tile * 128;
      w.sfa = a.sfa + ((size_t)(w.a_row0 >> 7) * a.katoms_a) * 512;
    } else {
      w.ma = &tmapA2; w.a_fp4 = 0;
      w.a_row0 = tile * 128;
      w.sfa = a.sfa2 + ((size_t)tile * a.katoms_a) * 512;
    }
    w.ks0 = 0; w.nks = skip ? 0 : ksteps;
    w.b_x0 = 0; w.b_row0 = seg * NP;
    w.sfb = a.sfb + (size_t)seg * a.katoms_b * 512;
    w.split = 0; w.splits = 1;
    w.tile_id = seg * n_tiles + tile; w.tiles_total = gridDim.x * gridDim.y;
    w.out_row0 = seg * NP; w.n_valid = skip ? 0 : a.seg_count[seg]; w.col0 = tile * 128; w.col_limit = a.d;
  } else {  // UM_DOWN: x = column tile of d, y = slot, z = token
    const int tile = blockIdx.x, slot = blockIdx.y, tok = blockIdx.z;
    const int ksteps = (a.inter + UM_BK - 1) / UM_BK;
    if (slot < a.top_k) {
      int e = a.ids[(size_t)tok * a.top_k + slot];
      if (e < 0) { skip = true; e = 0; }       // an expert this rank does not hold: the slot contributes zeros
      w.ma = &tmapA; w.a_fp4 = a.a_fp4;
      w.a_row0 = e * a.d + tile * 128;
      w.sfa = a.sfa + ((size_t)(w.a_row0 >> 7) * a.katoms_a) * 512;
    } else {
      w.ma = &tmapA2; w.a_fp4 = 0;
      w.a_row0 = tile * 128;
      w.sfa = a.sfa2 + ((size_t)tile * a.katoms_a) * 512;
    }
    w.ks0 = 0; w.nks = skip ? 0 : ksteps;
    w.b_x0 = 0; w.b_row0 = tok * a.slots + slot;
    w.sfb = a.sfb + (size_t)w.b_row0 * a.katoms_b * 512;
    w.split = slot; w.splits = a.slots;
    w.tile_id = tok * gridDim.x + tile; w.tiles_total = gridDim.x * gridDim.z;
    w.out_row0 = tok; w.n_valid = 1; w.col0 = tile * 128; w.col_limit = a.d;
  }
  // bytes TMA reports per stage: packed FP4 counts 4 bits per element although it lands in 8-bit containers
  const uint32_t STAGE_TX = (w.a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + (a.bf16 ? 0 : 1024);
  const uint32_t tmem = S.tmem_base;
  const uint32_t t_acc = tmem;               // NP fp32 columns
  const uint32_t t_sfa = tmem + NP;          // 2 x 4 columns
  const uint32_t t_sfb = tmem + NP + 8;      // 2 x 4 columns

  if (warp == 0) {
    if (elect_one()) {
      int gated = -1;
      um_mark(a, 2);
      for (int i = 0; i < w.nks; ++i) {
        const int s = i % UM_STAGES;
        if (i >= pre) {
          if (i >= UM_STAGES && !mbar_wait(&S.empty[s], ((i / UM_STAGES) - 1) & 1)) { S.fail = 1; break; }
          mbar_expect_tx(&S.full[s], STAGE_TX);
          tma_load_2d(S.a[s][0], w.ma, (w.ks0 + i) * UM_BK, w.a_row0, &S.full[s]);
        }
        if (BULK && a.b_maps) {
          // the k-slab belongs to the rank that owns this range of the hidden dimension: a plain (non-multicast) TMA load
          // from that rank's memory or from the local slot its owner pushed it into, and its scale atoms with a bulk copy
          const int k = (w.ks0 + i) * UM_BK, owner = k / a.b_k_per_map, kl = k - owner * a.b_k_per_map;
          if (owner != gated && a.gflag[owner]) {
            // a launch whose status word already holds an error (an earlier CTA ran out of time) does not wait again: the
            // loads below still read valid local memory, the epilogue writes nothing, and the host sees the status
            const bool dead = a.status && *reinterpret_cast<volatile int*>(&a.status->code) != 0;
            if (dead || !wait_flag_ge(a.gflag[owner], *a.gepoch_ptr + a.gepoch_add, a.gwait_ns)) {
              status_set(a.status, ST_TIMEOUT, 40, owner, (int)(*a.gepoch_ptr + a.gepoch_add));
              S.fail = 1;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          gated = owner;
          tma_load_2d(S.b[s], &a.b_maps[owner], kl, w.b_row0, &S.full[s]);
          bulk_load(S.sfb[s], a.sfb_maps[owner] + ((size_t)(w.b_row0 >> 7) * (a.b_k_per_map / UM_BK) + kl / UM_BK) * 512, 512, &S.full[s]);
        } else {
          tma_load_2d(S.b[s], &tmapB, w.b_x0 + i * UM_BK, w.b_row0, &S.full[s]);
          if (!a.bf16) bulk_load(S.sfb[s], w.sfb + (size_t)i * 512, 512, &S.full[s]);
        }
        if (i >= pre && !a.bf16) bulk_load(S.sfa[s][0], w.sfa + (size_t)i * 512, 512, &S.full[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(w.a_fp4 ? 5 : 0, 0, 128, NP);
      for (int i = 0; i < w.nks; ++i) {
        const int s = i % UM_STAGES;
        if (!mbar_wait(&S.full[s], (i / UM_STAGES) & 1)) { S.fail = 2; break; }
        tc_fence_after();
        if (i == 0) um_mark(a, 3);
        const uint32_t sf_slot = (uint32_t)(i & 1) * 4;
        const uint32_t a_addr = smem_u32(S.a[s][0]), b_addr = smem_u32(S.b[s]);
        if (a.bf16) {
          // a 128-byte stage row holds 64 bf16 elements = four K = 16 steps of 32 bytes
          const uint32_t idb = make_idesc_bf16(128, NP);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_f16(t_acc, make_desc(a_addr + kk * 32, 1024, 16, 2), make_desc(b_addr + kk * 32, 1024, 16, 2), idb,
                       (i > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&S.empty[s]);
          continue;
        }
        tc_cp_sf(t_sfa + sf_slot, make_desc(smem_u32(S.sfa[s][0]), 128, 0, 0));
        tc_cp_sf(t_sfb + sf_slot, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t ad = make_desc(a_addr + kk * 32, 1024, 16, 2);
          const uint64_t bd = make_desc(b_addr + kk * 32, 1024, 16, 2);
          const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);  // scale-factor byte ids
          tc_mma_bs(t_acc, ad, bd, id, t_sfa + sf_slot, t_sfb + sf_slot, (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&S.empty[s]);   // frees this stage's shared memory once the MMAs have read it
      }
      tc_commit(&S.acc_full);     // arrives even after a failed wait so the epilogue never hangs
      um_mark(a, 4);
    }
  } else {
    // ---- epilogue: warp w owns TMEM lanes 32*(w%4) .. +31 = weight rows of the tile ----
    const int q = warp & 3;
    const bool got = mbar_wait(&S.acc_full, 0);
    tc_fence_after();
    if (warp == 2 && lane == 0) um_mark(a, 5);
    const int col = w.col0 + q * 32 + lane;     // output column (row of A)
    const bool col_ok = col < w.col_limit;
    const bool single = w.splits == 1;
    const size_t lane_off = ((size_t)w.tile_id * 128 + q * 32 + lane) * NP;
    const size_t split_stride = (size_t)w.tiles_total * 128 * NP;
    float* part = a.scratch ? a.scratch + (size_t)w.split * split_stride + lane_off : nullptr;
    const int nv = (a.pair > 0 && !BULK) ? a.pair : w.n_valid;
    // bulk shapes: the bf16 tile is staged token-major in the (now idle) operand stages and leaves the SM as
    // 256-byte bulk copies, one per token row and destination - element stores to a peer serialise on NVLink
    const bool staged = BULK && a.pair == 0 && !a.out_f && !a.out_q && (a.out_b || a.n_peers > 0) &&
                        w.col0 + 128 <= w.col_limit && (a.out_stride & 7) == 0;
    __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(&S.a[0][0][0]);
    // grouped down projection with wide segments: the fp32 tile is staged token-major in the idle operand stages and leaves
    // as one 512-byte bulk copy per pair row (one element store per pair and thread took twice the main loop's time)
    constexpr bool STAGE_F_FITS = NP >= 32 && NP * 512 <= UM_STAGES * UM_A_BYTES;
    const bool stagedf = STAGE_F_FITS && !BULK && a.mode == UM_DOWN_GROUPED && a.out_f && !a.out_b && !a.out_q && single &&
                         a.pair == 0 && a.n_peers == 0 && w.col0 + 128 <= w.col_limit && (a.out_stride & 3) == 0;
    float* stagef = reinterpret_cast<float*>(&S.a[0][0][0]);
    // two-term activations in blocks, one split: the hi and lo accumulator columns of a token are added straight out of
    // TMEM (the same sum, 0 + hi + lo, that the scratch path forms), without the round trip through global memory
    const bool pair_direct = BULK && a.pair > 0 && single && 2 * a.pair <= NP && (a.pair & 15) == 0;
    // ... staged: bf16 rows, FP8 codes and the rows' scale bytes are collected in the idle operand stages and leave as one
    // bulk copy per token row (element stores from inside the column loop cost more than the main loop)
    const bool pd_stage = pair_direct && a.out_b && !a.out_f && w.col0 + 128 <= w.col_limit && (a.out_stride & 15) == 0 &&
                          a.pair * 384 <= UM_STAGES * UM_A_BYTES;
    if (pair_direct) {
      __nv_bfloat16* st_b = stage;                                                      // [pair][128] bf16
      uint8_t* st_q = reinterpret_cast<uint8_t*>(&S.a[0][0][0]) + (size_t)a.pair * 256;  // [pair][128] codes
      uint8_t* st_sf = &S.sfa[0][0][0];                                                  // [pair][4] scale bytes (pair <= 128)
      for (int c0 = 0; c0 < a.pair; c0 += 16) {
        uint32_t v[16], u[16];
        tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + c0, v);
        tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + c0 + a.pair, u);
        tc_wait_ld();
        if (!got || S.fail) continue;
        float sum[16];
        uint32_t amax_bits[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float t = 0.f;
          t += __uint_as_float(v[j]);
          t += __uint_as_float(u[j]);
          sum[j] = col_ok ? t : 0.f;
        }
        if (a.out_q && !pd_stage) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float r = bfr(sum[j]);
            const float ax = (r == r) ? fabsf(r) : 0.f;
            amax_bits[j] = __reduce_max_sync(0xffffffffu, __float_as_uint(ax));
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = c0 + j;
          if (tok < nv) {   // warp-uniform
            const int64_t o = (int64_t)(w.out_row0 + tok) * a.out_stride + col;
            if (pd_stage) {
              st_b[tok * 128 + q * 32 + lane] = __float2bfloat16_rn(sum[j]);
            } else if (col_ok) {
              if (a.out_b) a.out_b[o] = __float2bfloat16_rn(sum[j]);
              if (a.out_f) a.out_f[o] = sum[j];
            }
            if (a.out_q && !pd_stage) {
              const uint8_t sc = act_scale_code_fp8(__uint_as_float(amax_bits[j]));
              const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
              const uint8_t code = enc_e4m3(bfr(sum[j]) * inv);
              if (col_ok) {
                a.out_q[o] = code;
                if (lane == 0) a.out_q_atom[sf_offset(w.out_row0 + tok, col >> 5, (int)(a.out_stride >> 5))] = sc;
              }
            }
          }
        }
      }
      if (pd_stage && a.out_q) {       // CTA-uniform
        // the FP8 copy from the staged bf16 rows: sixteen consecutive columns of one token per thread and turn (two
        // neighbouring lanes share a 32-column scale block), packed conversions, 16-byte stores.  (Quantising from the TMEM
        // layout - one column per lane, one warp reduction per token - was most of this kernel's epilogue.)
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int tid = q * 32 + lane;
        for (int base = 0; base < nv * 8; base += 128) {      // the same trip count in every thread: the shuffle below is warp-wide
          const int sg = base + tid;
          const bool live = sg < nv * 8;
          const int tok = live ? sg >> 3 : 0, seg = sg & 7;
          const uint4* src = reinterpret_cast<const uint4*>(st_b + tok * 128 + seg * 16);
          const uint4 a0 = src[0], a1 = src[1];
          const uint32_t wv[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          float o[16];
          float amax = 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            o[2 * k] = __uint_as_float(wv[k] << 16);
            o[2 * k + 1] = __uint_as_float(wv[k] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(o[2 * k]), fabsf(o[2 * k + 1])));      // fmaxf drops a NaN operand: it counts as 0
          }
          amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
          if (!live) continue;
          const uint8_t sc = act_scale_code_fp8(amax);
          const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
          uint32_t cw[4];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t c2 = enc_e4m3x2(o[2 * k] * inv, o[2 * k + 1] * inv);
            if (k & 1) cw[k >> 1] |= c2 << 16; else cw[k >> 1] = c2;
          }
          *reinterpret_cast<uint4*>(st_q + tok * 128 + seg * 16) = make_uint4(cw[0], cw[1], cw[2], cw[3]);
          if (!(seg & 1)) st_sf[tok * 4 + (seg >> 1)] = sc;
        }
      }
      if (pd_stage) {       // CTA-uniform
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int tok = q * 32 + lane;
        if (tok < nv && got && !S.fail) {
          const int64_t row = w.out_row0 + tok;
          bulk_store(a.out_b + row * a.out_stride + w.col0, smem_u32(st_b + tok * 128), 256);
          if (a.out_q) bulk_store(a.out_q + row * a.out_stride + w.col0, smem_u32(st_q + tok * 128), 128);
          bulk_store_commit_wait_read();
          if (a.out_q)
            *reinterpret_cast<uint32_t*>(a.out_q_atom + sf_offset(row, w.col0 >> 5, (int)(a.out_stride >> 5))) =
                *reinterpret_cast<const uint32_t*>(st_sf + tok * 4);
        }
      }
    }
#pragma unroll
    for (int c0 = 0; c0 < NP; c0 += 16) {
      if (pair_direct) break;
      uint32_t v[16];
      tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + c0, v);
      tc_wait_ld();
      if (c0 == 0 && warp == 2 && lane == 0) um_mark(a, 8);
      if (!got || S.fail) continue;
      if (skip) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0u;
      }
      if (single && staged) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < nv) stage[(c0 + j) * 128 + q * 32 + lane] = __float2bfloat16_rn(__uint_as_float(v[j]));
      } else if (stagedf) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < nv) stagef[(c0 + j) * 128 + q * 32 + lane] = __uint_as_float(v[j]);
      } else if (single && a.pair == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = c0 + j;
          if (tok < nv) {   // warp-uniform
            const float f = col_ok ? __uint_as_float(v[j]) : 0.f;
            const int64_t o = (int64_t)(w.out_row0 + tok) * a.out_stride + col;
            if (col_ok) {
              const __nv_bfloat16 fb = __float2bfloat16_rn(f);
              if (a.out_b) a.out_b[o] = fb;
              if (a.out_f) a.out_f[o] = f;
              if (BULK && a.rs_rows > 0) {
                const int row = w.out_row0 + tok, pr = row / a.rs_rows;
                a.peer_out[pr][(int64_t)(row - pr * a.rs_rows) * a.out_stride + col] = fb;
              } else {
                for (int pr = 0; pr < a.n_peers; ++pr) a.peer_out[pr][o] = fb;
              }
            }
            if (a.out_q) {
              uint8_t sc;
              const uint8_t code = warp_quant_fp8(bfr(f), &sc);
              if (col_ok) {
                a.out_q[o] = code;
                if (lane == 0) a.out_q_atom[sf_offset(w.out_row0 + tok, col >> 5, (int)(a.out_stride >> 5))] = sc;
              }
            }
          }
        }
      } else {
        float4* p4 = reinterpret_cast<float4*>(part + c0);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          p4[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                              __uint_as_float(v[4 * j + 3]));
      }
    }
    if (!(single && a.pair == 0) && !a.defer_reduce && !pair_direct) {
      // last-arriving split of this tile reduces all splits in index order
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const unsigned int prev = atomicAdd(&a.tickets[w.tile_id], 1u);
        S.last_flag = (prev == (unsigned int)w.splits - 1) ? 1 : 0;
        if (S.last_flag) a.tickets[w.tile_id] = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (S.last_flag && staged) {
        __threadfence();
        for (int tok0 = 0; tok0 < nv; tok0 += 4) {
          float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp = 0; sp < w.splits; ++sp) {      // split order: the sum does not depend on arrival order
            const float4 t = __ldcg(reinterpret_cast<const float4*>(a.scratch + (size_t)sp * split_stride + lane_off + tok0));
            acc4.x += t.x; acc4.y += t.y; acc4.z += t.z; acc4.w += t.w;
          }
          const float r4[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (tok0 + j < nv) stage[(tok0 + j) * 128 + q * 32 + lane] = __float2bfloat16_rn(r4[j]);
        }
      } else if (S.last_flag) {
        __threadfence();
        const bool vec = a.pair == 0 || (a.pair & 3) == 0;     // four token columns per load when the layout allows it
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
        for (int tok = 0; tok < nv; ++tok) {
          float s = 0.f;
          if (vec) {
            if ((tok & 3) == 0) {
              s4[0] = s4[1] = s4[2] = s4[3] = 0.f;
              // split order, then the pair term: same sums as the scalar path.  Four splits' loads are issued before
              // their (ordered) adds so that the reduce is not one L2 round trip per split
              for (int sp0 = 0; sp0 < w.splits; sp0 += 4) {
                float4 t[4], u[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int sp = sp0 + i < w.splits ? sp0 + i : w.splits - 1;
                  const float* pp = a.scratch + (size_t)sp * split_stride + lane_off;
                  t[i] = __ldcg(reinterpret_cast<const float4*>(pp + tok));
                  u[i] = a.pair > 0 ? __ldcg(reinterpret_cast<const float4*>(pp + tok + a.pair)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  if (sp0 + i < w.splits) {
                    s4[0] += t[i].x; s4[1] += t[i].y; s4[2] += t[i].z; s4[3] += t[i].w;
                    if (a.pair > 0) { s4[0] += u[i].x; s4[1] += u[i].y; s4[2] += u[i].z; s4[3] += u[i].w; }
                  }
                }
              }
            }
            s = s4[tok & 3];
          } else {
            for (int sp = 0; sp < w.splits; ++sp) {
              const float* pp = a.scratch + (size_t)sp * split_stride + lane_off;
              s += __ldcg(pp + tok);
              if (a.pair > 0) s += __ldcg(pp + tok + a.pair);
            }
          }
          if (!col_ok) s = 0.f;
          const int64_t o = (int64_t)(w.out_row0 + tok) * a.out_stride + col;
          if (col_ok) {
            const __nv_bfloat16 sb = __float2bfloat16_rn(s);
            if (a.out_b) a.out_b[o] = sb;
            if (a.out_f) a.out_f[o] = s;
            if (BULK && a.rs_rows > 0) {
              const int row = w.out_row0 + tok, pr = row / a.rs_rows;
              a.peer_out[pr][(int64_t)(row - pr * a.rs_rows) * a.out_stride + col] = sb;
            } else {
              for (int pr = 0; pr < a.n_peers; ++pr) a.peer_out[pr][o] = sb;
            }
          }
          if (a.out_q) {
            uint8_t sc;
            const uint8_t code = warp_quant_fp8(bfr(s), &sc);
            if (col_ok) {
              a.out_q[o] = code;
              if (lane == 0) a.out_q_atom[sf_offset(w.out_row0 + tok, col >> 5, (int)(a.out_stride >> 5))] = sc;
            }
          }
        }
      }
    }
    if (stagedf) {        // CTA-uniform, so every epilogue warp reaches the barrier whatever its own wait returned
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int tok = q * 32 + lane;
      if (tok < nv && got && !S.fail) {
        bulk_store(a.out_f + (int64_t)(w.out_row0 + tok) * a.out_stride + w.col0, smem_u32(stagef + tok * 128), 512);
        bulk_store_commit_wait_read();
      }
    }
    if (staged && got && !S.fail && (single || S.last_flag)) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int tok = q * 32 + lane;
      if (tok < nv) {
        const int row = w.out_row0 + tok;
        const uint32_t src = smem_u32(stage + tok * 128);
        if (a.out_b) bulk_store(a.out_b + (int64_t)row * a.out_stride + w.col0, src, 256);
        if (a.rs_rows > 0) {
          const int pr = row / a.rs_rows;
          bulk_store(a.peer_out[pr] + (int64_t)(row - pr * a.rs_rows) * a.out_stride + w.col0, src, 256);
        } else {
          for (int pr = 0; pr < a.n_peers; ++pr) bulk_store(a.peer_out[pr] + (int64_t)row * a.out_stride + w.col0, src, 256);
        }
        if (a.n_peers > 0) bulk_store_commit_wait();      // the arrival flag below follows the writes
        else bulk_store_commit_wait_read();               // local rows: the grid's end orders them for the next kernel
      }
    }
    if (a.n_peers > 0) {
      // this CTA finalised its tile (directly, or as the last split): count it; the CTA that completes the
      // kernel's last tile raises this rank's arrival flag on every rank
      const bool finalised = (single && a.pair == 0) || pair_direct || S.last_flag;
      if (finalised) {
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const unsigned int prev = atomicAdd(a.done_counter, 1u);
          if (prev == (unsigned int)w.tiles_total - 1) {
            *a.done_counter = 0;
            __threadfence_system();
            const uint32_t ep = *a.epoch_ptr + a.epoch_add;
            for (int pr = 0; pr < a.n_peers; ++pr) st_release_sys(a.peer_flag[pr], ep);
          }
        }
      }
    }
    if ((!got || S.fail) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 10 + S.fail, blockIdx.x, blockIdx.y);
    if (warp == 2 && lane == 0) um_mark(a, 6);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) um_mark(a, 7);
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- persistent many-row dense GEMM ---------------------------------------------------------------------------------
// One CTA per SM walks over (weight tile, token tile) pairs.  The producer and the MMA thread run ahead into the next tile
// while the four epilogue warps drain the previous accumulator (two accumulator sets in TMEM), so a tile's epilogue - TMEM ->
// bf16 -> shared memory -> one 256-byte bulk copy per token row and destination, peer memory included - and the wait for
// those copies hide behind the next main loop.  Same arithmetic and the same output bits as umma_gemm_kernel<128, true>.
constexpr int PS_STAGES = 5;
struct UmmaPersistSmem {
  alignas(1024) uint8_t a[PS_STAGES][UM_A_BYTES];
  alignas(1024) uint8_t b[PS_STAGES][128 * UM_BK];
  alignas(1024) __nv_bfloat16 out[128 * 128];     // the tile on its way out, token-major
  alignas(128) uint8_t sfa[PS_STAGES][512];
  alignas(128) uint8_t sfb[PS_STAGES][512];
  alignas(8) uint64_t full[PS_STAGES];
  alignas(8) uint64_t empty[PS_STAGES];
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int fail;
  volatile int ep_ok;
};
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(UM_THREADS, 1)
umma_bulk_persistent_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, UmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  UmmaPersistSmem& S = *reinterpret_cast<UmmaPersistSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < PS_STAGES; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 1); }
    S.fail = 0;
    S.ep_ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, 512);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const int n_w = (a.N + 127) / 128, total = n_w * a.tok_tiles, ksteps = a.K / UM_BK;
  const uint32_t tmem = S.tmem_base;
  const uint32_t t_sfa = tmem + 256, t_sfb = tmem + 264;
  constexpr uint32_t STAGE_TX = UM_A_BYTES + 128 * UM_BK + 1024;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int wt = t % n_w, tt = t / n_w;
        const uint8_t* sfa = a.sfa + ((size_t)wt * a.katoms_a) * 512;
        const uint8_t* sfb = a.sfb + ((size_t)tt * a.katoms_b) * 512;
        for (int i = 0; i < ksteps; ++i, ++it) {
          const int s = it % PS_STAGES;
          if (it >= PS_STAGES && !mbar_wait(&S.empty[s], ((it / PS_STAGES) - 1) & 1)) { S.fail = 1; break; }
          mbar_expect_tx(&S.full[s], STAGE_TX);
          tma_load_2d(S.a[s], &tmapA, i * UM_BK, wt * 128, &S.full[s]);
          tma_load_2d(S.b[s], &tmapB, i * UM_BK, tt * 128, &S.full[s]);
          bulk_load(S.sfa[s], sfa + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfb[s], sfb + (size_t)i * 512, 512, &S.full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(0, 0, 128, 128);
      uint32_t it = 0;
      int lt = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x, ++lt) {
        const int buf = lt & 1;
        // the accumulator set is free once the epilogue of the tile before last has read it
        if (lt >= 2 && !mbar_wait(&S.acc_empty[buf], ((lt >> 1) - 1) & 1)) { S.fail = 3; break; }
        tc_fence_after();
        const uint32_t t_acc = tmem + (uint32_t)buf * 128;
        bool ok = true;
        for (int i = 0; i < ksteps; ++i, ++it) {
          const int s = it % PS_STAGES;
          if (!mbar_wait(&S.full[s], (it / PS_STAGES) & 1)) { S.fail = 2; ok = false; break; }
          tc_fence_after();
          const uint32_t sf_slot = (it & 1u) * 4;
          tc_cp_sf(t_sfa + sf_slot, make_desc(smem_u32(S.sfa[s]), 128, 0, 0));
          tc_cp_sf(t_sfb + sf_slot, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
          const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
            tc_mma_bs(t_acc, make_desc(a_addr + kk * 32, 1024, 16, 2), make_desc(b_addr + kk * 32, 1024, 16, 2), id, t_sfa + sf_slot,
                      t_sfb + sf_slot, (i > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&S.empty[s]);
        }
        tc_commit(&S.acc_full[buf]);      // arrives even after a failed wait, so the epilogue never waits for its limit
        if (!ok) break;
      }
    }
  } else {
    const int q = warp & 3;
    bool pending = false;      // this thread has bulk copies of the previous tile in flight
    int lt = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++lt) {
      const int buf = lt & 1, wt = t % n_w, tt = t / n_w;
      // one warp waits for the accumulator and tells the others through the barrier, so that all four take the same path
      if (warp == 2) {
        bool got = true;
        if (lane == 0) got = mbar_wait(&S.acc_full[buf], (lt >> 1) & 1) && !S.fail;
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (lane == 0 && !got) S.ep_ok = 0;
      }
      if (pending) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the staging tile has been read out (the
                                                                                      // plain loads of the peer stores are done when their loop ends)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!S.ep_ok) break;
      tc_fence_after();
      const int nv = min(128, a.n - tt * 128);
      const uint32_t t_acc = tmem + (uint32_t)buf * 128;
      // four 16-token chunks are requested before each wait (a load's round trip was paid once per chunk)
#pragma unroll
      for (int b0 = 0; b0 < 128; b0 += 64) {
        uint32_t v[4][16];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + b0 + ch * 16, v[ch]);
        tc_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int c0 = b0 + ch * 16;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < nv) S.out[(c0 + j) * 128 + q * 32 + lane] = __float2bfloat16_rn(__uint_as_float(v[ch][j]));
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) mbar_arrive(&S.acc_empty[buf]);       // every warp's TMEM reads of this set are done
      const int tok = q * 32 + lane;
      pending = false;
      if (a.out_b && tok < nv) {
        bulk_store(a.out_b + (int64_t)(tt * 128 + tok) * a.out_stride + wt * 128, smem_u32(S.out + tok * 128), 256);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        pending = true;
      }
      if (a.n_peers > 0) {
        // rows on their way to other GPUs go out as plain 16-byte stores, half a warp per 256-byte row segment (the form
        // NVLink moves best; one small bulk copy per row reached a quarter of the link rate)
        const int hw = lane >> 4, c8 = (lane & 15) * 8;
#pragma unroll 4
        for (int r0 = q * 32; r0 < q * 32 + 32; r0 += 2) {
          const int r = r0 + hw;
          if (r < nv) {
            const uint4 v = *reinterpret_cast<const uint4*>(S.out + r * 128 + c8);
            const int row = tt * 128 + r;
            if (a.rs_rows > 0) {
              const int pr = row / a.rs_rows;
              *reinterpret_cast<uint4*>(a.peer_out[pr] + (int64_t)(row - pr * a.rs_rows) * a.out_stride + wt * 128 + c8) = v;
            } else {
              for (int pr = 0; pr < a.n_peers; ++pr)
                *reinterpret_cast<uint4*>(a.peer_out[pr] + (int64_t)row * a.out_stride + wt * 128 + c8) = v;
            }
          }
        }
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // every copy of this thread has been written
    if (a.n_peers > 0) {
      // this CTA's tiles are out: count the CTA; the last one raises this rank's arrival flag on every rank
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        const unsigned int prev = atomicAdd(a.done_counter, 1u);
        if (prev == gridDim.x - 1) {
          *a.done_counter = 0;
          __threadfence_system();
          const uint32_t ep = *a.epoch_ptr + a.epoch_add;
          for (int pr = 0; pr < a.n_peers; ++pr) st_release_sys(a.peer_flag[pr], ep);
        }
      }
    }
    if ((S.fail || !S.ep_ok) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 60 + S.fail, blockIdx.x, lt);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---- MoE gate/up: two weight tiles (w1, w3) against one token, clamp-SwiGLU x route weight, FP8 re-quant ------
// grid: x = 128-column tile of the intermediate width, y = slot (top_k routed + shared), z = token
// UM_STAGES = 6 fills one SM's shared memory with a single CTA (few CTAs: decode); 3 lets two CTAs share an SM, so that one's
// prologue and epilogue hide behind the other's weight stream when a launch has many waves (grouped many-row steps)
// NP = token columns: 16 (a token, or a segment of up to 16 pairs) or 64 (many-row steps: segments of up to 64 pairs)
// Warps: 0 = TMA producer, 1 = MMA issue for the gate tile, 2..5 = epilogue, 6 = MMA issue for the up tile.  One thread
// issues a tcgen05 operation about every 75 cycles whatever its size, and with 16-column tiles that - not the data - paced
// the main loop; the two accumulators are independent, so each gets its own issuing thread (and its own copy of the
// activation scales in TMEM, because copies and MMAs of different threads are not ordered against each other).
constexpr int GU_THREADS = UM_THREADS + 96;      // + warp 6 (up MMAs), warps 7 / 8 (scale-factor copies for gate / up)
template <int UM_STAGES, int NP = 16>
__global__ void __launch_bounds__(GU_THREADS, UM_STAGES <= 3 ? 2 : 1)
umma_gateup_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapA2,
                   const __grid_constant__ CUtensorMap tmapB, UmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = UmmaSmem<NP, 2, UM_STAGES>;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = a.swap_xy ? blockIdx.y : blockIdx.x, slot = a.swap_xy ? blockIdx.x : blockIdx.y, tok = blockIdx.z;
  const int il = a.inter;
  const int nks = (a.d + UM_BK - 1) / UM_BK;
  // accumulators 2 NP columns; scale factors one 4-column slot per stage and operand (gate weights, gate's copy of the
  // activation scales, up weights, up's copy): a slot is rewritten only when its stage's previous MMAs are done
  constexpr uint32_t TMEM_NEED = 2 * NP + 16 * UM_STAGES;
  constexpr uint32_t TMEM_COLS = TMEM_NEED <= 64 ? 64 : (TMEM_NEED <= 128 ? 128 : 256);

  if (threadIdx.x == 0) {
    um_mark(a, 0);
    for (int s = 0; s < UM_STAGES; ++s) {      // both issuing threads free a stage
      mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 2);
      mbar_init(&S.sfready[s][0], 1); mbar_init(&S.sfready[s][1], 1);
    }
    mbar_init(&S.acc_full, 2);
    S.fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) um_mark(a, 1);
  pdl_wait();
  const CUtensorMap* ma;
  int a_fp4, row_g, row_u;
  const uint8_t *sf_g, *sf_u;
  float weight = 1.f;
  bool skip = false;
  const bool grouped = a.seg_expert != nullptr;     // blockIdx.y = segment, blockIdx.z = 0; tok = first pair slot of the segment
  int count = 1;
  if (grouped) {
    int e = a.seg_expert[slot];
    count = a.seg_count[slot];
    if (e == -1) { skip = true; e = 0; count = 0; }
    if (e >= 0) {
      ma = &tmapA; a_fp4 = a.a_fp4;
      row_g = (e * 2) * il + tile * 128; row_u = row_g + il;
      sf_g = a.sfa + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
      sf_u = a.sfa + ((size_t)(row_u >> 7) * a.katoms_a) * 512;
    } else {
      ma = &tmapA2; a_fp4 = 0;
      row_g = tile * 128; row_u = row_g + il;
      sf_g = a.sfa2 + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
      sf_u = a.sfa2 + ((size_t)(row_u >> 7) * a.katoms_a) * 512;
    }
  } else if (slot < a.top_k) {
    int e = a.ids[(size_t)tok * a.top_k + slot];
    if (e < 0) { skip = true; e = 0; }         // not this rank's expert: nothing is loaded, multiplied or written
    weight = a.wts[(size_t)tok * a.top_k + slot];
    ma = &tmapA; a_fp4 = a.a_fp4;
    row_g = (e * 2) * il + tile * 128; row_u = row_g + il;
    sf_g = a.sfa + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
    sf_u = a.sfa + ((size_t)(row_u >> 7) * a.katoms_a) * 512;
  } else {
    ma = &tmapA2; a_fp4 = 0;
    row_g = tile * 128; row_u = row_g + il;
    sf_g = a.sfa2 + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
    sf_u = a.sfa2 + ((size_t)(row_u >> 7) * a.katoms_a) * 512;
  }
  const int b_row = grouped ? slot * NP : tok;
  const uint8_t* sfb = a.sfb + (size_t)(grouped ? slot : tok) * a.katoms_b * 512;
  const uint32_t STAGE_TX = 2 * (a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + 3 * 512;
  const uint32_t tmem = S.tmem_base;
  const uint32_t t_g = tmem, t_u = tmem + NP;
  const uint32_t t_sfg = tmem + 2 * NP, t_sfb = t_sfg + 4 * UM_STAGES, t_sfu = t_sfb + 4 * UM_STAGES, t_sfb2 = t_sfu + 4 * UM_STAGES;
  const int nks_run = skip ? 0 : nks;

  if (warp == 0) {
    if (elect_one()) {
      um_mark(a, 2);
      for (int i = 0; i < nks_run; ++i) {
        const int s = i % UM_STAGES;
        if (i >= UM_STAGES && !mbar_wait(&S.empty[s], ((i / UM_STAGES) - 1) & 1)) { S.fail = 1; break; }
        mbar_expect_tx(&S.full[s], STAGE_TX);
        tma_load_2d(S.a[s][0], ma, i * UM_BK, row_g, &S.full[s]);
        tma_load_2d(S.a[s][1], ma, i * UM_BK, row_u, &S.full[s]);
        tma_load_2d(S.b[s], &tmapB, i * UM_BK, b_row, &S.full[s]);
        bulk_load(S.sfa[s][0], sf_g + (size_t)i * 512, 512, &S.full[s]);
        bulk_load(S.sfa[s][1], sf_u + (size_t)i * 512, 512, &S.full[s]);
        bulk_load(S.sfb[s], sfb + (size_t)i * 512, 512, &S.full[s]);
      }
    }
  } else if (warp == 1 || warp == 6) {
    if (elect_one()) {
      const int h = warp == 1 ? 0 : 1;           // 0: gate tile, 1: up tile
      const uint32_t idesc = make_idesc(a_fp4 ? 5 : 0, 0, 128, NP);
      const uint32_t t_d = h ? t_u : t_g, t_sa = h ? t_sfu : t_sfg, t_sb = h ? t_sfb2 : t_sfb;
      for (int i = 0; i < nks_run; ++i) {
        const int s = i % UM_STAGES;
        const long long tw0 = (SFB_MARKS_ON && a.marks && i == 8 && h == 0) ? clock64() : 0;
        if (!mbar_wait(&S.sfready[s][h], (i / UM_STAGES) & 1)) { S.fail = 2; break; }      // data landed and scales copied
        tc_fence_after();
        if (i == 0 && h == 0) um_mark(a, 3);
        const long long tw1 = (SFB_MARKS_ON && a.marks && i == 8 && h == 0) ? clock64() : 0;
        const uint32_t sl = (uint32_t)s * 4;
        const long long tw2 = (SFB_MARKS_ON && a.marks && i == 8 && h == 0) ? clock64() : 0;
        const uint32_t w_addr = smem_u32(S.a[s][h]), b_addr = smem_u32(S.b[s]);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t bd = make_desc(b_addr + kk * 32, 1024, 16, 2);
          const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
          const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
          tc_mma_bs(t_d, make_desc(w_addr + kk * 32, 1024, 16, 2), bd, id, t_sa + sl, t_sb + sl, acc);
        }
        tc_commit(&S.empty[s]);
        if (SFB_MARKS_ON && a.marks && i == 8 && h == 0) {      // cycle counts of one steady-state k-step of the issuing thread: wait, scale copies, MMAs + commit
          const long long tw3 = clock64();
          const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
          if (cta < a.marks_cap) {
            a.marks[(size_t)cta * 16 + 13] = (unsigned long long)(tw1 - tw0);
            a.marks[(size_t)cta * 16 + 14] = (unsigned long long)(tw2 - tw1);
            a.marks[(size_t)cta * 16 + 15] = (unsigned long long)(tw3 - tw2);
          }
        }
      }
      tc_commit(&S.acc_full);     // arrives even after a failed wait so the epilogue never hangs
      if (h == 0) um_mark(a, 4);
    }
  } else if (warp == 7 || warp == 8) {
    if (elect_one()) {      // scale-factor copies of one accumulator's operands, a thread of their own
      const int h = warp == 7 ? 0 : 1;
      const uint32_t t_sa = h ? t_sfu : t_sfg, t_sb = h ? t_sfb2 : t_sfb;
      for (int i = 0; i < nks_run; ++i) {
        const int s = i % UM_STAGES;
        if (!mbar_wait(&S.full[s], (i / UM_STAGES) & 1)) { S.fail = 4; break; }
        tc_fence_after();
        tc_cp_sf(t_sa + (uint32_t)s * 4, make_desc(smem_u32(S.sfa[s][h]), 128, 0, 0));
        tc_cp_sf(t_sb + (uint32_t)s * 4, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
        tc_commit(&S.sfready[s][h]);
      }
    }
  } else {
    const int q = warp & 3;
    const bool got = mbar_wait(&S.acc_full, 0);
    tc_fence_after();
    if (warp == 2 && lane == 0) um_mark(a, 5);
    const int col = tile * 128 + q * 32 + lane;   // column of the intermediate activation
    const int KBi = il / 32;
    const int ncol = grouped ? count : 1;         // accumulator column j = pair j of the segment (one column when ungrouped)
    const bool live = got && !S.fail && col < il;
    // segments: the FP8 codes of the tile are staged pair-major in the idle operand stages and leave as one 128-byte bulk
    // copy per pair row; the routing weights of a 16-pair chunk come in with one load (a load per pair inside the loop made
    // every pair wait for a trip to L2)
    // (16-pair segments keep their direct stores: one chunk of columns, and the barriers and the copy's latency cost more)
    const bool stq_cta = NP >= 32 && grouped && !skip && (tile + 1) * 128 <= il;      // CTA-uniform
    const bool stq = stq_cta && live;
    uint8_t* sq = &S.a[0][0][0];
    // the tile's scale bytes are one whole 512-byte atom of the segment's atom set (k-atom = tile): staged too
    uint8_t* ssf = &S.sfa[0][0][0];
    const bool stsf = stq_cta && a.act_sf && !a.act_s;
    if (stsf) {
      reinterpret_cast<uint32_t*>(ssf)[q * 32 + lane] = 0x7f7f7f7fu;      // rows past the segment's pairs: scale 1
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const float limit = a.limit;
    if (!grouped) {
      // one token per CTA: a single accumulator column, quantised and stored directly
      uint32_t vg[16], vu[16];
      tc_ld16(t_g + ((uint32_t)(q * 32) << 16), vg);
      tc_ld16(t_u + ((uint32_t)(q * 32) << 16), vu);
      tc_wait_ld();
      float act = 0.f;
      if (live) {
        const float g = fminf(bfr(__uint_as_float(vg[0])), limit);
        const float u = fminf(fmaxf(bfr(__uint_as_float(vu[0])), -limit), limit);
        act = bfr(g / (1.f + expf(-g)) * u * weight);
      }
      uint8_t sc;
      const uint8_t code = warp_quant_fp8(act, &sc);
      if (live && !skip) {
        const size_t row = (size_t)tok * a.slots + slot;
        a.act_q[row * il + col] = code;
        if (lane == 0) {
          if (a.act_s) a.act_s[row * KBi + col / 32] = sc;
          if (a.act_sf) a.act_sf[row * sf_bytes(1, KBi) + sf_offset(0, col / 32, KBi)] = sc;
        }
      }
    }
#pragma unroll 1
    for (int c0 = 0; grouped && c0 < NP && c0 < ncol; c0 += 16) {
      uint32_t vg[16], vu[16];
      tc_ld16(t_g + ((uint32_t)(q * 32) << 16) + c0, vg);
      tc_ld16(t_u + ((uint32_t)(q * 32) << 16) + c0, vu);
      float wv = weight;
      if (grouped) {
        const int jx = c0 + (lane & 15);
        wv = jx < ncol ? a.seg_weight[slot * NP + jx] : 0.f;
      }
      tc_wait_ld();
      if (c0 == 0 && warp == 2 && lane == 0) um_mark(a, 8);
      if (c0 == 16 && warp == 2 && lane == 0) um_mark(a, 12);
      // three passes over the chunk so that the sixteen columns' chains (exp, divide; reduction; encode) overlap instead
      // of running one after the other; per column the arithmetic is unchanged
      float act[16];
      const int nb = ncol - c0;                   // columns of this chunk that exist (warp-uniform); the passes skip the rest
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        act[jj] = 0.f;
        if (jj >= nb) continue;
        const float wj = grouped ? __shfl_sync(0xffffffffu, wv, jj) : weight;
        if (live) {
          const float g = fminf(bfr(__uint_as_float(vg[jj])), limit);
          const float u = fminf(fmaxf(bfr(__uint_as_float(vu[jj])), -limit), limit);
          act[jj] = bfr(g / (1.f + expf(-g)) * u * wj);
        }
      }
      uint32_t amax_bits[16];
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        amax_bits[jj] = 0u;
        if (jj >= nb) continue;
        const float ax = (act[jj] == act[jj]) ? fabsf(act[jj]) : 0.f;
        amax_bits[jj] = __reduce_max_sync(0xffffffffu, __float_as_uint(ax));
      }
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int j = c0 + jj;
        if (j < ncol) {                           // warp-uniform
          const uint8_t sc = act_scale_code_fp8(__uint_as_float(amax_bits[jj]));
          const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
          const uint8_t code = enc_e4m3(act[jj] * inv);
          if (live && !skip) {
            const size_t row = grouped ? (size_t)slot * NP + j : (size_t)tok * a.slots + slot;
            if (stq) sq[j * 128 + q * 32 + lane] = code;
            else a.act_q[row * il + col] = code;
            if (lane == 0) {
              if (a.act_s) a.act_s[row * KBi + col / 32] = sc;
              if (stsf) {
                ssf[(j & 31) * 16 + (j >> 5) * 4 + q] = sc;
              } else if (a.act_sf) {
                if (grouped) a.act_sf[(size_t)slot * sf_bytes(NP, KBi) + sf_offset(j, col / 32, KBi)] = sc;   // one atom set per segment, row j
                else a.act_sf[row * sf_bytes(1, KBi) + sf_offset(0, col / 32, KBi)] = sc;
              }
            }
          }
        }
      }
    }
    if (warp == 2 && lane == 0) um_mark(a, 9);
    if (stq_cta) {        // CTA-uniform, so every epilogue warp reaches the barrier whatever its own wait returned
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) um_mark(a, 10);
      const int j = q * 32 + lane;
      if (got && !S.fail) {
        bool any = false;
        if (j < ncol) { bulk_store(a.act_q + ((size_t)slot * NP + j) * il + tile * 128, smem_u32(sq + j * 128), 128); any = true; }
        if (stsf && j == 0) { bulk_store(a.act_sf + (size_t)slot * sf_bytes(NP, KBi) + (size_t)tile * 512, smem_u32(ssf), 512); any = true; }
        if (any) bulk_store_commit_wait_read();
      }
    }
    if ((!got || S.fail) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 20 + S.fail, blockIdx.x, blockIdx.y);
    if (warp == 2 && lane == 0) um_mark(a, 6);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) um_mark(a, 7);
  if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- persistent grouped gate/up for wide (64-pair) segments --------------------------------------------------------------
// One CTA per SM walks over (column tile of the intermediate width, segment) pairs.  While the four epilogue warps turn one
// tile's accumulators into FP8 activations (SwiGLU, routing weight, re-quantisation: 14 of a one-tile CTA's 48 us), the
// producer and the two MMA-issuing threads are already in the next tile's main loop on the other accumulator set.  The
// arithmetic, its order and the output bits are those of umma_gateup_kernel<2, 64>.
constexpr int PG_STAGES = 5;
constexpr int PG_NP = 64;
struct UmmaGateupPersistSmem {
  alignas(1024) uint8_t a[PG_STAGES][2][UM_A_BYTES];
  alignas(1024) uint8_t b[PG_STAGES][PG_NP * UM_BK];
  alignas(1024) uint8_t sq[PG_NP * 128];          // the tile's FP8 codes on their way out, pair-major
  alignas(128) uint8_t ssf[512];                  // and its scale atom
  alignas(128) uint8_t sfa[PG_STAGES][2][512];
  alignas(128) uint8_t sfb[PG_STAGES][512];
  alignas(8) uint64_t full[PG_STAGES];
  alignas(8) uint64_t empty[PG_STAGES];
  alignas(8) uint64_t sfready[PG_STAGES][2];      // the stage's scale factors are in TMEM (one barrier per accumulator)
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int fail;
  volatile int ep_ok;
};
// warps: 0 TMA producer, 1 / 6 MMA issue (gate / up), 2..5 epilogue, 7 / 8 scale-factor copies (gate / up) when
// copier_threads is set.  With single-thread roles entered through elect.sync an MMA thread issues its two scale copies and
// four MMAs per k-step well inside the stage's turn-over, and doing the copies itself saves one hand-over per stage (the
// shipped choice); the copier threads date from roles entered by lane index, where seven operations per k-step paced the loop.
constexpr int PG_THREADS = 288;

__global__ void __launch_bounds__(PG_THREADS, 1)
umma_gateup_persistent_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapA2,
                              const __grid_constant__ CUtensorMap tmapB, UmmaArgs a, int n_tiles, int n_segs, int copier_threads) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = UmmaGateupPersistSmem;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int NP = PG_NP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int il = a.inter;
  const int nks = (a.d + UM_BK - 1) / UM_BK;
  const int total = n_tiles * n_segs;
  if (threadIdx.x == 0) {
    for (int s = 0; s < PG_STAGES; ++s) {
      mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 2);
      mbar_init(&S.sfready[s][0], 1); mbar_init(&S.sfready[s][1], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 2); mbar_init(&S.acc_empty[b], 1); }
    S.fail = 0;
    S.ep_ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, 512);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem = S.tmem_base;
  // scale factors: one 4-column slot per stage and operand, so a slot is rewritten only after the MMAs of the stage's previous
  // use are done (the producer refills the stage only then): gate weights 256.., gate's activation copy 276.., up 296.., 316..
  const uint32_t t_sfg = tmem + 256, t_sfb = tmem + 276, t_sfu = tmem + 296, t_sfb2 = tmem + 316;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int tile = t % n_tiles, seg = t / n_tiles;
        const int e = a.seg_expert[seg];
        if (e == -1) continue;                                   // an unused segment: no role touches a barrier for it
        const CUtensorMap* ma;
        int a_fp4, row_g;
        const uint8_t *sf_g, *sf_u;
        if (e >= 0) {
          ma = &tmapA; a_fp4 = a.a_fp4;
          row_g = (e * 2) * il + tile * 128;
          sf_g = a.sfa + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
          sf_u = a.sfa + ((size_t)((row_g + il) >> 7) * a.katoms_a) * 512;
        } else {
          ma = &tmapA2; a_fp4 = 0;
          row_g = tile * 128;
          sf_g = a.sfa2 + ((size_t)(row_g >> 7) * a.katoms_a) * 512;
          sf_u = a.sfa2 + ((size_t)((row_g + il) >> 7) * a.katoms_a) * 512;
        }
        const int row_u = row_g + il;
        const uint8_t* sfb = a.sfb + (size_t)seg * a.katoms_b * 512;
        const uint32_t stage_tx = 2 * (a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + 3 * 512;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PG_STAGES;
          if (it >= PG_STAGES && !mbar_wait(&S.empty[s], ((it / PG_STAGES) - 1) & 1)) { S.fail = 1; break; }
          mbar_expect_tx(&S.full[s], stage_tx);
          tma_load_2d(S.a[s][0], ma, i * UM_BK, row_g, &S.full[s]);
          tma_load_2d(S.a[s][1], ma, i * UM_BK, row_u, &S.full[s]);
          tma_load_2d(S.b[s], &tmapB, i * UM_BK, seg * NP, &S.full[s]);
          bulk_load(S.sfa[s][0], sf_g + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfa[s][1], sf_u + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfb[s], sfb + (size_t)i * 512, 512, &S.full[s]);
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    if (elect_one()) {
      const int h = warp == 1 ? 0 : 1;           // 0: gate tile, 1: up tile
      const uint32_t t_sa = h ? t_sfu : t_sfg, t_sb = h ? t_sfb2 : t_sfb;
      uint32_t it = 0;
      int lt = 0;
      long long c_acc = 0, c_full = 0, c_all0 = SFB_MARKS_ON ? clock64() : 0;      // cycles waiting for a free accumulator set / for data
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int seg = t / n_tiles;
        const int e = a.seg_expert[seg];
        if (e == -1) continue;
        const uint32_t idesc = make_idesc((e >= 0 && a.a_fp4) ? 5 : 0, 0, 128, NP);
        const int buf = lt & 1;
        const long long w0 = SFB_MARKS_ON ? clock64() : 0;
        if (lt >= 2 && !mbar_wait(&S.acc_empty[buf], ((lt >> 1) - 1) & 1)) { S.fail = 3; break; }
        if (SFB_MARKS_ON) c_acc += clock64() - w0;
        tc_fence_after();
        const uint32_t t_d = tmem + (uint32_t)buf * 128 + (h ? NP : 0);
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PG_STAGES;
          const long long w1 = SFB_MARKS_ON ? clock64() : 0;
          if (!mbar_wait(copier_threads ? &S.sfready[s][h] : &S.full[s], (it / PG_STAGES) & 1)) { S.fail = 2; ok = false; break; }
          if (SFB_MARKS_ON) c_full += clock64() - w1;
          tc_fence_after();
          const uint32_t sl = (uint32_t)s * 4;
          if (!copier_threads) {      // this thread copies its own operands' scales: one hand-over less per stage
            tc_cp_sf(t_sa + sl, make_desc(smem_u32(S.sfa[s][h]), 128, 0, 0));
            tc_cp_sf(t_sb + sl, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
          }
          const uint32_t w_addr = smem_u32(S.a[s][h]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
            tc_mma_bs(t_d, make_desc(w_addr + kk * 32, 1024, 16, 2), make_desc(b_addr + kk * 32, 1024, 16, 2), id, t_sa + sl, t_sb + sl,
                      (i > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&S.empty[s]);
        }
        tc_commit(&S.acc_full[buf]);
        if (!ok) break;
        ++lt;
      }
      if (SFB_MARKS_ON && a.marks && h == 0 && (int)blockIdx.x < a.marks_cap) {      // per CTA: tiles, total, waiting-for-set, waiting-for-data cycles
        a.marks[(size_t)blockIdx.x * 16 + 0] = (unsigned long long)lt;
        a.marks[(size_t)blockIdx.x * 16 + 1] = (unsigned long long)(clock64() - c_all0);
        a.marks[(size_t)blockIdx.x * 16 + 2] = (unsigned long long)c_acc;
        a.marks[(size_t)blockIdx.x * 16 + 3] = (unsigned long long)c_full;
      }
    }
  } else if (warp == 7 || warp == 8) {
    if (copier_threads && elect_one()) {
      const int h = warp == 7 ? 0 : 1;
      const uint32_t t_sa = h ? t_sfu : t_sfg, t_sb = h ? t_sfb2 : t_sfb;
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        if (a.seg_expert[t / n_tiles] == -1) continue;
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PG_STAGES;
          if (!mbar_wait(&S.full[s], (it / PG_STAGES) & 1)) { S.fail = 4; ok = false; break; }
          tc_fence_after();
          tc_cp_sf(t_sa + (uint32_t)s * 4, make_desc(smem_u32(S.sfa[s][h]), 128, 0, 0));
          tc_cp_sf(t_sb + (uint32_t)s * 4, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
          tc_commit(&S.sfready[s][h]);
        }
        if (!ok) break;
      }
    }
  } else {
    const int q = warp & 3;
    const int KBi = il / 32;
    const float limit = a.limit;
    bool pending = false;
    int lt = 0;
    long long c_wait = 0;                          // cycles the epilogue waited for an accumulator (marks builds)
    const long long c_ep0 = SFB_MARKS_ON ? clock64() : 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      const int tile = t % n_tiles, seg = t / n_tiles;
      const int e = a.seg_expert[seg];
      if (e == -1) continue;                       // CTA-uniform (every thread reads the same word)
      const int ncol = a.seg_count[seg];
      const int buf = lt & 1;
      if (warp == 2) {
        bool got = true;
        const long long w2 = SFB_MARKS_ON ? clock64() : 0;
        if (lane == 0) got = mbar_wait(&S.acc_full[buf], (lt >> 1) & 1) && !S.fail;
        if (SFB_MARKS_ON && lane == 0) c_wait += clock64() - w2;
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (lane == 0 && !got) S.ep_ok = 0;
      }
      if (pending) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!S.ep_ok) break;
      tc_fence_after();
      reinterpret_cast<uint32_t*>(S.ssf)[q * 32 + lane] = 0x7f7f7f7fu;      // rows past the segment's pairs: scale 1
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t t_g = tmem + (uint32_t)buf * 128, t_u = t_g + NP;
      const int col = tile * 128 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < NP && c0 < ncol; c0 += 16) {
        uint32_t vg[16], vu[16];
        tc_ld16(t_g + ((uint32_t)(q * 32) << 16) + c0, vg);
        tc_ld16(t_u + ((uint32_t)(q * 32) << 16) + c0, vu);
        const int jx = c0 + (lane & 15);
        const float wv = jx < ncol ? a.seg_weight[seg * NP + jx] : 0.f;
        tc_wait_ld();
        // sixteen independent chains without branches (one warp per scheduler runs the epilogue: only instruction-level
        // parallelism hides the latency of the exponential and the division); pair slots past the segment's count carry
        // weight 0 and are never stored
        float act[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const float wj = __shfl_sync(0xffffffffu, wv, jj);
          const float g = fminf(bfr(__uint_as_float(vg[jj])), limit);
          const float u = fminf(fmaxf(bfr(__uint_as_float(vu[jj])), -limit), limit);
          act[jj] = bfr(g / (1.f + expf(-g)) * u * wj);
        }
        uint32_t amax_bits[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const float ax = (act[jj] == act[jj]) ? fabsf(act[jj]) : 0.f;
          amax_bits[jj] = __reduce_max_sync(0xffffffffu, __float_as_uint(ax));
        }
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int j = c0 + jj;
          const uint8_t sc = act_scale_code_fp8(__uint_as_float(amax_bits[jj]));
          const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
          const uint8_t code = enc_e4m3(act[jj] * inv);
          if (j < ncol) {                           // warp-uniform
            S.sq[j * 128 + q * 32 + lane] = code;
            if (lane == 0) S.ssf[(j & 31) * 16 + (j >> 5) * 4 + q] = sc;
          }
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) mbar_arrive(&S.acc_empty[buf]);
      const int j = q * 32 + lane;
      pending = false;
      if (j < ncol) { bulk_store(a.act_q + ((size_t)seg * NP + j) * il + tile * 128, smem_u32(S.sq + j * 128), 128); pending = true; }
      if (j == 0) { bulk_store(a.act_sf + (size_t)seg * sf_bytes(NP, KBi) + (size_t)tile * 512, smem_u32(S.ssf), 512); pending = true; }
      if (pending) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      ++lt;
    }
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if (SFB_MARKS_ON && a.marks && warp == 2 && lane == 0 && (int)blockIdx.x < a.marks_cap) {
      a.marks[(size_t)blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - c_ep0);
      a.marks[(size_t)blockIdx.x * 16 + 5] = (unsigned long long)c_wait;
    }
    if ((S.fail || !S.ep_ok) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 70 + S.fail, blockIdx.x, lt);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---- persistent grouped down projection for wide (64-pair) segments ---------------------------------------------------------
// One CTA per SM walks over (column tile of the model width, segment) pairs with seven operand stages in flight; the
// epilogue of one tile (TMEM -> fp32 tile in shared memory -> one 512-byte bulk copy per pair row) runs under the next
// tile's main loop on the other accumulator set.  One-tile CTAs spent a third of their life outside the main loop and, at
// three per SM with two stages each, kept too few bytes in flight for the weight stream.  The scale-factor copies have
// their own issuing thread (a thread issues one tcgen05 operation per ~80 cycles, and seven per k-step would pace the
// loop).  Arithmetic, order and output bits are those of umma_gemm_kernel<64, false, 2> in UM_DOWN_GROUPED mode.
constexpr int PD_STAGES = 7;
constexpr int PD_NP = 64;
constexpr int PD_THREADS = 224;      // warps: 0 TMA producer, 1 MMA issue, 2..5 epilogue, 6 scale-factor copies
struct UmmaDownPersistSmem {
  alignas(1024) uint8_t a[PD_STAGES][UM_A_BYTES];
  alignas(1024) uint8_t b[PD_STAGES][PD_NP * UM_BK];
  alignas(1024) float outf[PD_NP * 128];           // the tile on its way out, pair-major
  alignas(128) uint8_t sfa[PD_STAGES][512];
  alignas(128) uint8_t sfb[PD_STAGES][512];
  alignas(8) uint64_t full[PD_STAGES];
  alignas(8) uint64_t empty[PD_STAGES];
  alignas(8) uint64_t sfready[PD_STAGES];
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int fail;
  volatile int ep_ok;
};

__global__ void __launch_bounds__(PD_THREADS, 1)
umma_down_persistent_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapA2,
                            const __grid_constant__ CUtensorMap tmapB, UmmaArgs a, int n_tiles, int n_segs) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = UmmaDownPersistSmem;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int NP = PD_NP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nks = (a.inter + UM_BK - 1) / UM_BK;
  const int total = n_tiles * n_segs;
  if (threadIdx.x == 0) {
    for (int s = 0; s < PD_STAGES; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); mbar_init(&S.sfready[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 1); }
    S.fail = 0;
    S.ep_ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, 256);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem = S.tmem_base;
  // accumulator sets at columns 0 and 64; one 4-column scale-factor slot per stage and operand (a slot is rewritten only
  // after the MMAs of the stage's previous use are done, because the producer refills the stage only then)
  const uint32_t t_sfa = tmem + 128, t_sfb = tmem + 160;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      long long c_empty = 0;                                     // cycles the producer waited for a free stage (marks builds)
      const long long c_p0 = SFB_MARKS_ON ? clock64() : 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int tile = t % n_tiles, seg = t / n_tiles;
        const int e = a.seg_expert[seg];
        if (e == -1) continue;                                   // an unused segment: no role touches a barrier for it
        const CUtensorMap* ma;
        int a_fp4, row0;
        const uint8_t* sfa;
        if (e >= 0) {
          ma = &tmapA; a_fp4 = a.a_fp4;
          row0 = e * a.d + tile * 128;
          sfa = a.sfa + ((size_t)(row0 >> 7) * a.katoms_a) * 512;
        } else {
          ma = &tmapA2; a_fp4 = 0;
          row0 = tile * 128;
          sfa = a.sfa2 + ((size_t)tile * a.katoms_a) * 512;
        }
        const uint8_t* sfb = a.sfb + (size_t)seg * a.katoms_b * 512;
        const uint32_t stage_tx = (a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + 1024;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PD_STAGES;
          const long long w0 = SFB_MARKS_ON ? clock64() : 0;
          if (it >= PD_STAGES && !mbar_wait(&S.empty[s], ((it / PD_STAGES) - 1) & 1)) { S.fail = 1; break; }
          if (SFB_MARKS_ON) c_empty += clock64() - w0;
          mbar_expect_tx(&S.full[s], stage_tx);
          tma_load_2d(S.a[s], ma, i * UM_BK, row0, &S.full[s]);
          tma_load_2d(S.b[s], &tmapB, i * UM_BK, seg * NP, &S.full[s]);
          bulk_load(S.sfa[s], sfa + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfb[s], sfb + (size_t)i * 512, 512, &S.full[s]);
        }
      }
      if (SFB_MARKS_ON && a.marks && (int)blockIdx.x < a.marks_cap) {      // per CTA: k-steps, producer cycles, of which waiting
        a.marks[(size_t)blockIdx.x * 16 + 6] = (unsigned long long)it;
        a.marks[(size_t)blockIdx.x * 16 + 7] = (unsigned long long)(clock64() - c_p0);
        a.marks[(size_t)blockIdx.x * 16 + 8] = (unsigned long long)c_empty;
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      uint32_t it = 0;
      int lt = 0;
      long long c_acc = 0, c_sf = 0;               // cycles waiting for a free accumulator set / for the stage's scale factors
      const long long c_m0 = SFB_MARKS_ON ? clock64() : 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int e = a.seg_expert[t / n_tiles];
        if (e == -1) continue;
        const uint32_t idesc = make_idesc((e >= 0 && a.a_fp4) ? 5 : 0, 0, 128, NP);
        const int buf = lt & 1;
        const long long w0 = SFB_MARKS_ON ? clock64() : 0;
        if (lt >= 2 && !mbar_wait(&S.acc_empty[buf], ((lt >> 1) - 1) & 1)) { S.fail = 3; break; }
        if (SFB_MARKS_ON) c_acc += clock64() - w0;
        tc_fence_after();
        const uint32_t t_acc = tmem + (uint32_t)buf * NP;
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PD_STAGES;
          const long long w1 = SFB_MARKS_ON ? clock64() : 0;
          if (!mbar_wait(&S.sfready[s], (it / PD_STAGES) & 1)) { S.fail = 2; ok = false; break; }
          if (SFB_MARKS_ON) c_sf += clock64() - w1;
          tc_fence_after();
          const uint32_t sl = (uint32_t)s * 4;
          const uint32_t a_addr = smem_u32(S.a[s]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
            tc_mma_bs(t_acc, make_desc(a_addr + kk * 32, 1024, 16, 2), make_desc(b_addr + kk * 32, 1024, 16, 2), id, t_sfa + sl,
                      t_sfb + sl, (i > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&S.empty[s]);
        }
        tc_commit(&S.acc_full[buf]);      // arrives even after a failed wait, so the epilogue never waits for its limit
        if (!ok) break;
        ++lt;
      }
      if (SFB_MARKS_ON && a.marks && (int)blockIdx.x < a.marks_cap) {      // per CTA: tiles, MMA-thread cycles, waiting for a set / for data
        a.marks[(size_t)blockIdx.x * 16 + 0] = (unsigned long long)lt;
        a.marks[(size_t)blockIdx.x * 16 + 1] = (unsigned long long)(clock64() - c_m0);
        a.marks[(size_t)blockIdx.x * 16 + 2] = (unsigned long long)c_acc;
        a.marks[(size_t)blockIdx.x * 16 + 3] = (unsigned long long)c_sf;
      }
    }
  } else if (warp == 6) {
    if (elect_one()) {
      uint32_t it = 0;
      long long c_full = 0;                        // cycles the copier waited for a stage to land
      const long long c_c0 = SFB_MARKS_ON ? clock64() : 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        if (a.seg_expert[t / n_tiles] == -1) continue;
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % PD_STAGES;
          const long long w0 = SFB_MARKS_ON ? clock64() : 0;
          if (!mbar_wait(&S.full[s], (it / PD_STAGES) & 1)) { S.fail = 4; ok = false; break; }
          if (SFB_MARKS_ON) c_full += clock64() - w0;
          tc_fence_after();
          tc_cp_sf(t_sfa + (uint32_t)s * 4, make_desc(smem_u32(S.sfa[s]), 128, 0, 0));
          tc_cp_sf(t_sfb + (uint32_t)s * 4, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
          tc_commit(&S.sfready[s]);
        }
        if (!ok) break;
      }
      if (SFB_MARKS_ON && a.marks && (int)blockIdx.x < a.marks_cap) {
        a.marks[(size_t)blockIdx.x * 16 + 4] = (unsigned long long)(clock64() - c_c0);
        a.marks[(size_t)blockIdx.x * 16 + 5] = (unsigned long long)c_full;
      }
    }
  } else {
    const int q = warp & 3;
    bool pending = false;
    int lt = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      const int tile = t % n_tiles, seg = t / n_tiles;
      if (a.seg_expert[seg] == -1) continue;       // CTA-uniform (every thread reads the same word)
      const int nv = a.seg_count[seg];
      const int buf = lt & 1;
      if (warp == 2) {
        bool got = true;
        if (lane == 0) got = mbar_wait(&S.acc_full[buf], (lt >> 1) & 1) && !S.fail;
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (lane == 0 && !got) S.ep_ok = 0;
      }
      if (pending) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the staging tile has been read out
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!S.ep_ok) break;
      tc_fence_after();
      const uint32_t t_acc = tmem + (uint32_t)buf * NP;
      {
        uint32_t v[NP / 16][16];      // every chunk requested before the one wait
#pragma unroll
        for (int ch = 0; ch < NP / 16; ++ch) tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + ch * 16, v[ch]);
        tc_wait_ld();
#pragma unroll
        for (int ch = 0; ch < NP / 16; ++ch) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (ch * 16 + j < nv) S.outf[(ch * 16 + j) * 128 + q * 32 + lane] = __uint_as_float(v[ch][j]);
        }
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) mbar_arrive(&S.acc_empty[buf]);       // every warp's TMEM reads of this set are done
      const int tok = q * 32 + lane;
      pending = false;
      if (tok < nv) {
        bulk_store(a.out_f + (int64_t)(seg * NP + tok) * a.out_stride + tile * 128, smem_u32(S.outf + tok * 128), 512);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        pending = true;
      }
      ++lt;
    }
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if ((S.fail || !S.ep_ok) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 80 + S.fail, blockIdx.x, lt);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 256);
}

// ---- persistent grouped down projection, two column tiles per work item --------------------------------------------------------
// The one-tile form above carries 8 KB of weights and 8 KB of activations per stage, so only half of its ring of stages is
// HBM traffic.  Here a work item is a PAIR of neighbouring column tiles of one segment: both weight tiles share the stage's
// activation tile (stage = 2 x 16 KB + 8 KB, five stages: 80 KB of weights in flight per SM instead of 56), each has its own
// accumulator (two sets of two) and the fp32 tiles leave through a 16 KB staging buffer, 32 pair rows at a time.  Arithmetic,
// order and output bits are those of the one-tile kernels.
constexpr int PD2_STAGES = 5;
struct UmmaDownPersist2Smem {
  alignas(1024) uint8_t a[PD2_STAGES][2][UM_A_BYTES];
  alignas(1024) uint8_t b[PD2_STAGES][PD_NP * UM_BK];
  alignas(1024) float outf[32 * 128];              // 32 pair rows of one tile on their way out
  alignas(128) uint8_t sfa[PD2_STAGES][2][512];
  alignas(128) uint8_t sfb[PD2_STAGES][512];
  alignas(8) uint64_t full[PD2_STAGES];
  alignas(8) uint64_t empty[PD2_STAGES];
  alignas(8) uint64_t sfready[PD2_STAGES];
  alignas(8) uint64_t acc_full[2];
  alignas(8) uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int fail;
  volatile int ep_ok;
};

__global__ void __launch_bounds__(PD_THREADS, 1)
umma_down_persistent2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapA2,
                             const __grid_constant__ CUtensorMap tmapB, UmmaArgs a, int n_tile_pairs, int n_segs) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = UmmaDownPersist2Smem;
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int NP = PD_NP, ST = PD2_STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nks = (a.inter + UM_BK - 1) / UM_BK;
  const int total = n_tile_pairs * n_segs;
  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); mbar_init(&S.sfready[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 1); }
    S.fail = 0;
    S.ep_ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(&S.tmem_base, 512);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem = S.tmem_base;
  // accumulators: set b at columns 128 b (tile 0) and 128 b + 64 (tile 1); scale-factor slots per stage and operand from 256
  const uint32_t t_sfa0 = tmem + 256, t_sfa1 = tmem + 288, t_sfb = tmem + 320;

  if (warp == 0) {
    if (elect_one()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int tp = t % n_tile_pairs, seg = t / n_tile_pairs;
        const int e = a.seg_expert[seg];
        if (e == -1) continue;                                   // an unused segment: no role touches a barrier for it
        const CUtensorMap* ma;
        int a_fp4, row0;
        const uint8_t* sfa;
        if (e >= 0) {
          ma = &tmapA; a_fp4 = a.a_fp4;
          row0 = e * a.d + tp * 256;
          sfa = a.sfa + ((size_t)(row0 >> 7) * a.katoms_a) * 512;
        } else {
          ma = &tmapA2; a_fp4 = 0;
          row0 = tp * 256;
          sfa = a.sfa2 + ((size_t)(tp * 2) * a.katoms_a) * 512;
        }
        const uint8_t* sfa1 = sfa + (size_t)a.katoms_a * 512;      // the next 128 weight rows
        const uint8_t* sfb = a.sfb + (size_t)seg * a.katoms_b * 512;
        const uint32_t stage_tx = 2 * (a_fp4 ? UM_A_BYTES / 2 : UM_A_BYTES) + NP * UM_BK + 3 * 512;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % ST;
          if (it >= ST && !mbar_wait(&S.empty[s], ((it / ST) - 1) & 1)) { S.fail = 1; break; }
          mbar_expect_tx(&S.full[s], stage_tx);
          tma_load_2d(S.a[s][0], ma, i * UM_BK, row0, &S.full[s]);
          tma_load_2d(S.a[s][1], ma, i * UM_BK, row0 + 128, &S.full[s]);
          tma_load_2d(S.b[s], &tmapB, i * UM_BK, seg * NP, &S.full[s]);
          bulk_load(S.sfa[s][0], sfa + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfa[s][1], sfa1 + (size_t)i * 512, 512, &S.full[s]);
          bulk_load(S.sfb[s], sfb + (size_t)i * 512, 512, &S.full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      uint32_t it = 0;
      int lt = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        const int e = a.seg_expert[t / n_tile_pairs];
        if (e == -1) continue;
        const uint32_t idesc = make_idesc((e >= 0 && a.a_fp4) ? 5 : 0, 0, 128, NP);
        const int buf = lt & 1;
        if (lt >= 2 && !mbar_wait(&S.acc_empty[buf], ((lt >> 1) - 1) & 1)) { S.fail = 3; break; }
        tc_fence_after();
        const uint32_t t_acc = tmem + (uint32_t)buf * 128;
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % ST;
          if (!mbar_wait(&S.sfready[s], (it / ST) & 1)) { S.fail = 2; ok = false; break; }
          tc_fence_after();
          const uint32_t sl = (uint32_t)s * 4;
          const uint32_t a0_addr = smem_u32(S.a[s][0]), a1_addr = smem_u32(S.a[s][1]), b_addr = smem_u32(S.b[s]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t id = idesc | ((uint32_t)kk << 29) | ((uint32_t)kk << 4);
            const uint64_t bd = make_desc(b_addr + kk * 32, 1024, 16, 2);
            tc_mma_bs(t_acc, make_desc(a0_addr + kk * 32, 1024, 16, 2), bd, id, t_sfa0 + sl, t_sfb + sl, (i > 0 || kk > 0) ? 1u : 0u);
            tc_mma_bs(t_acc + NP, make_desc(a1_addr + kk * 32, 1024, 16, 2), bd, id, t_sfa1 + sl, t_sfb + sl, (i > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&S.empty[s]);
        }
        tc_commit(&S.acc_full[buf]);      // arrives even after a failed wait, so the epilogue never waits for its limit
        if (!ok) break;
        ++lt;
      }
    }
  } else if (warp == 6) {
    if (elect_one()) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total && !S.fail; t += gridDim.x) {
        if (a.seg_expert[t / n_tile_pairs] == -1) continue;
        bool ok = true;
        for (int i = 0; i < nks; ++i, ++it) {
          const int s = it % ST;
          if (!mbar_wait(&S.full[s], (it / ST) & 1)) { S.fail = 4; ok = false; break; }
          tc_fence_after();
          tc_cp_sf(t_sfa0 + (uint32_t)s * 4, make_desc(smem_u32(S.sfa[s][0]), 128, 0, 0));
          tc_cp_sf(t_sfa1 + (uint32_t)s * 4, make_desc(smem_u32(S.sfa[s][1]), 128, 0, 0));
          tc_cp_sf(t_sfb + (uint32_t)s * 4, make_desc(smem_u32(S.sfb[s]), 128, 0, 0));
          tc_commit(&S.sfready[s]);
        }
        if (!ok) break;
      }
    }
  } else {
    const int q = warp & 3;
    bool pending = false;
    int lt = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      const int tp = t % n_tile_pairs, seg = t / n_tile_pairs;
      if (a.seg_expert[seg] == -1) continue;       // CTA-uniform (every thread reads the same word)
      const int nv = a.seg_count[seg];
      const int buf = lt & 1;
      if (warp == 2) {
        bool got = true;
        if (lane == 0) got = mbar_wait(&S.acc_full[buf], (lt >> 1) & 1) && !S.fail;
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (lane == 0 && !got) S.ep_ok = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!S.ep_ok) break;
      tc_fence_after();
      // four rounds: (tile 0, pairs 0..31), (tile 0, pairs 32..63), (tile 1, ...); a round whose pairs do not exist is skipped
#pragma unroll 1
      for (int h = 0; h < 4; ++h) {
        const int j = h >> 1, p0 = (h & 1) * 32;
        if (p0 >= nv) continue;                    // CTA-uniform
        uint32_t v[2][16];
        const uint32_t t_acc = tmem + (uint32_t)buf * 128 + (uint32_t)j * NP + p0;
        tc_ld16(t_acc + ((uint32_t)(q * 32) << 16), v[0]);
        tc_ld16(t_acc + ((uint32_t)(q * 32) << 16) + 16, v[1]);
        tc_wait_ld();
        if (pending) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the staging rows have been read out
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int ch = 0; ch < 2; ++ch)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (p0 + ch * 16 + i < nv) S.outf[(ch * 16 + i) * 128 + q * 32 + lane] = __uint_as_float(v[ch][i]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        pending = false;
        if (q == 0 && p0 + lane < nv) {
          bulk_store(a.out_f + (int64_t)(seg * NP + p0 + lane) * a.out_stride + (tp * 2 + j) * 128, smem_u32(S.outf + lane * 128), 512);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          pending = true;
        }
      }
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) mbar_arrive(&S.acc_empty[buf]);       // every warp's TMEM reads of this set are done
      ++lt;
    }
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if ((S.fail || !S.ep_ok) && lane == 0 && q == 0) status_set(a.status, ST_TIMEOUT, 90 + S.fail, blockIdx.x, lt);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

}  // namespace sfb

using namespace sfb;

template <int NPV, bool BULK, int STO = 0>
static cudaError_t launch_umma_t(const CUtensorMap* mA, const CUtensorMap* mA2, const CUtensorMap* mB, const UmmaArgs& a, dim3 grid,
                                 cudaStream_t stream) {
  const size_t smem = sizeof(UmmaSmem<NPV, 1, (STO ? STO : (NPV <= 32 ? UM_STAGES_DENSE : ((BULK && NPV == 128) ? 3 : UM_STAGES_WIDE)))>) + 1024;
  static bool done = false;
  if (!done) {
    cudaFuncSetAttribute(umma_gemm_kernel<NPV, BULK, STO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    done = true;
  }
  return sfb_launch(umma_gemm_kernel<NPV, BULK, STO>, grid, dim3(UM_THREADS), smem, stream, *mA, *mA2, *mB, a);
}

extern "C" {

// Encode a 2-D K-major tensor map with a 128-byte swizzled box of `box_rows` rows x 128 K elements.
// fp4 != 0: packed E2M1 in memory (row_bytes = K/2), unpacked to 8-bit containers by TMA.
// Returns 0 on success, a CUresult otherwise (or -1 when the driver entry point is unavailable).
int sfb_tmap_encode(void* out_map /*128 bytes, 64-aligned*/, const void* base, int64_t rows, int64_t K,
                    int64_t row_bytes, int box_rows, int fp4) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  return (int)enc((CUtensorMap*)out_map, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

int sfb_umma_scratch_floats(int tiles_total, int splits, int NP) { return tiles_total * splits * 128 * NP; }

}  // extern "C"

namespace sfb {
// Split-K reduce for many-row dense launches: the GEMM leaves its fp32 partials in scratch ([split][tile][128 cols][NP
// tokens]) and this kernel adds them in split order - the order the in-kernel last-arriver uses, so a row's bits do not
// depend on which path ran - with every (tile, four-token group) on its own CTA instead of one CTA per tile.
struct SplitReduceArgs {
  const float* scratch;
  int splits, tiles_total, tiles_per_group, NP, n, N;
  int tok_tiles;              // > 1: tile ids run over (group, token tile, column tile); output row = token tile * NP + token
  __nv_bfloat16* out_b;
  float* out_f;
  int64_t out_stride;
};
__global__ void __launch_bounds__(128) splitk_reduce_kernel(SplitReduceArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile_id = blockIdx.x, c = threadIdx.x;
  const int z = tile_id / a.tiles_per_group, tile = tile_id - z * a.tiles_per_group;
  const int tt = a.tok_tiles > 1 ? a.tok_tiles : 1;
  const int g = z / tt, tok_tile = z - g * tt;
  const int tok_in = blockIdx.y * 4, tok0 = tok_tile * a.NP + tok_in;
  const int col = g * a.N + tile * 128 + c;
  const size_t split_stride = (size_t)a.tiles_total * 128 * a.NP;
  const float* pp = a.scratch + ((size_t)tile_id * 128 + c) * a.NP + tok_in;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp0 = 0; sp0 < a.splits; sp0 += 8) {
    float4 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int sp = sp0 + i < a.splits ? sp0 + i : a.splits - 1;
      t[i] = __ldcg(reinterpret_cast<const float4*>(pp + (size_t)sp * split_stride));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (sp0 + i < a.splits) { acc.x += t[i].x; acc.y += t[i].y; acc.z += t[i].z; acc.w += t[i].w; }
  }
  if (col >= (g + 1) * a.N) return;
  const float r[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (tok0 + j < a.n) {
      const int64_t o = (int64_t)(tok0 + j) * a.out_stride + col;
      if (a.out_b) a.out_b[o] = __float2bfloat16_rn(r[j]);
      if (a.out_f) a.out_f[o] = r[j];
    }
  }
}
}  // namespace sfb

extern "C" {

// Peer table of the next launch (set by sfb_umma_set_push, consumed and cleared by the launch).
struct PushSpec {
  void* out[8];
  void* flag[8];
  int n = 0;
  const void* epoch_ptr = nullptr;
  uint32_t epoch_add = 0;
  void* done = nullptr;
};
static thread_local PushSpec g_push;

// Arrival flags of the next all-gather -> GEMM launch (set by sfb_umma_set_gather, consumed and cleared by the launch).
struct GatherSpec {
  const void* flag[8];
  int n = 0;
  const void* epoch_ptr = nullptr;
  uint32_t epoch_add = 0;
  uint64_t wait_ns = 0;
};
static thread_local GatherSpec g_gather;

// Tuning switches for measurements (0 = the shipped choice): [1] stages of the 64-pair down projection (2 shipped; 3, 4),
// [2] stages of the 64-pair gate/up (2 = two CTAs per SM; 3, 5 = one CTA per SM), [3] / [4] segment-major grid order of the
// grouped down / gate-up kernels, [5] persistent many-row dense kernel, [6] persistent 64-pair gate/up kernel, [7] persistent 64-pair down kernel (1 = never, 2 = whenever the shape allows, 3 = the same with one column tile per work item).
static int g_tune[8] = {0, 0, 0, 0, 0, 0, 0, 0};
// Phase marks (um_mark) of the NEXT launch of a tensor-core GEMM of this library: cleared by that launch.
static thread_local unsigned long long* g_marks = nullptr;
static thread_local int g_marks_cap = 0;
int sfb_umma_set_marks(void* buf, int cap_ctas) {
  if (buf && !SFB_MARKS_ON) return (int)cudaErrorNotSupported;     // this library was built without the marks
  g_marks = (unsigned long long*)buf; g_marks_cap = buf ? cap_ctas : 0;
  return 0;
}
int sfb_umma_has_marks(void) { return SFB_MARKS_ON; }
static void apply_marks(UmmaArgs& a) {
  a.marks = g_marks; a.marks_cap = g_marks_cap;
  g_marks = nullptr; g_marks_cap = 0;
}
int sfb_umma_tune(int key, int value) {
  if (key < 0 || key >= 8) return (int)cudaErrorInvalidValue;
  g_tune[key] = value;
  return 0;
}

// An entry point that refuses its arguments must not leave a push or gather armed for some later, unrelated launch.
static int refuse_args() {
  g_push.n = 0;
  g_gather.n = 0;
  return (int)cudaErrorInvalidValue;
}

static void apply_gather(UmmaArgs& a) {
  for (int i = 0; i < 8; ++i) a.gflag[i] = i < g_gather.n ? (const uint32_t*)g_gather.flag[i] : nullptr;
  a.gepoch_ptr = (const uint32_t*)g_gather.epoch_ptr; a.gepoch_add = g_gather.epoch_add;
  a.gwait_ns = g_gather.wait_ns ? g_gather.wait_ns : 1000000000ull;
  g_gather.n = 0;
}

static void apply_marks(UmmaArgs& a);
static void apply_push(UmmaArgs& a) {
  apply_marks(a);
  a.n_peers = g_push.n;
  for (int i = 0; i < g_push.n; ++i) { a.peer_out[i] = (__nv_bfloat16*)g_push.out[i]; a.peer_flag[i] = (uint32_t*)g_push.flag[i]; }
  a.epoch_ptr = (const uint32_t*)g_push.epoch_ptr; a.epoch_add = g_push.epoch_add; a.done_counter = (unsigned int*)g_push.done;
  g_push.n = 0;
}

static int launch_umma(const void* tmapA, const void* tmapA2, const void* tmapB, const UmmaArgs& a_in, dim3 grid, int NP,
                       cudaStream_t stream) {
  const CUtensorMap* mA = (const CUtensorMap*)tmapA;
  const CUtensorMap* mA2 = (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA);
  const CUtensorMap* mB = (const CUtensorMap*)tmapB;
  cudaError_t launch_rc = cudaSuccess;
  UmmaArgs a = a_in;
  apply_push(a);
  apply_gather(a);
const bool bulk = a.force_bulk || a.tok_tiles > 1 || a.b_maps != nullptr || a.rs_rows > 0;
  if (a.tok_tiles < 1) a.tok_tiles = 1;
#define SFB_UM(NPV) { launch_rc = bulk ? launch_umma_t<NPV, true>(mA, mA2, mB, a, grid, stream) : launch_umma_t<NPV, false>(mA, mA2, mB, a, grid, stream); }
  if (NP == 16) SFB_UM(16) else if (NP == 32) SFB_UM(32) else if (NP == 64) SFB_UM(64) else if (NP == 128) SFB_UM(128)
  else return refuse_args();
#undef SFB_UM
  return (int)launch_rc;
}

// Arm the fused-collective epilogue for the next sfb_umma_dense / sfb_umma_down call of this thread: the bf16 output
// is also stored to out_ptrs[0..W) (this rank's slot on every rank) and flag_ptrs[0..W) are raised at the end.
int sfb_umma_set_push(const void* const* out_ptrs, const void* const* flag_ptrs, int W, const void* epoch_ptr,
                      uint32_t epoch_add, void* done_counter) {
  if (W < 0 || W > 8) return (int)cudaErrorInvalidValue;
  for (int i = 0; i < W; ++i) { g_push.out[i] = (void*)out_ptrs[i]; g_push.flag[i] = (void*)flag_ptrs[i]; }
  g_push.n = W; g_push.epoch_ptr = epoch_ptr; g_push.epoch_add = epoch_add; g_push.done = done_counter;
  return 0;
}

// Arm per-shard arrival flags for the next sfb_umma_bulk call with b_maps: flag_ptrs[r] (null = no wait) must reach
// *epoch_ptr + epoch_add before the kernel reads map r.
int sfb_umma_set_gather(const void* const* flag_ptrs, int W, const void* epoch_ptr, uint32_t epoch_add, uint64_t wait_ns) {
  if (W < 0 || W > 8) return (int)cudaErrorInvalidValue;
  for (int i = 0; i < W; ++i) g_gather.flag[i] = flag_ptrs[i];
  g_gather.n = W; g_gather.epoch_ptr = epoch_ptr; g_gather.epoch_add = epoch_add; g_gather.wait_ns = wait_ns;
  return 0;
}

// Dense / grouped block-scaled GEMM. NP = token columns (16/32/64/128) >= n (>= 2*pair when pair > 0).
// pair > 0: activations are two-term (hi rows 0..pair-1, lo rows pair..2*pair-1); out[t] = acc[t] + acc[t+pair].
int sfb_umma_dense(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb, int katoms_b,
                   int n, int NP, int N, int K, int groups, int a_fp4, int splits, float* scratch,
                   unsigned int* tickets, void* out_b, float* out_f, int64_t out_stride, void* status,
                   cudaStream_t stream) {
  if ((N % 128 && groups > 1) || K % UM_BK || n > NP || splits < 1 || splits > K / UM_BK)
    return refuse_args();
  if (splits > 1 && (!scratch || !tickets)) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.katoms_a = katoms_a; a.sfb = (const uint8_t*)sfb; a.katoms_b = katoms_b;
  a.n = n; a.K = K; a.a_fp4 = a_fp4; a.mode = UM_DENSE; a.N = N; a.groups = groups; a.splits = splits;
  a.scratch = scratch; a.tickets = tickets; a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f;
  a.out_stride = out_stride; a.status = (Status*)status;
  const int tiles = (N + 127) / 128;
  // many rows and many splits: one CTA per tile adding every split is the slow part, so the add runs as its own grid
  a.defer_reduce = (splits > 1 && NP >= 32 && g_push.n == 0) ? 1 : 0;
  // 64+ token rows: the staged epilogue (tile -> shared memory -> one 256-byte bulk store per token row) instead of one
  // 2-byte store per element; the values written are the same
  if (NP >= 64 && groups == 1 && out_b && !out_f && N % 128 == 0) a.force_bulk = 1;
  const int rc = launch_umma(tmapA, nullptr, tmapB, a, dim3(tiles, splits, groups), NP, stream);
  if (rc != 0 || !a.defer_reduce) return rc;
  SplitReduceArgs r{};
  r.scratch = scratch; r.splits = splits; r.tiles_total = tiles * groups; r.tiles_per_group = tiles; r.NP = NP; r.n = n;
  r.N = N; r.out_b = (__nv_bfloat16*)out_b; r.out_f = out_f; r.out_stride = out_stride;
  return (int)sfb_launch(splitk_reduce_kernel, dim3(tiles * groups, (n + 3) / 4), dim3(128), 0, stream, r);
}

// Bulk GEMM with the fused-collective options: any number of token rows (tiles of NP = 128 when n > 128),
//   b_maps != null : all-gather -> GEMM.  Activations are sharded along K; device array of n_maps tensor maps, map r
//                    = rank r's [rows, b_k_per_map] shard (peer memory is read with plain TMA loads), sfb_maps[r] its atoms
//   rs_rows > 0    : GEMM -> reduce-scatter.  With sfb_umma_set_push armed, token row t is stored only to rank t / rs_rows
//   (push armed, rs_rows == 0: GEMM -> all-reduce, every rank receives the whole partial)
int sfb_umma_bulk(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb, int katoms_b, int n,
                  int NP, int N, int K, int splits, float* scratch, unsigned int* tickets, void* out_b, float* out_f,
                  int64_t out_stride, const void* b_maps, int b_k_per_map, const void* const* sfb_maps, int n_maps,
                  int rs_rows, void* status, cudaStream_t stream) {
  const int tok_tiles = (n + NP - 1) / NP;
  if (K % UM_BK || splits < 1 || splits > K / UM_BK || n < 1 || (tok_tiles > 1 && NP != 128)) return refuse_args();
  if (splits > 1 && (!scratch || !tickets)) return refuse_args();
  if (b_maps && (n_maps < 1 || n_maps > 8 || b_k_per_map % UM_BK || b_k_per_map * n_maps != K)) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.katoms_a = katoms_a; a.sfb = (const uint8_t*)sfb; a.katoms_b = katoms_b;
  a.n = n; a.K = K; a.mode = UM_DENSE; a.N = N; a.groups = 1; a.splits = splits; a.scratch = scratch; a.tickets = tickets;
  a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f; a.out_stride = out_stride; a.status = (Status*)status;
  a.force_bulk = 1;
  a.tok_tiles = tok_tiles; a.b_maps = (const CUtensorMap*)b_maps; a.b_k_per_map = b_k_per_map; a.rs_rows = rs_rows;
  for (int i = 0; i < n_maps && b_maps; ++i) a.sfb_maps[i] = (const uint8_t*)sfb_maps[i];
  const int tiles = (N + 127) / 128;
  // many tiles of 128 x 128, one split, bf16 out (local and / or pushed): the persistent kernel, whose epilogues and copies
  // run under the next tile's main loop.  g_tune[5]: 1 = never, 2 = whenever the shape allows
  const bool can_persist = NP == 128 && splits == 1 && !b_maps && !out_f && (out_b || g_push.n > 0) && N % 128 == 0 &&
                           (out_stride % 8) == 0 && K >= UM_BK;
  // (for any reduction length: 320 tiles of K = 8192 on 296 one-tile CTA slots left a nearly empty second wave)
  if (can_persist && g_tune[5] != 1 && (g_tune[5] == 2 || tiles * tok_tiles >= 296)) {
    apply_push(a); apply_gather(a);
    static int sms = 0;
    if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    const size_t smem = sizeof(UmmaPersistSmem) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(umma_bulk_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    const int total = tiles * tok_tiles;
    return (int)sfb_launch(umma_bulk_persistent_kernel, dim3(total < sms ? total : sms), dim3(UM_THREADS), smem, stream,
                           *(const CUtensorMap*)tmapA, *(const CUtensorMap*)tmapB, a);
  }
  // many token tiles and several splits: the add of the partials runs as its own grid (one CTA per tile adding every split
  // is latency-bound); not with an armed push, whose epilogue needs the finished tile
  a.defer_reduce = (splits > 1 && NP >= 32 && g_push.n == 0) ? 1 : 0;
  const int rc = launch_umma(tmapA, nullptr, tmapB ? tmapB : tmapA, a, dim3(tiles, splits, tok_tiles), NP, stream);
  if (rc != 0 || !a.defer_reduce) return rc;
  SplitReduceArgs r{};
  r.scratch = scratch; r.splits = splits; r.tiles_total = tiles * tok_tiles; r.tiles_per_group = tiles; r.NP = NP; r.n = n;
  r.N = N; r.tok_tiles = tok_tiles; r.out_b = (__nv_bfloat16*)out_b; r.out_f = out_f; r.out_stride = out_stride;
  return (int)sfb_launch(splitk_reduce_kernel, dim3(tiles * tok_tiles, ((n < NP ? n : NP) + 3) / 4), dim3(128), 0, stream, r);
}

// Same with two-term activations (see k_quant.cu): rows [0, pair) are the hi terms, [pair, 2*pair) the lo terms.
int sfb_umma_dense_pair(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb,
                        int katoms_b, int pair, int NP, int N, int K, int groups, int a_fp4, int splits,
                        float* scratch, unsigned int* tickets, void* out_b, float* out_f, int64_t out_stride,
                        void* out_q, void* out_q_atom, void* status, cudaStream_t stream) {
  if (N % 128 || K % UM_BK || 2 * pair > NP || pair < 1 || splits < 1 || splits > K / UM_BK || !scratch || !tickets)
    return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.katoms_a = katoms_a; a.sfb = (const uint8_t*)sfb; a.katoms_b = katoms_b;
  a.n = 2 * pair; a.pair = pair; a.K = K; a.a_fp4 = a_fp4; a.mode = UM_DENSE; a.N = N; a.groups = groups;
  a.splits = splits; a.scratch = scratch; a.tickets = tickets; a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f;
  a.out_stride = out_stride; a.out_q = (uint8_t*)out_q; a.out_q_atom = (uint8_t*)out_q_atom; a.status = (Status*)status;
  return launch_umma(tmapA, nullptr, tmapB, a, dim3(N / 128, splits, groups), NP, stream);
}

// Two-term activations for any number of rows: the activation buffer holds blocks of 128 rows, each = 64 hi rows then 64 lo
// rows of 64 consecutive logical rows (scale atoms: one 128-row atom block per block); out row = logical row.
int sfb_umma_pair_bulk(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb, int katoms_b,
                       int n_rows, int N, int K, int groups, int splits, float* scratch, unsigned int* tickets, void* out_b,
                       float* out_f, int64_t out_stride, void* out_q, void* out_q_atom, void* status, cudaStream_t stream) {
  if (N % 128 || K % UM_BK || n_rows < 1 || splits < 1 || splits > K / UM_BK || !scratch || !tickets) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.katoms_a = katoms_a; a.sfb = (const uint8_t*)sfb; a.katoms_b = katoms_b;
  a.n = n_rows; a.pair = 64; a.K = K; a.mode = UM_DENSE; a.N = N; a.groups = groups; a.splits = splits;
  a.scratch = scratch; a.tickets = tickets; a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f; a.out_stride = out_stride;
  a.out_q = (uint8_t*)out_q; a.out_q_atom = (uint8_t*)out_q_atom; a.status = (Status*)status;
  a.force_bulk = 1;
  a.tok_tiles = (n_rows + 63) / 64;
  return launch_umma(tmapA, nullptr, tmapB, a, dim3(N / 128, splits, groups * a.tok_tiles), 128, stream);
}

// bf16 x bf16 -> fp32 GEMM (kind::f16): out[token, col] = sum_k W[col, k] X[token, k], both operands bf16 row-major.  The
// tensor maps are byte maps (sfb_tmap_encode with K = row_bytes = 2 * elements, fp4 = 0).  Any number of token rows
// (tiles of 128 when n > NP); split-K partials are added in split order.
int sfb_umma_bf16(const void* tmapA, const void* tmapB, int n, int NP, int N, int K_elems, int splits, float* scratch,
                  unsigned int* tickets, void* out_b, float* out_f, int64_t out_stride, void* status, cudaStream_t stream) {
  const int K = 2 * K_elems;
  const int tok_tiles = (n + NP - 1) / NP;
  if (K % UM_BK || n < 1 || splits < 1 || splits > K / UM_BK || (tok_tiles > 1 && NP != 128)) return refuse_args();
  if (splits > 1 && (!scratch || !tickets)) return refuse_args();
  UmmaArgs a{};
  a.bf16 = 1; a.n = n; a.K = K; a.mode = UM_DENSE; a.N = N; a.groups = 1; a.splits = splits; a.scratch = scratch; a.tickets = tickets;
  a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f; a.out_stride = out_stride; a.status = (Status*)status;
  const int tiles = (N + 127) / 128;
  if (tok_tiles > 1) {
    a.force_bulk = 1; a.tok_tiles = tok_tiles;
    a.defer_reduce = (splits > 1 && g_push.n == 0) ? 1 : 0;
    const int rc = launch_umma(tmapA, nullptr, tmapB, a, dim3(tiles, splits, tok_tiles), NP, stream);
    if (rc != 0 || !a.defer_reduce) return rc;
    SplitReduceArgs r{};
    r.scratch = scratch; r.splits = splits; r.tiles_total = tiles * tok_tiles; r.tiles_per_group = tiles; r.NP = NP; r.n = n;
    r.N = N; r.tok_tiles = tok_tiles; r.out_b = (__nv_bfloat16*)out_b; r.out_f = out_f; r.out_stride = out_stride;
    return (int)sfb_launch(splitk_reduce_kernel, dim3(tiles * tok_tiles, (NP + 3) / 4), dim3(128), 0, stream, r);
  }
  a.defer_reduce = (splits > 1 && NP >= 32 && g_push.n == 0) ? 1 : 0;
  const int rc = launch_umma(tmapA, nullptr, tmapB, a, dim3(tiles, splits, 1), NP, stream);
  if (rc != 0 || !a.defer_reduce) return rc;
  SplitReduceArgs r{};
  r.scratch = scratch; r.splits = splits; r.tiles_total = tiles; r.tiles_per_group = tiles; r.NP = NP; r.n = n;
  r.N = N; r.out_b = (__nv_bfloat16*)out_b; r.out_f = out_f; r.out_stride = out_stride;
  return (int)sfb_launch(splitk_reduce_kernel, dim3(tiles, (n + 3) / 4), dim3(128), 0, stream, r);
}

// MoE gate/up for n_tok tokens: tmapA = routed w13 [E*2*inter, d] (FP4), tmapA2 = shared [2*inter, d] (FP8, may be
// null when slots == top_k), tmapB = activations [rows, d] with a 16-row box; sfb = one atom set per token.
int sfb_umma_gate_up(const void* tmapA, const void* tmapA2, const void* tmapB, const void* sfa, const void* sfa2,
                     const void* sfb, const int* ids, const float* wts, void* act_q, void* act_s, void* act_sf,
                     int n_tok, int top_k, int slots, int d, int inter, float limit, void* status,
                     cudaStream_t stream) {
  if (inter % 128 || d % 32 || slots < top_k || slots > top_k + 1) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.sfa2 = (const uint8_t*)sfa2; a.katoms_a = (d / 32 + 3) / 4;
  a.sfb = (const uint8_t*)sfb; a.katoms_b = a.katoms_a; a.a_fp4 = 1; a.ids = ids; a.wts = wts; a.top_k = top_k;
  a.slots = slots; a.inter = inter; a.d = d; a.act_q = (uint8_t*)act_q; a.act_s = (uint8_t*)act_s;
  a.act_sf = (uint8_t*)act_sf; a.limit = limit; a.status = (Status*)status;
  apply_marks(a);
  const size_t smem = sizeof(UmmaSmem<16, 2, UM_STAGES_GATEUP>) + 1024;
  static bool done = false;
  if (!done) {
    cudaFuncSetAttribute(umma_gateup_kernel<UM_STAGES_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    done = true;
  }
  const CUtensorMap* mA = (const CUtensorMap*)tmapA;
  const CUtensorMap* mA2 = (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA);
  return (int)sfb_launch(umma_gateup_kernel<UM_STAGES_GATEUP>, dim3(inter / 128, slots, n_tok), dim3(GU_THREADS), smem, stream, *mA, *mA2,
                         *(const CUtensorMap*)tmapB, a);
}

// MoE down + combine: out[tok, :] = sum over slots of W2_slot . act[tok, slot, :] (fp32 partial per slot, added in
// slot order by the last CTA of each column tile).  tmapA = routed w2 [E*d, inter] (FP4), tmapA2 = shared [d, inter]
// (FP8), tmapB = activations [n_tok*slots, inter] with a 16-row box; sfb = one atom set per (token, slot).
int sfb_umma_down(const void* tmapA, const void* tmapA2, const void* tmapB, const void* sfa, const void* sfa2,
                  const void* sfb, const int* ids, void* out_b, float* out_f, int64_t out_stride, float* scratch,
                  unsigned int* tickets, int n_tok, int top_k, int slots, int d, int inter, void* status,
                  cudaStream_t stream) {
  if (d % 128 || inter % 128 || !scratch || !tickets) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.sfa2 = (const uint8_t*)sfa2; a.katoms_a = (inter / 32 + 3) / 4;
  a.sfb = (const uint8_t*)sfb; a.katoms_b = a.katoms_a; a.a_fp4 = 1; a.mode = UM_DOWN; a.ids = ids; a.top_k = top_k;
  a.slots = slots; a.inter = inter; a.d = d; a.scratch = scratch; a.tickets = tickets;
  a.out_b = (__nv_bfloat16*)out_b; a.out_f = out_f; a.out_stride = out_stride; a.status = (Status*)status;
  return launch_umma(tmapA, tmapA2, tmapB, a, dim3(d / 128, slots, n_tok), 16, stream);
}

}  // extern "C"

extern "C" {

// Grouped MoE (rows sorted by expert, see csrc/k_moe.cu moe_plan): gate/up over `segments` segments of up to 16 pairs.
// tmapB = permuted activations [segments*16, d] (16-row box); sfb = one atom set per segment (rows = pair slots).
int sfb_umma_gate_up_grouped(const void* tmapA, const void* tmapA2, const void* tmapB, const void* sfa, const void* sfa2, const void* sfb,
                             const int* seg_expert, const int* seg_count, const float* seg_weight, void* act_q, void* act_sf, int segments,
                             int d, int inter, float limit, int seg_size, void* status, cudaStream_t stream) {
  if (inter % 128 || d % 32 || segments < 1 || (seg_size != 16 && seg_size != 64)) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.sfa2 = (const uint8_t*)sfa2; a.katoms_a = (d / 32 + 3) / 4; a.sfb = (const uint8_t*)sfb; a.katoms_b = a.katoms_a;
  a.a_fp4 = 1; a.top_k = 0; a.slots = 1; a.inter = inter; a.d = d; a.act_q = (uint8_t*)act_q; a.act_sf = (uint8_t*)act_sf; a.limit = limit;
  a.seg_expert = seg_expert; a.seg_count = seg_count; a.seg_weight = seg_weight; a.status = (Status*)status;
  apply_marks(a);
  const CUtensorMap* mA = (const CUtensorMap*)tmapA;
  const CUtensorMap* mA2 = (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA);
  if (seg_size == 64 && g_tune[2] == 3) {      // tuning arm: one 3-stage CTA per SM
    const size_t smem = sizeof(UmmaSmem<64, 2, 3>) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(umma_gateup_kernel<3, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    return (int)sfb_launch(umma_gateup_kernel<3, 64>, dim3(inter / 128, segments, 1), dim3(GU_THREADS), smem, stream, *mA, *mA2,
                           *(const CUtensorMap*)tmapB, a);
  }
  if (seg_size == 64 && g_tune[2] == 5) {      // tuning arm: one 5-stage CTA per SM
    const size_t smem = sizeof(UmmaSmem<64, 2, 5>) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(umma_gateup_kernel<5, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    return (int)sfb_launch(umma_gateup_kernel<5, 64>, dim3(inter / 128, segments, 1), dim3(GU_THREADS), smem, stream, *mA, *mA2,
                           *(const CUtensorMap*)tmapB, a);
  }
  // many wide segments: the persistent kernel (g_tune[6]: 1 = never, 2 = whenever the shape allows)
  if (seg_size == 64 && inter % 128 == 0 && act_sf && g_tune[6] != 1 && (g_tune[6] == 2 || (inter / 128) * segments >= 296)) {
    static int sms = 0;
    if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    const size_t smem = sizeof(UmmaGateupPersistSmem) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(umma_gateup_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    const int total = (inter / 128) * segments;
    return (int)sfb_launch(umma_gateup_persistent_kernel, dim3(total < sms ? total : sms), dim3(PG_THREADS), smem, stream, *mA, *mA2,
                           *(const CUtensorMap*)tmapB, a, inter / 128, segments, g_tune[2] == 7 ? 1 : 0);
  }
  if (seg_size == 64) {      // segments of up to 64 pairs: two 2-stage CTAs per SM (a stage holds 32 KiB of weights and 8 KiB of tokens)
    const size_t smem64 = sizeof(UmmaSmem<64, 2, 2>) + 1024;
    static bool done64 = false;
    if (!done64) { cudaFuncSetAttribute(umma_gateup_kernel<2, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem64); done64 = true; }
    a.swap_xy = g_tune[4] ? 1 : 0;
    const dim3 grid = a.swap_xy ? dim3(segments, inter / 128, 1) : dim3(inter / 128, segments, 1);
    return (int)sfb_launch(umma_gateup_kernel<2, 64>, grid, dim3(GU_THREADS), smem64, stream, *mA, *mA2,
                           *(const CUtensorMap*)tmapB, a);
  }
  if ((inter / 128) * segments > 2 * 148) {      // several waves: two half-depth CTAs per SM
    const size_t smem3 = sizeof(UmmaSmem<16, 2, 3>) + 1024;
    static bool done3 = false;
    if (!done3) { cudaFuncSetAttribute(umma_gateup_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3); done3 = true; }
    return (int)sfb_launch(umma_gateup_kernel<3>, dim3(inter / 128, segments, 1), dim3(GU_THREADS), smem3, stream, *mA, *mA2,
                           *(const CUtensorMap*)tmapB, a);
  }
  const size_t smem = sizeof(UmmaSmem<16, 2, UM_STAGES_GATEUP>) + 1024;
  static bool done = false;
  if (!done) { cudaFuncSetAttribute(umma_gateup_kernel<UM_STAGES_GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
  return (int)sfb_launch(umma_gateup_kernel<UM_STAGES_GATEUP>, dim3(inter / 128, segments, 1), dim3(GU_THREADS), smem, stream, *mA, *mA2, *(const CUtensorMap*)tmapB, a);
}

// out_f [segments*16, d] fp32: one row per pair slot (the caller sums a token's pairs in slot order)
int sfb_umma_down_grouped(const void* tmapA, const void* tmapA2, const void* tmapB, const void* sfa, const void* sfa2, const void* sfb,
                          const int* seg_expert, const int* seg_count, float* out_f, int segments, int d, int inter, int seg_size,
                          void* status, cudaStream_t stream) {
  if (d % 128 || inter % 128 || segments < 1 || (seg_size != 16 && seg_size != 64)) return refuse_args();
  UmmaArgs a{};
  a.sfa = (const uint8_t*)sfa; a.sfa2 = (const uint8_t*)sfa2; a.katoms_a = (inter / 32 + 3) / 4; a.sfb = (const uint8_t*)sfb; a.katoms_b = a.katoms_a;
  a.a_fp4 = 1; a.mode = UM_DOWN_GROUPED; a.inter = inter; a.d = d; a.out_f = out_f; a.out_stride = d; a.seg_expert = seg_expert;
  a.seg_count = seg_count; a.status = (Status*)status; a.splits = 1;
  // many (column tile, segment) pairs: one persistent CTA per SM ([7]: 0 this rule, 1 never, 2 whenever the shape allows)
  if (seg_size == 64 && g_push.n == 0 && g_gather.n == 0 && g_tune[7] != 1 && (g_tune[7] >= 2 || (d / 128) * segments >= 296)) {
    apply_marks(a);
    static int sms = 0;
    if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    if ((d / 128) % 2 == 0 && g_tune[7] != 3) {      // pairs of column tiles sharing the activation tile ([7] = 3: one tile per item)
      const int total2 = (d / 256) * segments;
      const size_t smem2 = sizeof(UmmaDownPersist2Smem) + 1024;
      static bool done2 = false;
      if (!done2) { cudaFuncSetAttribute(umma_down_persistent2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2); done2 = true; }
      return (int)sfb_launch(umma_down_persistent2_kernel, dim3(total2 < sms ? total2 : sms), dim3(PD_THREADS), smem2, stream,
                             *(const CUtensorMap*)tmapA, *(const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA), *(const CUtensorMap*)tmapB, a,
                             d / 256, segments);
    }
    const int total = (d / 128) * segments;
    const size_t smem = sizeof(UmmaDownPersistSmem) + 1024;
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(umma_down_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); done = true; }
    return (int)sfb_launch(umma_down_persistent_kernel, dim3(total < sms ? total : sms), dim3(PD_THREADS), smem, stream,
                           *(const CUtensorMap*)tmapA, *(const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA), *(const CUtensorMap*)tmapB, a,
                           d / 128, segments);
  }
  if (seg_size == 64 && g_tune[1] != 3) {      // shipped: 2 stages, so that three CTAs share an SM (measured best); tuning arm 4 stages
    apply_push(a); apply_gather(a);
    a.tok_tiles = 1;
    a.swap_xy = g_tune[3] ? 1 : 0;
    if (g_tune[1] != 4)
      return (int)launch_umma_t<64, false, 2>((const CUtensorMap*)tmapA, (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA),
                                              (const CUtensorMap*)tmapB, a, a.swap_xy ? dim3(segments, d / 128, 1) : dim3(d / 128, segments, 1), stream);
    return (int)launch_umma_t<64, false, 4>((const CUtensorMap*)tmapA, (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA),
                                            (const CUtensorMap*)tmapB, a, dim3(d / 128, segments, 1), stream);
  }
  if (seg_size == 64) {
    apply_push(a); apply_gather(a);
    a.tok_tiles = 1;
    a.swap_xy = g_tune[3] ? 1 : 0;
    return (int)launch_umma_t<64, false, 3>((const CUtensorMap*)tmapA, (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA),
                                            (const CUtensorMap*)tmapB, a, a.swap_xy ? dim3(segments, d / 128, 1) : dim3(d / 128, segments, 1), stream);
  }
  if ((d / 128) * segments > 4 * 148) {      // many waves of 16-k-step CTAs: three 3-stage CTAs per SM
    apply_push(a); apply_gather(a);
    a.tok_tiles = 1;
    return (int)launch_umma_t<16, false, 3>((const CUtensorMap*)tmapA, (const CUtensorMap*)(tmapA2 ? tmapA2 : tmapA),
                                            (const CUtensorMap*)tmapB, a, dim3(d / 128, segments, 1), stream);
  }
  return launch_umma(tmapA, tmapA2, tmapB, a, dim3(d / 128, segments, 1), 16, stream);
}

}  // extern "C"

// ---- allocation-free entry point (declared and documented in sfb_noalloc.h) ---------------------------------
// The arrays below are device memory that belongs to the library image.  In host code their names
// are only handles for the runtime's symbol lookup - not device addresses - so the launcher asks
// cudaGetSymbolAddress once per device and hands the kernel the pointer it gets back.
static __device__ __align__(256) float g_noalloc_partials[SFB_NOALLOC_MAX_FLOATS];
static __device__ __align__(256) unsigned int g_noalloc_tickets[SFB_NOALLOC_MAX_TILES];

namespace {
constexpr int kMaxDevices = 64;
float* g_partials_ptr[kMaxDevices] = {};
unsigned int* g_tickets_ptr[kMaxDevices] = {};
thread_local char g_noalloc_err[256] = "";
}  // namespace

extern "C" {

const char* sfb_noalloc_last_error(void) { return g_noalloc_err; }

int sfb_umma_dense_noalloc(const void* tmapA, const void* tmapB, const void* sfa, int katoms_a, const void* sfb,
                           int katoms_b, int n, int NP, int N, int K, int groups, int a_fp4, int splits,
                           void* out_b, float* out_f, int64_t out_stride, void* status, cudaStream_t stream) {
  g_noalloc_err[0] = 0;
  if (N <= 0 || N % 128 || groups <= 0 || splits < 1 || NP <= 0) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err, "bad shape: N=%d groups=%d splits=%d NP=%d", N, groups, splits, NP);
    return (int)cudaErrorInvalidValue;
  }
  g_push.n = 0;      // this entry point never pushes to peers: a push armed for another call does not carry over
  g_gather.n = 0;
  if (splits == 1)   // a single split writes its output directly: no partial sums, no counters, no size limit
    return sfb_umma_dense(tmapA, tmapB, sfa, katoms_a, sfb, katoms_b, n, NP, N, K, groups, a_fp4, 1, nullptr, nullptr,
                          out_b, out_f, out_stride, status, stream);
  const long long tiles = (long long)groups * (N / 128);
  const long long floats = tiles * splits * 128 * NP;
  if (tiles > SFB_NOALLOC_MAX_TILES || floats > SFB_NOALLOC_MAX_FLOATS) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err,
             "problem needs %lld partial-sum floats and %lld tile counters; the built-in scratch holds %d and %d",
             floats, tiles, SFB_NOALLOC_MAX_FLOATS, SFB_NOALLOC_MAX_TILES);
    return SFB_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err, "cudaGetDevice failed (%d) or device index %d unsupported", (int)e, dev);
    return SFB_NOALLOC_SETUP_FAILED;
  }
  if (g_partials_ptr[dev] == nullptr || g_tickets_ptr[dev] == nullptr) {
    // first call on this device: resolve the arrays' device addresses (device `dev` is current)
    float* p = nullptr;
    unsigned int* t = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_partials);
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void**)&t, g_noalloc_tickets);
    if (e != cudaSuccess || p == nullptr || t == nullptr) {
      snprintf(g_noalloc_err, sizeof g_noalloc_err, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return SFB_NOALLOC_SETUP_FAILED;
    }
    g_partials_ptr[dev] = p;
    g_tickets_ptr[dev] = t;
  }
  // the counters must start at zero whatever an earlier (possibly failed) call left behind
  e = cudaMemsetAsync(g_tickets_ptr[dev], 0, (size_t)tiles * sizeof(unsigned int), stream);
  if (e != cudaSuccess) {
    snprintf(g_noalloc_err, sizeof g_noalloc_err, "clearing the tile counters failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  const int rc = sfb_umma_dense(tmapA, tmapB, sfa, katoms_a, sfb, katoms_b, n, NP, N, K, groups, a_fp4, splits,
                                g_partials_ptr[dev], g_tickets_ptr[dev], out_b, out_f, out_stride, status, stream);
  if (rc != 0) snprintf(g_noalloc_err, sizeof g_noalloc_err, "launch failed with CUDA error %d", rc);
  return rc;
}

}  // extern "C"
