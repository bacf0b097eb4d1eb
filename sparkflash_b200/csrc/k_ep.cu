// Expert-parallel all-to-all around the MoE: dispatch (route + MXFP8 activation quant + push to the expert's rank)
// and combine (push the expert output back to the token's rank, weighted sum in top-k order).
//
// Tokens are sharded over ranks; experts are sharded over ranks (rank r holds experts [r*epr, (r+1)*epr)).
//   dispatch : one block per local token quantises the row once (E4M3 per 32 + UE8M0, the W4A8 activation form), stages
//              it in shared memory and sends it with bulk copies to the receive region "from me" on every rank that
//              owns one of its top-k experts, together with a 16-byte record (local expert, token, k index, weight).
//              The slot inside the region comes from a local counter per destination.  The last block publishes the
//              counts and raises this rank's arrival flag everywhere.
//   plan     : the receiver waits (time-limited) for all flags and turns the records into the (expert id, weight)
//              arrays of the grouped-GEMM kernels; unused slots get expert id -1 and are skipped there.
//   combine  : one block per received row sends the expert output row back to the token's rank, slot (token, k).
//   fold     : the token's rank waits for all flags and adds its k rows in k order (fp32), plus an optional addend
//              (shared expert / residual).
// Peer traffic is plain stores and bulk copies over NVLink; nothing is multicast.  Reference behaviour replaced:
// crates/sparkflash-model-inkling2 ExpertSplit::Experts exchange (tensor.rs:49-78), kernels opt_exchange slot exchange.
#include "k_common.cuh"

namespace sfb {

__device__ __forceinline__ uint32_t ep_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ep_bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ep_bulk_wait() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

struct EpRecord { int expert; int tok; int k; float weight; };     // 16 bytes

struct EpDispatchArgs {
  const __nv_bfloat16* x;      // [t, d]
  const int* ids;              // [t, top_k] global expert ids
  const float* wts;            // [t, top_k]
  int t, d, top_k, epr, W, rank, cap;
  // per destination rank: the region "from this rank" of its receive buffers
  uint8_t* recv_q[8];          // [cap, d] E4M3
  uint8_t* recv_s[8];          // compact UE8M0 scales [cap, d/32]; the receiver expands them into scale atoms
  EpRecord* recv_rec[8];       // [cap]
  int* recv_count[8];          // one int
  uint32_t* flag[8];
  int* counters;               // [W] local, zero between launches
  unsigned int* done;          // zero between launches
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
};

// block = 256 threads, one token; dynamic shared memory: d bytes of codes + d/32 bytes of scales
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDispatchArgs a) {
  extern __shared__ __align__(128) uint8_t sm[];
  __shared__ int slot_of[8];
  __shared__ int is_last;
  const int tok = blockIdx.x;
  uint8_t* q = sm;
  uint8_t* scales = sm + a.d;
  for (int c = threadIdx.x; c < a.d; c += 256) {            // a warp covers one 32-group
    const float v = __bfloat162float(a.x[(size_t)tok * a.d + c]);
    uint8_t sc;
    q[c] = warp_quant_fp8(v, &sc);
    if ((threadIdx.x & 31) == 0) scales[c >> 5] = sc;
  }
  if (threadIdx.x < a.top_k) {
    const int e = a.ids[(size_t)tok * a.top_k + threadIdx.x];
    slot_of[threadIdx.x] = atomicAdd(&a.counters[e / a.epr], 1);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < a.top_k) {
    const int k = threadIdx.x;
    const int e = a.ids[(size_t)tok * a.top_k + k];
    const int dst = e / a.epr, slot = slot_of[k];
    if (slot < a.cap) {
      ep_bulk_store(a.recv_q[dst] + (size_t)slot * a.d, ep_smem_u32(q), (uint32_t)a.d);
      ep_bulk_store(a.recv_s[dst] + (size_t)slot * (a.d >> 5), ep_smem_u32(scales), (uint32_t)(a.d >> 5));
      EpRecord r{e - dst * a.epr, tok, k, a.wts[(size_t)tok * a.top_k + k]};
      *reinterpret_cast<int4*>(&a.recv_rec[dst][slot]) = *reinterpret_cast<int4*>(&r);
    }
    ep_bulk_wait();
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.done, 1u);
    is_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last && threadIdx.x < a.W) {
    const int r = threadIdx.x;
    const int n = min(atomicAdd(&a.counters[r], 0), a.cap);
    *a.recv_count[r] = n;
    a.counters[r] = 0;
    __threadfence_system();
    st_release_sys(a.flag[r], *a.epoch_ptr + a.epoch_add);
    if (r == 0) *a.done = 0;
  }
}

struct EpPlanArgs {
  const EpRecord* rec;          // [W, cap] this rank's receive records
  const int* count;             // [W]
  const uint32_t* flag[8];
  int W, cap;
  int* ids;                     // [W*cap] local expert id or -1
  float* wts;                   // [W*cap]
  const uint8_t* recv_s;        // [W*cap, KB] compact scales as received
  uint8_t* atoms;               // [W*cap, atom_bytes] one scale-atom set per row (what the grouped GEMM loads)
  int KB, atom_bytes;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  uint64_t wait_ns;
  Status* status;
};

__global__ void __launch_bounds__(256) ep_plan_kernel(EpPlanArgs a) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint32_t want = *a.epoch_ptr + a.epoch_add;
    for (int r = 0; r < a.W; ++r)
      if (!wait_flag_ge(a.flag[r], want, a.wait_ns)) { ok = 0; status_set(a.status, ST_TIMEOUT, 50, r, 0); break; }
  }
  __syncthreads();
  for (int i = blockIdx.x * 256 + threadIdx.x; i < a.W * a.cap; i += gridDim.x * 256) {
    const int src = i / a.cap, slot = i % a.cap;
    const bool live = ok && slot < a.count[src];
    a.ids[i] = live ? a.rec[i].expert : -1;
    a.wts[i] = live ? a.rec[i].weight : 0.f;
  }
  for (int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x; j < (int64_t)a.W * a.cap * a.KB; j += (int64_t)gridDim.x * 256) {
    const int i = (int)(j / a.KB), kb = (int)(j % a.KB);
    if (ok && (i % a.cap) < a.count[i / a.cap]) a.atoms[(size_t)i * a.atom_bytes + sf_offset(0, kb, a.KB)] = a.recv_s[j];
  }
}

struct EpCombineArgs {
  const __nv_bfloat16* y;       // [W*cap, d] expert outputs of the received rows
  const EpRecord* rec;
  const int* count;             // [W]
  int W, cap, d, top_k, rank;
  __nv_bfloat16* comb[8];       // on source rank s: [t, top_k, d]
  uint32_t* flag[8];
  unsigned int* done;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
};

// grid = W*cap blocks of 128 threads; a live row is staged in shared memory and leaves as one bulk copy
__global__ void __launch_bounds__(128) ep_combine_kernel(EpCombineArgs a) {
  extern __shared__ __align__(128) uint8_t sm[];
  __shared__ int is_last;
  const int i = blockIdx.x, src = i / a.cap, slot = i % a.cap;
  if (slot < a.count[src]) {
    const uint4* in = reinterpret_cast<const uint4*>(a.y + (size_t)i * a.d);
    uint4* st = reinterpret_cast<uint4*>(sm);
    for (int c = threadIdx.x; c < a.d / 8; c += 128) st[c] = in[c];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
      const EpRecord r = a.rec[i];
      ep_bulk_store(a.comb[src] + ((size_t)r.tok * a.top_k + r.k) * a.d, ep_smem_u32(sm), (uint32_t)(a.d * 2));
      ep_bulk_wait();
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.done, 1u);
    is_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last && threadIdx.x < a.W) {
    __threadfence_system();
    st_release_sys(a.flag[threadIdx.x], *a.epoch_ptr + a.epoch_add);
    if (threadIdx.x == 0) *a.done = 0;
  }
}

struct EpFoldArgs {
  const __nv_bfloat16* comb;    // [t, top_k, d]
  const __nv_bfloat16* addend;  // optional [t, d]
  __nv_bfloat16* out;           // [t, d]
  const uint32_t* flag[8];
  int W, t, d, top_k;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  uint64_t wait_ns;
  Status* status;
};

__global__ void __launch_bounds__(128) ep_fold_kernel(EpFoldArgs a) {
  __shared__ int ok;
  const int tok = blockIdx.x;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint32_t want = *a.epoch_ptr + a.epoch_add;
    for (int r = 0; r < a.W; ++r)
      if (!wait_flag_ge(a.flag[r], want, a.wait_ns)) { ok = 0; status_set(a.status, ST_TIMEOUT, 51, r, tok); break; }
  }
  __syncthreads();
  if (!ok) return;
  for (int c = threadIdx.x * 8; c < a.d; c += 128 * 8) {
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < a.top_k; ++k) {        // k order: the sum does not depend on which rank answered first
      const uint4 u = *reinterpret_cast<const uint4*>(a.comb + ((size_t)tok * a.top_k + k) * a.d + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); s[2 * j] += f.x; s[2 * j + 1] += f.y; }
    }
    if (a.addend) {
      const uint4 u = *reinterpret_cast<const uint4*>(a.addend + (size_t)tok * a.d + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); s[2 * j] += f.x; s[2 * j + 1] += f.y; }
    }
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(s[2 * j], s[2 * j + 1]);
    *reinterpret_cast<uint4*>(a.out + (size_t)tok * a.d + c) = o;
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_ep_dispatch(const void* x, const void* ids, const void* wts, int t, int d, int top_k, int epr, int W, int rank, int cap,
                    const void* const* recv_q, const void* const* recv_s, const void* const* recv_rec, const void* const* recv_count,
                    const void* const* flags, void* counters, void* done, const void* epoch_ptr, uint32_t epoch_add,
                    cudaStream_t stream) {
  if (W < 1 || W > 8 || top_k > 8 || d % 512 || t < 1) return (int)cudaErrorInvalidValue;
  EpDispatchArgs a{};
  a.x = (const __nv_bfloat16*)x; a.ids = (const int*)ids; a.wts = (const float*)wts; a.t = t; a.d = d; a.top_k = top_k; a.epr = epr;
  a.W = W; a.rank = rank; a.cap = cap; a.counters = (int*)counters; a.done = (unsigned int*)done;
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add;
  for (int r = 0; r < W; ++r) {
    a.recv_q[r] = (uint8_t*)recv_q[r]; a.recv_s[r] = (uint8_t*)recv_s[r]; a.recv_rec[r] = (EpRecord*)recv_rec[r];
    a.recv_count[r] = (int*)recv_count[r]; a.flag[r] = (uint32_t*)flags[r];
  }
  ep_dispatch_kernel<<<t, 256, (size_t)d + d / 32, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

int sfb_ep_plan(const void* rec, const void* count, const void* const* flags, int W, int cap, void* ids, void* wts, const void* recv_s,
                void* atoms, int KB, int atom_bytes, const void* epoch_ptr, uint32_t epoch_add, uint64_t wait_ns, void* status,
                cudaStream_t stream) {
  EpPlanArgs a{};
  a.rec = (const EpRecord*)rec; a.count = (const int*)count; a.W = W; a.cap = cap; a.ids = (int*)ids; a.wts = (float*)wts;
  a.recv_s = (const uint8_t*)recv_s; a.atoms = (uint8_t*)atoms; a.KB = KB; a.atom_bytes = atom_bytes;
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns; a.status = (Status*)status;
  for (int r = 0; r < W; ++r) a.flag[r] = (const uint32_t*)flags[r];
  ep_plan_kernel<<<(W * cap + 7) / 8 < 64 ? ((W * cap + 7) / 8 > 0 ? (W * cap + 7) / 8 : 1) : 64, 256, 0, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

int sfb_ep_combine(const void* y, const void* rec, const void* count, int W, int cap, int d, int top_k, int rank, const void* const* comb,
                   const void* const* flags, void* done, const void* epoch_ptr, uint32_t epoch_add, cudaStream_t stream) {
  if (d % 8) return (int)cudaErrorInvalidValue;
  EpCombineArgs a{};
  a.y = (const __nv_bfloat16*)y; a.rec = (const EpRecord*)rec; a.count = (const int*)count; a.W = W; a.cap = cap; a.d = d; a.top_k = top_k;
  a.rank = rank; a.done = (unsigned int*)done; a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add;
  for (int r = 0; r < W; ++r) { a.comb[r] = (__nv_bfloat16*)comb[r]; a.flag[r] = (uint32_t*)flags[r]; }
  ep_combine_kernel<<<W * cap, 128, (size_t)d * 2, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

int sfb_ep_fold(const void* comb, const void* addend, void* out, const void* const* flags, int W, int t, int d, int top_k,
                const void* epoch_ptr, uint32_t epoch_add, uint64_t wait_ns, void* status, cudaStream_t stream) {
  EpFoldArgs a{};
  a.comb = (const __nv_bfloat16*)comb; a.addend = (const __nv_bfloat16*)addend; a.out = (__nv_bfloat16*)out; a.W = W; a.t = t; a.d = d;
  a.top_k = top_k; a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns; a.status = (Status*)status;
  for (int r = 0; r < W; ++r) a.flag[r] = (const uint32_t*)flags[r];
  ep_fold_kernel<<<t, 128, 0, stream>>>(a);
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
