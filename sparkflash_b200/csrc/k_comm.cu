// Symmetric memory and the push half of the fused collectives.
//
// Every rank owns one symmetric allocation; all ranks map all allocations (CUDA IPC inside one box, the
// traffic goes over NVLink through NVSwitch).  A producer stores its partial result into "its" slot of
// every rank's buffer with plain peer stores and then raises an arrival flag on every rank; a consumer
// only ever reads its own memory and waits - with a time limit - on its own flags.  The reduction itself
// (rank-order fold in fp32) lives in the consumer, csrc/k_seam.cu.  No TMA, no multicast loads.
//
// Reference behaviour replaced: crates/sparkflash-comm/src/rdma/write_exchange.rs (one write per peer +
// arrival flag, doorbell deadline, abort word), kernels/opt_exchange_sm121.cuh (opt_exchange_stage_bf16:68),
// kernels/opt_misc_sm121.cu:399 (opt_sum_ranks_bf16, the canonical rank-order fold).
#include "k_common.cuh"

namespace sfb {

struct PushArgs {
  const uint4* src;        // n16 x 16 bytes
  uint4* dst[8];           // the same slot on every rank (including this one)
  uint32_t* flag[8];       // this rank's flag word on every rank
  int W;
  int64_t n16;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  unsigned int* done;      // zero between launches
};

__global__ void __launch_bounds__(256) push_rows_kernel(PushArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int is_last;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = a.src[i];
    for (int r = 0; r < a.W; ++r) a.dst[r][i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.done, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *a.done = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < a.W) {
    __threadfence_system();
    st_release_sys(a.flag[threadIdx.x], *a.epoch_ptr + a.epoch_add);
  }
}

// ---- two-shot all-reduce of a many-row partial: reduce-scatter, fold on the owner, all-gather -----------------------------------
// Shot 1: rank p sends rows [j rs, (j + 1) rs) of its partial to rows [0, rs) of slot p on rank j, then raises its flag on
// every rank.  Shot 2 (fold_push_rs_kernel): rank j waits for the W flags, adds the W slots' rows in rank order (fp32, one
// bf16 rounding: the sum a one-shot consumer forms), stores the result to rows [rs, 2 rs) of slot j on every rank and raises
// its flag to the second epoch.  A consumer then finds row t in slot t / rs at row rs + t % rs.  Each rank sends
// 2 (W - 1) / W of a partial instead of W - 1 partials.
struct PushRsArgs {
  const uint4* src;           // [n, src_row16] this rank's partial
  uint4* dst[8];              // this rank's slot on every rank
  uint32_t* flag[8];          // this rank's flag on every rank
  int W, n, rs_rows, row16, src_row16;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  unsigned int* done;         // zero between launches
};

__global__ void __launch_bounds__(256) push_rows_rs_kernel(PushRsArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int is_last;
  const int64_t total = (int64_t)a.n * a.row16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / a.row16), c = (int)(i - (int64_t)row * a.row16);
    const int j = row / a.rs_rows;
    a.dst[j][(int64_t)(row - j * a.rs_rows) * a.row16 + c] = a.src[(int64_t)row * a.src_row16 + c];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.done, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *a.done = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < a.W) {
    __threadfence_system();
    st_release_sys(a.flag[threadIdx.x], *a.epoch_ptr + a.epoch_add);
  }
}

struct FoldPushArgs {
  const uint4* slot[8];       // the W slots of this rank's own buffer
  const uint32_t* flag[8];    // their arrival flags (shot 1)
  uint4* dst[8];              // this rank's slot on every rank
  uint32_t* oflag[8];         // this rank's flag on every rank
  int W, rows, rs_rows, row16;
  const uint32_t* epoch_ptr;
  uint32_t epoch_wait, epoch_raise;
  uint64_t wait_ns;
  unsigned int* done;
  Status* status;
};

__global__ void __launch_bounds__(256) fold_push_rs_kernel(FoldPushArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int is_last, ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < a.W && !wait_flag_ge(a.flag[threadIdx.x], *a.epoch_ptr + a.epoch_wait, a.wait_ns)) {
    status_set(a.status, ST_TIMEOUT, 31, threadIdx.x, (int)(*a.epoch_ptr + a.epoch_wait));
    ok = 0;
  }
  __syncthreads();
  const int64_t total = (int64_t)a.rows * a.row16;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; ok && i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < a.W; ++r) {
      const uint4 v = a.slot[r][i];
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p2[e]);
        acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    const int64_t at = (int64_t)a.rs_rows * a.row16 + i;      // rows [rs, 2 rs) of the slot
    for (int r = 0; r < a.W; ++r) a.dst[r][at] = o;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(a.done, 1u);
    is_last = prev == gridDim.x - 1;
    if (is_last) *a.done = 0;
  }
  __syncthreads();
  if (is_last && threadIdx.x < a.W) {      // raised even after a timeout: the peers go on and the host reads the status word
    __threadfence_system();
    st_release_sys(a.oflag[threadIdx.x], *a.epoch_ptr + a.epoch_raise);
  }
}

__global__ void epoch_bump_kernel(uint32_t* epoch, uint32_t add) { *epoch += add; }

// Test / emulation helper: wait (bounded) until every flag reaches the epoch; records a timeout in status.
__global__ void wait_flags_kernel(const uint32_t* const* flags, int W, const uint32_t* epoch_ptr, uint32_t epoch_add,
                                  uint64_t budget_ns, Status* st) {
  if (threadIdx.x < W && !wait_flag_ge(flags[threadIdx.x], *epoch_ptr + epoch_add, budget_ns))
    status_set(st, ST_TIMEOUT, 30, threadIdx.x, (int)(*epoch_ptr + epoch_add));
}


// ---- consumer half of GEMM -> all-reduce / reduce-scatter: fold the W arrival slots, add the residual, RMSNorm ----
struct FoldArgs {
  const __nv_bfloat16* slot[8];   // rank r's partial for this rank's rows, [n, stride]
  const uint32_t* flag[8];        // arrival flags (null = do not wait)
  int W, n, d;
  int64_t stride;
  const uint32_t* epoch_ptr;
  uint32_t epoch_add;
  uint64_t wait_ns;
  const __nv_bfloat16* residual;  // optional [n, d]
  const float* norm_w;            // optional [d]: out = rmsnorm(sum + residual) * w
  float eps;
  __nv_bfloat16* out_sum;         // optional: sum + residual (the new residual stream)
  __nv_bfloat16* out;             // normalised (or plain sum when norm_w is null)
  uint8_t* out_q;                 // optional FP8 re-quantisation of `out` for the next GEMM, [n, d]
  uint8_t* out_atom;              //   its scale atoms (rows = tokens, d / 32 k-blocks)
  Status* status;
};

// one block per token row, 128 threads; a thread owns 8 consecutive columns per pass (16-byte loads), so four lanes
// hold one 32-column scale group
__global__ void __launch_bounds__(128) fold_slots_kernel(FoldArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  __shared__ int ok;
  const int row = blockIdx.x;
  if (threadIdx.x == 0) {
    ok = 1;
    if (a.flag[0]) {
      const uint32_t want = *a.epoch_ptr + a.epoch_add;
      for (int r = 0; r < a.W; ++r)
        if (!wait_flag_ge(a.flag[r], want, a.wait_ns)) { ok = 0; status_set(a.status, ST_TIMEOUT, 40, r, row); break; }
    }
  }
  __syncthreads();
  if (!ok) return;
  constexpr int PASS = 6;          // d <= 6 * 1024
  float vals[PASS][8];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PASS; ++p)
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[p][j] = 0.f;
  // one round trip per source instead of one per (source, pass): all of a source's 16-byte loads of this row are issued
  // before the first add.  Each element still adds slot 0, slot 1, ..., then the residual: same sums as before
  // two sources per round trip: both sources' loads are issued before either is added (slot order of the adds unchanged)
  for (int r = 0; r <= a.W; r += 2) {
    const __nv_bfloat16* src0 = r < a.W ? a.slot[r] + (int64_t)row * a.stride : (a.residual ? a.residual + (int64_t)row * a.d : nullptr);
    const __nv_bfloat16* src1 = r + 1 < a.W ? a.slot[r + 1] + (int64_t)row * a.stride
                                            : (r + 1 == a.W && a.residual ? a.residual + (int64_t)row * a.d : nullptr);
    if (!src0) break;
    uint4 u[PASS], u1[PASS];
#pragma unroll
    for (int p = 0; p < PASS; ++p) {
      const int c = (p * 128 + threadIdx.x) * 8;
      u[p] = c < a.d ? *reinterpret_cast<const uint4*>(src0 + c) : make_uint4(0, 0, 0, 0);
      u1[p] = (src1 && c < a.d) ? *reinterpret_cast<const uint4*>(src1 + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int p = 0; p < PASS; ++p) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[p]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); vals[p][2 * j] += f.x; vals[p][2 * j + 1] += f.y; }
    }
    if (src1) {
#pragma unroll
      for (int p = 0; p < PASS; ++p) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u1[p]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); vals[p][2 * j] += f.x; vals[p][2 * j + 1] += f.y; }
      }
    }
  }
#pragma unroll
  for (int p = 0; p < PASS; ++p) {
    const int c = (p * 128 + threadIdx.x) * 8;
    if (c >= a.d) break;
    if (a.out_sum) {
      uint4 o;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(vals[p][2 * j], vals[p][2 * j + 1]);
      *reinterpret_cast<uint4*>(a.out_sum + (int64_t)row * a.d + c) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += vals[p][j] * vals[p][j];
  }
  float scale = 1.f;
  if (a.norm_w) scale = rsqrtf(block_sum(ss, red) / (float)a.d + a.eps);
#pragma unroll
  for (int p = 0; p < PASS; ++p) {
    const int c = (p * 128 + threadIdx.x) * 8;
    if (c >= a.d) break;
    float y[8];
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = a.norm_w ? vals[p][j] * scale * a.norm_w[c + j] : vals[p][j];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
    *reinterpret_cast<uint4*>(a.out + (int64_t)row * a.d + c) = o;
    if (a.out_q) {
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) { y[j] = bfr(y[j]); amax = fmaxf(amax, fabsf(y[j])); }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const uint8_t sc = act_scale_code_fp8(amax);
      const float inv = bits_f32(((uint32_t)(254 - sc)) << 23);
      uint2 qv;
      uint8_t* qb = reinterpret_cast<uint8_t*>(&qv);
#pragma unroll
      for (int j = 0; j < 8; ++j) qb[j] = enc_e4m3(y[j] * inv);
      *reinterpret_cast<uint2*>(a.out_q + (int64_t)row * a.d + c) = qv;
      if ((threadIdx.x & 3) == 0) a.out_atom[sf_offset(row, c >> 5, a.d >> 5)] = sc;
    }
  }
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_symm_alloc(void** out, int64_t bytes) {
  cudaError_t e = cudaMalloc(out, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(*out, 0, (size_t)bytes);
  return (int)e;
}
int sfb_symm_free(void* p) { return (int)cudaFree(p); }
int sfb_ipc_get_handle(void* p, void* handle64) { return (int)cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, p); }
int sfb_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof h);
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
int sfb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }
int sfb_memcpy_d2h(void* dst, const void* src, int64_t bytes) { return (int)cudaMemcpy(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost); }
int sfb_memset_async(void* p, int v, int64_t bytes, cudaStream_t s) { return (int)cudaMemsetAsync(p, v, (size_t)bytes, s); }

// dst_ptrs / flag_ptrs: host arrays of W device addresses
int sfb_push_rows(const void* src, const void* const* dst_ptrs, const void* const* flag_ptrs, int W, int64_t bytes,
                  const void* epoch_ptr, uint32_t epoch_add, void* done, cudaStream_t stream) {
  if (bytes % 16 || W < 1 || W > 8) return (int)cudaErrorInvalidValue;
  PushArgs a{};
  a.src = (const uint4*)src;
  for (int r = 0; r < W; ++r) { a.dst[r] = (uint4*)dst_ptrs[r]; a.flag[r] = (uint32_t*)flag_ptrs[r]; }
  a.W = W; a.n16 = bytes / 16; a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add;
  a.done = (unsigned int*)done;
  int64_t blocks = (a.n16 + 255) / 256;
  const int64_t cap = bytes > (1 << 20) ? 148 * 4 : 64;     // megabytes need every SM's stores in flight to fill the links
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)sfb_launch(push_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, a);
}

// slots / flags: host arrays of W device addresses (flags may be null: no waiting)
int sfb_fold_slots(const void* const* slots, const void* const* flags, int W, int n, int d, int64_t stride, const void* epoch_ptr,
                   uint32_t epoch_add, uint64_t wait_ns, const void* residual, const void* norm_w, float eps, void* out_sum,
                   void* out, void* out_q, void* out_atom, void* status, cudaStream_t stream) {
  if (W < 1 || W > 8 || d > 6 * 1024 || d % 32 || n < 1 || (stride & 7)) return (int)cudaErrorInvalidValue;
  FoldArgs a{};
  for (int r = 0; r < W; ++r) { a.slot[r] = (const __nv_bfloat16*)slots[r]; a.flag[r] = flags ? (const uint32_t*)flags[r] : nullptr; }
  a.W = W; a.n = n; a.d = d; a.stride = stride; a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.wait_ns = wait_ns;
  a.residual = (const __nv_bfloat16*)residual; a.norm_w = (const float*)norm_w; a.eps = eps; a.out_sum = (__nv_bfloat16*)out_sum;
  a.out = (__nv_bfloat16*)out; a.out_q = (uint8_t*)out_q; a.out_atom = (uint8_t*)out_atom; a.status = (Status*)status;
  return (int)sfb_launch(fold_slots_kernel, dim3(n), dim3(128), 0, stream, a);
}

// shot 1 of the two-shot all-reduce: dst / flags = this rank's slot / flag on every rank; row_bytes a multiple of 16
int sfb_push_rows_rs(const void* src, int64_t src_row_bytes, const void* const* dst_ptrs, const void* const* flag_ptrs, int W, int n,
                     int rs_rows, int64_t row_bytes, const void* epoch_ptr, uint32_t epoch_add, void* done, cudaStream_t stream) {
  if (W < 1 || W > 8 || n < 1 || rs_rows < 1 || (int64_t)rs_rows * W < n || (row_bytes & 15) || (src_row_bytes & 15)) return (int)cudaErrorInvalidValue;
  PushRsArgs a{};
  a.src = (const uint4*)src;
  for (int r = 0; r < W; ++r) { a.dst[r] = (uint4*)dst_ptrs[r]; a.flag[r] = (uint32_t*)flag_ptrs[r]; }
  a.W = W; a.n = n; a.rs_rows = rs_rows; a.row16 = (int)(row_bytes / 16); a.src_row16 = (int)(src_row_bytes / 16);
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_add = epoch_add; a.done = (unsigned int*)done;
  int64_t blocks = ((int64_t)n * a.row16 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  return (int)sfb_launch(push_rows_rs_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, a);
}

// shot 2: slots / flags = the W slots of this rank's buffer and their flags; dst / oflags = this rank's slot / flag on every rank
int sfb_fold_push_rs(const void* const* slots, const void* const* flags, const void* const* dst_ptrs, const void* const* oflag_ptrs, int W,
                     int rows, int rs_rows, int64_t row_bytes, const void* epoch_ptr, uint32_t epoch_wait, uint32_t epoch_raise,
                     uint64_t wait_ns, void* done, void* status, cudaStream_t stream) {
  if (W < 1 || W > 8 || rows < 0 || rows > rs_rows || (row_bytes & 15)) return (int)cudaErrorInvalidValue;
  FoldPushArgs a{};
  for (int r = 0; r < W; ++r) {
    a.slot[r] = (const uint4*)slots[r]; a.flag[r] = (const uint32_t*)flags[r];
    a.dst[r] = (uint4*)dst_ptrs[r]; a.oflag[r] = (uint32_t*)oflag_ptrs[r];
  }
  a.W = W; a.rows = rows; a.rs_rows = rs_rows; a.row16 = (int)(row_bytes / 16);
  a.epoch_ptr = (const uint32_t*)epoch_ptr; a.epoch_wait = epoch_wait; a.epoch_raise = epoch_raise;
  a.wait_ns = wait_ns ? wait_ns : 2000000000ull; a.done = (unsigned int*)done; a.status = (Status*)status;
  int64_t blocks = ((int64_t)rows * a.row16 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  return (int)sfb_launch(fold_push_rs_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, a);
}

int sfb_epoch_bump(void* epoch, uint32_t add, cudaStream_t stream) {
  epoch_bump_kernel<<<1, 1, 0, stream>>>((uint32_t*)epoch, add);
  return SFB_CHECK_LAUNCH();
}

int sfb_wait_flags(const void* const* flags_dev_array, int W, const void* epoch_ptr, uint32_t epoch_add,
                   uint64_t budget_ns, void* status, cudaStream_t stream) {
  wait_flags_kernel<<<1, 32, 0, stream>>>((const uint32_t* const*)flags_dev_array, W, (const uint32_t*)epoch_ptr,
                                          epoch_add, budget_ns, (Status*)status);
  return SFB_CHECK_LAUNCH();
}

}  // extern "C"
