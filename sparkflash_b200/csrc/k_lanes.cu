// Lane memory: per-sequence KV regions in reserved virtual address space, backed lazily by 2 MiB physical
// chunks from a budgeted pool (CUDA virtual memory management).  A region is `lanes` spans laid out back to
// back, so the kernels see one dense [lanes, rows, row_bytes] array whose unused tails own no memory.
// Reference behaviour: crates/sparkflash-kernels/src/lane_memory.rs:93-586 (reserve, 2 MiB lazy backing, chunk
// pool with a byte budget, release, copy_prefix).  Driver entry points are resolved at run time, so the
// library loads on machines without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

namespace {

template <typename F>
F entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
  return (F)p;
}

struct Api {
  CUresult (*GetGran)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*Reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*AddrFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  bool ok = false;
  Api() {
    GetGran = entry<decltype(GetGran)>("cuMemGetAllocationGranularity");
    Reserve = entry<decltype(Reserve)>("cuMemAddressReserve");
    AddrFree = entry<decltype(AddrFree)>("cuMemAddressFree");
    Create = entry<decltype(Create)>("cuMemCreate");
    Release = entry<decltype(Release)>("cuMemRelease");
    Map = entry<decltype(Map)>("cuMemMap");
    Unmap = entry<decltype(Unmap)>("cuMemUnmap");
    SetAccess = entry<decltype(SetAccess)>("cuMemSetAccess");
    ok = GetGran && Reserve && AddrFree && Create && Release && Map && Unmap && SetAccess;
  }
};

struct Pool {                      // physical chunks shared by every region of one device
  Api api;
  int device = 0;
  size_t gran = 0;
  size_t budget_chunks = 0, created = 0;
  std::vector<CUmemGenericAllocationHandle> spare;
  CUmemAllocationProp prop{};
};

struct Region {
  Pool* pool;
  CUdeviceptr base = 0;
  size_t lanes = 0, span = 0;     // span: bytes per lane, a multiple of the granularity
  std::vector<std::vector<CUmemGenericAllocationHandle>> chunks;   // [lane][chunk] 0 = not backed
  size_t mapped = 0;
};

}  // namespace

extern "C" {

// status codes: 0 ok, 1 driver entry points missing, 2 budget exhausted, 3 bad argument, 100+ = 100 + CUresult
int sfb_lanepool_create(int device, long long budget_bytes, void** out) {
  Pool* p = new Pool();
  if (!p->api.ok) { delete p; return 1; }
  cudaFree(0);       // make sure the primary context exists
  p->device = device;
  p->prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p->prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p->prop.location.id = device;
  CUresult r = p->api.GetGran(&p->gran, &p->prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (r != CUDA_SUCCESS) { delete p; return 100 + (int)r; }
  p->budget_chunks = (size_t)budget_bytes / p->gran;
  *out = p;
  return 0;
}
long long sfb_lanepool_granularity(void* h) { return (long long)((Pool*)h)->gran; }
// [created, spare, budget] in chunks
void sfb_lanepool_stats(void* h, long long* out3) { Pool* p = (Pool*)h; out3[0] = p->created; out3[1] = p->spare.size(); out3[2] = p->budget_chunks; }
// give spare chunks back to the driver (at most `max_chunks`); returns how many
int sfb_lanepool_trim(void* h, int max_chunks) {
  Pool* p = (Pool*)h; int n = 0;
  while (!p->spare.empty() && n < max_chunks) { p->api.Release(p->spare.back()); p->spare.pop_back(); p->created--; ++n; }
  return n;
}
int sfb_lanepool_destroy(void* h) {
  Pool* p = (Pool*)h;
  for (auto c : p->spare) p->api.Release(c);
  delete p;
  return 0;
}

// Reserve lanes * span bytes of address space; span = lane_bytes rounded up to the granularity.
int sfb_laneregion_create(void* pool, int lanes, long long lane_bytes, void** out) {
  Pool* p = (Pool*)pool;
  if (lanes <= 0 || lane_bytes <= 0) return 3;
  Region* r = new Region();
  r->pool = p; r->lanes = lanes;
  r->span = ((size_t)lane_bytes + p->gran - 1) / p->gran * p->gran;
  CUresult e = p->api.Reserve(&r->base, r->lanes * r->span, p->gran, 0, 0);
  if (e != CUDA_SUCCESS) { delete r; return 100 + (int)e; }
  r->chunks.assign(lanes, std::vector<CUmemGenericAllocationHandle>(r->span / p->gran, 0));
  *out = r;
  return 0;
}
unsigned long long sfb_laneregion_base(void* h) { return (unsigned long long)((Region*)h)->base; }
long long sfb_laneregion_span(void* h) { return (long long)((Region*)h)->span; }
long long sfb_laneregion_mapped(void* h) { return (long long)((Region*)h)->mapped; }

// Back bytes [0, upto) of one lane.  Already-backed chunks are left alone.
int sfb_laneregion_ensure(void* h, int lane, long long upto) {
  Region* r = (Region*)h; Pool* p = r->pool;
  if (lane < 0 || (size_t)lane >= r->lanes || upto < 0 || (size_t)upto > r->span) return 3;
  size_t need = ((size_t)upto + p->gran - 1) / p->gran;
  auto& cs = r->chunks[lane];
  for (size_t c = 0; c < need; ++c) {
    if (cs[c]) continue;
    CUmemGenericAllocationHandle hnd;
    if (!p->spare.empty()) { hnd = p->spare.back(); p->spare.pop_back(); }
    else {
      if (p->created >= p->budget_chunks) return 2;
      CUresult e = p->api.Create(&hnd, p->gran, &p->prop, 0);
      if (e != CUDA_SUCCESS) return e == CUDA_ERROR_OUT_OF_MEMORY ? 2 : 100 + (int)e;
      p->created++;
    }
    CUdeviceptr at = r->base + (size_t)lane * r->span + c * p->gran;
    CUresult e = p->api.Map(at, p->gran, 0, hnd, 0);
    if (e != CUDA_SUCCESS) { p->spare.push_back(hnd); return 100 + (int)e; }
    CUmemAccessDesc acc{};
    acc.location = p->prop.location; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    e = p->api.SetAccess(at, p->gran, &acc, 1);
    if (e != CUDA_SUCCESS) { p->api.Unmap(at, p->gran); p->spare.push_back(hnd); return 100 + (int)e; }
    cs[c] = hnd;
    r->mapped += p->gran;
  }
  return 0;
}
// Give back the chunks of one lane that lie wholly at or above byte `from` (0 = the whole lane).  The caller
// has made sure that no kernel still uses them.
int sfb_laneregion_release(void* h, int lane, long long from) {
  Region* r = (Region*)h; Pool* p = r->pool;
  if (lane < 0 || (size_t)lane >= r->lanes || from < 0) return 3;
  auto& cs = r->chunks[lane];
  for (size_t c = ((size_t)from + p->gran - 1) / p->gran; c < cs.size(); ++c) {
    if (!cs[c]) continue;
    CUdeviceptr at = r->base + (size_t)lane * r->span + c * p->gran;
    CUresult e = p->api.Unmap(at, p->gran);
    if (e != CUDA_SUCCESS) return 100 + (int)e;
    p->spare.push_back(cs[c]);
    cs[c] = 0;
    r->mapped -= p->gran;
  }
  return 0;
}
long long sfb_laneregion_backed(void* h, int lane) {    // contiguous backed bytes from the start of the lane
  Region* r = (Region*)h;
  size_t n = 0;
  for (auto c : r->chunks[lane]) { if (!c) break; ++n; }
  return (long long)(n * r->pool->gran);
}
// Copy the first `bytes` of one lane to another (prefix adoption); the destination is backed first.
int sfb_laneregion_copy_prefix(void* h, int src, int dst, long long bytes, void* stream) {
  Region* r = (Region*)h;
  if (sfb_laneregion_backed(h, src) < bytes) return 3;
  int rc = sfb_laneregion_ensure(h, dst, bytes);
  if (rc) return rc;
  cudaError_t e = cudaMemcpyAsync((void*)(r->base + (size_t)dst * r->span), (const void*)(r->base + (size_t)src * r->span),
                                  (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  return e == cudaSuccess ? 0 : 100 + (int)e;
}
int sfb_laneregion_destroy(void* h) {
  Region* r = (Region*)h;
  for (size_t l = 0; l < r->lanes; ++l) sfb_laneregion_release(h, (int)l, 0);
  r->pool->api.AddrFree(r->base, r->lanes * r->span);
  delete r;
  return 0;
}

}  // extern "C"
