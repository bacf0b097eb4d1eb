// Device side of the tracer: a host-mapped ring of 32-byte events stamped with %globaltimer.
// The active scope mask is mirrored into the ring header, so an unarmed scope costs one load.
// Reference behaviour: kernels/trace_globaltimer_sm121.cuh, crates/sparkflash-kernels/src/device_trace.rs,
// crates/sparkflash-trace/src/controller.rs:186-198 (mask mirrored into the ring header).
#include <cuda_runtime.h>
#include <stdint.h>

namespace sfb {

struct TraceHeader {
  unsigned long long mask;      // armed scopes (written by the host)
  unsigned long long head;      // events pushed so far (written by the device)
  unsigned long long capacity;  // events in the ring
  unsigned long long dropped;
};
struct TraceEvent {             // 32 bytes
  unsigned long long t_ns;      // %globaltimer
  unsigned int scope_bit;       // index of the scope
  unsigned int tag;             // caller's id (layer, stage)
  unsigned int phase;           // 0 begin, 1 end, 2 instant
  unsigned int smid;
  unsigned long long aux;
};

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void trace_mark_kernel(TraceHeader* hdr, TraceEvent* ring, unsigned scope_bit, unsigned tag, unsigned phase,
                                  unsigned long long aux) {
  if (!((hdr->mask >> scope_bit) & 1ull)) return;
  unsigned long long i = atomicAdd(&hdr->head, 1ull);
  TraceEvent& e = ring[i % hdr->capacity];
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  e.scope_bit = scope_bit; e.tag = tag; e.phase = phase; e.smid = smid; e.aux = aux;
  e.t_ns = globaltimer();
  __threadfence_system();
}

}  // namespace sfb

extern "C" {

// One mapped allocation: header (64 bytes) followed by `capacity` events.  *host and *dev alias the same memory.
int sfb_trace_ring_create(long long capacity, void** host, void** dev) {
  size_t bytes = 64 + (size_t)capacity * sizeof(sfb::TraceEvent);
  cudaError_t e = cudaHostAlloc(host, bytes, cudaHostAllocMapped);
  if (e != cudaSuccess) return (int)e;
  memset(*host, 0, bytes);
  ((sfb::TraceHeader*)*host)->capacity = (unsigned long long)capacity;
  e = cudaHostGetDevicePointer(dev, *host, 0);
  return (int)e;
}
int sfb_trace_ring_destroy(void* host) { return (int)cudaFreeHost(host); }
int sfb_trace_mark(void* dev, unsigned scope_bit, unsigned tag, unsigned phase, unsigned long long aux, void* stream) {
  sfb::TraceHeader* h = (sfb::TraceHeader*)dev;
  sfb::trace_mark_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(h, (sfb::TraceEvent*)((char*)dev + 64), scope_bit, tag, phase, aux);
  return (int)cudaGetLastError();
}

}  // extern "C"
