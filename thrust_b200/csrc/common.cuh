// Shared device/host helpers of the thrust_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/thrust_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "thrust_b200 kernels are written for sm_100a only"
#endif

namespace tb200 {

constexpr int kWarp = 32;

// Every spin on another CTA's tile descriptor gives up after this many polls
// (with nanosleep back-off this is on the order of a second), raises the status
// word and lets the CTA finish without waiting again.
constexpr unsigned kSpinLimit = 1u << 22;

// Layout of the first 256 bytes of every scratch buffer.
struct TempHeader {
  int status;            // 0 or a tb200_error, written by kernels
  unsigned ticket;       // dynamic tile counter of single-kernel algorithms
  // aux[0..3]: where the first bounded wait gave up (note_timeout); aux[4..7]: shared-memory addresses of the
  // by-key kernel's mbarrier arrays (decode a recorded mbarrier time-out); aux[8]: the scouts' ticket counter
  unsigned long long aux[30];
};
static_assert(sizeof(TempHeader) <= 256, "header must fit the first 256 bytes");
constexpr size_t kHeaderBytes = 256;

__host__ __device__ constexpr size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ inline int dtype_bytes(int dt) {
  switch (dt) {
    case TB200_I8: case TB200_U8: case TB200_BOOL: return 1;
    case TB200_I16: case TB200_U16: return 2;
    case TB200_I32: case TB200_U32: case TB200_F32: return 4;
    case TB200_I64: case TB200_U64: case TB200_F64: return 8;
    default: return 0;
  }
}

// Launch tracing (tb200_trace_begin / tb200_trace_end): when the calling thread has
// tracing on, every kernel launch of the library is followed by an event record, so
// a benchmark can read per-launch device times without a profiler. Off by default.
enum TraceKind { kTraceOther = 0, kTraceSortHistogram = 1, kTraceSortPass = 2, kTraceSortCopyBack = 3, kTraceScan = 4,
                 kTraceReduceByKey = 5, kTraceHistogramSorted = 6, kTracePartitionHistogram = 7, kTracePartitionPass = 8, kTraceReduce = 9,
                 kTraceScanByKey = 10, kTraceUniqueByKey = 11, kTraceCopyFlagged = 12 };
void trace_mark(cudaStream_t stream, int kind = kTraceOther);

#define TB200_CUDA_TRY(expr)                       \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) return (int)_e;         \
  } while (0)

#ifdef __CUDACC__

__device__ __forceinline__ unsigned lane_id() {
  unsigned r;
  asm("mov.u32 %0, %%laneid;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned r;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(r));
  return r;
}

// Relaxed, gpu-scope 64-bit accesses: single-copy atomic, never cached in L1.
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_s32(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Raises the status word after a bounded wait ran out and records where: the FIRST wait to give
// up writes aux[0] = site, aux[1..2] = what it waited for, aux[3] = CTA | thread << 32 of the
// scratch header (every later time-out is a consequence of the first).
enum : unsigned { kSiteLookback = 1, kSiteBlockChain = 2, kSiteIdle = 4, kSiteMbarrier = 5 };
__device__ __forceinline__ void note_timeout(int* status, unsigned site, unsigned long long x, unsigned long long y) {
  unsigned long long* aux = reinterpret_cast<unsigned long long*>(status) + 1;  // TempHeader::aux
  if (atomicCAS(&aux[0], 0ull, (unsigned long long)site) == 0ull) {
    aux[1] = x;
    aux[2] = y;
    aux[3] = (unsigned long long)blockIdx.x | ((unsigned long long)threadIdx.x << 32);
  }
  atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
}

__device__ __forceinline__ void backoff(unsigned polls) {
  // a short sleep from the first retry on: tight polling of the few descriptor lines that
  // every look-back reads delays the very stores it is waiting for
  __nanosleep(polls > 256 ? 400 : 100);
}

// Tile descriptors of the decoupled look-back chains. A descriptor is W 64-bit
// words; each word carries {state:32 | payload:32}. A writer stores the words one
// by one with relaxed 8-byte stores; a reader accepts a descriptor only when all
// W words show the same state. States only move forward (EMPTY -> AGGREGATE ->
// PREFIX) and each word is written once per state, so equal states imply that the
// W payloads belong together. No fences are needed.
enum : unsigned { kStateEmpty = 0, kStateAggregate = 1, kStatePrefix = 2 };

template <int W>
struct alignas(W == 1 ? 8 : (W == 2 ? 16 : 32)) TileWords {
  unsigned long long w[W];
};

template <int W>
__device__ __forceinline__ void publish(TileWords<W>* d, unsigned state, const unsigned (&payload)[W]) {
#pragma unroll
  for (int i = 0; i < W; ++i)
    st_relaxed_u64(&d->w[i], ((unsigned long long)state << 32) | payload[i]);
}

// Returns the common state (kStateEmpty if the words disagree or are empty).
template <int W>
__device__ __forceinline__ unsigned peek(const TileWords<W>* d, unsigned (&payload)[W]) {
  unsigned long long v[W];
  if constexpr (W == 2) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "l"(d) : "memory");
  } else if constexpr (W == 4) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "l"(d) : "memory");
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(v[2]), "=l"(v[3]) : "l"(&d->w[2]) : "memory");
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = ld_relaxed_u64(&d->w[i]);
  }
  unsigned st = (unsigned)(v[0] >> 32);
  bool same = true;
#pragma unroll
  for (int i = 0; i < W; ++i) {
    payload[i] = (unsigned)v[i];
    same = same && ((unsigned)(v[i] >> 32) == st);
  }
  return same ? st : kStateEmpty;
}

// ---- bulk asynchronous copies (the TMA engine's untiled form) and their mbarriers -------
// One elected thread issues a global -> shared copy of a whole tile; the data lands without
// occupying registers or load-store slots and completion is signalled on an mbarrier.
// Source, destination and size must be multiples of 16 bytes. Never used with multicast.
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Orders earlier generic-proxy accesses to shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Barrier among the first `count` threads of the CTA (count a multiple of 32), id 1..15.
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for a bulk load. Returns false (after raising the status word) if the data
// did not arrive within the limit; the caller carries on without waiting again.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity, int* status) {
  for (unsigned spins = 0; spins < (1u << 20); ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 1023u) == 1023u && ld_relaxed_s32(status) != 0) return false;  // someone else gave up
  }
  note_timeout(status, kSiteMbarrier, smem_u32(bar), parity);
  return false;
}

#endif  // __CUDACC__

}  // namespace tb200
