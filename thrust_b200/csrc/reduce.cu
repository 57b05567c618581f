// thrust::reduce with thrust::plus on arithmetic types: one streaming read of the input.
//
// Replaces thrust::cuda_cub::detail::reduce_n_impl and the cub::DeviceReduce::Reduce call
// behind it (thrust/system/cuda/detail/reduce.h:930-1000). The accumulator has the type of
// `init` (reduce.h:1029-1062; sequential/reduce.h:43-62); integer sums wrap.
//
// One kernel: a resident grid of CTAs walks the input with 16-byte loads (four in flight per
// thread), every CTA leaves one partial in the scratch, and the last CTA to finish (atomic
// ticket) adds the partials in CTA order and `init`. The grid size depends only on n and on
// the device, and every partial is a fixed tree over fixed elements, so the result is
// reproducible from run to run; floating-point sums differ from the left-to-right order of
// the CPU systems only by rounding.
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kReduceThreads = 512;
constexpr int kReduceUnroll = 4;
constexpr int kReduceMaxCtas = 2048;

// 8- and 16-bit integers are summed in 32 bits and narrowed once (the same value modulo 2^width).
template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<uint8_t> { using type = unsigned; };
template <> struct AccOf<uint16_t> { using type = unsigned; };

template <typename T>
struct alignas(16) ReduceVec {
  T v[16 / sizeof(T)];
};

template <typename A>
__device__ __forceinline__ A cta_sum(A a, A* s_warp) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a += __shfl_down_sync(0xffffffffu, a, off);
  const unsigned lane = lane_id(), warp = threadIdx.x / kWarp;
  if (lane == 0) s_warp[warp] = a;
  __syncthreads();
  A t = A(0);
  if (warp == 0) {
    t = lane < kReduceThreads / kWarp ? s_warp[lane] : A(0);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += __shfl_down_sync(0xffffffffu, t, off);
  }
  __syncthreads();  // s_warp may be reused
  return t;         // valid in thread 0
}

template <typename T>
__global__ void __launch_bounds__(kReduceThreads)
reduce_kernel(const T* __restrict__ in, uint64_t n, T init, T* __restrict__ out, TempHeader* hdr,
              typename AccOf<T>::type* __restrict__ partials, int aligned) {
  using A = typename AccOf<T>::type;
  constexpr int VEC = 16 / sizeof(T);
  __shared__ A s_warp[kReduceThreads / kWarp];
  __shared__ unsigned s_last;

  A acc[kReduceUnroll];
#pragma unroll
  for (int u = 0; u < kReduceUnroll; ++u) acc[u] = A(0);

  constexpr uint64_t CHUNK = (uint64_t)kReduceThreads * VEC * kReduceUnroll;
  const uint64_t full_chunks = aligned ? n / CHUNK : 0;
  for (uint64_t c = blockIdx.x; c < full_chunks; c += gridDim.x) {
    const ReduceVec<T>* src = reinterpret_cast<const ReduceVec<T>*>(in + c * CHUNK);
    ReduceVec<T> v[kReduceUnroll];
#pragma unroll
    for (int u = 0; u < kReduceUnroll; ++u) v[u] = src[u * kReduceThreads + threadIdx.x];
#pragma unroll
    for (int u = 0; u < kReduceUnroll; ++u)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[u] += (A)v[u].v[j];
  }
  // remainder (and everything, when the pointer is not 16-byte aligned)
  for (uint64_t i = full_chunks * CHUNK + (uint64_t)blockIdx.x * kReduceThreads + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * kReduceThreads)
    acc[0] += (A)in[i];

  A a = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  a = cta_sum(a, s_warp);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = a;
    __threadfence();
    s_last = atomicAdd(&hdr->ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last CTA: partials in CTA order, thread t takes partials t, t + 512, ...
  A t = A(0);
  for (unsigned i = threadIdx.x; i < gridDim.x; i += kReduceThreads) t += __ldcg(&partials[i]);  // written by other CTAs: read through L2
  t = cta_sum(t, s_warp);
  if (threadIdx.x == 0) *out = (T)((A)init + t);
}

template <typename T>
int launch_reduce(void* d_temp, size_t* temp_bytes, const void* d_in, uint64_t n, const void* h_init, void* d_out,
                  cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  const size_t need = kHeaderBytes + (size_t)kReduceMaxCtas * sizeof(A);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (d_out == nullptr || (n && d_in == nullptr)) return TB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(d_out) % sizeof(T) || reinterpret_cast<uintptr_t>(d_in) % sizeof(T))
    return TB200_ERR_INVALID_ARGUMENT;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, kHeaderBytes, stream));
  T init = T(0);
  if (h_init) init = *static_cast<const T*>(h_init);
  int dev = 0, sms = 0, per_sm = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  TB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  TB200_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reduce_kernel<T>, kReduceThreads, 0));
  if (per_sm < 1) return TB200_ERR_UNSUPPORTED;
  constexpr uint64_t CHUNK = (uint64_t)kReduceThreads * (16 / sizeof(T)) * kReduceUnroll;
  uint64_t grid = (n + CHUNK - 1) / CHUNK;
  const uint64_t resident = (uint64_t)sms * per_sm;
  if (grid > resident) grid = resident;
  if (grid > (uint64_t)kReduceMaxCtas) grid = kReduceMaxCtas;
  if (grid == 0) grid = 1;  // n = 0: the result is init
  auto* hdr = static_cast<TempHeader*>(d_temp);
  auto* partials = reinterpret_cast<A*>(static_cast<char*>(d_temp) + kHeaderBytes);
  const int aligned = reinterpret_cast<uintptr_t>(d_in) % 16 == 0;
  reduce_kernel<T><<<(unsigned)grid, kReduceThreads, 0, stream>>>(static_cast<const T*>(d_in), n, init,
                                                                  static_cast<T*>(d_out), hdr, partials, aligned);
  trace_mark(stream, kTraceReduce);
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_reduce(void* d_temp, size_t* temp_bytes, const void* d_in, uint64_t n, int dtype,
                            const void* h_init, void* d_out, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  switch (dtype) {
    // signed integers are summed as unsigned: two's-complement addition is the same operation
    case TB200_I8: case TB200_U8: return launch_reduce<uint8_t>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    case TB200_I16: case TB200_U16: return launch_reduce<uint16_t>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    case TB200_I32: case TB200_U32: return launch_reduce<uint32_t>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    case TB200_I64: case TB200_U64:
      return launch_reduce<unsigned long long>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    case TB200_F32: return launch_reduce<float>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    case TB200_F64: return launch_reduce<double>(d_temp, temp_bytes, d_in, n, h_init, d_out, stream);
    default: return TB200_ERR_UNSUPPORTED;
  }
}
