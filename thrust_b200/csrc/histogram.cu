// Second half of the sort-based dense histogram: for every bin value the
// upper bound in the sorted data (cumulative count), then the difference of
// neighbouring cumulative counts, fused in one kernel. 65 536 bins touch well
// under a megabyte; the sort that precedes it carries all the bytes.
#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kHistThreads = 256;

template <typename T>
__device__ __forceinline__ uint64_t upper_bound_dev(const T* __restrict__ data, uint64_t n, T x) {
  uint64_t lo = 0, hi = n;
  while (lo < hi) {
    const uint64_t mid = lo + ((hi - lo) >> 1);
    if (x < data[mid]) hi = mid; else lo = mid + 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(kHistThreads)
histogram_sorted_kernel(const T* __restrict__ data, uint64_t n, const T* __restrict__ bins, uint32_t num_bins,
                        uint32_t* __restrict__ counts) {
  __shared__ uint64_t s_ub[kHistThreads + 1];
  const uint32_t b = blockIdx.x * kHistThreads + threadIdx.x;
  uint64_t ub = 0;
  if (b < num_bins) ub = upper_bound_dev(data, n, bins[b]);
  s_ub[threadIdx.x + 1] = ub;
  if (threadIdx.x == 0) {
    const uint32_t first = blockIdx.x * kHistThreads;
    s_ub[0] = first == 0 ? 0 : upper_bound_dev(data, n, bins[first - 1]);
  }
  __syncthreads();
  if (b < num_bins) counts[b] = (uint32_t)(ub - s_ub[threadIdx.x]);
}

template <typename T>
int launch_hist(const void* d_sorted, uint64_t n, const void* d_bins, uint32_t num_bins, uint32_t* d_counts,
                cudaStream_t stream) {
  const unsigned grid = (num_bins + kHistThreads - 1) / kHistThreads;
  histogram_sorted_kernel<T><<<grid, kHistThreads, 0, stream>>>(static_cast<const T*>(d_sorted), n,
                                                                 static_cast<const T*>(d_bins), num_bins, d_counts);
  trace_mark(stream, kTraceHistogramSorted);
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_histogram_sorted(const void* d_sorted, uint64_t n, int dtype, const void* d_bin_values,
                                      uint32_t num_bins, uint32_t* d_counts, tb200_stream_t stream) {
  using namespace tb200;
  if (num_bins == 0) return TB200_OK;
  if (!d_bin_values || !d_counts || (n && !d_sorted)) return TB200_ERR_INVALID_ARGUMENT;
  switch (dtype) {
    case TB200_I32: return launch_hist<int32_t>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    case TB200_U32: return launch_hist<uint32_t>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    case TB200_I64: return launch_hist<long long>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    case TB200_U64: return launch_hist<unsigned long long>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    case TB200_F32: return launch_hist<float>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    case TB200_F64: return launch_hist<double>(d_sorted, n, d_bin_values, num_bins, d_counts, stream);
    default: return TB200_ERR_UNSUPPORTED;
  }
}
