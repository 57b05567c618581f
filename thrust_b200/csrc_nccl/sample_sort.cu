// The sharded sample sort behind one C entry point: sampling, splitters, bucket counts, the
// count matrix, the exchange and the final local sort. The kernels are those of
// libthrust_b200.so (stable multi-way partition, onesweep radix sort); this file is the host
// orchestration over an NCCL communicator plus two tiny kernels for the sample.
//
// Steps (all ranks run them in lock step; collectives on `stream`):
//   1. every rank takes a regular sample of kSamples keys of its (unsorted) shard;
//   2. all-gather of the samples, sort, and the keys at ranks (len / G) * r become the G - 1
//      splitters: identical on every rank;
//      When one key makes up a sixteenth of a rank's share of the sample or more, elements and
//      splitters are compared as (key, global index) pairs instead, so that the copies of one key
//      can be divided between ranks (in input order): the sample carries its global indices;
//   3. bucket sizes of the shard (one read of the keys); all-gather of the G x G matrix; every
//      rank reads it on the host, so all take the same decision about overflow and know where
//      their buckets land: rank r's bucket for rank b starts behind the buckets of ranks < r, which
//      keeps the received runs in source-rank order (equal keys keep their global order);
//   4. exchange: ONE partition pass that stores bucket b straight into rank b's output buffer
//      (peer pointers given), or a local partition followed by grouped ncclSend / ncclRecv;
//   5. one stable local sort of what arrived.
#include <nccl.h>

#include <cstdint>
#include <vector>

#include "thrust_b200_nccl.h"

namespace {

constexpr unsigned kSamples = 16384;  // per rank: the largest share exceeds the mean by ~1.3 % at eight ranks (5 % with 1024)

#define TB200_TRY(expr)          \
  do {                           \
    const int rc_ = (expr);      \
    if (rc_ != 0) return rc_;    \
  } while (0)
#define TB200_CUDA(expr)                        \
  do {                                          \
    const cudaError_t e_ = (expr);              \
    if (e_ != cudaSuccess) return (int)e_;      \
  } while (0)
#define TB200_NCCL(expr)                              \
  do {                                                \
    if ((expr) != ncclSuccess) return TB200_ERR_NCCL; \
  } while (0)

// sample i = the key at the mid-point of the i-th of `s` equal strides of the shard, with its
// index in the global sequence (out[0..kSamples) keys, out[kSamples..2 kSamples) indices)
__global__ void take_samples(const unsigned long long* keys, unsigned long long n, unsigned s, unsigned long long base,
                             unsigned long long* out) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= kSamples) return;
  if (i >= s) {  // shards shorter than the sample: pad with the largest pair (sorts behind everything)
    out[i] = ~0ull;
    out[kSamples + i] = ~0ull;
    return;
  }
  unsigned long long idx = (2ull * i + 1ull) * n / (2ull * s);
  if (idx > n - 1) idx = n - 1;
  out[i] = keys[idx];
  out[kSamples + i] = base + idx;
}

// all-gathered samples arrive as [rank][keys | indices]: split them into two rank-major arrays
__global__ void unzip_samples(const unsigned long long* gathered, unsigned nranks, unsigned long long* keys,
                              unsigned long long* index) {
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nranks * kSamples) return;
  const unsigned r = i / kSamples, j = i % kSamples;
  keys[i] = gathered[(size_t)r * 2 * kSamples + j];
  index[i] = gathered[(size_t)r * 2 * kSamples + kSamples + j];
}

// splitters (keys and indices) at ranks (total / nranks) * r of the sorted sample; *heaviest = the
// largest number of equal keys in the sample (one block)
__global__ void pick_splitters(const unsigned long long* sorted, const unsigned long long* index, unsigned total,
                               unsigned nranks, unsigned long long* out_keys, unsigned long long* out_index,
                               unsigned* heaviest) {
  const unsigned r = threadIdx.x + 1;
  if (r < nranks) {
    out_keys[r - 1] = sorted[(unsigned long long)r * total / nranks];
    out_index[r - 1] = index[(unsigned long long)r * total / nranks];
  }
  // run lengths: thread t starts at every run head it owns and walks the run
  unsigned best = 0;
  for (unsigned i = threadIdx.x; i < total; i += blockDim.x) {
    if (sorted[i] == ~0ull) continue;  // padding of short shards
    if (i == 0 || sorted[i - 1] != sorted[i]) {
      unsigned len = 1;
      while (i + len < total && sorted[i + len] == sorted[i]) ++len;
      if (len > best) best = len;
    }
  }
  atomicMax(heaviest, best);
}

size_t align_up(size_t v) { return (v + 255) / 256 * 256; }

struct Layout {
  size_t own, gathered, sample_keys, sample_index, splitters, splitter_index, counts, matrix, barrier, work, part_keys,
      part_vals, total;
};

// work: the scratch of whichever library call is running (sample sort, partition, final sort)
int layout(int nranks, uint64_t n, uint64_t capacity, bool push, Layout& l) {
  size_t sample_sort = 0, part = 0, final_sort = 0;
  TB200_TRY(tb200_radix_sort(nullptr, &sample_sort, nullptr, nullptr, (uint64_t)nranks * kSamples, TB200_U64, 8, 0, 0, 64, nullptr));
  if (push) TB200_TRY(tb200_partition_count(nullptr, &part, nullptr, n, TB200_U64, 4, nullptr, (uint32_t)(nranks - 1), nullptr, nullptr));
  else TB200_TRY(tb200_partition(nullptr, &part, nullptr, nullptr, nullptr, nullptr, n, TB200_U64, 4, nullptr, (uint32_t)(nranks - 1), nullptr, nullptr));
  TB200_TRY(tb200_radix_sort(nullptr, &final_sort, nullptr, nullptr, capacity, TB200_U64, 4, 0, 0, 64, nullptr));
  size_t work = sample_sort > part ? sample_sort : part;
  if (final_sort > work) work = final_sort;
  size_t at = 0;
  l.own = at; at += align_up(2 * kSamples * 8);
  l.gathered = at; at += align_up((size_t)nranks * 2 * kSamples * 8);
  l.sample_keys = at; at += align_up((size_t)nranks * kSamples * 8);
  l.sample_index = at; at += align_up((size_t)nranks * kSamples * 8);
  l.splitters = at; at += align_up((size_t)nranks * 8);
  l.splitter_index = at; at += align_up((size_t)nranks * 8);
  l.counts = at; at += align_up((size_t)nranks * 8);
  l.matrix = at; at += align_up((size_t)nranks * nranks * 8);
  l.barrier = at; at += 256;
  l.work = at; at += align_up(work);
  l.part_keys = at; at += push ? 0 : align_up((size_t)n * 8);
  l.part_vals = at; at += push ? 0 : align_up((size_t)n * 4);
  l.total = at;
  return TB200_OK;
}

}  // namespace

extern "C" int tb200_sample_sort(tb200_nccl_comm_t comm, int rank, int nranks, void* d_temp, size_t* temp_bytes,
                                 const void* d_keys, const void* d_vals, uint64_t n, void* d_keys_out, void* d_vals_out,
                                 uint64_t capacity, void* const* peer_keys, void* const* peer_vals,
                                 uint64_t* h_count_out, tb200_stream_t stream_) {
  if (temp_bytes == nullptr || nranks < 1 || nranks > 256 || rank < 0 || rank >= nranks) return TB200_ERR_INVALID_ARGUMENT;
  const bool push = peer_keys != nullptr;
  if (push && peer_vals == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  Layout l;
  TB200_TRY(layout(nranks, n, capacity, push, l));
  if (d_temp == nullptr) {
    *temp_bytes = l.total;
    return TB200_OK;
  }
  if (*temp_bytes < l.total) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256 || h_count_out == nullptr || (nranks > 1 && comm == nullptr))
    return TB200_ERR_INVALID_ARGUMENT;
  if (n > capacity && nranks == 1) return TB200_ERR_OVERFLOW;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  char* base = static_cast<char*>(d_temp);
  void* work = base + l.work;
  size_t work_bytes = l.part_keys - l.work;
  const unsigned long long* keys = static_cast<const unsigned long long*>(d_keys);

  if (nranks == 1) {  // nothing to exchange
    TB200_CUDA(cudaMemcpyAsync(d_keys_out, d_keys, n * 8, cudaMemcpyDeviceToDevice, stream));
    TB200_CUDA(cudaMemcpyAsync(d_vals_out, d_vals, n * 4, cudaMemcpyDeviceToDevice, stream));
    TB200_TRY(tb200_radix_sort(work, &work_bytes, d_keys_out, d_vals_out, n, TB200_U64, 4, 0, 0, 64, stream_));
    *h_count_out = n;
    return tb200_temp_status(work, stream_);
  }

  // 0: where this shard starts in the global sequence (the shards may differ in length)
  auto* counts = reinterpret_cast<uint64_t*>(base + l.counts);
  auto* matrix = reinterpret_cast<uint64_t*>(base + l.matrix);
  std::vector<uint64_t> mat((size_t)nranks * nranks);
  TB200_CUDA(cudaMemcpyAsync(counts, &n, sizeof(uint64_t), cudaMemcpyHostToDevice, stream));
  TB200_NCCL(ncclAllGather(counts, matrix, 1, ncclUint64, comm, stream));
  TB200_CUDA(cudaMemcpyAsync(mat.data(), matrix, (size_t)nranks * 8, cudaMemcpyDeviceToHost, stream));
  TB200_CUDA(cudaStreamSynchronize(stream));
  uint64_t index_base = 0;
  for (int r = 0; r < rank; ++r) index_base += mat[r];

  // 1, 2: sample -> splitters
  auto* own = reinterpret_cast<unsigned long long*>(base + l.own);
  auto* gathered = reinterpret_cast<unsigned long long*>(base + l.gathered);
  auto* sample_keys = reinterpret_cast<unsigned long long*>(base + l.sample_keys);
  auto* sample_index = reinterpret_cast<unsigned long long*>(base + l.sample_index);
  auto* splitters = reinterpret_cast<unsigned long long*>(base + l.splitters);
  auto* splitter_index = reinterpret_cast<unsigned long long*>(base + l.splitter_index);
  unsigned* heaviest = reinterpret_cast<unsigned*>(base + l.barrier) + 8;
  const unsigned s = n < kSamples ? (unsigned)n : kSamples;
  take_samples<<<(kSamples + 255) / 256, 256, 0, stream>>>(keys, n, s, index_base, own);
  TB200_CUDA(cudaGetLastError());
  TB200_NCCL(ncclAllGather(own, gathered, 2 * kSamples, ncclUint64, comm, stream));
  const unsigned total = (unsigned)nranks * kSamples;
  unzip_samples<<<(total + 255) / 256, 256, 0, stream>>>(gathered, (unsigned)nranks, sample_keys, sample_index);
  TB200_CUDA(cudaGetLastError());
  // stable, and the sample is rank-major and position-ascending: equal keys stay in index order
  TB200_TRY(tb200_radix_sort(work, &work_bytes, sample_keys, sample_index, total, TB200_U64, 8, 0, 0, 64, stream_));
  TB200_CUDA(cudaMemsetAsync(heaviest, 0, sizeof(unsigned), stream));
  pick_splitters<<<1, 256, 0, stream>>>(sample_keys, sample_index, total, (unsigned)nranks, splitters, splitter_index,
                                        heaviest);
  TB200_CUDA(cudaGetLastError());
  unsigned h_heaviest = 0;
  TB200_CUDA(cudaMemcpyAsync(&h_heaviest, heaviest, sizeof(unsigned), cudaMemcpyDeviceToHost, stream));
  TB200_CUDA(cudaStreamSynchronize(stream));
  // one key holds a sixteenth of a rank's share of the sample or more: compare (key, index) pairs
  const uint64_t* ties = (uint64_t)h_heaviest * 16 >= kSamples ? reinterpret_cast<const uint64_t*>(splitter_index) : nullptr;

  // 3: bucket sizes and the count matrix
  void* part_keys = base + l.part_keys;
  void* part_vals = base + l.part_vals;
  if (push) {
    TB200_TRY(tb200_partition_count_ties(work, &work_bytes, d_keys, n, TB200_U64, 4, splitters, ties,
                                         (uint32_t)(nranks - 1), index_base, counts, stream_));
  } else {
    TB200_TRY(tb200_partition_ties(work, &work_bytes, d_keys, d_vals, part_keys, part_vals, n, TB200_U64, 4, splitters,
                                   ties, (uint32_t)(nranks - 1), index_base, counts, stream_));
  }
  TB200_NCCL(ncclAllGather(counts, matrix, (size_t)nranks, ncclUint64, comm, stream));
  TB200_CUDA(cudaMemcpyAsync(mat.data(), matrix, mat.size() * 8, cudaMemcpyDeviceToHost, stream));
  TB200_CUDA(cudaStreamSynchronize(stream));
  // mat[r * nranks + b] = pairs rank r sends to rank b
  uint64_t worst = 0, mine = 0;
  for (int b = 0; b < nranks; ++b) {
    uint64_t in = 0;
    for (int r = 0; r < nranks; ++r) in += mat[(size_t)r * nranks + b];
    if (in > worst) worst = in;
    if (b == rank) mine = in;
  }
  if (worst > capacity) return TB200_ERR_OVERFLOW;  // the same on every rank: nobody has sent anything

  // 4: exchange
  if (push) {
    std::vector<void*> bk(nranks), bv(nranks);
    for (int b = 0; b < nranks; ++b) {
      uint64_t off = 0;  // the buckets of lower source ranks come first in b's buffer
      for (int r = 0; r < rank; ++r) off += mat[(size_t)r * nranks + b];
      bk[b] = static_cast<char*>(peer_keys[b]) + off * 8;
      bv[b] = static_cast<char*>(peer_vals[b]) + off * 4;
    }
    TB200_TRY(tb200_partition_scatter_ties(work, &work_bytes, d_keys, d_vals, n, TB200_U64, 4, splitters, ties,
                                           (uint32_t)(nranks - 1), index_base, bk.data(), bv.data(), stream_));
    // Every rank's stores have landed once every rank's partition kernel has finished: a
    // collective that each rank enters behind that kernel on its stream.
    int* flag = reinterpret_cast<int*>(base + l.barrier);
    TB200_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), stream));
    TB200_NCCL(ncclAllReduce(flag, flag, 1, ncclInt32, ncclSum, comm, stream));
  } else {
    TB200_NCCL(ncclGroupStart());
    uint64_t send_at = 0, recv_at = 0;
    for (int b = 0; b < nranks; ++b) {
      const uint64_t out = mat[(size_t)rank * nranks + b], in = mat[(size_t)b * nranks + rank];
      if (out) {
        TB200_NCCL(ncclSend(static_cast<char*>(part_keys) + send_at * 8, out, ncclUint64, b, comm, stream));
        TB200_NCCL(ncclSend(static_cast<char*>(part_vals) + send_at * 4, out, ncclUint32, b, comm, stream));
      }
      if (in) {
        TB200_NCCL(ncclRecv(static_cast<char*>(d_keys_out) + recv_at * 8, in, ncclUint64, b, comm, stream));
        TB200_NCCL(ncclRecv(static_cast<char*>(d_vals_out) + recv_at * 4, in, ncclUint32, b, comm, stream));
      }
      send_at += out;
      recv_at += in;
    }
    TB200_NCCL(ncclGroupEnd());
  }

  // 5: the runs arrived in source-rank order: one stable sort
  TB200_TRY(tb200_radix_sort(work, &work_bytes, d_keys_out, d_vals_out, mine, TB200_U64, 4, 0, 0, 64, stream_));
  *h_count_out = mine;
  return tb200_temp_status(work, stream_);
}
