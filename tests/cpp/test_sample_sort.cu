// tb200_sample_sort called from C++ the way an application would (include/thrust_b200_nccl.h):
// size query, scratch from cudaMalloc, one call, result compared with std::stable_sort. One rank,
// so no communicator is needed; the multi-rank forms are covered by tests/test_sample_sort_c_gpu.py.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <numeric>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "thrust_b200_nccl.h"

#define CHECK(x)                                                      \
  do {                                                                \
    const int rc_ = (int)(x);                                         \
    if (rc_ != 0) {                                                   \
      std::printf("FAILED %s -> %d (%s:%d)\n", #x, rc_, __FILE__, __LINE__); \
      return 1;                                                       \
    }                                                                 \
  } while (0)

int main() {
  const uint64_t n = 300007;
  std::mt19937_64 rng(7);
  std::vector<uint64_t> keys(n);
  std::vector<uint32_t> vals(n);
  for (uint64_t i = 0; i < n; ++i) keys[i] = rng() >> 52;  // 4096 distinct keys: stability is visible
  std::iota(vals.begin(), vals.end(), 0u);
  void *dk, *dv, *ok, *ov, *temp;
  CHECK(cudaMalloc(&dk, n * 8));
  CHECK(cudaMalloc(&dv, n * 4));
  CHECK(cudaMalloc(&ok, n * 8));
  CHECK(cudaMalloc(&ov, n * 4));
  CHECK(cudaMemcpy(dk, keys.data(), n * 8, cudaMemcpyHostToDevice));
  CHECK(cudaMemcpy(dv, vals.data(), n * 4, cudaMemcpyHostToDevice));
  size_t bytes = 0;
  CHECK(tb200_sample_sort(nullptr, 0, 1, nullptr, &bytes, nullptr, nullptr, n, nullptr, nullptr, n, nullptr, nullptr,
                          nullptr, nullptr));
  CHECK(cudaMalloc(&temp, bytes));
  uint64_t count = 0;
  CHECK(tb200_sample_sort(nullptr, 0, 1, temp, &bytes, dk, dv, n, ok, ov, n, nullptr, nullptr, &count, nullptr));
  std::vector<uint64_t> gk(n);
  std::vector<uint32_t> gv(n);
  CHECK(cudaMemcpy(gk.data(), ok, n * 8, cudaMemcpyDeviceToHost));
  CHECK(cudaMemcpy(gv.data(), ov, n * 4, cudaMemcpyDeviceToHost));
  std::vector<uint32_t> order(n);
  std::iota(order.begin(), order.end(), 0u);
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return keys[a] < keys[b]; });
  if (count != n) {
    std::printf("FAILED count %llu\n", (unsigned long long)count);
    return 1;
  }
  for (uint64_t i = 0; i < n; ++i) {
    if (gk[i] != keys[order[i]] || gv[i] != order[i]) {
      std::printf("FAILED at %llu\n", (unsigned long long)i);
      return 1;
    }
  }
  std::printf("PASSED tb200_sample_sort on one rank: %llu pairs\n", (unsigned long long)n);
  return 0;
}
