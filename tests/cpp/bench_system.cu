// Times thrust::sort(thrust_b200::par.on(stream), ...) on 2^25 int32 keys, as a Thrust user calls
// it: the policy's scratch lease, every launch of the sort and the end-of-call status read-back
// are inside the timed region (CUDA events on the call's stream; the input is restored by a device
// copy outside them). Prints one JSON object. The reference's first example is this sort
// (README.md:42-54).
#include <thrust/copy.h>
#include <thrust/device_vector.h>
#include <thrust/sort.h>

#include <algorithm>
#include <cstdio>
#include <vector>

#include "thrust_b200/system.h"

int main() {
  namespace tb = thrust_b200;
  const size_t n = size_t(1) << 25;
  std::vector<int> h(n);
  unsigned long long x = 1337;
  for (size_t i = 0; i < n; ++i) {  // splitmix-style stream, seed 1337
    x += 0x9E3779B97F4A7C15ull;
    unsigned long long z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    h[i] = (int)(unsigned)(z ^ (z >> 31));
  }
  thrust::device_vector<int> d0(h.begin(), h.end()), d(n);
  cudaStream_t s;
  cudaStreamCreate(&s);
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  std::vector<float> ms;
  for (int i = 0; i < 13; ++i) {
    thrust::copy(thrust::cuda::par.on(s), d0.begin(), d0.end(), d.begin());
    cudaEventRecord(a, s);
    thrust::sort(tb::par.on(s), d.begin(), d.end());
    cudaEventRecord(b, s);
    cudaEventSynchronize(b);
    float t = 0;
    cudaEventElapsedTime(&t, a, b);
    if (i >= 3) ms.push_back(t);
  }
  std::sort(ms.begin(), ms.end());
  const bool sorted = thrust::is_sorted(d.begin(), d.end());
  const double med = ms[ms.size() / 2];
  std::printf("{\"value\": %.3f, \"unit\": \"Gkeys/s\", \"ms_median\": %.4f, \"ms_min\": %.4f, \"verified\": %s, "
              "\"api\": \"thrust::sort(thrust_b200::par.on(stream), first, last) incl. scratch lease and status read-back\"}\n",
              n / (med * 1e-3) / 1e9, med, (double)ms.front(), sorted ? "true" : "false");
  tb200_workspace_release_all();
  return sorted ? 0 : 1;
}
