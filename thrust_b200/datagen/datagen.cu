// Counter-based input generators, identical on host and device (see datagen.h), and the
// reference-free checker of sorted hashed pairs. Test and benchmark support: built into its own
// library (libtb200_datagen.so), not into the algorithm library.
#include "../csrc/common.cuh"
#include "datagen.h"

namespace tb200 {
namespace {

__host__ __device__ inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t hash64(uint64_t seed, uint64_t i) {
  return mix64(mix64(seed + 0x9E3779B97F4A7C15ull) + (i + 1) * 0x9E3779B97F4A7C15ull);
}

struct GenArgs {
  float flo, fhi;
  long long ilo, ihi;
  unsigned period;
  const double* cdf;
  unsigned cdf_len;
};

template <typename F>
__global__ void gen_kernel(uint64_t n, F f) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) f(i);
}

__host__ __device__ inline void gen_one(void* out, uint64_t j, uint64_t i, int kind, uint64_t seed,
                                        const GenArgs& a) {
  const uint64_t h = hash64(seed, i);
  switch (kind) {
    case TB200_GEN_BITS_U32: static_cast<uint32_t*>(out)[j] = (uint32_t)h; break;
    case TB200_GEN_BITS_U64: static_cast<uint64_t*>(out)[j] = h; break;
    case TB200_GEN_INDEX_U32: static_cast<uint32_t*>(out)[j] = (uint32_t)i; break;
    case TB200_GEN_UNIFORM_F32: {
      const float u = (float)(h >> 40) * (1.0f / 16777216.0f);  // 24 bits -> [0, 1)
      static_cast<float*>(out)[j] = a.flo + (a.fhi - a.flo) * u;
      break;
    }
    case TB200_GEN_UNIFORM_I64: {
      const uint64_t span = (uint64_t)(a.ihi - a.ilo) + 1;
      static_cast<long long*>(out)[j] = a.ilo + (long long)(h % span);
      break;
    }
    case TB200_GEN_HEAD_FLAGS_I32:
      static_cast<int*>(out)[j] = (i == 0 || h % a.period == 0) ? 1 : 0;
      break;
    case TB200_GEN_AND3_F32: {
      uint32_t w = 0;
      for (uint64_t attempt = 0; attempt < 64; ++attempt) {
        const uint64_t h1 = hash64(seed ^ (0xA5A5A5A5ull + attempt), i);
        const uint64_t h2 = hash64(seed + 0x51ED27ull + (attempt << 32), i);
        w = (uint32_t)h1 & (uint32_t)(h1 >> 32) & (uint32_t)h2;
        const bool is_nan = ((w >> 23) & 0xffu) == 0xffu && (w & 0x7fffffu) != 0;
        if (!is_nan) break;
        w = 0;
      }
      static_cast<uint32_t*>(out)[j] = w;
      break;
    }
    case TB200_GEN_ZIPF_RANK_U32: {
      const double u = (double)(h >> 11) * (1.0 / 9007199254740992.0);  // 53 bits -> [0, 1)
      unsigned lo = 0, hi = a.cdf_len - 1;  // first rank with cdf[r] > u
      while (lo < hi) {
        const unsigned mid = (lo + hi) >> 1;
        if (a.cdf[mid] > u) hi = mid; else lo = mid + 1;
      }
      static_cast<uint32_t*>(out)[j] = lo;
      break;
    }
    default: break;
  }
}

// Reference-free check of a sorted shard of (hash key, index value) pairs.
// result[0] order violations, [1] pairing violations, [2] sum of recovered global
// indices (mod 2^64), [3] number of pairs checked.
__global__ void check_pairs_kernel(const uint64_t* __restrict__ keys, const uint32_t* __restrict__ vals, uint64_t n,
                                   uint64_t seed, uint64_t total, unsigned long long* __restrict__ result) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const unsigned wraps = (unsigned)((total + 0xffffffffull) >> 32);
  auto recover = [&](uint64_t key, uint32_t v, bool& found) {
    found = false;
    for (unsigned c = 0; c < wraps; ++c) {
      const uint64_t gidx = ((uint64_t)c << 32) | v;
      if (gidx < total && hash64(seed, gidx) == key) { found = true; return gidx; }
    }
    return (uint64_t)0;
  };
  unsigned long long bad_order = 0, bad_pair = 0, sum = 0, cnt = 0;
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
    const uint64_t k = keys[j];
    bool found;
    const uint64_t gi = recover(k, vals[j], found);
    if (!found) ++bad_pair;
    sum += gi;
    ++cnt;
    if (j > 0) {
      const uint64_t kp = keys[j - 1];
      if (kp > k) ++bad_order;
      else if (kp == k) {
        bool fp;
        const uint64_t gp = recover(kp, vals[j - 1], fp);
        if (fp && found && !(gp < gi)) ++bad_order;
      }
    }
  }
  if (bad_order) atomicAdd(&result[0], bad_order);
  if (bad_pair) atomicAdd(&result[1], bad_pair);
  atomicAdd(&result[2], sum);
  atomicAdd(&result[3], cnt);
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_check_hashed_pairs(const void* d_keys, const void* d_vals, uint64_t n, uint64_t seed,
                                        uint64_t total, uint64_t* d_result4, tb200_stream_t stream) {
  using namespace tb200;
  if (!d_result4) return TB200_ERR_INVALID_ARGUMENT;
  TB200_CUDA_TRY(cudaMemsetAsync(d_result4, 0, 4 * sizeof(uint64_t), stream));
  if (n == 0) return TB200_OK;
  if (!d_keys || !d_vals) return TB200_ERR_INVALID_ARGUMENT;
  int dev = 0, sms = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  TB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  check_pairs_kernel<<<sms * 8, 256, 0, stream>>>(static_cast<const uint64_t*>(d_keys),
                                                  static_cast<const uint32_t*>(d_vals), n, seed, total,
                                                  reinterpret_cast<unsigned long long*>(d_result4));
  return (int)cudaGetLastError();
}

extern "C" uint64_t tb200_datagen_hash(uint64_t seed, uint64_t i) { return tb200::hash64(seed, i); }

extern "C" int tb200_datagen(void* out, uint64_t n, uint64_t first_index, int kind, uint64_t seed,
                             const void* aux, uint32_t aux_len, int on_device, tb200_stream_t stream) {
  using namespace tb200;
  if (n == 0) return TB200_OK;
  if (out == nullptr || kind < 0 || kind > TB200_GEN_ZIPF_RANK_U32) return TB200_ERR_INVALID_ARGUMENT;
  GenArgs a{};
  switch (kind) {
    case TB200_GEN_UNIFORM_F32:
      if (!aux) return TB200_ERR_INVALID_ARGUMENT;
      a.flo = static_cast<const float*>(aux)[0];
      a.fhi = static_cast<const float*>(aux)[1];
      break;
    case TB200_GEN_UNIFORM_I64:
      if (!aux) return TB200_ERR_INVALID_ARGUMENT;
      a.ilo = static_cast<const long long*>(aux)[0];
      a.ihi = static_cast<const long long*>(aux)[1];
      if (a.ihi < a.ilo) return TB200_ERR_INVALID_ARGUMENT;
      break;
    case TB200_GEN_HEAD_FLAGS_I32:
      if (!aux) return TB200_ERR_INVALID_ARGUMENT;
      a.period = static_cast<const unsigned*>(aux)[0];
      if (a.period == 0) return TB200_ERR_INVALID_ARGUMENT;
      break;
    case TB200_GEN_ZIPF_RANK_U32:
      if (!aux || aux_len == 0) return TB200_ERR_INVALID_ARGUMENT;
      a.cdf = static_cast<const double*>(aux);
      a.cdf_len = aux_len;
      break;
    default: break;
  }
  if (on_device) {
    int dev = 0, sms = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    TB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const uint64_t want = (n + 255) / 256;
    const unsigned grid = (unsigned)(want < (uint64_t)sms * 16 ? want : (uint64_t)sms * 16);
    gen_kernel<<<grid, 256, 0, stream>>>(n, [=] __device__(uint64_t j) {
      gen_one(out, j, first_index + j, kind, seed, a);
    });
    return (int)cudaGetLastError();
  }
#pragma omp parallel for schedule(static)
  for (long long j = 0; j < (long long)n; ++j) gen_one(out, (uint64_t)j, first_index + (uint64_t)j, kind, seed, a);
  return TB200_OK;
}
