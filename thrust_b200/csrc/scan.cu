// Single-pass prefix sum (inclusive / exclusive, plus) with a decoupled look-back
// chain of tile descriptors. Streaming kernel: 1 read + 1 write per element, no
// tensor cores (nothing here is a contraction).
//
// Data layout of one tile (kThreads * kVecs 16-byte vectors): warp w owns a
// contiguous slice; inside the slice lane l holds vectors l, l+32, l+64, ... so
// that every load/store instruction of a warp touches 512 contiguous bytes.
// Order of summation: left to right inside a vector, Kogge-Stone across the
// lanes of a warp, left to right across warps and tiles. Integer results are
// exact (two's complement wrap); floating-point results differ from a strictly
// sequential sum only by re-association.
#include "common.cuh"

#include <mutex>

namespace tb200 {
namespace {

// 512 threads x 8 vectors = 64 KiB per tile. Large tiles keep the number of tiles
// per microsecond (about 50 at full HBM speed) well below what the look-back chain
// can resolve: a warp inspects 64 predecessors per L2 round trip.
constexpr int kScanThreads = 512;
constexpr int kScanWarps = kScanThreads / kWarp;
constexpr int kScanVecs = 8;  // 16-byte vectors per thread

template <typename T>
struct alignas(16) Vec16 {
  T v[16 / sizeof(T)];
};

template <typename T>
struct Words {
  static constexpr int W = sizeof(T) / 4;
  __device__ static void pack(T x, unsigned (&p)[W]) {
    if constexpr (W == 1) {
      p[0] = __builtin_bit_cast(unsigned, x);
    } else {
      unsigned long long b = __builtin_bit_cast(unsigned long long, x);
      p[0] = (unsigned)b;
      p[1] = (unsigned)(b >> 32);
    }
  }
  __device__ static T unpack(const unsigned (&p)[W]) {
    if constexpr (W == 1) {
      return __builtin_bit_cast(T, p[0]);
    } else {
      return __builtin_bit_cast(T, ((unsigned long long)p[1] << 32) | p[0]);
    }
  }
};

// Warp 0 walks back over predecessor descriptors, 64 at a time (two per lane,
// both loads in flight together), until it meets one that carries a full prefix.
// Returns the sum of everything before `tile`.
template <typename T>
__device__ T lookback_sum(const TileWords<Words<T>::W>* tiles, unsigned tile, int* status) {
  constexpr int W = Words<T>::W;
  const unsigned lane = lane_id();
  T acc = T(0);
  long long base = (long long)tile - 1;
  bool timed_out = false;
  while (true) {
    // slot s = 0 is the nearer half of the window (tiles base-lane), s = 1 the farther one
    unsigned st[2] = {kStatePrefix, kStatePrefix};
    T val[2] = {T(0), T(0)};
    unsigned payload[2][W];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const long long idx = base - 32 * s - lane;
      if (idx >= 0) st[s] = peek<W>(&tiles[idx], payload[s]);
    }
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const long long idx = base - 32 * s - lane;
      if (idx >= 0) {
        unsigned polls = 0;
        while (st[s] == kStateEmpty) {
          backoff(++polls);
          if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(status) != 0)) {
            timed_out = true;
            st[s] = kStatePrefix;
            break;
          }
          st[s] = peek<W>(&tiles[idx], payload[s]);
        }
        val[s] = timed_out ? T(0) : Words<T>::unpack(payload[s]);
      }
    }
    bool found = false;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (found) break;
      const unsigned pm = __ballot_sync(0xffffffffu, st[s] == kStatePrefix);
      const unsigned first = pm ? (unsigned)(__ffs(pm) - 1) : 31u;
      T v = lane > first ? T(0) : val[s];
      // far predecessors (high lanes) are summed before near ones
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        T o = __shfl_down_sync(0xffffffffu, v, off);
        if (lane + off < 32) v = o + v;
      }
      v = __shfl_sync(0xffffffffu, v, 0);
      acc = v + acc;
      found = pm != 0;
    }
    if (found) break;
    base -= 64;
  }
  if (__any_sync(0xffffffffu, timed_out) && lane == 0) atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
  return acc;
}

template <typename T, bool EXCLUSIVE, bool ALIGNED>
__global__ void __launch_bounds__(kScanThreads, 2)
scan_kernel(const T* in, T* out, uint64_t n, T init, TempHeader* hdr,
            TileWords<Words<T>::W>* tiles) {
  constexpr int W = Words<T>::W;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int K = kScanVecs;
  constexpr int WARP_ITEMS = kWarp * K * VEC;
  constexpr int TILE = kScanThreads * K * VEC;

  __shared__ unsigned s_tile;
  __shared__ T s_warp_total[kScanWarps];
  __shared__ T s_tile_prefix;

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const unsigned tile = s_tile;
  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  const uint64_t tile_base = (uint64_t)tile * TILE;
  const uint64_t warp_base = tile_base + (uint64_t)warp * WARP_ITEMS;
  const bool full = tile_base + TILE <= n;

  T x[K][VEC];
  if (ALIGNED && full) {
    const Vec16<T>* src = reinterpret_cast<const Vec16<T>*>(in + warp_base);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      Vec16<T> v = src[k * kWarp + lane];
#pragma unroll
      for (int j = 0; j < VEC; ++j) x[k][j] = v.v[j];
    }
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const uint64_t i = warp_base + (uint64_t)(k * kWarp + lane) * VEC + j;
        x[k][j] = i < n ? in[i] : T(0);
      }
  }

  // inclusive sums inside each vector, then across the lanes of the warp
  T excl[K];
  T carry = T(0);
#pragma unroll
  for (int k = 0; k < K; ++k) {
#pragma unroll
    for (int j = 1; j < VEC; ++j) x[k][j] = x[k][j - 1] + x[k][j];
    T s = x[k][VEC - 1];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      T t = __shfl_up_sync(0xffffffffu, s, off);
      if (lane >= off) s = t + s;
    }
    T e = __shfl_up_sync(0xffffffffu, s, 1);
    if (lane == 0) e = T(0);
    excl[k] = carry + e;
    carry = carry + __shfl_sync(0xffffffffu, s, 31);
  }
  if (lane == 31) s_warp_total[warp] = carry;
  __syncthreads();

  T warp_prefix = T(0), tile_total = T(0);
#pragma unroll
  for (int w = 0; w < kScanWarps; ++w) {
    const T t = s_warp_total[w];
    if (w < (int)warp) warp_prefix = warp_prefix + t;
    tile_total = tile_total + t;
  }

  if (warp == 0) {
    unsigned payload[W];
    T prefix;
    if (tile == 0) {
      prefix = EXCLUSIVE ? init : T(0);
      if (lane == 0) {
        Words<T>::pack(prefix + tile_total, payload);
        publish<W>(&tiles[0], kStatePrefix, payload);
      }
    } else {
      if (lane == 0) {
        Words<T>::pack(tile_total, payload);
        publish<W>(&tiles[tile], kStateAggregate, payload);
      }
      prefix = lookback_sum<T>(tiles, tile, &hdr->status);
      if (lane == 0) {
        Words<T>::pack(prefix + tile_total, payload);
        publish<W>(&tiles[tile], kStatePrefix, payload);
      }
    }
    if (lane == 0) s_tile_prefix = prefix;
  }
  __syncthreads();
  const T base = s_tile_prefix + warp_prefix;

  if (ALIGNED && full) {
    Vec16<T>* dst = reinterpret_cast<Vec16<T>*>(out + warp_base);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const T p = base + excl[k];
      Vec16<T> v;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        if (EXCLUSIVE) v.v[j] = j == 0 ? p : p + x[k][j - 1];
        else           v.v[j] = p + x[k][j];
      }
      dst[k * kWarp + lane] = v;
    }
  } else {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const T p = base + excl[k];
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const uint64_t i = warp_base + (uint64_t)(k * kWarp + lane) * VEC + j;
        T r;
        if (EXCLUSIVE) r = j == 0 ? p : p + x[k][j - 1];
        else           r = p + x[k][j];
        if (i < n) out[i] = r;
      }
    }
  }
}

template <typename T>
int launch_scan(void* d_temp, size_t* temp_bytes, const void* d_in, void* d_out, uint64_t n,
                int exclusive, const void* h_init, cudaStream_t stream) {
  constexpr int W = Words<T>::W;
  constexpr uint64_t TILE = (uint64_t)kScanThreads * kScanVecs * (16 / sizeof(T));
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const size_t need = kHeaderBytes + (size_t)tiles * sizeof(TileWords<W>);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  if (n == 0) return TB200_OK;
  if (d_in == nullptr || d_out == nullptr) return TB200_ERR_INVALID_ARGUMENT;

  T init = T(0);
  if (exclusive && h_init) init = *static_cast<const T*>(h_init);
  auto* hdr = static_cast<TempHeader*>(d_temp);
  auto* desc = reinterpret_cast<TileWords<W>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  const T* in = static_cast<const T*>(d_in);
  T* out = static_cast<T*>(d_out);
  const bool aligned = ((reinterpret_cast<uintptr_t>(d_in) | reinterpret_cast<uintptr_t>(d_out)) % 16) == 0;
  const dim3 grid((unsigned)tiles), block(kScanThreads);
  if (exclusive) {
    if (aligned) scan_kernel<T, true, true><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
    else         scan_kernel<T, true, false><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
  } else {
    if (aligned) scan_kernel<T, false, true><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
    else         scan_kernel<T, false, false><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
  }
  trace_mark(stream);
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_scan(void* d_temp, size_t* temp_bytes, const void* d_in, void* d_out, uint64_t n,
                          int dtype, int exclusive, const void* h_init, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  switch (dtype) {
    // signed integers wrap like unsigned ones in two's complement
    case TB200_I32: case TB200_U32:
      return launch_scan<uint32_t>(d_temp, temp_bytes, d_in, d_out, n, exclusive, h_init, stream);
    case TB200_I64: case TB200_U64:
      return launch_scan<unsigned long long>(d_temp, temp_bytes, d_in, d_out, n, exclusive, h_init, stream);
    case TB200_F32:
      return launch_scan<float>(d_temp, temp_bytes, d_in, d_out, n, exclusive, h_init, stream);
    case TB200_F64:
      return launch_scan<double>(d_temp, temp_bytes, d_in, d_out, n, exclusive, h_init, stream);
    default:
      return TB200_ERR_UNSUPPORTED;
  }
}

// ---------------------------------------------------------------------------------------
// tb200_scan_static: the same scan, with its scratch in a fixed device array
// ---------------------------------------------------------------------------------------
namespace tb200 {
namespace {

// Look-back descriptors of tb200_scan_static. Lives in every GPU that loads this library,
// from load until the process exits. 1 MiB + header: up to 131072 tiles of a 4-byte type
// (n <= 2^31 elements) or 65536 tiles of an 8-byte type (n <= 2^29 elements).
constexpr size_t kStaticScanBytes = kHeaderBytes + (1u << 20);
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_scan_mutex;
void* g_static_scan_ptr[kMaxDevices] = {};

// In host code `g_static_scan_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up once per device, with that device current.
int static_scan_scratch(void** out) {
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return TB200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_scan_mutex);
  if (g_static_scan_ptr[dev] == nullptr) {
    void* p = nullptr;
    TB200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scan_scratch));
    g_static_scan_ptr[dev] = p;
  }
  *out = g_static_scan_ptr[dev];
  return TB200_OK;
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_scan_static(const void* d_in, void* d_out, uint64_t n, int dtype, int exclusive,
                                 const void* h_init, tb200_stream_t stream) {
  using namespace tb200;
  size_t need = 0;
  int rc = tb200_scan(nullptr, &need, nullptr, nullptr, n, dtype, exclusive, h_init, stream);
  if (rc) return rc;
  if (need > kStaticScanBytes) return TB200_ERR_OVERFLOW;  // n beyond the fixed scratch: use tb200_scan
  void* scratch = nullptr;
  rc = static_scan_scratch(&scratch);
  if (rc) return rc;
  size_t have = kStaticScanBytes;
  // tb200_scan clears the part of the scratch it uses (header and descriptors) on `stream`
  // before the kernel, so what the previous call left behind is never read.
  return tb200_scan(scratch, &have, d_in, d_out, n, dtype, exclusive, h_init, stream);
}
