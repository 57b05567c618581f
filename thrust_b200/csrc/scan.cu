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
constexpr int kScanMinCtas = 2;
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

// Warp 0 walks back over predecessor descriptors, 32 * kLookSlots at a time (kLookSlots
// per lane, all loads in flight together), until it meets one that carries a full prefix.
// Returns the sum of everything before `tile`.
constexpr int kLookSlots = 1;
template <typename T>
__device__ T lookback_sum(const TileWords<Words<T>::W>* tiles, unsigned tile, int* status) {
  constexpr int W = Words<T>::W;
  const unsigned lane = lane_id();
  T acc = T(0);
  long long base = (long long)tile - 1;
  bool timed_out = false;
  while (true) {
    // slot 0 is the nearest part of the window (tiles base-lane), higher slots lie farther
    // back. All loads are issued first; slots are then consumed nearest first and the
    // walk stops at the first prefix, so descriptors behind it are never waited for.
    unsigned st[kLookSlots];
    unsigned payload[kLookSlots][W];
#pragma unroll
    for (int s = 0; s < kLookSlots; ++s) {
      const long long idx = base - 32 * s - lane;
      st[s] = kStatePrefix;
      if (idx >= 0) st[s] = peek<W>(&tiles[idx], payload[s]);
    }
    bool found = false;
#pragma unroll
    for (int s = 0; s < kLookSlots; ++s) {
      if (found) break;
      const long long idx = base - 32 * s - lane;
      T v = T(0);
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
        v = timed_out ? T(0) : Words<T>::unpack(payload[s]);
      }
      const unsigned pm = __ballot_sync(0xffffffffu, st[s] == kStatePrefix);
      const unsigned first = pm ? (unsigned)(__ffs(pm) - 1) : 31u;
      if (lane > first) v = T(0);
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
    base -= 32 * kLookSlots;
  }
  if (__any_sync(0xffffffffu, timed_out) && lane == 0) atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
  return acc;
}

template <typename T, bool EXCLUSIVE, bool ALIGNED>
__global__ void __launch_bounds__(kScanThreads, kScanMinCtas)
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
      prefix = init;  // the seed: in front of the first element in both forms
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

// ---------------------------------------------------------------------------------------
// Streaming variant (16-byte aligned input and output): persistent CTAs, one per SM, each
// with 16 compute warps and one look-back warp.
//  * a ring of (park + 2) tiles in shared memory is filled by bulk asynchronous copies
//    (one elected thread, completion on an mbarrier), issued one to two tiles ahead of use;
//  * the compute warps scan tile i locally — thread t owns a contiguous run of the tile, so
//    one warp scan per tile suffices — publish the tile's aggregate and park the locally
//    resolved values in the tile's own ring slot;
//  * the look-back warp resolves the prefix of tile i while the compute warps go on with
//    tiles i+1 .. i+park, so the look-back latency (several L2 round trips) is off the
//    data path;
//  * the compute warps then re-read the parked tile lane-strided, add the prefix and store
//    it with coalesced 16-byte stores, after which the slot is refilled.
// Every tile, the first ring-full of a CTA included, is drawn from one atomic ticket counter:
// a tile is only ever owned by a CTA that is already running, so a look-back never waits for a
// CTA that has not been scheduled (whatever else occupies the GPU), and the tiles in flight
// are neighbours in the look-back chain.
// ---------------------------------------------------------------------------------------
constexpr int kStreamThreads = 512;  // compute threads; the CTA has one more warp
constexpr int kStreamWarps = kStreamThreads / kWarp;
constexpr int kStreamCta = kStreamThreads + kWarp;
// Per element size: 16-byte vectors per thread (tile = threads x vectors x 16 B) and the
// number of iterations a scanned tile stays parked waiting for its prefix. The ring has
// park + 2 slots. Measured best on B200: 40 KiB tiles parked for 3 iterations (4-byte
// types), 48 KiB tiles parked for 2 (8-byte types).
template <int ELEM_BYTES> struct StreamShape {
  static constexpr int kVecs = ELEM_BYTES == 4 ? 5 : 6;
  static constexpr int kPark = ELEM_BYTES == 4 ? 3 : 2;
  static constexpr int kStages = kPark + 2;
  static constexpr int kTileBytes = kStreamThreads * kVecs * 16;
};
constexpr unsigned kNoTile = 0xffffffffu;

template <typename T, bool EXCLUSIVE>
__global__ void __launch_bounds__(kStreamCta, 1)
scan_stream_kernel(const T* in, T* out, uint64_t n, T init, TempHeader* hdr, TileWords<Words<T>::W>* tiles,
                   unsigned num_tiles) {
  constexpr int W = Words<T>::W;
  constexpr int VEC = 16 / sizeof(T);
  constexpr int K = StreamShape<sizeof(T)>::kVecs;
  constexpr int kStreamPark = StreamShape<sizeof(T)>::kPark;
  constexpr int kStreamTileBytes = StreamShape<sizeof(T)>::kTileBytes;
  constexpr int WARP_ITEMS = kWarp * K * VEC;
  constexpr int TILE = kStreamThreads * K * VEC;
  constexpr int S = StreamShape<sizeof(T)>::kStages;

  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ __align__(8) unsigned long long s_full[S];    // bulk load of the slot has landed
  __shared__ __align__(8) unsigned long long s_handoff[S]; // slot's tile id and total are set
  __shared__ __align__(8) unsigned long long s_resolved[S];// slot's prefix is set
  __shared__ unsigned s_tile[S];      // tile loaded (or being loaded) into the slot
  __shared__ unsigned s_look_tile[S]; // tile handed to the look-back warp (kNoTile: stop)
  __shared__ T s_look_total[S];
  __shared__ T s_prefix[S];
  __shared__ T s_warp_total[kStreamWarps];

  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  int* status = &hdr->status;

  unsigned pending = 0;  // thread 0: the next tile of this CTA, already drawn
  auto start_load = [&](int slot, unsigned t) {
    s_tile[slot] = t;
    if (t < num_tiles && (uint64_t)(t + 1) * TILE <= n) {
      fence_proxy_async_smem();  // the slot was last touched by ordinary loads and stores
      mbar_expect_tx(&s_full[slot], kStreamTileBytes);
      bulk_load(ring + (size_t)slot * kStreamTileBytes, in + (uint64_t)t * TILE, kStreamTileBytes, &s_full[slot]);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_handoff[s], 1);
      mbar_init(&s_resolved[s], 1);
    }
    mbar_init_fence();
    unsigned first[S];
#pragma unroll
    for (int s = 0; s < S; ++s) first[s] = atomicAdd(&hdr->ticket, 1u);
#pragma unroll
    for (int s = 0; s < S; ++s) start_load(s, first[s]);
    pending = atomicAdd(&hdr->ticket, 1u);
  }
  __syncthreads();

  // ------------------------------------------------------------------ look-back warp
  if (warp == kStreamWarps) {
    for (unsigned j = 0;; ++j) {
      const int slot = j % S;
      if (!mbar_wait_bounded(&s_handoff[slot], (j / S) & 1u, status)) break;
      const unsigned tile = s_look_tile[slot];
      if (tile == kNoTile) break;
      const T total = s_look_total[slot];
      T prefix;
      if (tile == 0) {
        prefix = init;  // the seed: in front of the first element in both forms
      } else {
        prefix = lookback_sum<T>(tiles, tile, status);
      }
      if (lane == 0) {
        unsigned payload[W];
        Words<T>::pack(prefix + total, payload);
        publish<W>(&tiles[tile], kStatePrefix, payload);
        s_prefix[slot] = prefix;
        mbar_arrive(&s_resolved[slot]);
      }
      __syncwarp();
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps
  // adds the resolved prefix to the values parked in `slot` and stores the tile
  auto finalize = [&](unsigned it_prev, bool refill) {
    const int slot = it_prev % S;
    const unsigned tile = s_tile[slot];
    mbar_wait_bounded(&s_resolved[slot], (it_prev / S) & 1u, status);
    const T prefix = s_prefix[slot];
    const uint64_t warp_base = (uint64_t)tile * TILE + (uint64_t)warp * WARP_ITEMS;
    const Vec16<T>* parked = reinterpret_cast<const Vec16<T>*>(ring + (size_t)slot * kStreamTileBytes) +
                             warp * (kWarp * K);
    if ((uint64_t)(tile + 1) * TILE <= n) {
      Vec16<T>* dst = reinterpret_cast<Vec16<T>*>(out + warp_base);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        Vec16<T> v = parked[k * kWarp + lane];
#pragma unroll
        for (int j = 0; j < VEC; ++j) v.v[j] = prefix + v.v[j];
        dst[k * kWarp + lane] = v;
      }
    } else {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const Vec16<T> v = parked[k * kWarp + lane];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const uint64_t i = warp_base + (uint64_t)(k * kWarp + lane) * VEC + j;
          if (i < n) out[i] = prefix + v.v[j];
        }
      }
    }
    if (refill) {
      named_barrier(1, kStreamThreads);  // the slot has been read by every compute thread
      if (threadIdx.x == 0) {
        start_load(slot, pending);
        pending = atomicAdd(&hdr->ticket, 1u);
      }
    }
  };

  unsigned it = 0;
  for (;; ++it) {
    const int slot = it % S;
    const unsigned tile = s_tile[slot];
    if (tile >= num_tiles) break;  // tickets only grow: no load of this CTA is still in flight
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const bool full = tile_base + TILE <= n;
    // blocked layout for the local scan: thread t owns vectors [t*K, (t+1)*K) of the tile,
    // so one warp scan per tile suffices (the parked tile is re-read lane-strided later)
    Vec16<T>* mine = reinterpret_cast<Vec16<T>*>(ring + (size_t)slot * kStreamTileBytes) + threadIdx.x * K;

    T x[K][VEC];
    if (full) {
      mbar_wait_bounded(&s_full[slot], (it / S) & 1u, status);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const Vec16<T> v = mine[k];
#pragma unroll
        for (int j = 0; j < VEC; ++j) x[k][j] = v.v[j];
      }
    } else {
#pragma unroll
      for (int k = 0; k < K; ++k)
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const uint64_t i = tile_base + (uint64_t)(threadIdx.x * K + k) * VEC + j;
          x[k][j] = i < n ? in[i] : T(0);
        }
    }

    // sequential inclusive scan of the thread's K*VEC elements, then one scan across lanes
    T run = T(0);
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        run = (k == 0 && j == 0) ? x[0][0] : run + x[k][j];
        x[k][j] = run;
      }
    T s = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      T t = __shfl_up_sync(0xffffffffu, s, off);
      if (lane >= off) s = t + s;
    }
    T lane_excl = __shfl_up_sync(0xffffffffu, s, 1);
    if (lane == 0) lane_excl = T(0);
    if (lane == 31) s_warp_total[warp] = s;
    named_barrier(1, kStreamThreads);

    T warp_prefix = T(0), tile_total = T(0);
#pragma unroll
    for (int w = 0; w < kStreamWarps; ++w) {
      const T t = s_warp_total[w];
      if (w < (int)warp) warp_prefix = warp_prefix + t;
      tile_total = tile_total + t;
    }
    if (threadIdx.x == 0) {
      if (tile != 0) {
        unsigned payload[W];
        Words<T>::pack(tile_total, payload);
        publish<W>(&tiles[tile], kStateAggregate, payload);
      }
      s_look_tile[slot] = tile;
      s_look_total[slot] = tile_total;
      mbar_arrive(&s_handoff[slot]);
    }
    // park the locally resolved values in the tile's own slot
    {
      const T p = warp_prefix + lane_excl;
      T before = p;  // exclusive form: value in front of the element
#pragma unroll
      for (int k = 0; k < K; ++k) {
        Vec16<T> v;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const T incl = p + x[k][j];
          v.v[j] = EXCLUSIVE ? before : incl;
          before = incl;
        }
        mine[k] = v;
      }
    }
    // the barrier inside finalize (or this one) also orders this tile's parking stores
    // before other threads read them when the tile is finalized kStreamPark iterations on
    if (it >= (unsigned)kStreamPark) finalize(it - kStreamPark, true);
    else named_barrier(1, kStreamThreads);
  }
  // tiles of this CTA that are still parked
  named_barrier(1, kStreamThreads);
#pragma unroll
  for (int p = kStreamPark; p >= 1; --p)
    if (it >= (unsigned)p) finalize(it - p, false);
  if (threadIdx.x == 0) {  // release the look-back warp
    const int slot = it % S;
    s_look_tile[slot] = kNoTile;
    mbar_arrive(&s_handoff[slot]);
  }
}

template <typename T>
int launch_scan(void* d_temp, size_t* temp_bytes, const void* d_in, void* d_out, uint64_t n,
                int exclusive, const void* h_init, cudaStream_t stream) {
  constexpr int W = Words<T>::W;
  constexpr uint64_t TILE = (uint64_t)kScanThreads * kScanVecs * (16 / sizeof(T));
  constexpr uint64_t STREAM_TILE = (uint64_t)kStreamThreads * StreamShape<sizeof(T)>::kVecs * (16 / sizeof(T));
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const uint64_t stream_tiles = (n + STREAM_TILE - 1) / STREAM_TILE;  // the smaller tile sizes the scratch
  const size_t need = kHeaderBytes + (size_t)stream_tiles * sizeof(TileWords<W>);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (stream_tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  if (n == 0) return TB200_OK;
  if (d_in == nullptr || d_out == nullptr) return TB200_ERR_INVALID_ARGUMENT;

  T init = T(0);
  if (h_init) init = *static_cast<const T*>(h_init);
  auto* hdr = static_cast<TempHeader*>(d_temp);
  auto* desc = reinterpret_cast<TileWords<W>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  const T* in = static_cast<const T*>(d_in);
  T* out = static_cast<T*>(d_out);
  const bool aligned = ((reinterpret_cast<uintptr_t>(d_in) | reinterpret_cast<uintptr_t>(d_out)) % 16) == 0;
  if (aligned && stream_tiles >= 8) {
    int dev = 0, sms = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    TB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    constexpr int smem = StreamShape<sizeof(T)>::kStages * StreamShape<sizeof(T)>::kTileBytes;
    auto run = [&](auto kernel) -> int {
      TB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      int per_sm = 0;
      TB200_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kStreamCta, smem));
      if (per_sm < 1) return TB200_ERR_UNSUPPORTED;
      // one CTA per slot of the GPU: more would only queue behind them
      const uint64_t resident = (uint64_t)sms * per_sm;
      const unsigned grid = (unsigned)(stream_tiles < resident ? stream_tiles : resident);
      kernel<<<grid, kStreamCta, smem, stream>>>(in, out, n, init, hdr, desc, (unsigned)stream_tiles);
      return TB200_OK;
    };
    const int rc = exclusive ? run(scan_stream_kernel<T, true>) : run(scan_stream_kernel<T, false>);
    if (rc) return rc;
    trace_mark(stream, kTraceScan);
    return (int)cudaGetLastError();
  }
  const dim3 grid((unsigned)tiles), block(kScanThreads);
  if (exclusive) {
    if (aligned) scan_kernel<T, true, true><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
    else         scan_kernel<T, true, false><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
  } else {
    if (aligned) scan_kernel<T, false, true><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
    else         scan_kernel<T, false, false><<<grid, block, 0, stream>>>(in, out, n, init, hdr, desc);
  }
  trace_mark(stream, kTraceScan);
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
// from load until the process exits. The size is whatever the streaming kernel's tiles need
// at the documented limits (checked below), rounded up to 2 MiB.
constexpr uint64_t kStaticScanMaxN4 = 1ull << 31;  // 4-byte element types
constexpr uint64_t kStaticScanMaxN8 = 1ull << 29;  // 8-byte element types
constexpr size_t kStaticScanBytes = kHeaderBytes + (2u << 20);
template <int ELEM_BYTES>
constexpr size_t static_scan_need(uint64_t n) {
  constexpr uint64_t tile = (uint64_t)kStreamThreads * StreamShape<ELEM_BYTES>::kVecs * (16 / ELEM_BYTES);
  return kHeaderBytes + (size_t)((n + tile - 1) / tile) * sizeof(TileWords<ELEM_BYTES / 4>);
}
static_assert(static_scan_need<4>(kStaticScanMaxN4) <= kStaticScanBytes, "static scratch too small for 2^31 4-byte elements");
static_assert(static_scan_need<8>(kStaticScanMaxN8) <= kStaticScanBytes, "static scratch too small for 2^29 8-byte elements");
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
  const int eb = dtype_bytes(dtype);
  if (eb != 4 && eb != 8) return TB200_ERR_UNSUPPORTED;
  // the documented limits, checked before anything touches the device
  if (n > (eb == 4 ? kStaticScanMaxN4 : kStaticScanMaxN8)) return TB200_ERR_OVERFLOW;
  size_t need = 0;
  int rc = tb200_scan(nullptr, &need, nullptr, nullptr, n, dtype, exclusive, h_init, stream);
  if (rc) return rc;
  if (need > kStaticScanBytes) return TB200_ERR_OVERFLOW;  // cannot happen inside the limits (static_assert above)
  void* scratch = nullptr;
  rc = static_scan_scratch(&scratch);
  if (rc) return rc;
  size_t have = kStaticScanBytes;
  // tb200_scan clears the part of the scratch it uses (header and descriptors) on `stream`
  // before the kernel, so what the previous call left behind is never read.
  return tb200_scan(scratch, &have, d_in, d_out, n, dtype, exclusive, h_init, stream);
}

extern "C" int tb200_scan_static_status(tb200_stream_t stream) {
  using namespace tb200;
  void* scratch = nullptr;
  const int rc = static_scan_scratch(&scratch);
  if (rc) return rc;
  return tb200_temp_status(scratch, stream);
}
