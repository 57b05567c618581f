// inclusive_scan_by_key / exclusive_scan_by_key (equal_to, plus): the segmented scan of
// reduce_by_key with every element written. The streaming kernel is seg::stream_kernel
// (seg_stream.cuh); the one-tile-per-CTA kernel below serves unaligned pointers and tiny inputs.
#include "common.cuh"
#include "seg_stream.cuh"

namespace tb200 {
namespace {

// 256 threads x 8 chunks: 8192 elements (64 KiB of keys + values for 4-byte types)
// per tile, two tiles resident per SM. Large tiles keep the tile rate below what the
// look-back chain resolves (64 predecessors per L2 round trip).
constexpr int kRbkThreads = 256;
constexpr int kRbkWarps = kRbkThreads / kWarp;
constexpr int kRbkChunks = 8;

using seg::Pack;
template <typename V> using Seg = seg::SegPair<V>;
template <typename V>
__device__ __forceinline__ Seg<V> seg_combine(const Seg<V>& a, const Seg<V>& b) { return seg::combine(a, b); }
template <typename V> using SegWords = seg::DescWords<V>;
template <typename V>
__device__ __forceinline__ void lookback_seg(const TileWords<4>* tiles, unsigned tile, int* status,
                                             unsigned long long& out_cnt, V& out_val) {
  seg::lookback_chain<V>(tiles, tile, status, out_cnt, out_val);
}

// ---------------------------------------------------------------------------------------
// inclusive_scan_by_key / exclusive_scan_by_key (equal_to, plus): the same segmented scan
// with every element written. out[i] = sum of the elements of i's run up to and including i
// (inclusive), or init + the sum of those before i (exclusive; every run restarts at init).
// Replaces thrust::cuda_cub::detail::{inclusive,exclusive}_scan_by_key_n and their
// cub::DispatchScanByKey (thrust/system/cuda/detail/scan_by_key.h:96-290); semantics of
// thrust/system/detail/sequential/scan_by_key.h:34-146 (consecutive keys are compared).
// One tile per CTA, tiles taken by atomic ticket, look-back by warp 0; the output may be the
// value input (every CTA holds its tile in registers before it writes).
// ---------------------------------------------------------------------------------------
template <typename K, typename V, bool ALIGNED, bool EXCLUSIVE>
__global__ void __launch_bounds__(kRbkThreads, 2)
scan_by_key_kernel(const K* __restrict__ keys, const V* vals, V* out, V init, uint64_t n, unsigned num_tiles,
                   TempHeader* hdr, TileWords<4>* tiles) {
  constexpr int E = 16 / (sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V));
  constexpr int C = kRbkChunks;
  constexpr int WARP_ITEMS = kWarp * C * E;
  constexpr int TILE = kRbkThreads * C * E;

  __shared__ unsigned s_tile;
  __shared__ unsigned s_warp_cnt[kRbkWarps];
  __shared__ V s_warp_val[kRbkWarps];
  __shared__ V s_prefix_val;

  if (threadIdx.x == 0) s_tile = atomicAdd(&hdr->ticket, 1u);
  __syncthreads();
  const unsigned tile = s_tile;
  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  const uint64_t tile_base = (uint64_t)tile * TILE;
  const uint64_t warp_base = tile_base + (uint64_t)warp * WARP_ITEMS;
  const bool full = tile_base + TILE <= n;

  K k[C][E];
  V v[C][E];
  if (ALIGNED && full) {
    const Pack<K, E>* ksrc = reinterpret_cast<const Pack<K, E>*>(keys + warp_base);
    const Pack<V, E>* vsrc = reinterpret_cast<const Pack<V, E>*>(vals + warp_base);
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const Pack<K, E> kk = ksrc[c * kWarp + lane];
      const Pack<V, E> vv = vsrc[c * kWarp + lane];
#pragma unroll
      for (int e = 0; e < E; ++e) { k[c][e] = kk.v[e]; v[c][e] = vv.v[e]; }
    }
  } else {
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const uint64_t i = warp_base + (uint64_t)(c * kWarp + lane) * E + e;
        k[c][e] = i < n ? keys[i] : K(0);
        v[c][e] = i < n ? vals[i] : V(0);
      }
  }
  K slice_prev = K(0);
  if (lane == 0 && warp_base > 0 && warp_base <= n) slice_prev = keys[warp_base - 1];

  unsigned heads = 0;
  Seg<V> excl[C];
  Seg<V> carry{0u, V(0)};
  K prev_chunk_last = slice_prev;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    K prev = __shfl_up_sync(0xffffffffu, k[c][E - 1], 1);
    if (lane == 0) prev = prev_chunk_last;
    prev_chunk_last = __shfl_sync(0xffffffffu, k[c][E - 1], 31);
    Seg<V> mine{0u, V(0)};
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const uint64_t i = warp_base + (uint64_t)(c * kWarp + lane) * E + e;
      const bool head = i < n && (i == 0 || !(k[c][e] == prev));
      prev = k[c][e];
      if (head) { heads |= 1u << (c * E + e); mine.cnt += 1; mine.val = v[c][e]; }
      else mine.val = mine.val + v[c][e];
    }
    Seg<V> s = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      Seg<V> o;
      o.cnt = __shfl_up_sync(0xffffffffu, s.cnt, off);
      o.val = __shfl_up_sync(0xffffffffu, s.val, off);
      if (lane >= off) s = seg_combine(o, s);
    }
    Seg<V> e1;
    e1.cnt = __shfl_up_sync(0xffffffffu, s.cnt, 1);
    e1.val = __shfl_up_sync(0xffffffffu, s.val, 1);
    if (lane == 0) { e1.cnt = 0; e1.val = V(0); }
    excl[c] = seg_combine(carry, e1);
    Seg<V> tot;
    tot.cnt = __shfl_sync(0xffffffffu, s.cnt, 31);
    tot.val = __shfl_sync(0xffffffffu, s.val, 31);
    carry = seg_combine(carry, tot);
  }
  if (lane == 31) { s_warp_cnt[warp] = carry.cnt; s_warp_val[warp] = carry.val; }
  __syncthreads();

  Seg<V> warp_prefix{0u, V(0)}, tile_total{0u, V(0)};
#pragma unroll
  for (int w = 0; w < kRbkWarps; ++w) {
    const Seg<V> t{s_warp_cnt[w], s_warp_val[w]};
    if (w < (int)warp) warp_prefix = seg_combine(warp_prefix, t);
    tile_total = seg_combine(tile_total, t);
  }
  if (warp == 0) {
    unsigned payload[4];
    unsigned long long pc = 0;
    V pv = V(0);
    if (tile != 0) {
      if (lane == 0) {
        SegWords<V>::pack(tile_total.cnt, tile_total.val, payload);
        publish<4>(&tiles[tile], kStateAggregate, payload);
      }
      lookback_seg<V>(tiles, tile, &hdr->status, pc, pv);
    }
    if (lane == 0) {
      const unsigned long long ic = pc + tile_total.cnt;
      const V iv = tile_total.cnt ? tile_total.val : pv + tile_total.val;
      SegWords<V>::pack(ic, iv, payload);
      publish<4>(&tiles[tile], kStatePrefix, payload);
      s_prefix_val = pv;  // sum of the run that is open at the end of the predecessor tiles
    }
  }
  __syncthreads();

  const V tile_val = s_prefix_val;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const Seg<V> local = seg_combine(warp_prefix, excl[c]);
    V run = local.cnt ? local.val : tile_val + local.val;  // the open run's sum before this thread's elements
    Pack<V, E> res;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if (heads & (1u << (c * E + e))) run = V(0);
      if (EXCLUSIVE) res.v[e] = init + run;
      run = run + v[c][e];
      if (!EXCLUSIVE) res.v[e] = run;
    }
    if (ALIGNED && full) {
      reinterpret_cast<Pack<V, E>*>(out + warp_base)[c * kWarp + lane] = res;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const uint64_t i = warp_base + (uint64_t)(c * kWarp + lane) * E + e;
        if (i < n) out[i] = res.v[e];
      }
    }
  }
}

template <typename K, typename V>
int launch_sbk(void* d_temp, size_t* temp_bytes, const void* kin, const void* vin, void* vout, uint64_t n,
               int exclusive, const void* h_init, cudaStream_t stream) {
  constexpr int E = 16 / (sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V));
  constexpr uint64_t TILE = (uint64_t)kRbkThreads * kRbkChunks * E;
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const uint64_t stream_tiles = (n + seg::tile_elems<K, V>() - 1) / seg::tile_elems<K, V>();  // the smaller tile sizes the scratch
  const size_t need = seg::scratch_bytes<K, V>(n);  // tile and block descriptors of the streaming kernel
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (stream_tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  if (n == 0) return TB200_OK;
  if (!kin || !vin || !vout) return TB200_ERR_INVALID_ARGUMENT;
  V init = V(0);
  if (exclusive && h_init) init = *static_cast<const V*>(h_init);
  const bool aligned16 = (reinterpret_cast<uintptr_t>(kin) | reinterpret_cast<uintptr_t>(vin) |
                          reinterpret_cast<uintptr_t>(vout)) % 16 == 0;
  if (aligned16 && stream_tiles >= 8) {
    const int rc = exclusive
        ? seg::launch<seg::kScanByKeyExcl, K, V>(static_cast<const K*>(kin), static_cast<const V*>(vin), nullptr,
                                                 static_cast<V*>(vout), nullptr, n, init, true, d_temp, stream)
        : seg::launch<seg::kScanByKeyIncl, K, V>(static_cast<const K*>(kin), static_cast<const V*>(vin), nullptr,
                                                 static_cast<V*>(vout), nullptr, n, init, true, d_temp, stream);
    trace_mark(stream, kTraceScanByKey);
    return rc;
  }
  auto* hdr = static_cast<TempHeader*>(d_temp);
  auto* desc = reinterpret_cast<TileWords<4>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  const bool aligned = reinterpret_cast<uintptr_t>(kin) % (sizeof(K) * E) == 0 &&
                       reinterpret_cast<uintptr_t>(vin) % (sizeof(V) * E) == 0 &&
                       reinterpret_cast<uintptr_t>(vout) % (sizeof(V) * E) == 0;
  const dim3 grid((unsigned)tiles), block(kRbkThreads);
  auto go = [&](auto kernel) {
    kernel<<<grid, block, 0, stream>>>(static_cast<const K*>(kin), static_cast<const V*>(vin), static_cast<V*>(vout),
                                       init, n, (unsigned)tiles, hdr, desc);
  };
  if (aligned) {
    if (exclusive) go(scan_by_key_kernel<K, V, true, true>); else go(scan_by_key_kernel<K, V, true, false>);
  } else {
    if (exclusive) go(scan_by_key_kernel<K, V, false, true>); else go(scan_by_key_kernel<K, V, false, false>);
  }
  trace_mark(stream, kTraceScanByKey);
  return (int)cudaGetLastError();
}

template <typename K>
int launch_sbk_vals(int val_dtype, void* d_temp, size_t* temp_bytes, const void* kin, const void* vin, void* vout,
                    uint64_t n, int exclusive, const void* h_init, cudaStream_t stream) {
  switch (val_dtype) {
    case TB200_I32: case TB200_U32:
      return launch_sbk<K, uint32_t>(d_temp, temp_bytes, kin, vin, vout, n, exclusive, h_init, stream);
    case TB200_I64: case TB200_U64:
      return launch_sbk<K, unsigned long long>(d_temp, temp_bytes, kin, vin, vout, n, exclusive, h_init, stream);
    case TB200_F32: return launch_sbk<K, float>(d_temp, temp_bytes, kin, vin, vout, n, exclusive, h_init, stream);
    case TB200_F64: return launch_sbk<K, double>(d_temp, temp_bytes, kin, vin, vout, n, exclusive, h_init, stream);
    default: return TB200_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_scan_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals_in,
                                 void* d_vals_out, uint64_t n, int key_dtype, int val_dtype, int exclusive,
                                 const void* h_init, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
#define SBK_KEYS(K) \
  return launch_sbk_vals<K>(val_dtype, d_temp, temp_bytes, d_keys, d_vals_in, d_vals_out, n, exclusive, h_init, stream)
  switch (key_dtype) {
    // integer keys compare by bit pattern; floating-point keys with IEEE ==
    case TB200_I8: case TB200_U8: case TB200_BOOL: SBK_KEYS(uint8_t);
    case TB200_I16: case TB200_U16: SBK_KEYS(uint16_t);
    case TB200_I32: case TB200_U32: SBK_KEYS(uint32_t);
    case TB200_I64: case TB200_U64: SBK_KEYS(unsigned long long);
    case TB200_F32: SBK_KEYS(float);
    case TB200_F64: SBK_KEYS(double);
    default: return TB200_ERR_UNSUPPORTED;
  }
#undef SBK_KEYS
}
