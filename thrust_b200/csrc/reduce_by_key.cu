// reduce_by_key (equal_to / plus) as ONE streaming kernel: a segmented scan of
// (head-count, open-run sum) pairs with a decoupled look-back chain across tiles.
//
// For element i let head(i) = (i == 0 || key[i] != key[i-1]). The scan state
// before element i is (c, s): c = number of heads in [0, i), s = sum of the run
// that is open at i-1. At every head i > 0 the run that just closed is emitted:
// values_out[c-1] = s, and the new run's FIRST key: keys_out[c] = key[i]. The
// last tile emits the final open run and the run count. Sums are formed left to
// right inside a thread and in scan-tree order across lanes, warps and tiles:
// exact for integers, re-associated for floating point.
//
// Tile layout is the one of the scan kernel (warp-contiguous slices, lane-strided
// vectors), so key and value loads are full-width and coalesced.
#include "common.cuh"

namespace tb200 {
namespace {

// 256 threads x 8 chunks: 8192 elements (64 KiB of keys + values for 4-byte types)
// per tile, two tiles resident per SM. Large tiles keep the tile rate below what the
// look-back chain resolves (64 predecessors per L2 round trip).
constexpr int kRbkThreads = 256;
constexpr int kRbkWarps = kRbkThreads / kWarp;
constexpr int kRbkChunks = 8;

template <typename T, int E>
struct alignas(sizeof(T) * E) Pack {
  T v[E];
};

template <typename V>
struct Seg {
  unsigned cnt;
  V val;
};

template <typename V>
__device__ __forceinline__ Seg<V> seg_combine(const Seg<V>& a, const Seg<V>& b) {
  Seg<V> r;
  r.cnt = a.cnt + b.cnt;
  r.val = b.cnt ? b.val : a.val + b.val;
  return r;
}

template <typename V>
struct SegWords {
  static constexpr int W = 4;  // {count lo, count hi, value lo, value hi}
  __device__ static void pack(unsigned long long cnt, V val, unsigned (&p)[W]) {
    p[0] = (unsigned)cnt;
    p[1] = (unsigned)(cnt >> 32);
    if constexpr (sizeof(V) == 4) {
      p[2] = __builtin_bit_cast(unsigned, val);
      p[3] = 0;
    } else {
      unsigned long long b = __builtin_bit_cast(unsigned long long, val);
      p[2] = (unsigned)b;
      p[3] = (unsigned)(b >> 32);
    }
  }
  __device__ static void unpack(const unsigned (&p)[W], unsigned long long& cnt, V& val) {
    cnt = ((unsigned long long)p[1] << 32) | p[0];
    if constexpr (sizeof(V) == 4) val = __builtin_bit_cast(V, p[2]);
    else val = __builtin_bit_cast(V, ((unsigned long long)p[3] << 32) | p[2]);
  }
};

// Look-back over (count, value) descriptors by one warp, 32 predecessors per round. The
// operator is not commutative, so far predecessors are combined on the left of near ones.
// (Wider windows were measured to be slower: every extra polled descriptor adds traffic
// on the few cache lines all look-back warps read.)
template <typename V>
__device__ void lookback_seg(const TileWords<4>* tiles, unsigned tile, int* status,
                             unsigned long long& out_cnt, V& out_val) {
  const unsigned lane = lane_id();
  unsigned long long acc_cnt = 0;
  V acc_val = V(0);
  long long base = (long long)tile - 1;
  bool timed_out = false;
  while (true) {
    const long long idx = base - lane;
    unsigned st = kStatePrefix;
    unsigned long long cnt = 0;
    V val = V(0);
    if (idx >= 0) {
      unsigned payload[4];
      unsigned polls = 0;
      while ((st = peek<4>(&tiles[idx], payload)) == kStateEmpty) {
        backoff(++polls);
        if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(status) != 0)) {
          timed_out = true;
          st = kStatePrefix;
          break;
        }
      }
      if (!timed_out) SegWords<V>::unpack(payload, cnt, val);
    }
    const unsigned pm = __ballot_sync(0xffffffffu, st == kStatePrefix);
    const unsigned first = pm ? (unsigned)(__ffs(pm) - 1) : 31u;
    if (lane > first) { cnt = 0; val = V(0); }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long oc = __shfl_down_sync(0xffffffffu, cnt, off);
      const V ov = __shfl_down_sync(0xffffffffu, val, off);
      if (lane + off < 32) {  // (oc, ov) lies to the LEFT of (cnt, val)
        val = cnt ? val : ov + val;
        cnt = oc + cnt;
      }
    }
    cnt = __shfl_sync(0xffffffffu, cnt, 0);
    val = __shfl_sync(0xffffffffu, val, 0);
    // this window lies to the left of everything accumulated so far
    acc_val = acc_cnt ? acc_val : val + acc_val;
    acc_cnt = cnt + acc_cnt;
    if (pm) break;
    base -= 32;
  }
  if (__any_sync(0xffffffffu, timed_out) && lane == 0) atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
  out_cnt = acc_cnt;
  out_val = acc_val;
}

template <typename K, typename V, bool ALIGNED>
__global__ void __launch_bounds__(kRbkThreads, 2)
reduce_by_key_kernel(const K* __restrict__ keys, const V* __restrict__ vals, K* __restrict__ keys_out,
                     V* __restrict__ vals_out, unsigned long long* __restrict__ num_runs, uint64_t n,
                     unsigned num_tiles, TempHeader* hdr, TileWords<4>* tiles) {
  constexpr int E = 16 / (sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V));
  constexpr int C = kRbkChunks;
  constexpr int WARP_ITEMS = kWarp * C * E;
  constexpr int TILE = kRbkThreads * C * E;

  __shared__ unsigned s_tile;
  __shared__ unsigned s_warp_cnt[kRbkWarps];
  __shared__ V s_warp_val[kRbkWarps];
  __shared__ unsigned long long s_prefix_cnt;
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

  // key just before this warp's slice (lane 0 of chunk 0 needs it)
  K slice_prev = K(0);
  if (lane == 0 && warp_base > 0 && warp_base <= n) slice_prev = keys[warp_base - 1];

  unsigned heads = 0;  // bit (c*E+e) set when the element starts a run
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
      s_prefix_cnt = pc;
      s_prefix_val = pv;
      if (tile == num_tiles - 1) {  // close the last run and report the count
        if (ic > 0) vals_out[ic - 1] = iv;
        *num_runs = ic;
      }
    }
  }
  __syncthreads();

  // exclusive state of this thread's first element of every chunk, then walk
  const unsigned long long tile_cnt = s_prefix_cnt;
  const V tile_val = s_prefix_val;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    // (tile prefix) (+) (warp prefix) (+) (lane-exclusive inside the warp)
    Seg<V> local = seg_combine(warp_prefix, excl[c]);
    unsigned long long cnt = tile_cnt + local.cnt;
    V run = local.cnt ? local.val : tile_val + local.val;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      if (heads & (1u << (c * E + e))) {
        if (cnt > 0) vals_out[cnt - 1] = run;
        keys_out[cnt] = k[c][e];
        cnt += 1;
        run = v[c][e];
      } else {
        run = run + v[c][e];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Streaming variant (16-byte aligned inputs): the structure of the streaming scan kernel.
// Persistent CTAs, one per SM, 10 compute warps + one look-back warp; a ring of four slots,
// each holding one tile of keys and one of values, filled by bulk asynchronous copies.
// Thread t owns 5*E consecutive elements of the tile (80 bytes of the wider type: a
// bank-conflict-free stride), so head flags need one shuffle and the tile-local
// segmented scan one warp scan. Every value is then replaced in place by the sum of its
// run inside the thread and the tile stays parked for two iterations while the
// look-back warp resolves its prefix; the compute warps finally emit the parked tile's runs.
// ---------------------------------------------------------------------------------------
// 10 compute warps with 5 packs each: the per-thread stride (80 bytes of the wider type) is an odd
// multiple of 16 bytes, so the 16-byte shared-memory accesses stay bank-conflict-free, and the
// per-warp cost of the two shuffle scans is spread over more elements than with 16 warps x 3
// packs (measured 3.5 % faster; even pack counts lose more to bank conflicts than they gain).
#ifndef TB200_RS_THREADS
#define TB200_RS_THREADS 320
#define TB200_RS_PACKS 5
#define TB200_RS_PARK 2
#endif
#ifndef TB200_RS_LOADING
#define TB200_RS_LOADING 1
#endif
constexpr int kRsThreads = TB200_RS_THREADS;
constexpr int kRsWarps = kRsThreads / kWarp;
#ifndef TB200_RS_LOOK_WARPS
#define TB200_RS_LOOK_WARPS 1
#endif
constexpr int kRsLookWarps = TB200_RS_LOOK_WARPS;  // look-back warps; tile j of a CTA is resolved by warp j % count
constexpr int kRsCta = kRsThreads + kRsLookWarps * kWarp;
constexpr int kRsPacks = TB200_RS_PACKS;  // packs of E elements per thread
constexpr int kRsPark = TB200_RS_PARK;
constexpr int kRsLoading = TB200_RS_LOADING;  // tiles in flight from HBM beside the one being scanned
constexpr int kRsStages = kRsPark + 1 + kRsLoading;
constexpr unsigned kRsNoTile = 0xffffffffu;

template <typename K, typename V>
struct RsShape {
  static constexpr int E = 16 / (sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V));
  static constexpr int kItems = kRsPacks * E;
  static constexpr int kTile = kRsThreads * kItems;
  static constexpr int kKeyBytes = kTile * (int)sizeof(K);
  static constexpr int kValBytes = kTile * (int)sizeof(V);
  static constexpr int kSlotBytes = ((kKeyBytes + 127) / 128) * 128 + ((kValBytes + 127) / 128) * 128;
  static constexpr int kValOffset = ((kKeyBytes + 127) / 128) * 128;
  static constexpr int kSmem = kRsStages * kSlotBytes;
};

template <typename K, typename V>
__global__ void __launch_bounds__(kRsCta, 1)
rbk_stream_kernel(const K* __restrict__ keys, const V* __restrict__ vals, K* __restrict__ keys_out,
                  V* __restrict__ vals_out, unsigned long long* __restrict__ num_runs, uint64_t n,
                  unsigned num_tiles, TempHeader* hdr, TileWords<4>* tiles) {
  using Shape = RsShape<K, V>;
  constexpr int E = Shape::E;
  constexpr int P = kRsPacks;
  constexpr int ITEMS = Shape::kItems;
  constexpr int TILE = Shape::kTile;
  constexpr int S = kRsStages;

  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ __align__(8) unsigned long long s_full[S], s_handoff[S], s_resolved[S];
  __shared__ unsigned s_tile[S], s_look_tile[S], s_look_cnt[S];
  __shared__ V s_look_val[S];
  __shared__ unsigned long long s_prefix_cnt[S];
  __shared__ V s_prefix_val[S];
  __shared__ unsigned short s_park_cnt[S][kRsThreads];
  __shared__ unsigned s_park_heads[S][kRsThreads];
  __shared__ V s_park_val[S][kRsThreads];
  __shared__ unsigned s_warp_cnt[kRsWarps];
  __shared__ V s_warp_val[kRsWarps];

  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  int* status = &hdr->status;
  auto slot_keys = [&](int slot) { return reinterpret_cast<K*>(ring + (size_t)slot * Shape::kSlotBytes); };
  auto slot_vals = [&](int slot) {
    return reinterpret_cast<V*>(ring + (size_t)slot * Shape::kSlotBytes + Shape::kValOffset);
  };

  const unsigned first_dynamic = S * gridDim.x;
  unsigned pending = 0;
  auto start_load = [&](int slot, unsigned t) {
    s_tile[slot] = t;
    if (t < num_tiles && (uint64_t)(t + 1) * TILE <= n) {
      fence_proxy_async_smem();  // the slot was last touched by ordinary loads and stores
      mbar_expect_tx(&s_full[slot], Shape::kKeyBytes + Shape::kValBytes);
      bulk_load(slot_keys(slot), keys + (uint64_t)t * TILE, Shape::kKeyBytes, &s_full[slot]);
      bulk_load(slot_vals(slot), vals + (uint64_t)t * TILE, Shape::kValBytes, &s_full[slot]);
    }
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_handoff[s], 1);
      mbar_init(&s_resolved[s], 1);
    }
    mbar_init_fence();
    for (int s = 0; s < S; ++s) start_load(s, s * gridDim.x + blockIdx.x);
    pending = first_dynamic + atomicAdd(&hdr->ticket, 1u);
  }
  __syncthreads();

  // ------------------------------------------------------------------ look-back warps
  // kRsLookWarps warps take turns, each resolving its tiles independently of the others. One
  // warp measured fastest: a second poller slows the chain it waits on more than it overlaps.
  if (warp >= kRsWarps) {
    for (unsigned j = warp - kRsWarps;; j += kRsLookWarps) {
      const int slot = j % S;
      if (!mbar_wait_bounded(&s_handoff[slot], (j / S) & 1u, status)) break;
      const unsigned tile = s_look_tile[slot];
      if (tile == kRsNoTile) break;
      const unsigned tot_cnt = s_look_cnt[slot];
      const V tot_val = s_look_val[slot];
      unsigned long long pc = 0;
      V pv = V(0);
#ifndef TB200_EXPERIMENT_NO_LOOKBACK
      if (tile != 0) lookback_seg<V>(tiles, tile, status, pc, pv);
#endif
      if (lane == 0) {
        const unsigned long long ic = pc + tot_cnt;
        const V iv = tot_cnt ? tot_val : pv + tot_val;
        unsigned payload[4];
        SegWords<V>::pack(ic, iv, payload);
        publish<4>(&tiles[tile], kStatePrefix, payload);
        if (tile == num_tiles - 1) {  // close the last run and report the count
          if (ic > 0) vals_out[ic - 1] = iv;
          *num_runs = ic;
        }
        s_prefix_cnt[slot] = pc;
        s_prefix_val[slot] = pv;
        mbar_arrive(&s_resolved[slot]);
      }
      __syncwarp();
    }
    return;
  }

  // ------------------------------------------------------------------ compute warps
  // emits the runs that close inside the tile parked at iteration it_prev (each thread
  // re-reads only what it parked itself)
  auto finalize = [&](unsigned it_prev, bool refill) {
    const int slot = it_prev % S;
    mbar_wait_bounded(&s_resolved[slot], (it_prev / S) & 1u, status);
    unsigned heads = s_park_heads[slot][threadIdx.x];
#ifdef TB200_EXPERIMENT_NO_FINALIZE
    heads = 0;
#endif
    if (heads) {
      const unsigned long long pc = s_prefix_cnt[slot];
      const V pv = s_prefix_val[slot];
      const K* pk = slot_keys(slot) + threadIdx.x * ITEMS;
      const V* pr = slot_vals(slot) + threadIdx.x * ITEMS;  // parked: run sums inside the thread
      unsigned cnt = s_park_cnt[slot][threadIdx.x];
      // the run that closes at the thread's FIRST head began before the thread
      V carried = s_park_val[slot][threadIdx.x];
      while (heads) {  // one iteration per run that starts in this thread's elements
        const int i = __ffs(heads) - 1;
        heads &= heads - 1;
        const unsigned long long at = pc + cnt;
        const V r = carried + (i ? pr[i - 1] : V(0));
        if (at > 0) vals_out[at - 1] = cnt ? r : pv + r;
        keys_out[at] = pk[i];
        carried = V(0);
        ++cnt;
      }
    }
    if (refill) {
      named_barrier(1, kRsThreads);  // the slot has been read by every compute thread
      if (threadIdx.x == 0) {
        start_load(slot, pending);
        pending = first_dynamic + atomicAdd(&hdr->ticket, 1u);
      }
    }
  };

  unsigned it = 0;
  for (;; ++it) {
    const int slot = it % S;
    const unsigned tile = s_tile[slot];
    if (tile >= num_tiles) break;
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const uint64_t my_base = tile_base + (uint64_t)threadIdx.x * ITEMS;
    const bool full = tile_base + TILE <= n;
    Pack<K, E>* mk = reinterpret_cast<Pack<K, E>*>(slot_keys(slot)) + threadIdx.x * P;
    Pack<V, E>* mv = reinterpret_cast<Pack<V, E>*>(slot_vals(slot)) + threadIdx.x * P;

    K k[ITEMS];
    V v[ITEMS];
    if (full) {
      mbar_wait_bounded(&s_full[slot], (it / S) & 1u, status);
#pragma unroll
      for (int p = 0; p < P; ++p) {
        const Pack<K, E> kk = mk[p];
        const Pack<V, E> vv = mv[p];
#pragma unroll
        for (int e = 0; e < E; ++e) { k[p * E + e] = kk.v[e]; v[p * E + e] = vv.v[e]; }
      }
    } else {
#pragma unroll
      for (int p = 0; p < P; ++p) {
        Pack<K, E> kk;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const uint64_t i = my_base + p * E + e;
          k[p * E + e] = i < n ? keys[i] : K(0);
          v[p * E + e] = i < n ? vals[i] : V(0);
          kk.v[e] = k[p * E + e];
        }
        mk[p] = kk;  // the final pass reads keys from the slot
      }
    }
    // key in front of this thread's run of elements
    K prev = __shfl_up_sync(0xffffffffu, k[ITEMS - 1], 1);
    if (lane == 0) prev = (my_base > 0 && my_base <= n) ? keys[my_base - 1] : K(0);

    // head flags; full tiles need no bounds checks (only element 0 of the array is special)
    unsigned heads = 0;
    if (full) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) heads |= (unsigned)!(k[i] == (i == 0 ? prev : k[i - 1])) << i;
      if (my_base == 0) heads |= 1u;
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const uint64_t g = my_base + i;
        const bool head = g < n && (g == 0 || !(k[i] == (i == 0 ? prev : k[i - 1])));
        heads |= (unsigned)head << i;
      }
    }
    // one pass of run sums inside the thread: incl[i] = sum of element i's run so far,
    // counted from the thread's first element
    V incl[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      incl[i] = (i == 0 || (heads & (1u << i))) ? v[i] : incl[i - 1] + v[i];
    Seg<V> s{(unsigned)__popc(heads), incl[ITEMS - 1]};
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      Seg<V> o;
      o.cnt = __shfl_up_sync(0xffffffffu, s.cnt, off);
      o.val = __shfl_up_sync(0xffffffffu, s.val, off);
      if (lane >= off) s = seg_combine(o, s);
    }
    Seg<V> lane_excl;
    lane_excl.cnt = __shfl_up_sync(0xffffffffu, s.cnt, 1);
    lane_excl.val = __shfl_up_sync(0xffffffffu, s.val, 1);
    if (lane == 0) { lane_excl.cnt = 0; lane_excl.val = V(0); }
    if (lane == 31) { s_warp_cnt[warp] = s.cnt; s_warp_val[warp] = s.val; }
    named_barrier(1, kRsThreads);

    // scan of the warp totals: lane w holds warp w's total (kRsWarps <= 32)
    Seg<V> wt{0u, V(0)};
    if (lane < kRsWarps) { wt.cnt = s_warp_cnt[lane]; wt.val = s_warp_val[lane]; }
#pragma unroll
    for (int off = 1; off < kRsWarps; off <<= 1) {
      Seg<V> o;
      o.cnt = __shfl_up_sync(0xffffffffu, wt.cnt, off);
      o.val = __shfl_up_sync(0xffffffffu, wt.val, off);
      if (lane >= off) wt = seg_combine(o, wt);
    }
    Seg<V> warp_prefix, tile_total;
    warp_prefix.cnt = __shfl_sync(0xffffffffu, wt.cnt, warp == 0 ? 0 : warp - 1);
    warp_prefix.val = __shfl_sync(0xffffffffu, wt.val, warp == 0 ? 0 : warp - 1);
    if (warp == 0) { warp_prefix.cnt = 0; warp_prefix.val = V(0); }
    tile_total.cnt = __shfl_sync(0xffffffffu, wt.cnt, kRsWarps - 1);
    tile_total.val = __shfl_sync(0xffffffffu, wt.val, kRsWarps - 1);
    if (threadIdx.x == 0) {
      if (tile != 0) {
        unsigned payload[4];
        SegWords<V>::pack(tile_total.cnt, tile_total.val, payload);
        publish<4>(&tiles[tile], kStateAggregate, payload);
      }
      s_look_tile[slot] = tile;
      s_look_cnt[slot] = tile_total.cnt;
      s_look_val[slot] = tile_total.val;
      mbar_arrive(&s_handoff[slot]);
    }
    // park what the final pass needs: the run sums inside the thread (in place of the
    // values), the thread's head mask, and the state of the scan in front of the thread
#ifndef TB200_EXPERIMENT_NO_PARK
    {
      const Seg<V> local = seg_combine(warp_prefix, lane_excl);
      s_park_heads[slot][threadIdx.x] = heads;
      s_park_cnt[slot][threadIdx.x] = (unsigned short)local.cnt;
      s_park_val[slot][threadIdx.x] = local.val;
#pragma unroll
      for (int p = 0; p < P; ++p) {
        Pack<V, E> rr;
#pragma unroll
        for (int e = 0; e < E; ++e) rr.v[e] = incl[p * E + e];
        mv[p] = rr;
      }
    }
#endif
    if (it >= (unsigned)kRsPark) finalize(it - kRsPark, true);
    else named_barrier(1, kRsThreads);  // s_warp_* are rewritten by the next tile
  }
#pragma unroll
  for (int p = kRsPark; p >= 1; --p)
    if (it >= (unsigned)p) finalize(it - p, false);
  if (threadIdx.x == 0) {  // release the look-back warps (the next kRsLookWarps hand-offs)
    for (unsigned j = it; j < it + kRsLookWarps; ++j) {
      const int slot = j % S;
      s_look_tile[slot] = kRsNoTile;
      mbar_arrive(&s_handoff[slot]);
    }
  }
}

template <typename K, typename V>
int launch_rbk(void* d_temp, size_t* temp_bytes, const void* kin, const void* vin, void* kout, void* vout,
               uint64_t* d_num_runs, uint64_t n, cudaStream_t stream) {
  constexpr int E = 16 / (sizeof(K) > sizeof(V) ? sizeof(K) : sizeof(V));
  constexpr uint64_t TILE = (uint64_t)kRbkThreads * kRbkChunks * E;
  constexpr uint64_t STREAM_TILE = RsShape<K, V>::kTile;  // the smaller tile sizes the scratch
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const uint64_t stream_tiles = (n + STREAM_TILE - 1) / STREAM_TILE;
  const size_t need = kHeaderBytes + (size_t)stream_tiles * sizeof(TileWords<4>);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (stream_tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  if (d_num_runs == nullptr || reinterpret_cast<uintptr_t>(d_num_runs) % 8) return TB200_ERR_INVALID_ARGUMENT;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  TB200_CUDA_TRY(cudaMemsetAsync(d_num_runs, 0, sizeof(uint64_t), stream));
  if (n == 0) return TB200_OK;
  if (!kin || !vin || !kout || !vout) return TB200_ERR_INVALID_ARGUMENT;
  auto* hdr = static_cast<TempHeader*>(d_temp);
  auto* desc = reinterpret_cast<TileWords<4>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  const bool aligned = reinterpret_cast<uintptr_t>(kin) % (sizeof(K) * E) == 0 &&
                       reinterpret_cast<uintptr_t>(vin) % (sizeof(V) * E) == 0;
  auto* nr = reinterpret_cast<unsigned long long*>(d_num_runs);
  const bool aligned16 = (reinterpret_cast<uintptr_t>(kin) | reinterpret_cast<uintptr_t>(vin)) % 16 == 0;
  if (aligned16 && stream_tiles >= 8) {
    int dev = 0, sms = 0, per_sm = 0;
    TB200_CUDA_TRY(cudaGetDevice(&dev));
    TB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    auto kernel = rbk_stream_kernel<K, V>;
    constexpr int smem = RsShape<K, V>::kSmem;
    TB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    TB200_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRsCta, smem));
    if (per_sm < 1) return TB200_ERR_UNSUPPORTED;
    const uint64_t resident = (uint64_t)sms * per_sm;  // all CTAs resident: the first tiles are dealt statically
    const unsigned sgrid = (unsigned)(stream_tiles < resident ? stream_tiles : resident);
    kernel<<<sgrid, kRsCta, smem, stream>>>(static_cast<const K*>(kin), static_cast<const V*>(vin),
                                            static_cast<K*>(kout), static_cast<V*>(vout), nr, n,
                                            (unsigned)stream_tiles, hdr, desc);
    trace_mark(stream, kTraceReduceByKey);
    return (int)cudaGetLastError();
  }
  const dim3 grid((unsigned)tiles), block(kRbkThreads);
  if (aligned)
    reduce_by_key_kernel<K, V, true><<<grid, block, 0, stream>>>(
        static_cast<const K*>(kin), static_cast<const V*>(vin), static_cast<K*>(kout), static_cast<V*>(vout), nr,
        n, (unsigned)tiles, hdr, desc);
  else
    reduce_by_key_kernel<K, V, false><<<grid, block, 0, stream>>>(
        static_cast<const K*>(kin), static_cast<const V*>(vin), static_cast<K*>(kout), static_cast<V*>(vout), nr,
        n, (unsigned)tiles, hdr, desc);
  trace_mark(stream, kTraceReduceByKey);
  return (int)cudaGetLastError();
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
  const size_t need = kHeaderBytes + (size_t)tiles * sizeof(TileWords<4>);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  if (n == 0) return TB200_OK;
  if (!kin || !vin || !vout) return TB200_ERR_INVALID_ARGUMENT;
  V init = V(0);
  if (exclusive && h_init) init = *static_cast<const V*>(h_init);
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

template <typename K>
int launch_rbk_vals(int val_dtype, void* d_temp, size_t* temp_bytes, const void* kin, const void* vin,
                    void* kout, void* vout, uint64_t* d_num_runs, uint64_t n, cudaStream_t stream) {
  switch (val_dtype) {
    case TB200_I32: case TB200_U32:
      return launch_rbk<K, uint32_t>(d_temp, temp_bytes, kin, vin, kout, vout, d_num_runs, n, stream);
    case TB200_I64: case TB200_U64:
      return launch_rbk<K, unsigned long long>(d_temp, temp_bytes, kin, vin, kout, vout, d_num_runs, n, stream);
    case TB200_F32:
      return launch_rbk<K, float>(d_temp, temp_bytes, kin, vin, kout, vout, d_num_runs, n, stream);
    case TB200_F64:
      return launch_rbk<K, double>(d_temp, temp_bytes, kin, vin, kout, vout, d_num_runs, n, stream);
    default:
      return TB200_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_reduce_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys_in,
                                   const void* d_vals_in, void* d_keys_out, void* d_vals_out,
                                   uint64_t* d_num_runs, uint64_t n, int key_dtype, int val_dtype,
                                   tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
#define RBK_KEYS(K) \
  return launch_rbk_vals<K>(val_dtype, d_temp, temp_bytes, d_keys_in, d_vals_in, d_keys_out, d_vals_out, \
                            d_num_runs, n, stream)
  switch (key_dtype) {
    // integer keys compare by bit pattern; floating-point keys with IEEE ==
    case TB200_I8: case TB200_U8: case TB200_BOOL: RBK_KEYS(uint8_t);
    case TB200_I16: case TB200_U16: RBK_KEYS(uint16_t);
    case TB200_I32: case TB200_U32: RBK_KEYS(uint32_t);
    case TB200_I64: case TB200_U64: RBK_KEYS(unsigned long long);
    case TB200_F32: RBK_KEYS(float);
    case TB200_F64: RBK_KEYS(double);
    default: return TB200_ERR_UNSUPPORTED;
  }
#undef RBK_KEYS
}

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
