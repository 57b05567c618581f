// Streaming skeleton of the by-key algorithms (reduce_by_key, inclusive / exclusive
// scan_by_key, unique_by_key, copy of flagged elements): ONE pass over the input, a decoupled
// look-back chain across tiles, and no barrier that spans the whole CTA on the data path.
//
// A persistent CTA (one per SM) has three kinds of warps:
//   * one producer thread draws tiles from an atomic ticket counter and fills a ring of
//     shared-memory slots with bulk asynchronous copies (the untiled TMA form), keys and values
//     of a tile per slot, completion signalled on the slot's `full` mbarrier;
//   * kComputeWarps compute warps, each working on its own 32 x kItems slice of every tile
//     WITHOUT synchronising with the other compute warps: phase A (head flags, run sums inside
//     the thread, one segmented warp scan, warp total to shared memory, arrive on the slot's
//     `scanned` mbarrier) and, kPark tiles later, phase C (wait for the slot's `resolved`
//     mbarrier, read the warp's prefix, emit, arrive on the slot's `freed` mbarrier);
//   * one look-back warp that, per tile, scans the compute warps' totals, publishes the tile
//     aggregate, resolves the tile's prefix over the predecessor tiles and hands every compute
//     warp its own prefix.
// Because every warp runs at its own pace, the latency chains of different warps (shared-memory
// loads, dependent adds, shuffles, scattered stores) overlap instead of adding up behind CTA
// barriers. Every tile, the first ring-full included, is drawn by ticket, so a tile is only
// ever owned by a CTA that is already running: no look-back waits for an unscheduled CTA.
// Every wait (mbarrier or look-back poll) is bounded and reports through the status word.
#pragma once

#include "common.cuh"

#include <type_traits>

namespace tb200 {
namespace seg {

template <typename T, int E>
struct alignas(sizeof(T) * E) Pack {
  T v[E];
};

// Opaque payloads (compared never, only moved) of the selection kernels.
template <int BYTES> struct Blob;
template <> struct Blob<1> { using type = uint8_t; };
template <> struct Blob<2> { using type = uint16_t; };
template <> struct Blob<4> { using type = uint32_t; };
template <> struct Blob<8> { using type = unsigned long long; };
template <> struct Blob<16> { using type = uint4; };
// Value type of the keys-only forms (unique): nothing is loaded, staged or stored for it.
struct NoVal {};

enum Mode : int {
  kReduceByKey = 0,    // emit (first key, run sum) per run
  kScanByKeyIncl = 1,  // write every element's running sum of its run
  kScanByKeyExcl = 2,  // same, exclusive, every run restarts at init
  kUniqueByKey = 3,    // emit (key, value) of the first element of every run
  kCopyFlagged = 4     // "keys" are flags: emit the value of every element whose flag is non-zero
};

template <typename A>
struct SegPair {
  unsigned cnt;
  A val;
};
template <typename A>
__device__ __forceinline__ SegPair<A> combine(const SegPair<A>& a, const SegPair<A>& b) {
  SegPair<A> r;
  r.cnt = a.cnt + b.cnt;
  r.val = b.cnt ? b.val : a.val + b.val;
  return r;
}

// {count lo, count hi, value lo, value hi} of one tile descriptor
template <typename A>
struct DescWords {
  __device__ static void pack(unsigned long long cnt, A val, unsigned (&p)[4]) {
    p[0] = (unsigned)cnt;
    p[1] = (unsigned)(cnt >> 32);
    if constexpr (sizeof(A) == 4) {
      p[2] = __builtin_bit_cast(unsigned, val);
      p[3] = 0;
    } else {
      unsigned long long b = __builtin_bit_cast(unsigned long long, val);  // not const: the front end must not try to fold it
      p[2] = (unsigned)b;
      p[3] = (unsigned)(b >> 32);
    }
  }
  __device__ static void unpack(const unsigned (&p)[4], unsigned long long& cnt, A& val) {
    cnt = ((unsigned long long)p[1] << 32) | p[0];
    if constexpr (sizeof(A) == 4) val = __builtin_bit_cast(A, p[2]);
    else val = __builtin_bit_cast(A, ((unsigned long long)p[3] << 32) | p[2]);
  }
};

// Look-back over (count, value) descriptors by one warp, 32 predecessors per round. The
// operator is not commutative: far predecessors are combined on the left of near ones.
template <typename A>
__device__ void lookback(const TileWords<4>* tiles, unsigned tile, int* status, unsigned long long& out_cnt,
                         A& out_val) {
  const unsigned lane = lane_id();
  unsigned long long acc_cnt = 0;
  A acc_val = A(0);
  long long base = (long long)tile - 1;
  bool timed_out = false;
  while (true) {
    const long long idx = base - lane;
    unsigned st = kStatePrefix;
    unsigned long long cnt = 0;
    A val = A(0);
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
      if (!timed_out) DescWords<A>::unpack(payload, cnt, val);
    }
    const unsigned pm = __ballot_sync(0xffffffffu, st == kStatePrefix);
    const unsigned first = pm ? (unsigned)(__ffs(pm) - 1) : 31u;
    if (lane > first) { cnt = 0; val = A(0); }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long oc = __shfl_down_sync(0xffffffffu, cnt, off);
      const A ov = __shfl_down_sync(0xffffffffu, val, off);
      if (lane + off < 32) {  // (oc, ov) lies to the LEFT of (cnt, val)
        val = cnt ? val : ov + val;
        cnt = oc + cnt;
      }
    }
    cnt = __shfl_sync(0xffffffffu, cnt, 0);
    val = __shfl_sync(0xffffffffu, val, 0);
    acc_val = acc_cnt ? acc_val : val + acc_val;  // this window lies to the left of the accumulated part
    acc_cnt = cnt + acc_cnt;
    if (pm) break;
    base -= 32;
  }
  if (__any_sync(0xffffffffu, timed_out) && lane == 0) atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
  out_cnt = acc_cnt;
  out_val = acc_val;
}

constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * kWarp;
constexpr int kCtaThreads = kComputeThreads + 2 * kWarp;  // + look-back warp + producer warp
constexpr int kPacks = 5;  // 16-byte packs of the wider type per thread: an 80-byte stride has no bank conflicts
constexpr int kPark = 2;   // tiles a scanned tile waits for its prefix while the warp goes on
constexpr int kStages = 5; // ring slots: kPark parked, one in phase A, two loading
constexpr unsigned kNoTile = 0xffffffffu;

template <typename K, typename V>
struct Shape {
  static constexpr bool kHasVals = !std::is_same<V, NoVal>::value;
  static constexpr int kValSize = kHasVals ? (int)sizeof(V) : 0;
  static constexpr int kWide = (int)sizeof(K) > kValSize ? (int)sizeof(K) : kValSize;
  static constexpr int E = 16 / kWide > 4 ? 4 : 16 / kWide;  // elements per pack (head masks have 32 bits)
  static constexpr int kItems = kPacks * E;                  // per thread
  static constexpr int kWarpItems = kWarp * kItems;
  static constexpr int kTile = kComputeThreads * kItems;
  static constexpr int kKeyBytes = kTile * (int)sizeof(K);
  static constexpr int kValBytes = kTile * kValSize;
  static constexpr int kValOffset = (kKeyBytes + 127) / 128 * 128;
  static constexpr int kSlotBytes = kValOffset + (kValBytes + 127) / 128 * 128;
  static constexpr int kSmem = kStages * kSlotBytes;
  static_assert(kKeyBytes % 16 == 0 && kValBytes % 16 == 0, "bulk copies move multiples of 16 bytes");
  static_assert(kItems <= 32, "one head bit per item");
};

template <typename K, typename V>
struct Args {
  const K* keys;
  const V* vals;
  K* keys_out;                  // reduce_by_key, unique_by_key
  V* vals_out;                  // every mode
  unsigned long long* num_out;  // number of runs / selected elements (not for scan_by_key)
  uint64_t n;
  unsigned num_tiles;
  int bulk;                     // inputs are 16-byte aligned: tiles arrive by bulk copy
  V init;                       // exclusive scan_by_key
  TempHeader* hdr;
  TileWords<4>* tiles;
};

template <int MODE, typename V> struct AccOf { using type = unsigned; };
template <typename V> struct AccOf<kReduceByKey, V> { using type = V; };
template <typename V> struct AccOf<kScanByKeyIncl, V> { using type = V; };
template <typename V> struct AccOf<kScanByKeyExcl, V> { using type = V; };

template <int MODE, typename K, typename V>
__global__ void __launch_bounds__(kCtaThreads, 1) stream_kernel(const Args<K, V> a) {
  using S = Shape<K, V>;
  using A = typename AccOf<MODE, V>::type;
  constexpr bool kSum = MODE == kReduceByKey || MODE == kScanByKeyIncl || MODE == kScanByKeyExcl;
  constexpr bool kScanOut = MODE == kScanByKeyIncl || MODE == kScanByKeyExcl;
  constexpr bool kHasVals = S::kHasVals;
  static_assert(kHasVals || MODE == kUniqueByKey, "only unique has a keys-only form");
  constexpr int E = S::E;
  constexpr int ITEMS = S::kItems;
  constexpr int TILE = S::kTile;
  constexpr int NS = kStages;
  constexpr int NW = kComputeWarps;

  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ __align__(8) unsigned long long s_full[NS], s_scanned[NS], s_resolved[NS], s_freed[NS];
  __shared__ unsigned s_tile[NS];
  __shared__ unsigned s_wtot_cnt[NS][NW];
  __shared__ A s_wtot_val[NS][NW];
  __shared__ unsigned long long s_wpre_cnt[NS][NW];
  __shared__ A s_wpre_val[NS][NW];

  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  int* status = &a.hdr->status;
  const uint64_t n = a.n;
  const unsigned num_tiles = a.num_tiles;
  auto slot_keys = [&](int slot) { return reinterpret_cast<K*>(ring + (size_t)slot * S::kSlotBytes); };
  auto slot_vals = [&](int slot) { return reinterpret_cast<V*>(ring + (size_t)slot * S::kSlotBytes + S::kValOffset); };

  // a wait whose outcome all lanes of the calling warp agree on (a time-out ends the whole warp's role)
  auto wait_all = [&](unsigned long long* bar, unsigned parity) -> bool {
    return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, status));
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_scanned[s], NW);
      mbar_init(&s_resolved[s], 1);
      mbar_init(&s_freed[s], NW);
    }
    mbar_init_fence();
  }
  __syncthreads();  // the only CTA-wide barrier of the kernel

  // ---------------------------------------------------------------------- producer
  if (warp == NW + 1) {
    if (lane != 0) return;
    // tile t goes into `slot`; false when the tickets have run past the last tile
    auto issue = [&](int slot, unsigned t) -> bool {
      if (t >= num_tiles) {
        s_tile[slot] = kNoTile;
        mbar_arrive(&s_full[slot]);
        return false;
      }
      s_tile[slot] = t;
      if (a.bulk && (uint64_t)(t + 1) * TILE <= n) {
        fence_proxy_async_smem();  // the slot was last written by ordinary stores (parked values)
        mbar_expect_tx(&s_full[slot], S::kKeyBytes + S::kValBytes);
        bulk_load(slot_keys(slot), a.keys + (uint64_t)t * TILE, S::kKeyBytes, &s_full[slot]);
        if constexpr (kHasVals)
          bulk_load(slot_vals(slot), a.vals + (uint64_t)t * TILE, S::kValBytes, &s_full[slot]);
      } else {
        mbar_arrive(&s_full[slot]);  // ragged last tile or unaligned input: the compute warps load it themselves
      }
      return true;
    };
    unsigned first[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) first[s] = atomicAdd(&a.hdr->ticket, 1u);
    bool more = true;
#pragma unroll
    for (int s = 0; s < NS; ++s)
      if (more) more = issue(s, first[s]);
    if (!more) return;
    unsigned pending = atomicAdd(&a.hdr->ticket, 1u);
    for (unsigned j = NS;; ++j) {
      const int slot = j % NS;
      const unsigned t = pending;
      pending = atomicAdd(&a.hdr->ticket, 1u);  // in flight while this thread waits for the slot
      if (!mbar_wait_bounded(&s_freed[slot], ((j / NS) - 1u) & 1u, status)) return;
      if (!issue(slot, t)) return;
    }
  }

  // ---------------------------------------------------------------------- look-back warp
  if (warp == NW) {
    for (unsigned j = 0;; ++j) {
      const int slot = j % NS;
      const unsigned par = (j / NS) & 1u;
      if (!wait_all(&s_full[slot], par)) return;
      const unsigned tile = s_tile[slot];
      if (tile == kNoTile) return;
      if (!wait_all(&s_scanned[slot], par)) return;
      SegPair<A> tot{0u, A(0)};
      if (lane < NW) {
        tot.cnt = s_wtot_cnt[slot][lane];
        if constexpr (kSum) tot.val = s_wtot_val[slot][lane];
      }
      SegPair<A> inc = tot;
#pragma unroll
      for (int off = 1; off < NW; off <<= 1) {
        SegPair<A> o;
        o.cnt = __shfl_up_sync(0xffffffffu, inc.cnt, off);
        o.val = kSum ? __shfl_up_sync(0xffffffffu, inc.val, off) : A(0);
        if (lane >= off) inc = combine(o, inc);
      }
      SegPair<A> exc;  // warps in front of warp `lane`
      exc.cnt = __shfl_up_sync(0xffffffffu, inc.cnt, 1);
      exc.val = kSum ? __shfl_up_sync(0xffffffffu, inc.val, 1) : A(0);
      if (lane == 0) { exc.cnt = 0; exc.val = A(0); }
      SegPair<A> total;
      total.cnt = __shfl_sync(0xffffffffu, inc.cnt, NW - 1);
      total.val = kSum ? __shfl_sync(0xffffffffu, inc.val, NW - 1) : A(0);

      unsigned long long pc = 0;
      A pv = A(0);
      if (tile != 0) {
        if (lane == 0) {
          unsigned payload[4];
          DescWords<A>::pack(total.cnt, total.val, payload);
          publish<4>(&a.tiles[tile], kStateAggregate, payload);
        }
        lookback<A>(a.tiles, tile, status, pc, pv);
      }
      if (lane == 0) {
        const unsigned long long ic = pc + total.cnt;
        const A iv = total.cnt ? total.val : pv + total.val;
        unsigned payload[4];
        DescWords<A>::pack(ic, iv, payload);
        publish<4>(&a.tiles[tile], kStatePrefix, payload);
        if (tile == num_tiles - 1) {
          if constexpr (MODE == kReduceByKey) {  // close the last run
            if (ic > 0) a.vals_out[ic - 1] = iv;
          }
          if constexpr (!kScanOut) *a.num_out = ic;
        }
      }
      if (lane < NW) {  // state of the scan in front of compute warp `lane`
        s_wpre_cnt[slot][lane] = pc + exc.cnt;
        if constexpr (kSum) s_wpre_val[slot][lane] = exc.cnt ? exc.val : pv + exc.val;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_resolved[slot]);
    }
  }

  // ---------------------------------------------------------------------- compute warps
  const unsigned my_off = threadIdx.x * ITEMS;  // first element of this thread inside a tile
  struct Parked {
    unsigned heads;  // head / selection flags of the thread's items
    unsigned cnt;    // flags set in earlier lanes of the warp
    A val;           // sum of the run that is open in front of the thread, counted from the warp's first element
    unsigned fh;     // scan_by_key: first head of the warp's slice (kWarpItems: none)
  };

  // Phase C of the tile parked in `slot` at iteration jj.
  auto phase_c = [&](unsigned jj, const Parked& st) -> bool {
    const int slot = jj % NS;
    if (!wait_all(&s_resolved[slot], (jj / NS) & 1u)) return false;
    const unsigned tile = s_tile[slot];
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const K* sk = slot_keys(slot);
    const V* sv = slot_vals(slot);
    const unsigned long long wcnt = s_wpre_cnt[slot][warp];
    A wval = A(0);
    if constexpr (kSum) wval = s_wpre_val[slot][warp];
    if constexpr (kScanOut) {
      // the parked values are complete up to the warp's first head; in front of it the run
      // that was open at the start of the slice continues
      const Pack<V, E>* src = reinterpret_cast<const Pack<V, E>*>(sv + warp * S::kWarpItems);
      const uint64_t warp_base = tile_base + (uint64_t)warp * S::kWarpItems;
      const bool whole = (uint64_t)(tile + 1) * TILE <= n && a.bulk;  // a.bulk: the output is 16-byte aligned too
#pragma unroll
      for (int p = 0; p < kPacks; ++p) {
        const unsigned e0 = (p * kWarp + lane) * E;
        Pack<V, E> y = src[p * kWarp + lane];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          if (e0 + e < st.fh) y.v[e] = wval + y.v[e];
          if constexpr (MODE == kScanByKeyExcl) y.v[e] = a.init + y.v[e];
        }
        if (whole) {
          reinterpret_cast<Pack<V, E>*>(a.vals_out + warp_base)[p * kWarp + lane] = y;
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e)
            if (warp_base + e0 + e < n) a.vals_out[warp_base + e0 + e] = y.v[e];
        }
      }
    } else {
      unsigned heads = st.heads;
      if (heads) {
        unsigned long long at = wcnt + st.cnt;
        if constexpr (MODE == kReduceByKey) {
          // the run that closes at the thread's first head began in front of the thread
          A carried = st.cnt ? st.val : wval + st.val;
          while (heads) {
            const int i = __ffs(heads) - 1;
            heads &= heads - 1;
            const A r = i ? carried + sv[my_off + i - 1] : carried;
            if (at > 0) a.vals_out[at - 1] = r;
            a.keys_out[at] = sk[my_off + i];
            carried = A(0);
            ++at;
          }
        } else {
          while (heads) {
            const int i = __ffs(heads) - 1;
            heads &= heads - 1;
            if constexpr (MODE == kUniqueByKey) a.keys_out[at] = sk[my_off + i];
            if constexpr (kHasVals) a.vals_out[at] = sv[my_off + i];
            ++at;
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_freed[slot]);
    return true;
  };

  Parked parked[kPark];
#pragma unroll
  for (int p = 0; p < kPark; ++p) parked[p] = Parked{0u, 0u, A(0), 0u};
  unsigned j = 0;
  bool alive = true;
  for (;; ++j) {
    const int slot = j % NS;
    if (!wait_all(&s_full[slot], (j / NS) & 1u)) { alive = false; break; }
    const unsigned tile = s_tile[slot];
    if (tile == kNoTile) break;
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const uint64_t my_base = tile_base + my_off;
    const bool staged = a.bulk && (uint64_t)(tile + 1) * TILE <= n;  // the tile came by bulk copy
    K* sk = slot_keys(slot);
    V* sv = slot_vals(slot);
    Pack<K, E>* mk = reinterpret_cast<Pack<K, E>*>(sk + my_off);
    Pack<V, E>* mv = reinterpret_cast<Pack<V, E>*>(sv + my_off);

    // ---- phase A: this thread's items
    K k[ITEMS];
    V v[kHasVals ? ITEMS : 1];
    if (staged) {
#pragma unroll
      for (int p = 0; p < kPacks; ++p) {
        const Pack<K, E> kk = mk[p];
#pragma unroll
        for (int e = 0; e < E; ++e) k[p * E + e] = kk.v[e];
        if constexpr (kSum) {  // the selection kernels move values in phase C only
          const Pack<V, E> vv = mv[p];
#pragma unroll
          for (int e = 0; e < E; ++e) v[p * E + e] = vv.v[e];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const uint64_t g = my_base + i;
        k[i] = g < n ? a.keys[g] : K{};
        if constexpr (kHasVals) v[i] = g < n ? a.vals[g] : V{};
      }
      // phase C reads keys (and the selection kernels values) from the slot
#pragma unroll
      for (int p = 0; p < kPacks; ++p) {
        Pack<K, E> kk;
#pragma unroll
        for (int e = 0; e < E; ++e) kk.v[e] = k[p * E + e];
        mk[p] = kk;
        if constexpr (!kSum && kHasVals) {
          Pack<V, E> vv;
#pragma unroll
          for (int e = 0; e < E; ++e) vv.v[e] = v[p * E + e];
          mv[p] = vv;
        }
      }
    }
    unsigned heads = 0;
    if constexpr (MODE == kCopyFlagged) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) heads |= (unsigned)(k[i] != K(0)) << i;
    } else {
      // key in front of this thread's items
      K prev = __shfl_up_sync(0xffffffffu, k[ITEMS - 1], 1);
      if (lane == 0) {
        if (staged && warp > 0) prev = sk[my_off - 1];
        else prev = (my_base > 0 && my_base <= n) ? a.keys[my_base - 1] : K{};
      }
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) heads |= (unsigned)!(k[i] == (i == 0 ? prev : k[i - 1])) << i;
      if (my_base == 0) heads |= 1u;
    }
    if (!staged) {  // elements past the end are neither heads nor selected
      const uint64_t left = my_base < n ? n - my_base : 0;
      if (left < (uint64_t)ITEMS) heads &= (1u << (unsigned)left) - 1u;
    }

    Parked now;
    now.heads = heads;
    now.fh = 0;
    SegPair<A> s{(unsigned)__popc(heads), A(0)};
    A incl[kSum ? ITEMS : 1];
    if constexpr (kSum) {
      // run sums inside the thread: incl[i] = sum of element i's run, counted from the thread's first item
      incl[0] = v[0];
#pragma unroll
      for (int i = 1; i < ITEMS; ++i) incl[i] = (heads & (1u << i)) ? v[i] : incl[i - 1] + v[i];
      s.val = incl[ITEMS - 1];
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      SegPair<A> o;
      o.cnt = __shfl_up_sync(0xffffffffu, s.cnt, off);
      o.val = kSum ? __shfl_up_sync(0xffffffffu, s.val, off) : A(0);
      if (lane >= off) s = combine(o, s);
    }
    now.cnt = __shfl_up_sync(0xffffffffu, s.cnt, 1);
    now.val = kSum ? __shfl_up_sync(0xffffffffu, s.val, 1) : A(0);
    if (lane == 0) { now.cnt = 0; now.val = A(0); }
    if (lane == 31) {
      s_wtot_cnt[slot][warp] = s.cnt;
      if constexpr (kSum) s_wtot_val[slot][warp] = s.val;
    }
    // ---- park what phase C needs in the tile's own slot
    if constexpr (MODE == kReduceByKey) {
#pragma unroll
      for (int p = 0; p < kPacks; ++p) {
        Pack<V, E> rr;
#pragma unroll
        for (int e = 0; e < E; ++e) rr.v[e] = incl[p * E + e];
        mv[p] = rr;
      }
    } else if constexpr (kScanOut) {
      // values resolved inside the warp: the sum of the element's run counted from the warp's
      // first element (inclusive), or of the elements in front of it (exclusive)
      const A carry = now.val;  // open run in front of the thread
#pragma unroll
      for (int p = 0; p < kPacks; ++p) {
        Pack<V, E> rr;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int i = p * E + e;
          const bool no_head_yet = (heads & ((2u << i) - 1u)) == 0;  // no head among items 0..i
          const A inc_i = no_head_yet ? carry + incl[i] : incl[i];
          if constexpr (MODE == kScanByKeyIncl) {
            rr.v[e] = inc_i;
          } else {
            const bool head_i = heads & (1u << i);
            const bool none_before = i == 0 || (heads & ((1u << i) - 1u)) == 0;  // no head among items 0..i-1
            const A before = i == 0 ? carry : (none_before ? carry + incl[i - 1] : incl[i - 1]);
            rr.v[e] = head_i ? A(0) : before;
          }
        }
        mv[p] = rr;
      }
      const unsigned with_head = __ballot_sync(0xffffffffu, heads != 0);
      unsigned fh = S::kWarpItems;
      if (with_head) {
        const int fl = __ffs(with_head) - 1;
        const unsigned fheads = __shfl_sync(0xffffffffu, heads, fl);
        fh = (unsigned)fl * ITEMS + (unsigned)(__ffs(fheads) - 1);
      }
      now.fh = fh;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s_scanned[slot]);

    // ---- phase C of the tile this warp scanned kPark iterations ago
    if (j >= (unsigned)kPark) {
      if (!phase_c(j - kPark, parked[kPark - 1])) { alive = false; break; }
    }
#pragma unroll
    for (int p = kPark - 1; p > 0; --p) parked[p] = parked[p - 1];
    parked[0] = now;
  }
  if (alive) {
#pragma unroll
    for (int p = kPark; p >= 1; --p)
      if (j >= (unsigned)p && alive) alive = phase_c(j - p, parked[p - 1]);
  }
}

inline int sm_count(int* sms) {
  static int cached[64] = {};
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev]) { *sms = cached[dev]; return TB200_OK; }
  TB200_CUDA_TRY(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 64) cached[dev] = *sms;
  return TB200_OK;
}

template <typename K, typename V>
constexpr uint64_t tile_elems() { return (uint64_t)Shape<K, V>::kTile; }

// Scratch: header + one 32-byte descriptor per tile.
template <typename K, typename V>
size_t scratch_bytes(uint64_t n) {
  const uint64_t tiles = (n + tile_elems<K, V>() - 1) / tile_elems<K, V>();
  return kHeaderBytes + (size_t)tiles * sizeof(TileWords<4>);
}

// Launches the streaming kernel (n > 0, scratch cleared by the caller). `bulk`: keys, values and,
// for scan_by_key, the output are 16-byte aligned.
template <int MODE, typename K, typename V>
int launch(const K* keys, const V* vals, K* keys_out, V* vals_out, unsigned long long* num_out, uint64_t n, V init,
           bool bulk, void* d_temp, cudaStream_t stream) {
  using S = Shape<K, V>;
  const uint64_t tiles = (n + S::kTile - 1) / S::kTile;
  if (tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  Args<K, V> a;
  a.keys = keys;
  a.vals = vals;
  a.keys_out = keys_out;
  a.vals_out = vals_out;
  a.num_out = num_out;
  a.n = n;
  a.num_tiles = (unsigned)tiles;
  a.bulk = bulk ? 1 : 0;
  a.init = init;
  a.hdr = static_cast<TempHeader*>(d_temp);
  a.tiles = reinterpret_cast<TileWords<4>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  auto kernel = stream_kernel<MODE, K, V>;
  // opt in to the kernel's dynamic shared memory once per device (this function is one
  // instantiation per kernel, so the flag below belongs to this kernel alone)
  static unsigned long long prepared = 0;  // bit d: done on device d (benign race: the call is idempotent)
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 64 || !((prepared >> dev) & 1ull)) {
    TB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmem));
    if (dev < 64) prepared |= 1ull << dev;
  }
  int sms = 0;
  const int rc = sm_count(&sms);
  if (rc) return rc;
  const unsigned grid = (unsigned)(tiles < (uint64_t)sms ? tiles : (uint64_t)sms);
  kernel<<<grid, kCtaThreads, S::kSmem, stream>>>(a);
  return (int)cudaGetLastError();
}

}  // namespace seg
}  // namespace tb200
