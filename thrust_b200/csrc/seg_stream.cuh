// Streaming skeleton of the by-key algorithms (reduce_by_key, inclusive / exclusive
// scan_by_key, unique_by_key, copy of flagged elements): ONE pass over the input and no barrier
// that spans the whole CTA on the data path.
//
// A persistent CTA (one per SM) has these warps:
//   * one producer thread draws tiles from an atomic ticket counter and fills a ring of
//     shared-memory slots with bulk asynchronous copies (the untiled TMA form), keys and values
//     of a tile per slot, completion signalled on the slot's `full` mbarrier;
//   * two teams of kComputeWarps compute warps; tile j of the CTA belongs to team j % 2, and each
//     warp works on its own 32 x kItems slice of the tile WITHOUT synchronising with the other
//     warps: phase A (head flags, run sums inside the thread, one segmented warp scan, warp total
//     to shared memory; the LAST warp to get there combines the warp totals, publishes what other
//     tiles need with plain stores and arrives on the slot's `scanned` mbarrier) and, once the
//     slot's `resolved` mbarrier completes, phase C (emit, arrive on the slot's `freed`
//     mbarrier). A warp scans the next tile as soon as it has landed and emits as soon as a
//     parked tile is resolved; two teams keep sixteen such latency chains in flight per SM;
//   * look-back warps that take the CTA's tiles in turn and supply what a tile needs from the
//     tiles in front of it;
//   * scout warps (compacting algorithms only), see below.
//
// What a tile needs from its predecessors differs by algorithm, and nothing waits for more:
//   * scan_by_key needs the sum of the run that is open where the tile starts. A tile that holds
//     a head is final for its successors the moment it is scanned, so the look-back goes to the
//     NEAREST such tile (usually the one directly in front) instead of waiting for the slowest
//     of the hundreds of tiles in flight;
//   * reduce_by_key, unique and the copy of flagged elements need the NUMBER of heads in front of
//     the tile: that depends on all predecessors, so it is produced ahead of the data by the
//     scout warps (keys only, from L2-prefetched global memory) with a block-level chain, and is
//     read by the look-back warp while the tile is still loading. reduce_by_key's one value that
//     depends on other tiles (the run that the tile's first head closes) is stored by the
//     look-back warp from the same nearest-final-tile chain as scan_by_key; the compute warps
//     never wait for it.
// A tile therefore stays in its slot for load + scan + emit and no longer for the prefix of
// the whole grid. Every tile is drawn by ticket, so a tile is only ever owned by a CTA that is
// already running: no wait depends on an unscheduled CTA. Every wait (mbarrier, descriptor
// poll, idle loop, the scouts' throttle) is bounded and reports through the status word; the
// first one to give up records where.
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

// Single-level look-back over (count, value) descriptors by one warp, 32 predecessors per round
// (states EMPTY -> AGGREGATE -> PREFIX): the chain of the one-tile-per-CTA kernels that serve
// unaligned and tiny inputs. The operator is not commutative: far predecessors are combined on
// the left of near ones.
template <typename A>
__device__ void lookback_chain(const TileWords<4>* tiles, unsigned tile, int* status, unsigned long long& out_cnt,
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

// Look-back of the segmented scans (scan_by_key). Only the run that is open at the end of the
// predecessors matters, so a tile that contains a head is final the moment it is scanned: such a
// tile publishes its trailing run sum as PREFIX at once, a tile without a head publishes its
// total as AGGREGATE and, once its own look-back is done, the open run's sum as PREFIX. The walk
// goes back to the NEAREST prefix and waits for nothing older: with a head in most tiles that is
// the tile directly in front, not the slowest of all tiles in flight.
template <typename A>
__device__ void lookback_short(const TileWords<4>* tiles, unsigned tile, int* status, A& out_val) {
  const unsigned lane = lane_id();
  A acc = A(0);
  long long base = (long long)tile - 1;
  bool timed_out = false;
  unsigned long long missing = 0;
  while (base >= 0 && !timed_out) {
    const long long idx = base - lane;
    unsigned st = kStatePrefix;  // in front of the first tile: an empty prefix
    unsigned payload[4] = {0u, 0u, 0u, 0u};
    unsigned polls = 0, first = 0;
    bool unread = idx >= 0;  // this lane's descriptor has not been seen published yet
    while (true) {
      if (unread) {
        st = peek<4>(&tiles[idx], payload);
        unread = st == kStateEmpty;
      }
      const unsigned pm = __ballot_sync(0xffffffffu, st == kStatePrefix);
      const unsigned em = __ballot_sync(0xffffffffu, st == kStateEmpty);
      first = pm ? (unsigned)(__ffs(pm) - 1) : 31u;
      const unsigned needed = first == 31u ? 0xffffffffu : ((2u << first) - 1u);  // lanes up to the nearest prefix
      if ((em & needed) == 0u) break;
      backoff(++polls);
      if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(status) != 0)) {
        timed_out = true;
        missing = (unsigned long long)(base - (__ffs(em & needed) - 1));
        break;
      }
    }
    unsigned long long cnt = 0;
    A val = A(0);
    if (idx >= 0 && lane <= first && st != kStateEmpty) DescWords<A>::unpack(payload, cnt, val);
    const bool done = __any_sync(0xffffffffu, st == kStatePrefix);
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {  // ordered sum: farther tiles (higher lanes) on the left
      const A ov = __shfl_down_sync(0xffffffffu, val, off);
      if (lane + off < 32) val = ov + val;
    }
    val = __shfl_sync(0xffffffffu, val, 0);
    acc = val + acc;
    if (done) break;
    base -= 32;
  }
  if (timed_out && lane == 0) note_timeout(status, kSiteLookback, tile, missing);
  out_val = acc;
}

constexpr int kBlockTiles = 32;  // tiles per block of the count chain (one lane per tile)

// ---- the count chain of the compacting algorithms (reduce_by_key, unique, copy of flagged) ----
// Where a tile's output goes depends on the number of heads in ALL tiles in front of it, and a
// GPU at full HBM speed has hundreds of tiles in flight, some of them always a few microseconds
// late: a tile that waited for that count with its data parked in shared memory would hold its
// slot for most of its life. The counts are therefore produced AHEAD of the data by scout warps:
// a scout draws a tile from its own ticket counter, reads only the tile's keys (plain loads, no
// shared memory), counts the heads and publishes the count; the scout of a block's last tile
// adds up the block and resolves the block's prefix by look-back over the block descriptors.
// The scouts run a bounded number of tiles in front of the data tickets, so the keys they read
// are still in L2 when the data path loads them again, and a data tile finds its prefix already
// resolved: two descriptor reads, no waiting.
//   ctiles[t]  one word {state | heads in tile t}                         EMPTY -> AGGREGATE
//   cblocks[b] {0, heads in block b} then {0, heads in blocks 0..b}       EMPTY -> AGGREGATE -> PREFIX
__device__ __forceinline__ bool poll_count(const TileWords<1>* d, unsigned& cnt, int* status) {
  unsigned polls = 0;
  while (true) {
    const unsigned long long v = ld_relaxed_u64(&d->w[0]);
    if ((unsigned)(v >> 32) != kStateEmpty) {
      cnt = (unsigned)v;
      return true;
    }
    backoff(++polls);
    if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(status) != 0)) return false;
  }
}

// Heads in tiles [first, first + count) of one block, count <= 32 (one warp, all lanes).
__device__ __forceinline__ unsigned long long block_part(const TileWords<1>* ctiles, unsigned first, unsigned count,
                                                         int* status) {
  const unsigned lane = lane_id();
  unsigned c = 0;
  bool ok = true;
  if (lane < count) ok = poll_count(&ctiles[first + lane], c, status);
  if (!__all_sync(0xffffffffu, ok)) {
    if (lane == 0) note_timeout(status, kSiteBlockChain, first, count);
    return 0;
  }
  return (unsigned long long)__reduce_add_sync(0xffffffffu, c);
}

// Number of heads in front of `tile` (one warp, all lanes).
__device__ __forceinline__ unsigned long long count_prefix(const TileWords<1>* ctiles, const TileWords<4>* cblocks,
                                                           unsigned tile, int* status) {
  const unsigned b = tile / kBlockTiles;
  const unsigned long long inside = block_part(ctiles, b * kBlockTiles, tile % kBlockTiles, status);
  unsigned long long before = 0;
  lookback_short<unsigned long long>(cblocks, b, status, before);
  return before + inside;
}

// The scout of a block's last tile: the block's aggregate, then its inclusive prefix.
__device__ __forceinline__ void close_block(const TileWords<1>* ctiles, TileWords<4>* cblocks, unsigned b,
                                            unsigned tiles_in_block, int* status) {
  const unsigned lane = lane_id();
  const unsigned long long agg = block_part(ctiles, b * kBlockTiles, tiles_in_block, status);
  unsigned payload[4];
  if (lane == 0) {
    DescWords<unsigned long long>::pack(0ull, agg, payload);
    publish<4>(&cblocks[b], kStateAggregate, payload);
  }
  unsigned long long before = 0;
  lookback_short<unsigned long long>(cblocks, b, status, before);
  if (lane == 0) {  // same thread as the aggregate: the two sets of words cannot mix
    DescWords<unsigned long long>::pack(0ull, before + agg, payload);
    publish<4>(&cblocks[b], kStatePrefix, payload);
  }
}

// Asks the memory system to bring [p, p + bytes) into L2 (16-byte aligned, a multiple of 16 bytes):
// the bytes are in flight without a register or a shared-memory destination waiting for them.
__device__ __forceinline__ void prefetch_l2(const void* p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// L2 eviction priorities. The keys are read twice, a few microseconds apart (scouts, then the data
// path): they are brought in to stay (evict_last) and read the second time, like everything that is
// read once, as the first to go (evict_first).
__device__ __forceinline__ unsigned long long policy_evict_last() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ unsigned long long policy_evict_first() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void prefetch_l2_hint(const void* p, unsigned bytes, unsigned long long pol) {
  asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(p), "r"(bytes), "l"(pol) : "memory");
}
__device__ __forceinline__ void bulk_load_hint(void* smem_dst, const void* gmem_src, unsigned bytes,
                                               unsigned long long* bar, unsigned long long pol) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
               : "memory");
}
// read-only 16-byte load that the compiler may schedule freely (measured: keeping the lines in L1 and
// dropping `volatile` took unique_by_key from 0.48 to 0.45 ms)
__device__ __forceinline__ uint4 ld_stream_v4(const uint4* p) {
  uint4 r;
  asm("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Heads (FLAGS: non-zero elements) of one whole tile of NP 16-byte packs that starts at the
// 16-byte aligned keys + base; one warp. The scouts share their SM's issue slots with sixteen
// compute warps, so what counts here is the number of instructions per pack: lane-strided
// 16-byte loads kept U deep in flight (a pack is counted, then its buffer is loaded again), and
// the element in front of a pack by a small load of its own that travels with the pack (it hits
// L1: the line belongs to the neighbouring lane's pack). No shuffle: nothing orders the rows, so
// their latencies overlap.
template <typename K, bool FLAGS, int NP>
__device__ unsigned count_heads_tile(const K* keys, uint64_t base) {
  constexpr int EP = 16 / (int)sizeof(K);
  constexpr int ROWS = (NP + kWarp - 1) / kWarp;
  constexpr int U = ROWS < 8 ? ROWS : 8;
  constexpr bool kRagged = NP % kWarp != 0;  // the last row is not full
  const unsigned lane = lane_id();
  const uint4* src = reinterpret_cast<const uint4*>(keys + base);
  const K* first = keys + base;
  uint4 q[U];
  K front[U];  // the element in front of the pack: the line is in L1 (the neighbouring lane's pack)
  auto load = [&](int r, uint4& qq, K& ff) {
    const unsigned pk = (unsigned)r * kWarp + lane;
    const bool in = !kRagged || pk < (unsigned)NP;
    qq = in ? ld_stream_v4(src + pk) : uint4{0u, 0u, 0u, 0u};
    if constexpr (!FLAGS) ff = (in && (base != 0 || pk != 0)) ? first[(long long)pk * EP - 1] : K{};
  };
#pragma unroll
  for (int u = 0; u < U; ++u) load(u, q[u], front[u]);
  unsigned cnt = 0;
#pragma unroll 1
  for (int r0 = 0; r0 < ROWS; r0 += U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + u;
      if (ROWS % U == 0 || r < ROWS) {  // the same for all lanes
        const Pack<K, EP> e = *reinterpret_cast<const Pack<K, EP>*>(&q[u]);
        const K prev = front[u];
        if (r + U < ROWS) load(r + U, q[u], front[u]);
        const unsigned pk = (unsigned)r * kWarp + lane;
        const bool in = !kRagged || pk < (unsigned)NP;
        unsigned c = 0;
        if constexpr (FLAGS) {
#pragma unroll
          for (int i = 0; i < EP; ++i) c += (unsigned)(e.v[i] != K(0));
        } else {
          c = (unsigned)((base == 0 && pk == 0) || !(e.v[0] == prev));  // the input's first element is a head
#pragma unroll
          for (int i = 1; i < EP; ++i) c += (unsigned)!(e.v[i] == e.v[i - 1]);
        }
        cnt += in ? c : 0u;
      }
    }
  }
  return __reduce_add_sync(0xffffffffu, cnt);
}

// The same for any `count` elements of keys[base, base + count): the last tile of an input and
// inputs that are not 16-byte aligned. Element-wise, coalesced; one warp.
template <typename K, bool FLAGS>
__device__ unsigned count_heads_any(const K* keys, uint64_t base, unsigned count, uint64_t n) {
  const unsigned lane = lane_id();
  constexpr int U = 8;
  unsigned cnt = 0;
  K carry = K{};  // element in front of lane 0's next one
  if (!FLAGS && base > 0) carry = keys[base - 1];
  for (unsigned i0 = 0; i0 < count; i0 += kWarp * U) {
    K e[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t g = base + i0 + u * kWarp + lane;
      e[u] = (i0 + u * kWarp + lane < count && g < n) ? keys[g] : K{};
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t g = base + i0 + u * kWarp + lane;
      const bool in = i0 + u * kWarp + lane < count && g < n;
      if constexpr (FLAGS) {
        cnt += (unsigned)(in && e[u] != K(0));
      } else {
        K prev = __shfl_up_sync(0xffffffffu, e[u], 1);
        const K wrap = __shfl_sync(0xffffffffu, e[u], 31);
        if (lane == 0) prev = carry;
        carry = wrap;
        cnt += (unsigned)(in && (g == 0 || !(e[u] == prev)));
      }
    }
  }
  return __reduce_add_sync(0xffffffffu, cnt);
}

constexpr int kComputeWarps = 8;  // warps of one team: a tile is split over them
constexpr int kComputeThreads = kComputeWarps * kWarp;
constexpr int kTeams = 2;      // teams of compute warps; tile j of a CTA belongs to team j % kTeams
constexpr int kLookWarps = 2;  // look-back warps; tile j of a CTA is resolved by warp j % kLookWarps
// Warps that count heads ahead of the data (compacting algorithms only). Measured: the scouts take issue
// slots from the compute warps, so an algorithm gets as few as keep its counts ahead: reduce_by_key and
// the copy of flagged elements (whose compute warps do the most per tile) 4, unique_by_key 5, keys-only
// unique (the cheapest tiles, so the fastest consumer) 6.
constexpr int scout_warps(int mode, bool has_vals) {
  return (mode == 1 || mode == 2) ? 0 : (mode == 0 || mode == 4) ? 4 : (has_vals ? 5 : 6);
}
constexpr unsigned kScoutAhead = 1536;  // tiles a scout may run in front of the data tickets (their keys stay in L2)
constexpr unsigned kScoutPrefetch = 512;  // a scout that draws tile u asks for the keys of tile u + kScoutPrefetch
constexpr int kStops = kLookWarps > kTeams ? kLookWarps : kTeams;  // "no tile" slots that end the roles
constexpr int kRoleWarp0 = kTeams * kComputeWarps;  // first warp that is not a compute warp
// compute warps + look-back warps + producer (+ scouts: the segmented scans compact nothing and run without)
constexpr int cta_threads(int mode, bool has_vals) {
  return (kRoleWarp0 + kLookWarps + 1 + scout_warps(mode, has_vals)) * kWarp;
}
constexpr int kScoutTicket = 8;  // TempHeader::aux word that deals tiles to the scouts
constexpr int kPacks = 5;   // 16-byte packs of the wider type per thread: an 80-byte stride has no bank conflicts
constexpr int kStages = 5;  // ring slots: one or two loading, one being scanned, the rest parked
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
  int inplace;                  // an output overlaps its input (unique): a tile is overwritten only after it was read
  V init;                       // exclusive scan_by_key
  TempHeader* hdr;
  TileWords<4>* tiles;    // value chain, one descriptor per tile: EMPTY -> AGGREGATE -> PREFIX
  TileWords<4>* cblocks;  // count chain, one per block of kBlockTiles tiles
  TileWords<1>* ctiles;   // count chain, one word per tile
};

template <int MODE, typename V> struct AccOf { using type = unsigned; };
template <typename V> struct AccOf<kReduceByKey, V> { using type = V; };
template <typename V> struct AccOf<kScanByKeyIncl, V> { using type = V; };
template <typename V> struct AccOf<kScanByKeyExcl, V> { using type = V; };

template <int MODE, typename K, typename V>
__global__ void __launch_bounds__(cta_threads(MODE, !std::is_same<V, NoVal>::value), 1) stream_kernel(const Args<K, V> a) {
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
  __shared__ __align__(8) unsigned long long s_full[NS], s_scanned[NS], s_resolved[NS], s_freed[NS], s_issued[NS];
  __shared__ unsigned s_tile[NS];
  __shared__ __align__(16) unsigned char s_halo[NS][16];  // the 16 bytes of keys in front of the slot's tile
  __shared__ unsigned s_arrivals[NS];        // compute warps that have finished phase A of the slot's tile
  __shared__ unsigned s_wtot_cnt[NS][NW];    // warp totals, then (same cells) the warps' exclusive prefixes inside the tile
  __shared__ A s_wtot_val[NS][NW];
  __shared__ unsigned s_tot_cnt[NS];         // tile aggregate
  __shared__ A s_tot_val[NS];
  __shared__ A s_wlead[NS][NW];              // reduce_by_key: sum of the warp's elements in front of its first head
  __shared__ A s_lead[NS];                   // reduce_by_key: the same for the whole tile
  __shared__ unsigned long long s_pc[NS];  // compacting algorithms: heads in front of the tile, set by the look-back warp
  __shared__ A s_wpre_val[NS][NW];         // scan_by_key: run open in front of every warp, set by the look-back warp
  // what a thread keeps of a scanned tile until its prefix is known (per slot)
  __shared__ unsigned s_park_heads[NS][kComputeThreads];  // head / selection flags of the thread's items
  __shared__ unsigned s_park_cnt[NS][kComputeThreads];    // flags set in earlier lanes of the warp
  __shared__ A s_park_val[kSum ? NS : 1][kComputeThreads];  // run open in front of the thread, from the warp's first element
  __shared__ unsigned s_park_fh[NS][NW];  // scan_by_key: first head of the warp's slice (kWarpItems: none)

  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  const unsigned team = warp / NW;                         // compute warps: the team ...
  const unsigned w = warp % NW;                            // ... the warp's place in it ...
  const unsigned tid = threadIdx.x % kComputeThreads;      // ... and the thread's
  int* status = &a.hdr->status;
  const uint64_t n = a.n;
  const unsigned num_tiles = a.num_tiles;
  auto slot_keys = [&](int slot) { return reinterpret_cast<K*>(ring + (size_t)slot * S::kSlotBytes); };
  auto slot_vals = [&](int slot) { return reinterpret_cast<V*>(ring + (size_t)slot * S::kSlotBytes + S::kValOffset); };

  // a wait whose outcome all lanes of the calling warp agree on (a time-out ends the whole warp's role)
  auto wait_all = [&](unsigned long long* bar, unsigned parity) -> bool {
    return __all_sync(0xffffffffu, mbar_wait_bounded(bar, parity, status));
  };
  // non-blocking: has the phase completed? (one answer for the whole warp: lane 0's)
  auto ready = [&](unsigned long long* bar, unsigned parity) -> bool {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
  };

  // A parity wait tells "phase r completed" apart from "not yet" only for an observer that is at
  // most one phase away from the barrier. A slot's successive tiles go to DIFFERENT teams and
  // look-back warps, and tiles land out of order when several loads are in flight, so a warp that
  // has finished tile j-2 or j-3 may ask for tile j while the slot's previous tenant, tile j-NS, has
  // not even landed: the parity test would then answer for the phase before. Whoever did not
  // handle the previous tenant itself therefore first checks that the tenant has been FREED
  // (that barrier it cannot be two phases away from: tile j-NS is issued before every tile the
  // warp has seen, and only after tile j-2NS was freed).
  auto landed = [&](unsigned jj) -> bool {  // non-blocking: tile jj of the CTA is in its slot
    const int s = jj % NS;
    const unsigned r = jj / NS;
    return (r == 0 || ready(&s_freed[s], (r - 1u) & 1u)) && ready(&s_full[s], r & 1u);
  };
  auto wait_issued = [&](unsigned jj) -> bool {  // blocking (bounded): s_tile of tile jj is set
    const int s = jj % NS;
    const unsigned r = jj / NS;
    return (r == 0 || wait_all(&s_freed[s], (r - 1u) & 1u)) && wait_all(&s_issued[s], r & 1u);
  };
  auto wait_landed = [&](unsigned jj) -> bool {  // blocking (bounded)
    const int s = jj % NS;
    const unsigned r = jj / NS;
    return (r == 0 || wait_all(&s_freed[s], (r - 1u) & 1u)) && wait_all(&s_full[s], r & 1u);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_scanned[s], 1);
      mbar_init(&s_resolved[s], 1);
      mbar_init(&s_freed[s], NW);
      mbar_init(&s_issued[s], 1);
      s_arrivals[s] = 0;
    }
    if (blockIdx.x == 0) {  // decodes a recorded mbarrier time-out
      a.hdr->aux[4] = smem_u32(&s_full[0]);
      a.hdr->aux[5] = smem_u32(&s_scanned[0]);
      a.hdr->aux[6] = smem_u32(&s_resolved[0]);
      a.hdr->aux[7] = smem_u32(&s_freed[0]);
    }
    mbar_init_fence();
  }
  __syncthreads();  // the only CTA-wide barrier of the kernel

  // ---------------------------------------------------------------------- producer
  if (warp == kRoleWarp0 + kLookWarps) {
    if (lane != 0) return;
    const unsigned long long pol_first = policy_evict_first();
    // tile t goes into `slot`; false when the tickets have run past the last tile
    auto issue = [&](int slot, unsigned t) -> bool {
      if (t >= num_tiles) {
        s_tile[slot] = kNoTile;
        mbar_arrive(&s_issued[slot]);
        mbar_arrive(&s_full[slot]);
        return false;
      }
      s_tile[slot] = t;
      mbar_arrive(&s_issued[slot]);  // the look-back warp may resolve the tile's count while the tile loads
      if (a.bulk && (uint64_t)(t + 1) * TILE <= n) {
        fence_proxy_async_smem();  // the slot was last written by ordinary stores (parked values)
        constexpr bool kNeedsPrev = MODE != kCopyFlagged;  // the key in front of the tile decides its first head
        mbar_expect_tx(&s_full[slot], S::kKeyBytes + S::kValBytes + ((kNeedsPrev && t != 0) ? 16 : 0));
        if (kNeedsPrev && t != 0)
          bulk_load(s_halo[slot], reinterpret_cast<const unsigned char*>(a.keys + (uint64_t)t * TILE) - 16, 16, &s_full[slot]);
        if constexpr (kScanOut) {
          bulk_load(slot_keys(slot), a.keys + (uint64_t)t * TILE, S::kKeyBytes, &s_full[slot]);
          bulk_load(slot_vals(slot), a.vals + (uint64_t)t * TILE, S::kValBytes, &s_full[slot]);
        } else {  // second and last read of the keys, only read of the values: first to leave L2
          bulk_load_hint(slot_keys(slot), a.keys + (uint64_t)t * TILE, S::kKeyBytes, &s_full[slot], pol_first);
          if constexpr (kHasVals)
            bulk_load_hint(slot_vals(slot), a.vals + (uint64_t)t * TILE, S::kValBytes, &s_full[slot], pol_first);
        }
      } else {
        mbar_arrive(&s_full[slot]);  // ragged last tile or unaligned input: the compute warps load it themselves
      }
      return true;
    };
    // After the last tile, kStops further slots are marked "no tile": every look-back warp and
    // every team of compute warps meets one and stops.
    // The first ring-full is drawn one ticket at a time, each after the previous tile has landed:
    // all CTAs start together, so their draws interleave and a CTA's k-th tile comes k rounds
    // after its first in ticket order too. (Drawn in one burst, a CTA's first tiles would be
    // consecutive tickets; every other CTA's first look-back would then wait for tiles this CTA
    // scans several iterations later, and the whole grid would start up one CTA after the other.)
    int stops = 0;
    for (int s = 0; s < NS && stops < kStops; ++s) {
      if (!issue(s, stops ? kNoTile : atomicAdd(&a.hdr->ticket, 1u))) ++stops;
      if (!mbar_wait_bounded(&s_full[s], 0u, status)) return;
    }
    // A ticket is drawn only when its slot is free: a drawn tile starts loading at once, so no
    // tile that successors will wait for sits idle.
    for (unsigned j = NS; stops < kStops; ++j) {
      const int slot = j % NS;
      if (!mbar_wait_bounded(&s_freed[slot], ((j / NS) - 1u) & 1u, status)) return;
      if (!issue(slot, stops ? kNoTile : atomicAdd(&a.hdr->ticket, 1u))) ++stops;
    }
    return;
  }

  // ---------------------------------------------------------------------- scout warps
  if (warp > kRoleWarp0 + kLookWarps) {
    if constexpr (kScanOut) {
      return;  // the segmented scans compact nothing
    } else {
      unsigned long long* scout_ticket = &a.hdr->aux[kScoutTicket];
      const unsigned long long pol_last = policy_evict_last();
      unsigned seen = 0;  // data tickets known to have been drawn
      while (true) {
        // (a ticket drawn ahead of its turn would sit idle for a whole tile while others wait for it)
        unsigned u = 0;
        if (lane == 0) u = (unsigned)atomicAdd(scout_ticket, 1ull);
        u = __shfl_sync(0xffffffffu, u, 0);
        if (u >= num_tiles) return;
        // The scouts read half of what the kernel takes from HBM; registers cannot hold that many
        // bytes in flight, an L2 prefetch issued a few microseconds ahead can. Every tile is asked
        // for exactly once, by the scout that draws the ticket kScoutPrefetch below it.
        if (lane == 0 && reinterpret_cast<uintptr_t>(a.keys) % 16 == 0) {
          const uint64_t pf = (uint64_t)u + kScoutPrefetch;
          if ((pf + 1) * TILE <= n) prefetch_l2_hint(a.keys + pf * TILE, S::kKeyBytes, pol_last);
        }
        // stay within reach of the data path, so that the keys read here are still in L2 when the
        // tile is loaded again. (Tile u only waits while a data ticket below u - kScoutAhead is
        // still to be drawn, and no data tile ever waits for a scout in front of it.)
        unsigned waits = 0;
        while (u > seen + kScoutAhead) {
          seen = ld_relaxed_u32(&a.hdr->ticket);
          if (u <= seen + kScoutAhead) break;
          __nanosleep(500);
          if (++waits >= kSpinLimit || ((waits & 255u) == 0 && ld_relaxed_s32(status) != 0)) {
            if (lane == 0 && waits >= kSpinLimit) note_timeout(status, kSiteIdle, u, 1);
            return;
          }
        }
        const uint64_t base = (uint64_t)u * TILE;
        const bool whole = (uint64_t)(u + 1) * TILE <= n;
        const unsigned heads = (whole && reinterpret_cast<uintptr_t>(a.keys) % 16 == 0)
            ? count_heads_tile<K, MODE == kCopyFlagged, S::kKeyBytes / 16>(a.keys, base)
            : count_heads_any<K, MODE == kCopyFlagged>(a.keys, base, whole ? (unsigned)TILE : (unsigned)(n - base), n);
        if (lane == 0) {
          const unsigned payload[1] = {heads};
          publish<1>(&a.ctiles[u], kStateAggregate, payload);
        }
        if (u % kBlockTiles == kBlockTiles - 1 || u == num_tiles - 1)  // the block's last tile
          close_block(a.ctiles, a.cblocks, u / kBlockTiles, u % kBlockTiles + 1, status);
      }
    }
  }

  // ---------------------------------------------------------------------- look-back warps
  if (warp >= kRoleWarp0) {
    unsigned checked = 0;  // in-place runs: every tile in [first tile the last output touched, checked) has been read
    for (unsigned j = warp - kRoleWarp0;; j += kLookWarps) {
      const int slot = j % NS;
      const unsigned par = (j / NS) & 1u;
      if (!wait_issued(j)) return;
      const unsigned tile = s_tile[slot];
      if (tile == kNoTile) return;
      unsigned long long pc = 0;  // heads in front of the tile: the scouts' work, read while the tile loads
      if constexpr (!kScanOut) {
        pc = count_prefix(a.ctiles, a.cblocks, tile, status);
        if (a.inplace) {
          // The output overwrites the input from element pc on: every tile from there up to this
          // one must have been read (scanned tiles have published a descriptor). Tiles below
          // `checked` are known to be.
          unsigned t0 = (unsigned)(pc / TILE);
          if (t0 < checked) t0 = checked;
          unsigned polls = 0;
          while (t0 < tile) {
            const unsigned idx = t0 + lane;
            const bool done = idx >= tile || (unsigned)(ld_relaxed_u64(&a.tiles[idx].w[0]) >> 32) != kStateEmpty;
            const unsigned waiting = __ballot_sync(0xffffffffu, !done);
            if (waiting == 0) { t0 += kWarp; continue; }
            t0 += (unsigned)(__ffs(waiting) - 1);
            backoff(++polls);
            if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(status) != 0)) {
              if (lane == 0 && polls >= kSpinLimit) note_timeout(status, kSiteLookback, tile, t0);
              return;
            }
          }
          checked = tile;
          // ... and by its scout: the scouts of the tiles in front are done (their counts are in
          // pc), this tile's own may still be reading the keys this tile is about to overwrite
          unsigned own = 0;
          if (!poll_count(&a.ctiles[tile], own, status)) {
            if (lane == 0) note_timeout(status, kSiteBlockChain, tile, 1);
            return;
          }
        }
      }
      if (!wait_landed(j)) return;
      if (!wait_all(&s_scanned[slot], par)) return;
      SegPair<A> total{s_tot_cnt[slot], A(0)};
      if constexpr (kSum) total.val = s_tot_val[slot];
      A pv = A(0);
      if constexpr (kScanOut) {
        A exc = A(0);  // warps in front of warp `lane` inside the tile
        unsigned exc_cnt = 0;
        if (lane < NW) {
          exc_cnt = s_wtot_cnt[slot][lane];
          exc = s_wtot_val[slot][lane];
        }
        lookback_short<A>(a.tiles, tile, status, pv);
        if (total.cnt == 0 && lane == 0) {  // no head in the tile: the run open in front of it goes on
          unsigned payload[4];
          DescWords<A>::pack(0ull, pv + total.val, payload);
          publish<4>(&a.tiles[tile], kStatePrefix, payload);  // second writer of the descriptor, ordered after the first by the `scanned` barrier
        }
        if (lane < NW) s_wpre_val[slot][lane] = exc_cnt ? exc : pv + exc;  // run open in front of compute warp `lane`
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_resolved[slot]);
      } else {
        // The compute warps need only the count: hand it over, then settle the one value that
        // depends on other tiles (the run that the tile's first head closes).
        A lead = A(0);
        if constexpr (MODE == kReduceByKey) lead = s_lead[slot];
        if (lane == 0) s_pc[slot] = pc;
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_resolved[slot]);
        if (tile == num_tiles - 1 && lane == 0) *a.num_out = pc + total.cnt;
        if constexpr (MODE == kReduceByKey) {
          lookback_short<A>(a.tiles, tile, status, pv);
          if (lane == 0) {
            if (total.cnt == 0) {
              unsigned payload[4];
              DescWords<A>::pack(0ull, pv + total.val, payload);
              publish<4>(&a.tiles[tile], kStatePrefix, payload);
            } else if (pc > 0) {
              a.vals_out[pc - 1] = pv + lead;
            }
            if (tile == num_tiles - 1) {  // close the last run
              const unsigned long long ic = pc + total.cnt;
              if (ic > 0) a.vals_out[ic - 1] = total.cnt ? total.val : pv + total.val;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- compute warps
  const unsigned my_off = tid * ITEMS;  // first element of this thread inside a tile
  struct Parked {
    unsigned heads, cnt;
    A val;
    unsigned fh;
  };

  // Phase C of the tile parked in the slot of iteration jj (its prefix has been resolved).
  auto phase_c = [&](unsigned jj) -> bool {
    const int slot = jj % NS;
    if (!wait_all(&s_resolved[slot], (jj / NS) & 1u)) return false;  // returns at once: the caller saw it complete
    Parked st;
    st.heads = s_park_heads[slot][tid];
    st.cnt = s_park_cnt[slot][tid];
    st.val = A(0);
    if constexpr (kSum) st.val = s_park_val[slot][tid];
    st.fh = s_park_fh[slot][w];
    const unsigned tile = s_tile[slot];
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const K* sk = slot_keys(slot);
    const V* sv = slot_vals(slot);
    const unsigned wexc = s_wtot_cnt[slot][w];  // heads in the warps in front of this one inside the tile
    unsigned long long wcnt = 0;                // heads in front of the warp
    if constexpr (!kScanOut) wcnt = s_pc[slot] + wexc;
    A wval = A(0);  // run open in front of the warp: over all tiles (scan_by_key), inside the tile (reduce_by_key)
    if constexpr (kScanOut) wval = s_wpre_val[slot][w];
    else if constexpr (kSum) wval = s_wtot_val[slot][w];
    if constexpr (kScanOut) {
      // the parked values are complete up to the warp's first head; in front of it the run
      // that was open at the start of the slice continues
      const Pack<V, E>* src = reinterpret_cast<const Pack<V, E>*>(sv + w * S::kWarpItems);
      const uint64_t warp_base = tile_base + (uint64_t)w * S::kWarpItems;
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
      bool emitted = false;
      if constexpr (MODE != kReduceByKey) {
        // Many selected in the warp's slice: compact the slice in place in shared memory (read
        // everything, synchronise, write each selected element to its rank), then copy it out with
        // consecutive lanes writing consecutive elements. (Per-thread stores of ten elements each
        // would touch thirty-two lines per instruction.)
        const unsigned wtotal = __reduce_add_sync(0xffffffffu, (unsigned)__popc(heads));
        if (wtotal * 3 > (unsigned)S::kWarpItems) {
          K* wk = const_cast<K*>(sk) + w * S::kWarpItems;
          V* wv = const_cast<V*>(sv) + w * S::kWarpItems;
          const unsigned lo = lane * ITEMS;  // this thread's items inside the slice
          K kk[MODE == kUniqueByKey ? ITEMS : 1];
          V vv[kHasVals ? ITEMS : 1];
#pragma unroll
          for (int i = 0; i < ITEMS; ++i) {
            if constexpr (MODE == kUniqueByKey) kk[i] = wk[lo + i];
            if constexpr (kHasVals) vv[i] = wv[lo + i];
          }
          __syncwarp();
          unsigned r = st.cnt;  // selected in the lanes in front
#pragma unroll
          for (int i = 0; i < ITEMS; ++i) {
            if (heads & (1u << i)) {
              if constexpr (MODE == kUniqueByKey) wk[r] = kk[i];
              if constexpr (kHasVals) wv[r] = vv[i];
              ++r;
            }
          }
          __syncwarp();
          for (unsigned i = lane; i < wtotal; i += kWarp) {
            if constexpr (MODE == kUniqueByKey) a.keys_out[wcnt + i] = wk[i];
            if constexpr (kHasVals) a.vals_out[wcnt + i] = wv[i];
          }
          emitted = true;
        }
      }
      if (heads && !emitted) {
        unsigned long long at = wcnt + st.cnt;
        if constexpr (MODE == kReduceByKey) {
          // the run that closes at the thread's first head began in front of the thread
          A carried = st.cnt ? st.val : wval + st.val;
          // The run that the TILE's first head closes began in another tile: its sum is stored by
          // the look-back warp, the only one to wait for other tiles' values.
          bool other_tile = wexc == 0 && st.cnt == 0;
          while (heads) {
            const int i = __ffs(heads) - 1;
            heads &= heads - 1;
            const A r = i ? carried + sv[my_off + i - 1] : carried;
            if (at > 0 && !other_tile) a.vals_out[at - 1] = r;
            other_tile = false;
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

  // Every warp schedules itself: it scans the next tile as soon as the tile has landed (so the
  // tile's aggregate reaches the other CTAs as early as possible, whatever this CTA is still
  // waiting for) and emits the oldest parked tile as soon as its prefix is resolved; it idles
  // only when neither is possible.
  unsigned j = team;       // next tile of the CTA for this team to scan
  unsigned j_emit = team;  // the team's oldest scanned tile not yet emitted
  bool more = true;     // the producer has not run out of tiles
  unsigned idle = 0;
  while (more || j_emit < j) {
    if (j_emit < j && ready(&s_resolved[j_emit % NS], (j_emit / NS) & 1u)) {
      if (!phase_c(j_emit)) return;
      j_emit += kTeams;
      idle = 0;
      continue;
    }
    if (!(more && landed(j))) {
      if (++idle > (1u << 24) || ((idle & 4095u) == 0 && ld_relaxed_s32(status) != 0)) {  // bounded
        if (lane == 0 && idle > (1u << 24)) note_timeout(status, kSiteIdle, ((unsigned long long)j << 32) | j_emit, team);
        return;
      }
      if (idle > 64) __nanosleep(40);
      continue;
    }
    idle = 0;
    const int slot = j % NS;
    if (!wait_all(&s_full[slot], (j / NS) & 1u)) return;  // returns at once
    const unsigned tile = s_tile[slot];
    if (tile == kNoTile) { more = false; continue; }
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
        if (staged && w > 0) prev = sk[my_off - 1];
        else if (staged && tile != 0) prev = *reinterpret_cast<const K*>(&s_halo[slot][16 - sizeof(K)]);
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

    int lead_lane = -1;  // reduce_by_key: the lane that holds the warp's first head
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
      s_wtot_cnt[slot][w] = s.cnt;
      if constexpr (kSum) s_wtot_val[slot][w] = s.val;
    }
    if constexpr (MODE == kReduceByKey) {
      // sum of the warp's elements in front of its first head (the whole warp if it has none)
      const unsigned with_head = __ballot_sync(0xffffffffu, heads != 0);
      if (with_head == 0) {
        if (lane == 31) s_wlead[slot][w] = s.val;
      }
      lead_lane = with_head ? __ffs(with_head) - 1 : -1;
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
    if constexpr (MODE == kReduceByKey) {
      if ((int)lane == lead_lane) {  // the lanes in front of this one have no head; its run sums are parked above
        const int i0 = __ffs(heads) - 1;
        s_wlead[slot][w] = i0 ? now.val + sv[my_off + i0 - 1] : now.val;
      }
    }
    s_park_heads[slot][tid] = now.heads;
    s_park_cnt[slot][tid] = now.cnt;
    if constexpr (kSum) s_park_val[slot][tid] = now.val;
    if (lane == 0) s_park_fh[slot][w] = now.fh;
    __syncwarp();
    // The last warp to finish phase A of this tile combines the warp totals (in warp order) and
    // publishes the tile's aggregate.
    unsigned last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(&s_arrivals[slot], 1u) == (unsigned)(NW - 1);
      __threadfence_block();
    }
    if (__shfl_sync(0xffffffffu, last, 0)) {
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
      SegPair<A> exc;
      exc.cnt = __shfl_up_sync(0xffffffffu, inc.cnt, 1);
      exc.val = kSum ? __shfl_up_sync(0xffffffffu, inc.val, 1) : A(0);
      if (lane == 0) { exc.cnt = 0; exc.val = A(0); }
      if (lane < NW) {  // the totals have been read by this warp: the cells now hold the exclusive prefixes
        s_wtot_cnt[slot][lane] = exc.cnt;
        if constexpr (kSum) s_wtot_val[slot][lane] = exc.val;
      }
      if constexpr (MODE == kReduceByKey) {
        const unsigned hm = __ballot_sync(0xffffffffu, lane < NW && tot.cnt != 0);
        if (hm && lane == (unsigned)(__ffs(hm) - 1)) s_lead[slot] = exc.val + s_wlead[slot][lane];
      }
      if (lane == NW - 1) {
        s_tot_cnt[slot] = inc.cnt;
        if constexpr (kSum) {
          s_tot_val[slot] = inc.val;
          unsigned payload[4];
          DescWords<A>::pack(inc.cnt, inc.val, payload);
          // The value chain (plain stores: nothing is waited for). Only the run open at the end
          // of a tile matters to its successors, so a tile that holds a head is final at once.
          publish<4>(&a.tiles[tile], inc.cnt ? kStatePrefix : kStateAggregate, payload);
        }
        else if (a.inplace) {  // the tile's input is in shared memory now: it may be overwritten
          st_relaxed_u64(&a.tiles[tile].w[0], (unsigned long long)kStateAggregate << 32);
        }
        s_arrivals[slot] = 0;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_scanned[slot]);  // hands the tile to its look-back warp
    }

    j += kTeams;
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

// Scratch: header + a 32-byte value descriptor per tile + a 32-byte count descriptor per block
// of tiles + an 8-byte count word per tile.
template <typename K, typename V>
size_t scratch_bytes(uint64_t n) {
  const uint64_t tiles = (n + tile_elems<K, V>() - 1) / tile_elems<K, V>();
  const uint64_t blocks = (tiles + kBlockTiles - 1) / kBlockTiles;
  return kHeaderBytes + (size_t)(tiles + blocks) * sizeof(TileWords<4>) + (size_t)tiles * sizeof(TileWords<1>);
}

// Launches the streaming kernel (n > 0, scratch cleared by the caller). `bulk`: keys, values and,
// for scan_by_key, the output are 16-byte aligned.
template <int MODE, typename K, typename V>
int launch(const K* keys, const V* vals, K* keys_out, V* vals_out, unsigned long long* num_out, uint64_t n, V init,
           bool bulk, void* d_temp, cudaStream_t stream, bool inplace = false) {
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
  a.inplace = inplace ? 1 : 0;
  a.init = init;
  a.hdr = static_cast<TempHeader*>(d_temp);
  a.tiles = reinterpret_cast<TileWords<4>*>(static_cast<char*>(d_temp) + kHeaderBytes);
  a.cblocks = a.tiles + tiles;
  a.ctiles = reinterpret_cast<TileWords<1>*>(a.cblocks + (tiles + kBlockTiles - 1) / kBlockTiles);
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
  kernel<<<grid, cta_threads(MODE, S::kHasVals), S::kSmem, stream>>>(a);
  return (int)cudaGetLastError();
}

}  // namespace seg
}  // namespace tb200
