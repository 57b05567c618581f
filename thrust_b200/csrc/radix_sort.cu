// Onesweep LSD radix sort, 8-bit digits, written for sm_100a.
//
//   1. histogram_kernel   one read of the keys builds the digit histogram of EVERY
//                         pass (shared-memory atomics, then 64-bit global atomics);
//                         the last CTA to finish turns each histogram into exclusive
//                         global digit offsets, marks passes in which one digit holds
//                         all n keys as skipped, and fixes the ping-pong parity.
//   2. onesweep_kernel    one launch per pass, 1 read + 1 write per element. A CTA
//                         takes the next tile by atomic ticket, ranks its keys with
//                         warp-level match (per-warp digit counters in shared memory),
//                         publishes its 256 digit counts to a decoupled look-back
//                         chain, resolves its global digit prefixes from predecessor
//                         tiles, reorders keys (and values) through shared memory so
//                         each digit leaves as one contiguous run, and scatters them.
//   3. copy_back_kernel   only when an odd number of passes ran (result in the
//                         alternate buffer); decided on the device, no host sync.
//
// Stability: inside a warp keys are ranked in (round, lane) order, which is their
// order in memory (round j of lane l holds element j*32+l of the warp's slice);
// warps, tiles and passes are combined in order. Equal keys therefore keep their
// input order, which is what makes sort_by_key's values bit-exact.
//
// Key encoding (order-preserving map to unsigned, applied on the first executed
// pass's load and undone on the last executed pass's store): signed -> flip the
// sign bit; floating point -> flip all bits of negatives, the sign bit of the
// rest (bitwise total order); descending -> complement.
#include "common.cuh"

#include <type_traits>

namespace tb200 {
namespace {

constexpr int kRadix = 256;
constexpr int kMaxPasses = 8;

struct SortCtl {
  int status;                    // must stay first: tb200_temp_status reads it
  unsigned hist_done;            // CTAs of the histogram kernel that have finished
  unsigned total_exec;           // number of passes that are not skipped
  unsigned last_pass;            // index of the last executed pass
  unsigned tickets[kMaxPasses];  // dynamic tile counters, one per pass
  unsigned skip[kMaxPasses];
  unsigned exec_before[kMaxPasses];  // executed passes before pass p (ping-pong parity)
  unsigned long long hist[kMaxPasses][kRadix];
  unsigned long long offs[kMaxPasses][kRadix];
};

struct Encoding {
  unsigned long long cmask;  // constant xor (sign bit for signed and float keys)
  unsigned long long fmask;  // all ones for floating point, else 0
  unsigned long long dmask;  // all ones for descending, else 0
};

template <typename UK>
__device__ __forceinline__ UK encode_key(UK x, const Encoding& e) {
  using SK = typename std::make_signed<UK>::type;
  const UK sra = (UK)((SK)x >> (8 * sizeof(UK) - 1));
  return x ^ (UK)((sra & (UK)e.fmask) | (UK)e.cmask) ^ (UK)e.dmask;
}
template <typename UK>
__device__ __forceinline__ UK decode_key(UK y, const Encoding& e) {
  using SK = typename std::make_signed<UK>::type;
  y ^= (UK)e.dmask;
  const UK sra = (UK)((SK)y >> (8 * sizeof(UK) - 1));
  return y ^ (UK)(((UK)~sra & (UK)e.fmask) | (UK)e.cmask);
}

// Digit of an encoded key. 64-bit keys: the 32-bit window that starts at bit `shift` is
// taken with one funnel shift (or from the high word alone), never a 64-bit shift.
template <typename UK>
__device__ __forceinline__ unsigned digit_of(UK k, int shift, unsigned mask) {
  if constexpr (sizeof(UK) == 8) {
    const unsigned lo = (unsigned)k, hi = (unsigned)(k >> 32);
    const unsigned w = shift < 32 ? __funnelshift_r(lo, hi, shift) : hi >> (shift - 32);
    return w & mask;
  } else {
    return ((unsigned)k >> shift) & mask;
  }
}

template <int BYTES> struct ValueOf;
template <> struct ValueOf<1> { using type = uint8_t; };
template <> struct ValueOf<2> { using type = uint16_t; };
template <> struct ValueOf<4> { using type = uint32_t; };
template <> struct ValueOf<8> { using type = unsigned long long; };
template <> struct ValueOf<16> { using type = uint4; };
template <> struct ValueOf<0> { using type = uint8_t; };  // unused

// ---------------------------------------------------------------------------------
// 1. upfront histogram of all passes
// ---------------------------------------------------------------------------------
constexpr int kHistThreads = 512;
constexpr int kHistUnroll = 4;

template <typename UK>
struct alignas(16) KeyVec {
  UK v[16 / sizeof(UK)];
};

// One CTA of kHistThreads threads: exclusive offsets per pass, skip flags, ping-pong bookkeeping.
__device__ __forceinline__ void finalize_histograms(SortCtl* ctl, int num_passes, uint64_t n,
                                                    unsigned long long* s_warp_tot) {
  unsigned exec = 0, last = 0;
  for (int p = 0; p < num_passes; ++p) {
    unsigned long long c = 0;
    if (threadIdx.x < kRadix) c = ld_relaxed_u64(&ctl->hist[p][threadIdx.x]);
    const int all_here = __syncthreads_or(threadIdx.x < kRadix && c == n);
    // block-exclusive scan over the 256 digits (threads 0..255 = 8 warps)
    unsigned long long s = c;
    const unsigned lane = lane_id(), warp = threadIdx.x / kWarp;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, s, off);
      if (lane >= off) s += t;
    }
    if (threadIdx.x < kRadix && lane == 31) s_warp_tot[warp] = s;
    __syncthreads();
    if (threadIdx.x < kRadix) {
      unsigned long long base = 0;
      for (unsigned w = 0; w < warp; ++w) base += s_warp_tot[w];
      ctl->offs[p][threadIdx.x] = base + s - c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ctl->skip[p] = all_here ? 1u : 0u;
      ctl->exec_before[p] = exec;
    }
    if (!all_here) { last = p; ++exec; }
  }
  if (threadIdx.x == 0) {
    ctl->total_exec = exec;
    ctl->last_pass = last;
  }
}

template <typename UK>
__global__ void __launch_bounds__(kHistThreads)
histogram_kernel(const UK* __restrict__ keys, uint64_t n, int begin_bit, int end_bit, int num_passes,
                 Encoding enc, SortCtl* ctl, int aligned) {
  constexpr int P = sizeof(UK);
  constexpr int VEC = 16 / sizeof(UK);
  __shared__ unsigned s_hist[P][kRadix];
  __shared__ unsigned s_last;
  __shared__ unsigned long long s_warp_tot[8];

  for (int i = threadIdx.x; i < P * kRadix; i += kHistThreads) (&s_hist[0][0])[i] = 0;
  __syncthreads();

  auto count = [&](UK raw) {
    const UK k = encode_key(raw, enc);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      if (p < num_passes) {
        const int shift = begin_bit + 8 * p;
        const int bits = min(8, end_bit - shift);
        atomicAdd(&s_hist[p][digit_of(k, shift, (1u << bits) - 1u)], 1u);
      }
    }
  };

  constexpr uint64_t CHUNK = (uint64_t)kHistThreads * VEC * kHistUnroll;
  const uint64_t full_chunks = aligned ? n / CHUNK : 0;
  for (uint64_t c = blockIdx.x; c < full_chunks; c += gridDim.x) {
    const KeyVec<UK>* src = reinterpret_cast<const KeyVec<UK>*>(keys + c * CHUNK);
    KeyVec<UK> v[kHistUnroll];
#pragma unroll
    for (int u = 0; u < kHistUnroll; ++u) v[u] = src[u * kHistThreads + threadIdx.x];
#pragma unroll
    for (int u = 0; u < kHistUnroll; ++u)
#pragma unroll
      for (int j = 0; j < VEC; ++j) count(v[u].v[j]);
  }
  // remainder (and everything, when the pointer is not 16-byte aligned)
  for (uint64_t i = full_chunks * CHUNK + (uint64_t)blockIdx.x * kHistThreads + threadIdx.x; i < n;
       i += (uint64_t)gridDim.x * kHistThreads)
    count(keys[i]);
  __syncthreads();

  for (int i = threadIdx.x; i < num_passes * kRadix; i += kHistThreads) {
    const unsigned c = (&s_hist[0][0])[i];
    if (c) atomicAdd(&ctl->hist[0][0] + i, (unsigned long long)c);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&ctl->hist_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  finalize_histograms(ctl, num_passes, n, s_warp_tot);
}

// Whole-key variant of histogram_kernel (begin_bit = 0, end_bit = key width: what every sort of
// the Thrust front end asks for). Every digit is a byte of the key at a compile-time position,
// and the counters are laid out [pass][digit pair][lane]: each lane of a warp owns a bank, so the
// one shared-memory atomic per key and pass meets no bank conflict (a single shared copy costs a
// random-digit warp about 3.2 conflict cycles per atomic), and the address needs three
// instructions. Two digits share a 32-bit word as 16-bit halves (16 KiB per pass); the CTA folds
// the words into per-thread 64-bit totals before any half can reach 65536.
constexpr int kByteHistThreads = 1024;

// One count: byte (PASS & 3) of `w` is the digit of pass PASS; lane_base is the shared-memory
// address of the calling lane's column of counters.
template <int PASS>
__device__ __forceinline__ void count_byte(unsigned w, unsigned lane_base) {
  constexpr int b = 8 * (PASS & 3);
  unsigned off;  // byte offset of the word of digit pair (d >> 1): ((w >> b) & 0xfe) << 6
  if constexpr (b == 0) off = (w << 6) & 0x3f80u;
  else off = (w >> (b - 6)) & 0x3f80u;
  const unsigned inc = (w & (1u << b)) ? 0x10000u : 1u;
  asm volatile("red.shared.add.u32 [%0 + %2], %1;" ::"r"(lane_base + off), "r"(inc), "n"(PASS * 16384) : "memory");
}

template <typename UK>
__global__ void __launch_bounds__(kByteHistThreads, 1)
histogram_bytes_kernel(const UK* __restrict__ keys, uint64_t n, Encoding enc, SortCtl* ctl, int aligned) {
  constexpr int P = sizeof(UK);
  constexpr int VEC = 16 / sizeof(UK);
  constexpr int T = kByteHistThreads;
  constexpr unsigned kHalfMax = 65535u;
  constexpr int kEntries = P * (kRadix / 2);  // thread e owns digits 2e' and 2e'+1 of one pass
  extern __shared__ __align__(16) unsigned s_cnt[];  // [P][128][32]
  __shared__ unsigned s_last;
  __shared__ unsigned long long s_warp_tot[8];

  const unsigned lane = lane_id();
  for (int i = threadIdx.x; i < kEntries * kWarp; i += T) s_cnt[i] = 0;
  __syncthreads();
  const unsigned lane_base = (unsigned)__cvta_generic_to_shared(s_cnt) + lane * 4u;

  unsigned long long tot_lo = 0, tot_hi = 0;
  unsigned pending = 0;  // upper bound of any 16-bit half since the last fold

  auto count = [&](UK raw) {
    const UK k = encode_key(raw, enc);
    const unsigned lo = (unsigned)k;
    count_byte<0>(lo, lane_base);
    if constexpr (sizeof(UK) >= 2) count_byte<1>(lo, lane_base);
    if constexpr (sizeof(UK) >= 4) {
      count_byte<2>(lo, lane_base);
      count_byte<3>(lo, lane_base);
    }
    if constexpr (sizeof(UK) == 8) {
      const unsigned hi = (unsigned)((unsigned long long)k >> 32);
      count_byte<4>(hi, lane_base);
      count_byte<5>(hi, lane_base);
      count_byte<6>(hi, lane_base);
      count_byte<7>(hi, lane_base);
    }
  };
  auto fold = [&]() {
    __syncthreads();
    if ((int)threadIdx.x < kEntries) {
      unsigned* row = s_cnt + ((unsigned)threadIdx.x << 5);
      unsigned lo = 0, hi = 0;
#pragma unroll 8
      for (unsigned j = 0; j < kWarp; ++j) {
        const unsigned idx = (j + lane) & 31u;  // rotated: one bank per lane
        const unsigned w = row[idx];
        row[idx] = 0;
        lo += w & 0xffffu;
        hi += w >> 16;
      }
      tot_lo += lo;
      tot_hi += hi;
    }
    __syncthreads();
    pending = 0;
  };

  constexpr uint64_t CHUNK = (uint64_t)T * VEC * kHistUnroll;
  constexpr unsigned kPerChunk = (T / kWarp) * VEC * kHistUnroll;  // adds one lane's counters can see
  const uint64_t full_chunks = aligned ? n / CHUNK : 0;
  for (uint64_t c = blockIdx.x; c < full_chunks; c += gridDim.x) {
    if (pending + kPerChunk > kHalfMax) fold();
    pending += kPerChunk;
    const KeyVec<UK>* src = reinterpret_cast<const KeyVec<UK>*>(keys + c * CHUNK);
    KeyVec<UK> v[kHistUnroll];
#pragma unroll
    for (int u = 0; u < kHistUnroll; ++u) v[u] = src[u * T + threadIdx.x];
#pragma unroll
    for (int u = 0; u < kHistUnroll; ++u)
#pragma unroll
      for (int j = 0; j < VEC; ++j) count(v[u].v[j]);
  }
  // remainder (and everything, when the pointer is not 16-byte aligned); every thread of the
  // CTA makes the same number of trips because fold() synchronises
  for (uint64_t base = full_chunks * CHUNK + (uint64_t)blockIdx.x * T; base < n; base += (uint64_t)gridDim.x * T) {
    if (pending + T / kWarp > kHalfMax) fold();
    pending += T / kWarp;
    const uint64_t i = base + threadIdx.x;
    if (i < n) count(keys[i]);
  }
  fold();

  if ((int)threadIdx.x < kEntries) {
    unsigned long long* h = &ctl->hist[0][0] + 2 * threadIdx.x;
    if (tot_lo) atomicAdd(h, tot_lo);
    if (tot_hi) atomicAdd(h + 1, tot_hi);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&ctl->hist_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  finalize_histograms(ctl, P, n, s_warp_tot);
}

// Finalisation alone, for histograms that another kernel accumulated (the gather of the
// sharded sort counts the digits of the keys it moves).
__global__ void __launch_bounds__(kHistThreads)
histogram_finalize_kernel(SortCtl* ctl, int num_passes, uint64_t n) {
  __shared__ unsigned long long s_warp_tot[8];
  finalize_histograms(ctl, num_passes, n, s_warp_tot);
}

// ---------------------------------------------------------------------------------
// 2. one onesweep pass
// ---------------------------------------------------------------------------------
struct PassParams {
  void* keys_main;
  void* keys_alt;
  void* vals_main;
  void* vals_alt;
  uint64_t n;
  unsigned num_tiles;
  int pass;
  int shift;
  unsigned mask;
  Encoding enc;
  SortCtl* ctl;
  void* desc;
  const void* splitters;   // partition mode: ascending splitters (device), else unused
  unsigned num_splitters;
  // (The pair form of the partition, TIES, finds its two extra arguments in the control block,
  // ctl->offs[3][0..1]: the splitters' indices and the index of the input's first element. They are
  // kept out of this struct on purpose: a larger parameter block changed the register allocation of
  // the plain radix pass and cost it 3 %.)
  // partition mode: device tables of num_splitters + 1 pointers, the first element of every
  // bucket's output (keys, values); the buckets may live in different allocations, another
  // GPU's memory included. Null: bucket b starts at element offs[0][b] of the alternate arrays.
  void* const* bucket_keys;
  void* const* bucket_vals;
};

template <typename DescT> struct DescBits;
template <> struct DescBits<unsigned> {
  static constexpr int kShift = 30;
  static constexpr unsigned kValueMask = (1u << 30) - 1;
};
template <> struct DescBits<unsigned long long> {
  static constexpr int kShift = 62;
  static constexpr unsigned long long kValueMask = (1ull << 62) - 1;
};

template <typename DescT>
__device__ __forceinline__ DescT ld_desc(const DescT* p) {
  if constexpr (sizeof(DescT) == 4) return ld_relaxed_u32(p);
  else return ld_relaxed_u64(p);
}
template <typename DescT>
__device__ __forceinline__ void st_desc(DescT* p, DescT v) {
  if constexpr (sizeof(DescT) == 4) st_relaxed_u32(p, v);
  else st_relaxed_u64(p, v);
}

template <int B>
__device__ __forceinline__ void match_bit(unsigned& peers, unsigned d) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b32 t, m, nm;\n"
      "and.b32 t, %1, %2;\n"
      "setp.ne.u32 p, t, 0;\n"
      "vote.sync.ballot.b32 m, p, 0xffffffff;\n"
      "not.b32 nm, m;\n"
      "@p and.b32 %0, %0, m;\n"
      "@!p and.b32 %0, %0, nm;\n"
      "}\n"
      : "+r"(peers)
      : "r"(d), "n"(1 << B));
}

// Lanes of the warp that hold the same 8-bit digit. One ballot per bit; a lane keeps
// the voters that agree with its own bit: peers &= ~(ballot ^ sign_extend(bit)).
__device__ __forceinline__ unsigned match_digit(unsigned d) {
  // four instructions per bit: test, vote, and one predicated AND for either polarity
  unsigned peers = 0xffffffffu;
  match_bit<0>(peers, d); match_bit<1>(peers, d); match_bit<2>(peers, d); match_bit<3>(peers, d);
  match_bit<4>(peers, d); match_bit<5>(peers, d); match_bit<6>(peers, d); match_bit<7>(peers, d);
  return peers;
}
// Same, for digits known to fit in `bits` bits (bucket ids of a partition): fewer ballots.
__device__ __forceinline__ unsigned match_digit_bits(unsigned d, int bits) {
  unsigned peers = 0xffffffffu;
  switch (bits) {  // bits is the same for the whole grid
    case 8: match_bit<7>(peers, d); [[fallthrough]];
    case 7: match_bit<6>(peers, d); [[fallthrough]];
    case 6: match_bit<5>(peers, d); [[fallthrough]];
    case 5: match_bit<4>(peers, d); [[fallthrough]];
    case 4: match_bit<3>(peers, d); [[fallthrough]];
    case 3: match_bit<2>(peers, d); [[fallthrough]];
    case 2: match_bit<1>(peers, d); [[fallthrough]];
    case 1: match_bit<0>(peers, d); [[fallthrough]];
    default: break;
  }
  return peers;
}

// Copies `len` elements from shared memory to global memory with all THREADS threads of the CTA:
// element by element up to the first 16-byte boundary of the destination, 16 bytes per thread
// from there, element by element for what is left.
template <typename T, int THREADS>
__device__ __forceinline__ void copy_run(T* __restrict__ dst, const T* __restrict__ src, unsigned len) {
  constexpr unsigned VEC = 16 / sizeof(T);
  if constexpr (VEC <= 1) {
    for (unsigned i = threadIdx.x; i < len; i += THREADS) dst[i] = src[i];
  } else {
    unsigned head = (unsigned)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(dst) & 15u)) & 15u) / sizeof(T));
    if (head > len) head = len;
    if (threadIdx.x < head) dst[threadIdx.x] = src[threadIdx.x];
    const unsigned nvec = (len - head) / VEC;
    struct alignas(16) Vec { T v[VEC]; };
    Vec* vdst = reinterpret_cast<Vec*>(dst + head);
    for (unsigned i = threadIdx.x; i < nvec; i += THREADS) {
      Vec x;
#pragma unroll
      for (unsigned e = 0; e < VEC; ++e) x.v[e] = src[head + i * VEC + e];
      vdst[i] = x;
    }
    const unsigned done = head + nvec * VEC;
    if (threadIdx.x < len - done) dst[done + threadIdx.x] = src[done + threadIdx.x];
  }
}

template <typename UK, int VB, int THREADS, int ITEMS>
struct PassShape {
  using V = typename ValueOf<VB>::type;
  static constexpr int kWarps = THREADS / kWarp;
  static constexpr int kTile = THREADS * ITEMS;
  static constexpr int kWarpItems = kWarp * ITEMS;
  static constexpr size_t kKeysBytes = (size_t)kTile * sizeof(UK);
  static constexpr size_t kValsBytes = VB ? align_up((size_t)kTile * VB, 16) : 0;
  static constexpr size_t kWhistBytes = (size_t)kWarps * kRadix * sizeof(unsigned);
  static constexpr size_t kSmem = align_up(kKeysBytes, 16) + kValsBytes + kWhistBytes;
  // the partition form also keeps one byte per sorted slot: the bucket of the key parked there
  static constexpr size_t kSmemSplit = kSmem + align_up((size_t)kTile, 16);
};

// Persistent CTAs: the grid holds as many CTAs as fit on the GPU at once and every
// CTA loops over tiles taken from an atomic ticket counter. The ticket of the NEXT
// tile is taken one iteration ahead and its keys are loaded into the key registers
// as soon as the current tile's keys have been moved to shared memory, so the load
// latency hides behind the look-back and the scatter of the current tile.
// SPLIT = true turns the pass into a stable multi-way partition: the "digit" of a key is the
// number of splitters strictly below it (bucket b holds keys in (s[b-1], s[b]]).
template <typename UK, int VB, int THREADS, int ITEMS, int MIN_CTAS, typename DescT, bool SPLIT = false,
          bool TIES = false>
__global__ void __launch_bounds__(THREADS, MIN_CTAS)
onesweep_kernel(const PassParams prm) {
  using Shape = PassShape<UK, VB, THREADS, ITEMS>;
  using V = typename Shape::V;
  // 32-bit output indices whenever n fits (the narrow descriptor is used for n <= 2^30)
  using IdxT = typename std::conditional<sizeof(DescT) == 4, unsigned, unsigned long long>::type;
  constexpr int WARPS = Shape::kWarps;
  constexpr int TILE = Shape::kTile;
  constexpr int DSH = DescBits<DescT>::kShift;
  static_assert(THREADS >= kRadix && THREADS % kRadix == 0, "one or more threads per digit");
  constexpr int GROUPS = THREADS / kRadix;          // thread groups that share the per-digit loops
  constexpr int WARPS_PER_GROUP = WARPS / GROUPS;

  extern __shared__ __align__(16) unsigned char smem[];
  UK* s_keys = reinterpret_cast<UK*>(smem);
  V* s_vals = reinterpret_cast<V*>(smem + align_up(Shape::kKeysBytes, 16));
  unsigned* s_whist = reinterpret_cast<unsigned*>(smem + align_up(Shape::kKeysBytes, 16) + Shape::kValsBytes);
  unsigned char* s_bkt = smem + Shape::kSmem;  // partition form only: bucket of every parked key
  __shared__ IdxT s_gbase[kRadix];
  __shared__ unsigned s_part[GROUPS][kRadix];  // per-group digit totals
  __shared__ unsigned s_scan[kRadix / kWarp];
  __shared__ unsigned s_next;
  __shared__ UK s_split[SPLIT ? kRadix : 1];
  __shared__ unsigned long long s_split_idx[TIES ? kRadix : 1];
  __shared__ unsigned s_run_start[SPLIT ? kRadix : 1], s_run_len[SPLIT ? kRadix : 1];  // partition: runs of the parked tile
  __shared__ UK* s_bucket_keys[SPLIT ? kRadix : 1];
  __shared__ V* s_bucket_vals[SPLIT ? kRadix : 1];

  SortCtl* ctl = prm.ctl;
  const int pass = prm.pass;
  if (ctl->skip[pass]) return;
  const unsigned before = ctl->exec_before[pass];
  const bool first_exec = before == 0;
  const bool last_exec = ctl->last_pass == (unsigned)pass;
  const bool from_alt = before & 1u;
  const UK* src_keys = static_cast<const UK*>(from_alt ? prm.keys_alt : prm.keys_main);
  UK* dst_keys = static_cast<UK*>(from_alt ? prm.keys_main : prm.keys_alt);
  const V* src_vals = static_cast<const V*>(from_alt ? prm.vals_alt : prm.vals_main);
  V* dst_vals = static_cast<V*>(from_alt ? prm.vals_main : prm.vals_alt);
  // descriptor states rotate with the parity of executed passes, so the chain
  // needs zeroing only once per sort: after a pass every entry reads kPrefix of
  // that pass, which is kEmpty of the next one.
  const unsigned st_empty = (2u * (before & 1u)) & 3u;
  const unsigned st_agg = (st_empty + 1u) & 3u;
  const unsigned st_prefix = (st_empty + 2u) & 3u;

  const unsigned warp = threadIdx.x / kWarp;
  const unsigned lane = lane_id();
  const unsigned warp_off = warp * Shape::kWarpItems;
  const int shift = prm.shift;
  const unsigned mask = prm.mask;
  const unsigned num_tiles = prm.num_tiles;
  unsigned* whist = s_whist + warp * kRadix;
  const unsigned num_split = SPLIT ? prm.num_splitters : 0u;
  const int split_bits = 32 - __clz(num_split | 1u);  // bucket ids are 0..num_split
  // Partition form: the bucket of a key is the number of splitters strictly below it. It is
  // computed ONCE per key (while ranking) and kept: in a byte per item in registers until the
  // reorder, in a byte per sorted slot in shared memory until the scatter. Up to seven splitters
  // (eight GPUs) live in registers, padded with the largest key: three compare-and-select levels.
  UK sp[SPLIT ? 7 : 1];
  unsigned long long spi[TIES ? 7 : 1];  // TIES: the splitters' indices (padding: the largest index)
  const bool few = SPLIT && num_split <= 7;
  static_assert(SPLIT || !TIES, "ties belong to the partition form");
  // TIES: splitter i is the PAIR (splitters[i], splitter_index[i]) and element g of the input is the pair
  // (key, index_base + g); pairs compare by key, then by index
  const unsigned long long* splitter_index = nullptr;
  unsigned long long index_base = 0;
  if constexpr (TIES) {
    splitter_index = reinterpret_cast<const unsigned long long*>(ctl->offs[3][0]);
    index_base = ctl->offs[3][1];
  }
  if constexpr (SPLIT) {
#pragma unroll
    for (int j = 0; j < 7; ++j) {
      const bool real = few && (unsigned)j < num_split;
      sp[j] = real ? static_cast<const UK*>(prm.splitters)[j] : (UK)~(UK)0;
      if constexpr (TIES) spi[j] = real ? splitter_index[j] : ~0ull;
    }
    for (unsigned i = threadIdx.x; i < num_split; i += THREADS) {
      s_split[i] = static_cast<const UK*>(prm.splitters)[i];
      if constexpr (TIES) s_split_idx[i] = splitter_index[i];
    }
  }
  auto digit = [&](UK k) -> unsigned {
    if constexpr (SPLIT) {
      if (few) {
        const bool c1 = sp[3] < k;
        const bool c2 = (c1 ? sp[5] : sp[1]) < k;
        const bool c3 = (c1 ? (c2 ? sp[6] : sp[4]) : (c2 ? sp[2] : sp[0])) < k;
        return 4u * c1 + 2u * c2 + (unsigned)c3;
      }
      unsigned lo = 0, hi = num_split;  // binary search over the ascending splitters
      while (lo < hi) {
        const unsigned mid = (lo + hi) >> 1;
        if (s_split[mid] < k) lo = mid + 1; else hi = mid;
      }
      return lo;
    } else {
      return digit_of(k, shift, mask);
    }
  };
  // TIES: the bucket of the PAIR (k, g): the number of splitter pairs strictly below it
  auto digit_pair = [&](UK k, unsigned long long g) -> unsigned {
    if constexpr (TIES) {
      auto below = [&](UK s_, unsigned long long si) -> bool { return s_ < k || (s_ == k && si < g); };
      if (few) {
        const bool c1 = below(sp[3], spi[3]);
        const bool c2 = below(c1 ? sp[5] : sp[1], c1 ? spi[5] : spi[1]);
        const bool c3 = below(c1 ? (c2 ? sp[6] : sp[4]) : (c2 ? sp[2] : sp[0]),
                              c1 ? (c2 ? spi[6] : spi[4]) : (c2 ? spi[2] : spi[0]));
        return 4u * c1 + 2u * c2 + (unsigned)c3;
      }
      unsigned lo = 0, hi = num_split;
      while (lo < hi) {
        const unsigned mid = (lo + hi) >> 1;
        if (below(s_split[mid], s_split_idx[mid])) lo = mid + 1; else hi = mid;
      }
      return lo;
    } else {
      return 0u;
    }
  };

  // warp-striped load: round j of lane l is element j*32+l of the warp's slice
  UK key[ITEMS];
  auto load_keys = [&](unsigned t) {
    const uint64_t base = (uint64_t)t * TILE;
    const uint64_t remaining = prm.n - base;
    const UK* p = src_keys + base + warp_off + lane;
    if (remaining >= (uint64_t)TILE) {  // full tile: no bounds checks, constant offsets
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) key[j] = p[j * kWarp];
    } else {
      const unsigned valid = (unsigned)remaining;
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) {
        const unsigned local = warp_off + j * kWarp + lane;
        key[j] = local < valid ? p[j * kWarp] : (UK)0;
      }
    }
    if (first_exec) {
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) key[j] = encode_key(key[j], prm.enc);
    }
    if (remaining < (uint64_t)TILE) {  // padding sorts to the end of the tile
#pragma unroll
      for (int j = 0; j < ITEMS; ++j)
        if (warp_off + j * kWarp + lane >= (unsigned)remaining) key[j] = (UK)~(UK)0;
    }
  };

  // global offset of this thread's digit in this pass: read once, used for every tile
  unsigned long long pass_offset = ctl->offs[pass][threadIdx.x % kRadix];
  if constexpr (SPLIT) {  // buckets are addressed through their own base pointers
    if (threadIdx.x < kRadix) {
      const unsigned b = threadIdx.x;
      UK* bk = dst_keys + pass_offset;
      V* bv = VB ? dst_vals + pass_offset : nullptr;
      if (prm.bucket_keys != nullptr && b <= num_split) {
        bk = static_cast<UK*>(prm.bucket_keys[b]);
        if (VB) bv = static_cast<V*>(prm.bucket_vals[b]);
      }
      s_bucket_keys[b] = bk;
      s_bucket_vals[b] = bv;
    }
    pass_offset = 0;
  }
  if (threadIdx.x == 0) s_next = atomicAdd(&ctl->tickets[pass], 1u);
  __syncthreads();
  unsigned tile = s_next;
  if (tile >= num_tiles) return;
  load_keys(tile);
  __syncthreads();  // everyone has read s_next before it is overwritten

  // The sorted keys and values of a tile stay parked in shared memory while the CTA ranks the
  // NEXT tile (ranking needs only registers and the per-warp counters). The parked tile's
  // look-back and scatter run after that ranking: by then the predecessor tiles it waits for
  // have had a whole ranking phase to publish their counts, so the in-order dependency of
  // the chained scan costs almost no idle time.
  bool parked = false;
  unsigned p_tile = 0, p_valid = 0, p_count = 0, p_digit_start = 0;
  const unsigned d_own = threadIdx.x % kRadix;
  const unsigned grp = threadIdx.x / kRadix;
  auto flush_parked = [&]() {
      // ---- look-back: global prefix of every digit over the predecessor tiles. A thread
      // fetches kWindow descriptors at once and consumes them nearest first.
      if (grp == 0) {
        const unsigned d = d_own;
        unsigned long long excl = 0;
        if (p_tile != 0) {
          constexpr int kWindow = 4;
          const DescT* chain = static_cast<const DescT*>(prm.desc) + d;
          const DescT below_first = (DescT)st_prefix << DSH;  // virtual prefix 0 before tile 0
          long long t = (long long)p_tile - 1;
          bool timed_out = false, done = false;
          while (!done && !timed_out) {
            DescT v[kWindow];
  #pragma unroll
            for (int i = 0; i < kWindow; ++i)
              v[i] = t - i >= 0 ? ld_desc<DescT>(chain + (size_t)(t - i) * kRadix) : below_first;
  #pragma unroll
            for (int i = 0; i < kWindow; ++i) {
              if (done || timed_out) break;
              unsigned polls = 0;
              while ((unsigned)(v[i] >> DSH) == st_empty) {
                backoff(++polls);
                if (polls >= kSpinLimit || ((polls & 255u) == 0 && ld_relaxed_s32(&ctl->status) != 0)) {
                  timed_out = true;
                  break;
                }
                v[i] = ld_desc<DescT>(chain + (size_t)(t - i) * kRadix);
              }
              if (timed_out) break;
              excl += (unsigned long long)(v[i] & DescBits<DescT>::kValueMask);
              done = (unsigned)(v[i] >> DSH) == st_prefix;
            }
            t -= kWindow;
          }
          if (timed_out) atomicExch(&ctl->status, (int)TB200_ERR_WAIT_TIMEOUT);
          DescT* mine = static_cast<DescT*>(prm.desc) + (size_t)p_tile * kRadix + d;
          st_desc<DescT>(mine, ((DescT)st_prefix << DSH) | (DescT)((excl + p_count) & DescBits<DescT>::kValueMask));
        }
        s_gbase[d] = (IdxT)(pass_offset + excl - p_digit_start);
        if constexpr (SPLIT) {
          s_run_start[d] = p_digit_start;
          s_run_len[d] = p_count;
        }
      }
      __syncthreads();
      // ---- scatter: every digit leaves as one contiguous run
      if constexpr (SPLIT) {
        if (num_split < 16u) {
          // Few buckets (one per GPU): every bucket's run is long, so the CTA copies run after run
          // with 16-byte stores once the destination is 16-byte aligned (a few elements in front
          // and behind go one by one). Wide stores matter when the destination is another GPU:
          // NVLink moves them in larger packets.
          for (unsigned b = 0; b <= num_split; ++b) {
            const unsigned start = s_run_start[b], len = s_run_len[b];
            const IdxT g0 = s_gbase[b] + start;
            copy_run<UK, THREADS>(s_bucket_keys[b] + g0, s_keys + start, len);
            if constexpr (VB != 0) copy_run<V, THREADS>(s_bucket_vals[b] + g0, s_vals + start, len);
          }
          return;
        }
      }
      auto emit = [&](unsigned pos) {
        const UK k = s_keys[pos];
        if constexpr (SPLIT) {
          const unsigned b = s_bkt[pos];
          const IdxT g = s_gbase[b] + pos;  // index inside bucket b (the sum never wraps)
          s_bucket_keys[b][g] = k;
          if constexpr (VB != 0) s_bucket_vals[b][g] = s_vals[pos];
        } else {
          const IdxT g = s_gbase[digit(k)] + pos;
          dst_keys[g] = last_exec ? decode_key(k, prm.enc) : k;
          if constexpr (VB != 0) dst_vals[g] = s_vals[pos];
        }
      };
      if (p_valid == (unsigned)TILE) {
  #pragma unroll
        for (int i = 0; i < ITEMS; ++i) emit(threadIdx.x + i * THREADS);
      } else {
  #pragma unroll
        for (int i = 0; i < ITEMS; ++i)
          if (threadIdx.x + i * THREADS < p_valid) emit(threadIdx.x + i * THREADS);
      }
  };

  while (true) {
    const uint64_t tile_base = (uint64_t)tile * TILE;
    const uint64_t remaining = prm.n - tile_base;
    const unsigned tile_valid = remaining < (uint64_t)TILE ? (unsigned)remaining : (unsigned)TILE;

    for (int i = threadIdx.x; i < WARPS * kRadix / 4; i += THREADS)
      reinterpret_cast<uint4*>(s_whist)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    // ---- rank inside the warp. All lanes read the warp's running count of their
    // digit, then the lowest lane of every group of equal digits advances it. The
    // shared-memory accesses of one warp execute in program order, so round j+1 reads
    // what round j wrote; the only register dependency inside a round is
    // load -> add -> store.
    unsigned short rank[ITEMS];
    unsigned char bkt[SPLIT ? ITEMS : 1];
    const unsigned lt_mask = lanemask_lt();
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      // (warp-striped: round j of lane l is element warp_off + j * 32 + l of the tile)
      // padding (all-ones keys behind the input's end) lies above every splitter pair
      unsigned d;
      if constexpr (TIES) {
        const unsigned at_ = warp_off + j * kWarp + lane;
        d = digit_pair(key[j], at_ < tile_valid ? index_base + tile_base + at_ : ~0ull);
      } else {
        d = digit(key[j]);
      }
      if constexpr (SPLIT) bkt[j] = (unsigned char)d;
      const unsigned peers = SPLIT ? match_digit_bits(d, split_bits) : match_digit(d);
      const unsigned ahead = __popc(peers & lt_mask);
      const unsigned old = whist[d];
      if (ahead == 0) whist[d] = old + __popc(peers);
      __syncwarp();
      rank[j] = (unsigned short)(old + ahead);
    }
    // values of this tile: requested now, consumed after the per-digit phases below, so the
    // global-load latency overlaps two barriers' worth of work
    V val[VB ? ITEMS : 1];
    if constexpr (VB != 0) {
      const V* pv = src_vals + tile_base + warp_off + lane;
      if (tile_valid == (unsigned)TILE) {
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) val[j] = pv[j * kWarp];
      } else {
#pragma unroll
        for (int j = 0; j < ITEMS; ++j)
          if (warp_off + j * kWarp + lane < tile_valid) val[j] = pv[j * kWarp];
      }
    }
    __syncthreads();

    // ---- per-digit tile totals and warp offsets: thread (g, d) walks the warps of its
    // group; group totals are combined through shared memory. The tile's counts are
    // published BEFORE any local reordering so that successor tiles can use them
    // while this CTA is still busy.
    unsigned part = 0;
#pragma unroll 4
    for (int w = 0; w < WARPS_PER_GROUP; ++w) {
      unsigned* cell = &s_whist[(grp * WARPS_PER_GROUP + w) * kRadix + d_own];
      const unsigned c = *cell;
      *cell = part;
      part += c;
    }
    s_part[grp][d_own] = part;
    __syncthreads();
    unsigned count = 0, grp_off = 0;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const unsigned c = s_part[g][d_own];
      if (g < (int)grp) grp_off += c;
      count += c;
    }
    // padding (all-ones keys at the end of the tile) carries the largest digit in use
    if (d_own == (SPLIT ? (TIES ? num_split : digit((UK)~(UK)0)) : mask)) count -= (unsigned)TILE - tile_valid;
    if (grp == 0) {
      DescT* mine = static_cast<DescT*>(prm.desc) + (size_t)tile * kRadix + d_own;
      if (tile == 0) st_desc<DescT>(mine, ((DescT)st_prefix << DSH) | count);
      else           st_desc<DescT>(mine, ((DescT)st_agg << DSH) | count);
    }
    // exclusive scan of the 256 tile totals -> first slot of each digit in the sorted tile
    unsigned incl = count;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (grp == 0 && lane == 31) s_scan[warp] = incl;
    __syncthreads();
    unsigned digit_start = incl - count;
    for (unsigned w = 0; w < (warp % (kRadix / kWarp)); ++w) digit_start += s_scan[w];
    {
      const unsigned add = digit_start + grp_off;
#pragma unroll 4
      for (int w = 0; w < WARPS_PER_GROUP; ++w) s_whist[(grp * WARPS_PER_GROUP + w) * kRadix + d_own] += add;
    }

    // The next tile's ticket is drawn as late as its latency can still hide behind the scatter:
    // a drawn tile that waits long before it is ranked holds back every later tile's look-back.
    unsigned drawn = 0;  // thread 0: in flight during the look-back and the scatter
    if (threadIdx.x == 0) drawn = atomicAdd(&ctl->tickets[pass], 1u);
    if (parked) flush_parked();  // tile i-1 leaves while tile i's counts are already published
    if (threadIdx.x == 0) s_next = drawn;
    __syncthreads();  // counters hold slot offsets; the shared tile buffers are free
    const unsigned next = s_next;

    // ---- reorder keys and values through shared memory (tile-local, needs no prefix)
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      unsigned d;
      if constexpr (SPLIT) d = bkt[j]; else d = digit(key[j]);
      const unsigned q = whist[d] + rank[j];
      rank[j] = (unsigned short)q;
      s_keys[q] = key[j];
      if constexpr (SPLIT) s_bkt[q] = (unsigned char)d;
    }
    // the key registers are free: fetch the next tile's keys now
    if (next < num_tiles) load_keys(next);
    if constexpr (VB != 0) {
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) s_vals[rank[j]] = val[j];  // padding slots lie beyond tile_valid
    }

    parked = true;
    p_tile = tile;
    p_valid = tile_valid;
    p_count = count;
    p_digit_start = digit_start;
    if (next >= num_tiles) break;
    tile = next;
    __syncthreads();  // counters are cleared and the tile buffers read by the next iteration
  }
  if (parked) {
    __syncthreads();
    flush_parked();
  }
}

// ---------------------------------------------------------------------------------
// 3. copy back when the result ended in the alternate buffer
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
copy_back_kernel(uint4* __restrict__ keys_main, const uint4* __restrict__ keys_alt, uint64_t key_bytes,
                 uint4* __restrict__ vals_main, const uint4* __restrict__ vals_alt, uint64_t val_bytes,
                 const SortCtl* ctl) {
  if ((ctl->total_exec & 1u) == 0) return;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // both buffers are at least 16-byte aligned only when the caller's are; copy the
  // bulk as bytes if not. The alternate buffer is always 256-byte aligned.
  auto copy = [&](uint4* dst, const uint4* src, uint64_t bytes) {
    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      const uint64_t nvec = bytes / 16;
      for (uint64_t i = tid; i < nvec; i += stride) dst[i] = src[i];
      unsigned char* d8 = reinterpret_cast<unsigned char*>(dst);
      const unsigned char* s8 = reinterpret_cast<const unsigned char*>(src);
      for (uint64_t i = nvec * 16 + tid; i < bytes; i += stride) d8[i] = s8[i];
    } else {
      unsigned char* d8 = reinterpret_cast<unsigned char*>(dst);
      const unsigned char* s8 = reinterpret_cast<const unsigned char*>(src);
      for (uint64_t i = tid; i < bytes; i += stride) d8[i] = s8[i];
    }
  };
  copy(keys_main, keys_alt, key_bytes);
  if (val_bytes) copy(vals_main, vals_alt, val_bytes);
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
// tb200_radix_sort runs both phases; the sharded sort splits them around its gather kernel,
// which accumulates the digit histograms itself.
enum { kPhaseAll = 0, kPhaseBegin = 1, kPhaseFinish = 2 };

template <typename UK, int VB>
struct Tuning {
  // threads x items per thread of one onesweep tile, and CTAs that must fit the register file of one SM
  // Measured on B200: few threads with many items each (more independent work per thread,
  // no register spills at 128 registers, fewer per-warp counters to combine) beat 512-thread
  // CTAs by about 10 %; two CTAs per SM (three CTAs of 16 items or four of 12 measured 2 % and
  // 8 % slower on 64-bit pairs, 13-25 % slower on 32-bit keys).
  static constexpr int kThreads = 256;
  static constexpr int kItems = sizeof(UK) == 8 ? (VB == 16 ? 12 : (VB == 8 ? 16 : 24))
                                                : (VB == 16 ? 12 : (VB == 8 ? 24 : (VB == 0 ? 40 : 32)));
  static constexpr int kMinCtas = 2;
};

// Shared-memory opt-in and residency (CTAs per SM) of one kernel, asked of the runtime once per
// device. Tag names the kernel's instantiation: all instantiations share one function-pointer type.
template <typename Tag, typename Kernel>
int resident_ctas(Kernel kernel, int threads, size_t smem, int* per_sm) {
  static int cached[64] = {};  // 0: not asked yet (benign race: the answer is always the same)
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev] > 0) { *per_sm = cached[dev]; return TB200_OK; }
  TB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  TB200_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, kernel, threads, smem));
  if (*per_sm < 1) return TB200_ERR_UNSUPPORTED;
  if (dev < 64) cached[dev] = *per_sm;
  return TB200_OK;
}
inline int sm_count_of_device(int* sms) {
  static int cached[64] = {};
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && cached[dev]) { *sms = cached[dev]; return TB200_OK; }
  TB200_CUDA_TRY(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 64) cached[dev] = *sms;
  return TB200_OK;
}
template <typename UK, int VB, typename DescT, bool SPLIT, bool TIES = false> struct PassTag {};
template <typename UK> struct ByteHistTag {};

struct Layout {
  size_t ctl_off, desc_off, keys_off, vals_off, total, clear_bytes;
};

inline Layout make_layout(uint64_t n, int key_bytes, int val_bytes, uint64_t tiles, size_t desc_elem) {
  Layout l;
  l.ctl_off = 0;
  l.desc_off = align_up(sizeof(SortCtl), 256);
  l.clear_bytes = l.desc_off + align_up((size_t)tiles * kRadix * desc_elem, 256);
  l.keys_off = l.clear_bytes;
  l.vals_off = l.keys_off + align_up((size_t)n * key_bytes, 256);
  l.total = l.vals_off + align_up((size_t)n * val_bytes, 256);
  return l;
}

template <typename UK, int VB>
int sort_impl(void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n, int kind,
              int descending, int begin_bit, int end_bit, cudaStream_t stream, int phase = kPhaseAll) {
  using T = Tuning<UK, VB>;
  using Shape = PassShape<UK, VB, T::kThreads, T::kItems>;
  constexpr uint64_t TILE = Shape::kTile;
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const bool wide = n > (1ull << 30);
  const Layout lay = make_layout(n, sizeof(UK), VB, tiles, wide ? 8 : 4);
  if (d_temp == nullptr) {
    *temp_bytes = lay.total;
    return TB200_OK;
  }
  if (*temp_bytes < lay.total) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  char* base = static_cast<char*>(d_temp);
  auto* ctl = reinterpret_cast<SortCtl*>(base + lay.ctl_off);
  if (n <= 1 || begin_bit >= end_bit) {
    if (phase != kPhaseFinish) TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, sizeof(int), stream));
    return TB200_OK;
  }
  if (phase != kPhaseFinish) TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, lay.clear_bytes, stream));
  if (phase == kPhaseBegin) return TB200_OK;
  if (d_keys == nullptr || (VB && d_vals == nullptr)) return TB200_ERR_INVALID_ARGUMENT;

  Encoding enc;
  const unsigned long long sign = 1ull << (8 * sizeof(UK) - 1);
  enc.cmask = kind == 0 ? 0ull : sign;
  enc.fmask = kind == 2 ? ~0ull : 0ull;
  enc.dmask = descending ? ~0ull : 0ull;
  const int num_passes = (end_bit - begin_bit + 7) / 8;

  int sms = 0;
  {
    const int rc = sm_count_of_device(&sms);
    if (rc) return rc;
  }

  if (phase == kPhaseFinish) {
    histogram_finalize_kernel<<<1, kHistThreads, 0, stream>>>(ctl, num_passes, n);
    trace_mark(stream, kTraceSortHistogram);
    TB200_CUDA_TRY(cudaGetLastError());
  } else {
    const int aligned = reinterpret_cast<uintptr_t>(d_keys) % 16 == 0;
    if (begin_bit == 0 && end_bit == 8 * (int)sizeof(UK)) {
      constexpr int kSmem = (int)sizeof(UK) * (kRadix / 2) * kWarp * (int)sizeof(unsigned);
      const uint64_t chunk = (uint64_t)kByteHistThreads * (16 / sizeof(UK)) * kHistUnroll;
      const uint64_t want = (n + chunk - 1) / chunk;
      auto kernel = histogram_bytes_kernel<UK>;
      int per_sm = 0;
      const int prc = resident_ctas<ByteHistTag<UK>>(kernel, kByteHistThreads, (size_t)kSmem, &per_sm);
      if (prc) return prc;
      const uint64_t resident = (uint64_t)per_sm * sms;
      const unsigned grid = (unsigned)(want < resident ? (want ? want : 1) : resident);
      kernel<<<grid, kByteHistThreads, kSmem, stream>>>(static_cast<const UK*>(d_keys), n, enc, ctl, aligned);
    } else {
      const uint64_t chunk = (uint64_t)kHistThreads * (16 / sizeof(UK)) * kHistUnroll;
      const uint64_t want = (n + chunk - 1) / chunk;
      const unsigned grid = (unsigned)(want < (uint64_t)sms * 4 ? want : (uint64_t)sms * 4);
      histogram_kernel<UK><<<grid, kHistThreads, 0, stream>>>(static_cast<const UK*>(d_keys), n, begin_bit,
                                                              end_bit, num_passes, enc, ctl, aligned);
    }
    trace_mark(stream, kTraceSortHistogram);
    TB200_CUDA_TRY(cudaGetLastError());
  }

  PassParams prm;
  prm.keys_main = d_keys;
  prm.keys_alt = base + lay.keys_off;
  prm.vals_main = d_vals;
  prm.vals_alt = base + lay.vals_off;
  prm.n = n;
  prm.num_tiles = (unsigned)tiles;
  prm.enc = enc;
  prm.ctl = ctl;
  prm.desc = base + lay.desc_off;
  prm.splitters = nullptr;
  prm.num_splitters = 0;
  prm.bucket_keys = nullptr;
  prm.bucket_vals = nullptr;
  auto launch = [&](auto kernel, auto tag) -> int {
    int per_sm = 0;
    const int prc = resident_ctas<decltype(tag)>(kernel, T::kThreads, Shape::kSmem, &per_sm);
    if (prc) return prc;
    const uint64_t resident = (uint64_t)per_sm * sms;
    const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
    for (int p = 0; p < num_passes; ++p) {
      prm.pass = p;
      prm.shift = begin_bit + 8 * p;
      const int bits = end_bit - prm.shift < 8 ? end_bit - prm.shift : 8;
      prm.mask = (1u << bits) - 1u;
      kernel<<<grid, T::kThreads, Shape::kSmem, stream>>>(prm);
      trace_mark(stream, kTraceSortPass);
      TB200_CUDA_TRY(cudaGetLastError());
    }
    return TB200_OK;
  };
  int rc = wide ? launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned long long>,
                         PassTag<UK, VB, unsigned long long, false>{})
                : launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned>,
                         PassTag<UK, VB, unsigned, false>{});
  if (rc) return rc;

  copy_back_kernel<<<sms * 4, 256, 0, stream>>>(
      static_cast<uint4*>(d_keys), reinterpret_cast<const uint4*>(base + lay.keys_off), n * sizeof(UK),
      static_cast<uint4*>(d_vals), reinterpret_cast<const uint4*>(base + lay.vals_off), n * (uint64_t)VB, ctl);
  trace_mark(stream, kTraceSortCopyBack);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// stable multi-way partition by splitters (one onesweep pass with bucket ids as digits)
// ---------------------------------------------------------------------------------
template <typename UK, bool TIES>
__global__ void __launch_bounds__(kHistThreads)
bucket_histogram_kernel(const UK* __restrict__ keys, uint64_t n, const UK* __restrict__ splitters, unsigned num_split,
                        SortCtl* ctl, const unsigned long long* __restrict__ splitter_index,
                        unsigned long long index_base) {
  __shared__ unsigned s_hist[kRadix];
  __shared__ UK s_split[kRadix];
  __shared__ unsigned long long s_split_idx[TIES ? kRadix : 1];  // TIES: splitters and elements are (key, index) pairs
  __shared__ unsigned s_last;
  __shared__ unsigned long long s_warp_tot[8];
  for (int i = threadIdx.x; i < kRadix; i += kHistThreads) s_hist[i] = 0;
  for (unsigned i = threadIdx.x; i < num_split; i += kHistThreads) {
    s_split[i] = splitters[i];
    if constexpr (TIES) s_split_idx[i] = splitter_index[i];
  }
  __syncthreads();
  // Two forms. Up to seven splitters (eight GPUs): the splitters live in registers, padded with
  // the largest key, the search is at most three compare-and-select levels, and every thread
  // counts into eight 8-bit fields of one register that it adds to the shared counters every
  // 248 keys. More splitters: binary search in shared memory; equal buckets inside a warp are
  // found with one ballot per bucket-id bit and counted by one lane, so the shared-memory
  // atomics do not serialise.
  const bool few = num_split <= 7;
  UK sp[7];
  unsigned long long spi[TIES ? 7 : 1];
#pragma unroll
  for (int j = 0; j < 7; ++j) {
    const bool real = few && (unsigned)j < num_split;
    sp[j] = real ? s_split[j] : (UK)~(UK)0;
    if constexpr (TIES) spi[j] = real ? s_split_idx[j] : ~0ull;
  }
  auto below = [&](UK s_, unsigned long long si, UK k, unsigned long long g) -> bool {
    if constexpr (TIES) return s_ < k || (s_ == k && si < g);
    else return s_ < k;
  };
  auto idx_of = [&](int a, int b, bool pick_a) -> unsigned long long {
    if constexpr (TIES) return pick_a ? spi[a] : spi[b];
    else return 0ull;
  };
  unsigned long long packed = 0;
  unsigned since = 0;
  auto flush = [&]() {
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const unsigned c = (unsigned)(packed >> (8 * b)) & 0xffu;
      if (c) atomicAdd(&s_hist[b], c);
    }
    packed = 0;
    since = 0;
  };
  auto bucket_few = [&](UK k, unsigned long long g) -> unsigned {  // number of splitters strictly below (k, g)
    if (num_split <= 1) return below(sp[0], idx_of(0, 0, true), k, g);
    if (num_split <= 3) {
      const bool c1 = below(sp[1], idx_of(1, 1, true), k, g);
      return 2u * c1 + (unsigned)below(c1 ? sp[2] : sp[0], idx_of(2, 0, c1), k, g);
    }
    const bool c1 = below(sp[3], idx_of(3, 3, true), k, g);
    const bool c2 = below(c1 ? sp[5] : sp[1], idx_of(5, 1, c1), k, g);
    const bool c3 = below(c1 ? (c2 ? sp[6] : sp[4]) : (c2 ? sp[2] : sp[0]), c1 ? idx_of(6, 4, c2) : idx_of(2, 0, c2), k, g);
    return 4u * c1 + 2u * c2 + (unsigned)c3;
  };
  const int split_bits = 32 - __clz(num_split | 1u);
  const unsigned lt_mask = lanemask_lt();
  auto count_many = [&](UK k, unsigned long long g, bool valid) {
    unsigned lo = 0, hi = num_split;
    while (lo < hi) {
      const unsigned mid = (lo + hi) >> 1;
      unsigned long long si = 0;
      if constexpr (TIES) si = s_split_idx[mid];
      if (below(s_split[mid], si, k, g)) lo = mid + 1; else hi = mid;
    }
    unsigned peers = match_digit_bits(lo, split_bits) & __ballot_sync(0xffffffffu, valid);
    if (valid && (peers & lt_mask) == 0) atomicAdd(&s_hist[lo], (unsigned)__popc(peers));
  };
  constexpr int VEC = 16 / sizeof(UK);
  constexpr uint64_t CHUNK = (uint64_t)kHistThreads * VEC * kHistUnroll;
  const uint64_t full_chunks = reinterpret_cast<uintptr_t>(keys) % 16 == 0 ? n / CHUNK : 0;
  for (uint64_t c = blockIdx.x; c < full_chunks; c += gridDim.x) {
    const KeyVec<UK>* src = reinterpret_cast<const KeyVec<UK>*>(keys + c * CHUNK);
    KeyVec<UK> v[kHistUnroll];
#pragma unroll
    for (int u = 0; u < kHistUnroll; ++u) v[u] = src[u * kHistThreads + threadIdx.x];
    if (few) {
#pragma unroll
      for (int u = 0; u < kHistUnroll; ++u)
#pragma unroll
        for (int j = 0; j < VEC; ++j)
          packed += 1ull << (8 * bucket_few(v[u].v[j], index_base + c * CHUNK + (uint64_t)(u * kHistThreads + threadIdx.x) * VEC + j));
      since += VEC * kHistUnroll;
      if (since + VEC * kHistUnroll > 255u) flush();
    } else {
#pragma unroll
      for (int u = 0; u < kHistUnroll; ++u)
#pragma unroll
        for (int j = 0; j < VEC; ++j)
          count_many(v[u].v[j], index_base + c * CHUNK + (uint64_t)(u * kHistThreads + threadIdx.x) * VEC + j, true);
    }
  }
  for (uint64_t base = full_chunks * CHUNK + (uint64_t)blockIdx.x * kHistThreads; base < n;
       base += (uint64_t)gridDim.x * kHistThreads) {
    const uint64_t i = base + threadIdx.x;
    const bool valid = i < n;
    if (few) {
      if (valid) {
        packed += 1ull << (8 * bucket_few(keys[i], index_base + i));
        if (++since >= 255u) flush();
      }
    } else {
      count_many(valid ? keys[i] : UK(0), index_base + i, valid);
    }
  }
  if (few) flush();
  __syncthreads();
  for (int i = threadIdx.x; i <= (int)num_split; i += kHistThreads)
    if (s_hist[i]) atomicAdd(&ctl->hist[0][i], (unsigned long long)s_hist[i]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&ctl->hist_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  unsigned long long c = 0;
  if (threadIdx.x < kRadix) c = ld_relaxed_u64(&ctl->hist[0][threadIdx.x]);
  unsigned long long s = c;
  const unsigned lane = lane_id(), warp = threadIdx.x / kWarp;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, s, off);
    if (lane >= off) s += t;
  }
  if (threadIdx.x < kRadix && lane == 31) s_warp_tot[warp] = s;
  __syncthreads();
  if (threadIdx.x < kRadix) {
    unsigned long long base = 0;
    for (unsigned w = 0; w < warp; ++w) base += s_warp_tot[w];
    ctl->offs[0][threadIdx.x] = base + s - c;
  }
  if (threadIdx.x == 0) {  // one pass, never skipped, input in the caller's array, output in the other
    ctl->skip[0] = 0;
    ctl->exec_before[0] = 0;
    ctl->total_exec = 1;
    ctl->last_pass = 0;
  }
}

// phase kPhaseAll: count and scatter into d_keys_out / d_vals_out; kPhaseBegin: count only (the
// bucket sizes reach d_counts); kPhaseFinish: scatter only, bucket b to h_bucket_keys[b] /
// h_bucket_vals[b] (host arrays of num_splitters + 1 device pointers) after a kPhaseBegin call
// on the same scratch and input.
template <typename UK, int VB>
int partition_impl(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals, void* d_keys_out,
                   void* d_vals_out, uint64_t n, const void* d_splitters, unsigned num_splitters,
                   uint64_t* d_counts, cudaStream_t stream, int phase = kPhaseAll,
                   void* const* h_bucket_keys = nullptr, void* const* h_bucket_vals = nullptr,
                   const uint64_t* d_splitter_index = nullptr, uint64_t index_base = 0) {
  using T = Tuning<UK, VB>;
  using Shape = PassShape<UK, VB, T::kThreads, T::kItems>;
  constexpr uint64_t TILE = Shape::kTile;
  const uint64_t tiles = (n + TILE - 1) / TILE;
  const bool wide = n > (1ull << 30);
  const Layout lay = make_layout(0, sizeof(UK), VB, tiles, wide ? 8 : 4);  // control block + descriptors only
  if (d_temp == nullptr) {
    *temp_bytes = lay.total;
    return TB200_OK;
  }
  if (*temp_bytes < lay.total) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (tiles > 0x7fffffffull) return TB200_ERR_UNSUPPORTED;
  if ((phase != kPhaseFinish && !d_counts) || (num_splitters && !d_splitters)) return TB200_ERR_INVALID_ARGUMENT;
  if (phase == kPhaseFinish && (!h_bucket_keys || (VB && !h_bucket_vals))) return TB200_ERR_INVALID_ARGUMENT;
  char* base = static_cast<char*>(d_temp);
  auto* ctl = reinterpret_cast<SortCtl*>(base + lay.ctl_off);
  if (phase != kPhaseFinish) {
    TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, lay.clear_bytes, stream));
    if (n == 0) {
      TB200_CUDA_TRY(cudaMemsetAsync(d_counts, 0, (num_splitters + 1) * sizeof(uint64_t), stream));
      return TB200_OK;
    }
  }
  if (n == 0) return TB200_OK;
  if (!d_keys) return TB200_ERR_INVALID_ARGUMENT;
  if (phase != kPhaseBegin && VB && !d_vals) return TB200_ERR_INVALID_ARGUMENT;
  if (phase == kPhaseAll && (!d_keys_out || (VB && !d_vals_out))) return TB200_ERR_INVALID_ARGUMENT;
  int sms = 0;
  {
    const int rc = sm_count_of_device(&sms);
    if (rc) return rc;
  }
  if (phase != kPhaseFinish) {
    const uint64_t want = (n + kHistThreads * 16 - 1) / (kHistThreads * 16);
    const unsigned grid = (unsigned)(want < (uint64_t)sms * 4 ? want : (uint64_t)sms * 4);
    if (d_splitter_index != nullptr)
      bucket_histogram_kernel<UK, true><<<grid, kHistThreads, 0, stream>>>(
          static_cast<const UK*>(d_keys), n, static_cast<const UK*>(d_splitters), num_splitters, ctl,
          reinterpret_cast<const unsigned long long*>(d_splitter_index), index_base);
    else
      bucket_histogram_kernel<UK, false><<<grid, kHistThreads, 0, stream>>>(
          static_cast<const UK*>(d_keys), n, static_cast<const UK*>(d_splitters), num_splitters, ctl, nullptr, 0);
    trace_mark(stream, kTracePartitionHistogram);
    TB200_CUDA_TRY(cudaGetLastError());
    TB200_CUDA_TRY(cudaMemcpyAsync(d_counts, &ctl->hist[0][0], (num_splitters + 1) * sizeof(uint64_t),
                                   cudaMemcpyDeviceToDevice, stream));
    if (phase == kPhaseBegin) return TB200_OK;
  }
  // the bucket pointer tables travel in two rows of the control block that a one-pass
  // partition never touches
  void* const* d_bucket_keys = nullptr;
  void* const* d_bucket_vals = nullptr;
  if (phase == kPhaseFinish) {
    static_assert(sizeof(void*) == sizeof(unsigned long long), "pointer tables reuse 64-bit rows");
    TB200_CUDA_TRY(cudaMemcpyAsync(&ctl->offs[1][0], h_bucket_keys, (num_splitters + 1) * sizeof(void*),
                                   cudaMemcpyHostToDevice, stream));
    d_bucket_keys = reinterpret_cast<void* const*>(&ctl->offs[1][0]);
    if (VB) {
      TB200_CUDA_TRY(cudaMemcpyAsync(&ctl->offs[2][0], h_bucket_vals, (num_splitters + 1) * sizeof(void*),
                                     cudaMemcpyHostToDevice, stream));
      d_bucket_vals = reinterpret_cast<void* const*>(&ctl->offs[2][0]);
    }
  }
  PassParams prm;
  prm.keys_main = const_cast<void*>(d_keys);
  prm.keys_alt = d_keys_out;
  prm.vals_main = const_cast<void*>(d_vals);
  prm.vals_alt = d_vals_out;
  prm.n = n;
  prm.num_tiles = (unsigned)tiles;
  prm.enc = Encoding{0ull, 0ull, 0ull};
  prm.ctl = ctl;
  prm.desc = base + lay.desc_off;
  prm.pass = 0;
  prm.shift = 0;
  prm.mask = num_splitters;
  prm.splitters = d_splitters;
  prm.num_splitters = num_splitters;
  if (d_splitter_index != nullptr) {
    const unsigned long long pair_args[2] = {reinterpret_cast<unsigned long long>(d_splitter_index), index_base};
    TB200_CUDA_TRY(cudaMemcpyAsync(&ctl->offs[3][0], pair_args, sizeof(pair_args), cudaMemcpyHostToDevice, stream));
  }
  prm.bucket_keys = d_bucket_keys;
  prm.bucket_vals = d_bucket_vals;
  auto launch = [&](auto kernel, auto tag) -> int {
    int per_sm = 0;
    const int prc = resident_ctas<decltype(tag)>(kernel, T::kThreads, Shape::kSmemSplit, &per_sm);
    if (prc) return prc;
    const uint64_t resident = (uint64_t)per_sm * sms;
    const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
    kernel<<<grid, T::kThreads, Shape::kSmemSplit, stream>>>(prm);
    trace_mark(stream, kTracePartitionPass);
    return (int)cudaGetLastError();
  };
  // pairs (key, index) are a kernel of their own: the indices cost registers that the plain form keeps
  if (d_splitter_index != nullptr)
    return wide ? launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned long long, true, true>,
                         PassTag<UK, VB, unsigned long long, true, true>{})
                : launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned, true, true>,
                         PassTag<UK, VB, unsigned, true, true>{});
  const int rc = wide ? launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned long long, true>,
                               PassTag<UK, VB, unsigned long long, true>{})
                      : launch(onesweep_kernel<UK, VB, T::kThreads, T::kItems, T::kMinCtas, unsigned, true>,
                               PassTag<UK, VB, unsigned, true>{});
  return rc;
}

template <typename UK>
int sort_vals(int val_bytes, void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n, int kind,
              int descending, int begin_bit, int end_bit, cudaStream_t stream, int phase = kPhaseAll) {
  switch (val_bytes) {
    case 0: return sort_impl<UK, 0>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    case 1: return sort_impl<UK, 1>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    case 2: return sort_impl<UK, 2>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    case 4: return sort_impl<UK, 4>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    case 8: return sort_impl<UK, 8>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    case 16: return sort_impl<UK, 16>(d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream, phase);
    default: return TB200_ERR_UNSUPPORTED;
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_radix_sort(void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n,
                                int key_dtype, int val_bytes, int descending, int begin_bit, int end_bit,
                                tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  const int kb = dtype_bytes(key_dtype);
  if (kb == 0) return TB200_ERR_UNSUPPORTED;
  if (begin_bit < 0 || end_bit > 8 * kb || begin_bit > end_bit) return TB200_ERR_INVALID_ARGUMENT;
  int kind = 0;  // 0 unsigned / bool, 1 signed, 2 floating point
  switch (key_dtype) {
    case TB200_I8: case TB200_I16: case TB200_I32: case TB200_I64: kind = 1; break;
    case TB200_F32: case TB200_F64: kind = 2; break;
    default: kind = 0;
  }
  switch (kb) {
    case 1: return sort_vals<uint8_t>(val_bytes, d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream);
    case 2: return sort_vals<uint16_t>(val_bytes, d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream);
    case 4: return sort_vals<uint32_t>(val_bytes, d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream);
    default: return sort_vals<unsigned long long>(val_bytes, d_temp, temp_bytes, d_keys, d_vals, n, kind, descending, begin_bit, end_bit, stream);
  }
}

extern "C" int tb200_partition_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                                    void* d_keys_out, void* d_vals_out, uint64_t n, int key_dtype, int val_bytes,
                                    const void* d_splitters, const uint64_t* d_splitter_index, uint32_t num_splitters,
                                    uint64_t index_base, uint64_t* d_counts, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  if (num_splitters > 255) return TB200_ERR_INVALID_ARGUMENT;
#define TB200_PART(UK, VB) \
  return partition_impl<UK, VB>(d_temp, temp_bytes, d_keys, d_vals, d_keys_out, d_vals_out, n, d_splitters, \
                                num_splitters, d_counts, stream, kPhaseAll, nullptr, nullptr, d_splitter_index, index_base)
  if (key_dtype == TB200_U64) {
    if (val_bytes == 0) TB200_PART(unsigned long long, 0);
    if (val_bytes == 4) TB200_PART(unsigned long long, 4);
    if (val_bytes == 8) TB200_PART(unsigned long long, 8);
  } else if (key_dtype == TB200_U32) {
    if (val_bytes == 0) TB200_PART(uint32_t, 0);
    if (val_bytes == 4) TB200_PART(uint32_t, 4);
    if (val_bytes == 8) TB200_PART(uint32_t, 8);
  }
#undef TB200_PART
  return TB200_ERR_UNSUPPORTED;
}

extern "C" int tb200_partition(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                               void* d_keys_out, void* d_vals_out, uint64_t n, int key_dtype, int val_bytes,
                               const void* d_splitters, uint32_t num_splitters, uint64_t* d_counts,
                               tb200_stream_t stream) {
  return tb200_partition_ties(d_temp, temp_bytes, d_keys, d_vals, d_keys_out, d_vals_out, n, key_dtype, val_bytes,
                              d_splitters, nullptr, num_splitters, 0, d_counts, stream);
}

namespace tb200 {
namespace {
int partition_phase(int phase, void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals, uint64_t n,
                    int key_dtype, int val_bytes, const void* d_splitters, uint32_t num_splitters,
                    uint64_t* d_counts, void* const* h_bucket_keys, void* const* h_bucket_vals, cudaStream_t stream,
                    const uint64_t* d_splitter_index = nullptr, uint64_t index_base = 0) {
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  if (num_splitters > 255) return TB200_ERR_INVALID_ARGUMENT;
#define TB200_PART(UK, VB) \
  return partition_impl<UK, VB>(d_temp, temp_bytes, d_keys, d_vals, nullptr, nullptr, n, d_splitters, num_splitters, \
                                d_counts, stream, phase, h_bucket_keys, h_bucket_vals, d_splitter_index, index_base)
  if (key_dtype == TB200_U64) {
    if (val_bytes == 0) TB200_PART(unsigned long long, 0);
    if (val_bytes == 4) TB200_PART(unsigned long long, 4);
    if (val_bytes == 8) TB200_PART(unsigned long long, 8);
  } else if (key_dtype == TB200_U32) {
    if (val_bytes == 0) TB200_PART(uint32_t, 0);
    if (val_bytes == 4) TB200_PART(uint32_t, 4);
    if (val_bytes == 8) TB200_PART(uint32_t, 8);
  }
#undef TB200_PART
  return TB200_ERR_UNSUPPORTED;
}
}  // namespace
}  // namespace tb200

extern "C" int tb200_partition_count(void* d_temp, size_t* temp_bytes, const void* d_keys, uint64_t n, int key_dtype,
                                     int val_bytes, const void* d_splitters, uint32_t num_splitters,
                                     uint64_t* d_counts, tb200_stream_t stream) {
  return tb200::partition_phase(tb200::kPhaseBegin, d_temp, temp_bytes, d_keys, nullptr, n, key_dtype, val_bytes,
                                d_splitters, num_splitters, d_counts, nullptr, nullptr, stream);
}

extern "C" int tb200_partition_scatter(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                                       uint64_t n, int key_dtype, int val_bytes, const void* d_splitters,
                                       uint32_t num_splitters, void* const* h_bucket_keys,
                                       void* const* h_bucket_vals, tb200_stream_t stream) {
  return tb200::partition_phase(tb200::kPhaseFinish, d_temp, temp_bytes, d_keys, d_vals, n, key_dtype, val_bytes,
                                d_splitters, num_splitters, nullptr, h_bucket_keys, h_bucket_vals, stream);
}

extern "C" int tb200_partition_count_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, uint64_t n,
                                          int key_dtype, int val_bytes, const void* d_splitters,
                                          const uint64_t* d_splitter_index, uint32_t num_splitters, uint64_t index_base,
                                          uint64_t* d_counts, tb200_stream_t stream) {
  return tb200::partition_phase(tb200::kPhaseBegin, d_temp, temp_bytes, d_keys, nullptr, n, key_dtype, val_bytes,
                                d_splitters, num_splitters, d_counts, nullptr, nullptr, stream, d_splitter_index,
                                index_base);
}

extern "C" int tb200_partition_scatter_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                                            uint64_t n, int key_dtype, int val_bytes, const void* d_splitters,
                                            const uint64_t* d_splitter_index, uint32_t num_splitters,
                                            uint64_t index_base, void* const* h_bucket_keys,
                                            void* const* h_bucket_vals, tb200_stream_t stream) {
  return tb200::partition_phase(tb200::kPhaseFinish, d_temp, temp_bytes, d_keys, d_vals, n, key_dtype, val_bytes,
                                d_splitters, num_splitters, nullptr, h_bucket_keys, h_bucket_vals, stream,
                                d_splitter_index, index_base);
}

// ---------------------------------------------------------------------------------------
// Exchange step of the sharded sort, fused with the first step of the sort that follows it:
// one kernel pulls this GPU's runs out of the peers' buffers (plain loads over NVLink) and,
// for the keys, counts the digits of all eight passes on the way.
// ---------------------------------------------------------------------------------------
namespace tb200 {
namespace {

constexpr int kMaxSegments = 16;

struct GatherArgs {
  const void* src[kMaxSegments];     // may point into another GPU's memory (peer mapping)
  unsigned long long count[kMaxSegments];
  unsigned long long dst_off[kMaxSegments];
  int num_segments;
  int rotate;
};

// Every CTA walks all segments with a grid-stride loop. The source side (possibly across
// NVLink) is read with 16-byte loads, eight in flight per thread, after peeling the few
// elements in front of the first 16-byte boundary of the source; the destination is local
// and is written element by element (its alignment is independent of the source's).
// CTAs start on different segments (CTA b on segment (b + rotate) mod count) and then walk
// all of them cyclically, so at any moment the loads of one GPU are spread over all source
// GPUs, and with `rotate` = the caller's rank the pullers are spread over the sources too.
// HIST (64-bit keys only): the digits of every moved key are counted for all eight radix
// passes in shared memory and added to the sort's control block at the end.
template <typename T, bool HIST>
__global__ void __launch_bounds__(512)
gather_segments_kernel(T* __restrict__ dst, const GatherArgs args, SortCtl* ctl) {
  constexpr int U = 8;
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte load
  __shared__ unsigned s_hist[HIST ? 8 : 1][HIST ? kRadix : 1];
  if constexpr (HIST) {
    for (int i = threadIdx.x; i < 8 * kRadix; i += blockDim.x) (&s_hist[0][0])[i] = 0;
    __syncthreads();
  }
  auto count = [&](T e) {
    if constexpr (HIST) {
      const unsigned long long k = (unsigned long long)e;
#pragma unroll
      for (int p = 0; p < 8; ++p) atomicAdd(&s_hist[p][(unsigned)(k >> (8 * p)) & 0xffu], 1u);
    }
  };
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long tid = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (int k = 0; k < args.num_segments; ++k) {
    const int s = (int)((blockIdx.x + (unsigned)args.rotate + (unsigned)k) % (unsigned)args.num_segments);
    const T* __restrict__ src = static_cast<const T*>(args.src[s]);
    T* __restrict__ out = dst + args.dst_off[s];
    const unsigned long long n = args.count[s];
    if constexpr (V == 1) {
      unsigned long long i = tid;
      for (; i + (U - 1) * stride < n; i += U * stride) {
        T v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = src[i + u * stride];
#pragma unroll
        for (int u = 0; u < U; ++u) out[i + u * stride] = v[u];
      }
      for (; i < n; i += stride) out[i] = src[i];
    } else {
      unsigned long long head = ((16 - (reinterpret_cast<uintptr_t>(src) & 15)) & 15) / sizeof(T);
      if (head > n) head = n;
      if (tid < head) { const T e = src[tid]; out[tid] = e; count(e); }
      const uint4* __restrict__ vsrc = reinterpret_cast<const uint4*>(src + head);
      T* __restrict__ vout = out + head;
      const unsigned long long nvec = (n - head) / V;
      unsigned long long i = tid;
      auto emit = [&](unsigned long long at, const uint4& q) {
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int j = 0; j < V; ++j) { vout[at * V + j] = e[j]; count(e[j]); }
      };
      for (; i + (U - 1) * stride < nvec; i += U * stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = vsrc[i + u * stride];
#pragma unroll
        for (int u = 0; u < U; ++u) emit(i + u * stride, v[u]);
      }
      for (; i < nvec; i += stride) emit(i, vsrc[i]);
      const unsigned long long done = head + nvec * V;
      if (tid < n - done) { const T e = src[done + tid]; out[done + tid] = e; count(e); }
    }
  }
  if constexpr (HIST) {
    __syncthreads();
    for (int i = threadIdx.x; i < 8 * kRadix; i += blockDim.x) {
      const unsigned c = (&s_hist[0][0])[i];
      if (c) atomicAdd(&ctl->hist[0][0] + i, (unsigned long long)c);
    }
  }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_gather_segments(void* d_dst, const void* const* h_src, const uint64_t* h_src_offset,
                                     const uint64_t* h_count, uint32_t num_segments, int elem_bytes,
                                     uint32_t rotate, void* d_sort_temp, tb200_stream_t stream) {
  using namespace tb200;
  if (num_segments > (uint32_t)kMaxSegments) return TB200_ERR_UNSUPPORTED;
  if (num_segments && (!d_dst || !h_src || !h_src_offset || !h_count)) return TB200_ERR_INVALID_ARGUMENT;
  if (elem_bytes != 4 && elem_bytes != 8 && elem_bytes != 16) return TB200_ERR_UNSUPPORTED;
  if (d_sort_temp && elem_bytes != 8) return TB200_ERR_UNSUPPORTED;
  GatherArgs a{};
  a.num_segments = (int)num_segments;
  a.rotate = (int)(num_segments ? rotate % num_segments : 0);
  unsigned long long off = 0;
  for (uint32_t s = 0; s < num_segments; ++s) {
    a.src[s] = static_cast<const char*>(h_src[s]) + h_src_offset[s] * (uint64_t)elem_bytes;
    a.count[s] = h_count[s];
    a.dst_off[s] = off;
    off += h_count[s];
  }
  if (off == 0) return TB200_OK;
  int sms = 0;
  {
    const int rc = tb200::sm_count_of_device(&sms);
    if (rc) return rc;
  }
  const unsigned grid = (unsigned)sms * 4;
  auto* ctl = static_cast<SortCtl*>(d_sort_temp);
  switch (elem_bytes) {
    case 4:
      gather_segments_kernel<uint32_t, false><<<grid, 512, 0, stream>>>(static_cast<uint32_t*>(d_dst), a, nullptr);
      break;
    case 8:
      if (ctl) gather_segments_kernel<unsigned long long, true><<<grid, 512, 0, stream>>>(static_cast<unsigned long long*>(d_dst), a, ctl);
      else     gather_segments_kernel<unsigned long long, false><<<grid, 512, 0, stream>>>(static_cast<unsigned long long*>(d_dst), a, nullptr);
      break;
    default:
      gather_segments_kernel<uint4, false><<<grid, 512, 0, stream>>>(static_cast<uint4*>(d_dst), a, nullptr);
      break;
  }
  trace_mark(stream, kTraceOther);
  return (int)cudaGetLastError();
}

// The two halves of tb200_radix_sort for uint64 keys sorted whole, around a gather that counts.
extern "C" int tb200_radix_sort_begin(void* d_temp, size_t* temp_bytes, uint64_t n, int key_dtype, int val_bytes,
                                      tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr || d_temp == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  if (key_dtype != TB200_U64) return TB200_ERR_UNSUPPORTED;
  return sort_vals<unsigned long long>(val_bytes, d_temp, temp_bytes, nullptr, nullptr, n, 0, 0, 0, 64, stream, kPhaseBegin);
}

extern "C" int tb200_radix_sort_finish(void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n,
                                       int key_dtype, int val_bytes, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr || d_temp == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  if (key_dtype != TB200_U64) return TB200_ERR_UNSUPPORTED;
  return sort_vals<unsigned long long>(val_bytes, d_temp, temp_bytes, d_keys, d_vals, n, 0, 0, 0, 64, stream, kPhaseFinish);
}
