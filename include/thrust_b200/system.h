// thrust_b200::system — a Thrust custom system (in the style of the reference's
// examples/minimal_custom_backend.cu:17-37) that routes sort / stable_sort /
// sort_by_key / stable_sort_by_key / inclusive_scan / exclusive_scan / inclusive_scan_by_key /
// exclusive_scan_by_key / reduce / reduce_by_key / unique / unique_copy / unique_by_key /
// unique_by_key_copy / copy_if (stencil form), and the asynchronous forms thrust::async::sort /
// stable_sort / inclusive_scan / exclusive_scan,
// on contiguous arithmetic data to the sm_100a kernels behind the C ABI of
// thrust_b200.h, and everything else to the CUDA system it derives from.
//
//   thrust::sort(thrust_b200::par, v.begin(), v.end());
//   thrust::inclusive_scan(thrust_b200::par.on(stream), in, in + n, out);
//   thrust::reduce_by_key(thrust_b200::par_nosync.on(stream), ...);   // still syncs for the count
//   thrust::sort(thrust_b200::par(my_allocator).on(stream), ...);      // scratch from the caller's allocator
//
// The thrust:: signatures and the execution-policy API are untouched: dispatch reaches
// the overloads below by ADL on the policy type (thrust/detail/sort.inl:30-38,
// scan.inl:36-43, reduce.inl:125-136). Every arity is overloaded because the CUDA
// system forwards its default-argument forms with QUALIFIED calls
// (thrust/system/cuda/detail/sort.h:585-623, scan.h:256-349, reduce_by_key.h:1149-1200),
// which would bypass a system that only overloads the full form.
//
// Fast-path rule (same as the reference's, thrust/system/cuda/detail/sort.h:389-407,
// 431-484): contiguous iterators, arithmetic keys, comparator exactly thrust::less /
// thrust::greater; scans and reduce_by_key additionally need plus / equal_to and one
// 4- or 8-byte numeric type for input, output and accumulator. Anything else is
// forwarded to thrust::cuda::par.on(stream) — the inherited GPU path, never a CPU one.
//
// Requires C++17 and the toolkit's Thrust headers (CCCL); link with libthrust_b200.so.
#pragma once

#include <thrust/execution_policy.h>
#include <thrust/functional.h>
#include <thrust/iterator/iterator_traits.h>
#include <thrust/memory.h>
#include <thrust/pair.h>
#include <thrust/reduce.h>
#include <thrust/scan.h>
#include <thrust/sort.h>
#include <thrust/copy.h>
#include <thrust/unique.h>
#include <thrust/async/scan.h>
#include <thrust/async/sort.h>
#include <thrust/system/cuda/error.h>
#include <thrust/system/cuda/execution_policy.h>
#include <thrust/system/system_error.h>
#include <thrust/type_traits/is_contiguous_iterator.h>

#include <atomic>
#include <cstddef>
#include <memory>
#include <tuple>
#include <cstdint>
#include <new>
#include <string>
#include <type_traits>
#include <utility>

#include "../thrust_b200.h"

namespace thrust_b200 {

// The policy object. Like the reference's policies it is passed by reference through
// dispatch and never copied by the algorithms (testing/unittest/special_types.h:135-168).
struct system : thrust::device_execution_policy<system> {
  cudaStream_t stream = nullptr;  // legacy default stream, like thrust::cuda::par
  bool sync = true;               // false: par_nosync semantics (cuda/detail/par.h:100-107)
  // Scratch allocator attached with par(alloc) (thrust/detail/allocator_aware_execution_policy.h:41-96,
  // examples/cuda/custom_temporary_allocation.cu), type-erased so that one policy type serves every
  // overload below. Null: scratch is leased from the library's workspace pool.
  void* alloc_ctx = nullptr;
  void* (*alloc_fn)(void* ctx, std::size_t bytes) = nullptr;
  void (*free_fn)(void* ctx, void* ptr, std::size_t bytes) = nullptr;

  constexpr system() = default;
  constexpr system(cudaStream_t s, bool sy) : stream(s), sync(sy) {}
  // par.on(stream), cf. thrust/system/cuda/detail/par.h:45-70
  system on(cudaStream_t s) const { system r = *this; r.stream = s; return r; }
  // par(alloc): every call made with the returned policy takes its scratch from `alloc`
  // (allocate(n) / deallocate(p, n) in units of Alloc::value_type, like the reference's
  // temporary_allocator, thrust/detail/allocator/temporary_allocator.inl:40-74) and returns it
  // before the call returns. The allocator must outlive the policy object.
  template <typename Alloc>
  system operator()(Alloc& alloc) const {
    using T = typename Alloc::value_type;
    system r = *this;
    r.alloc_ctx = &alloc;
    r.alloc_fn = [](void* ctx, std::size_t bytes) -> void* {
      auto p = static_cast<Alloc*>(ctx)->allocate((bytes + sizeof(T) - 1) / sizeof(T));
      return static_cast<void*>(thrust::raw_pointer_cast(p));
    };
    r.free_fn = [](void* ctx, void* ptr, std::size_t bytes) {
      using pointer = decltype(std::declval<Alloc&>().allocate(std::size_t(0)));
      static_cast<Alloc*>(ctx)->deallocate(pointer(static_cast<T*>(ptr)), (bytes + sizeof(T) - 1) / sizeof(T));
    };
    return r;
  }
};

inline constexpr system par{};
inline constexpr system par_nosync{nullptr, false};

namespace detail {

// Calls that took the sm_100a path / were forwarded to the inherited CUDA path
// (tests use these the way the reference's dispatch tests use `is_valid`).
inline std::atomic<unsigned long long>& fast_calls() { static std::atomic<unsigned long long> c{0}; return c; }
inline std::atomic<unsigned long long>& forwarded_calls() { static std::atomic<unsigned long long> c{0}; return c; }

inline void throw_on_error(int code, const char* what) {
  if (code == 0) return;
  const std::string msg = std::string(what) + ": " + tb200_error_string(code);
  // cudaError_t codes keep their value; library codes are reported as cudaErrorUnknown
  // with the library's message (thrust/system/cuda/detail/util.h:251-299).
  throw thrust::system_error(code > 0 ? code : (int)cudaErrorUnknown, thrust::cuda_category(), msg);
}

// Scratch of one call: from the policy's allocator if it has one (the reference's
// temporary_array over the policy, thrust/detail/temporary_array.inl:74-80), else a lease of the
// library's workspace pool. Given back when the call leaves; a block of the caller's allocator
// only after the stream has drained, because that allocator may hand it to anyone next.
class scratch {
 public:
  scratch(const system& s, std::size_t bytes) : sys_(s), bytes_(bytes + 256) {
    if (s.alloc_fn) {
      raw_ = s.alloc_fn(s.alloc_ctx, bytes_);
      if (raw_ == nullptr) throw std::bad_alloc();
    } else {
      const int rc = tb200_workspace_acquire(bytes_, s.stream, &raw_);
      if (rc == (int)cudaErrorMemoryAllocation) throw std::bad_alloc();  // malloc_and_free.h:77-82
      throw_on_error(rc, "tb200_workspace_acquire");
    }
  }
  scratch(const scratch&) = delete;
  scratch& operator=(const scratch&) = delete;
  ~scratch() {
    if (raw_ == nullptr) return;
    if (sys_.free_fn) {
      cudaStreamSynchronize(sys_.stream);
      sys_.free_fn(sys_.alloc_ctx, raw_, bytes_);
    } else {
      tb200_workspace_release(raw_);
    }
  }
  // 256-byte aligned, as the C ABI asks of d_temp
  char* get() const { return reinterpret_cast<char*>((reinterpret_cast<std::uintptr_t>(raw_) + 255) / 256 * 256); }

 private:
  const system& sys_;
  void* raw_ = nullptr;
  std::size_t bytes_;
};

inline void finish(const system& s, const void* temp, const char* what) {
  if (s.sync) throw_on_error(tb200_temp_status(temp, s.stream), what);
}

template <typename T> struct is_plain_arithmetic
    : std::integral_constant<bool, std::is_arithmetic<T>::value && !std::is_same<T, long double>::value> {};

template <typename T> constexpr int dtype_of() {
  if (std::is_same<T, bool>::value) return TB200_BOOL;
  if (std::is_floating_point<T>::value) return sizeof(T) == 4 ? TB200_F32 : TB200_F64;
  switch (sizeof(T)) {
    case 1: return std::is_signed<T>::value ? TB200_I8 : TB200_U8;
    case 2: return std::is_signed<T>::value ? TB200_I16 : TB200_U16;
    case 4: return std::is_signed<T>::value ? TB200_I32 : TB200_U32;
    default: return std::is_signed<T>::value ? TB200_I64 : TB200_U64;
  }
}

template <typename T> struct is_scan_type
    : std::integral_constant<bool, is_plain_arithmetic<T>::value && !std::is_same<T, bool>::value &&
                                       (sizeof(T) == 4 || sizeof(T) == 8)> {};

template <typename It> using value_t = typename thrust::iterator_traits<It>::value_type;
template <typename It> constexpr bool contiguous_v = thrust::is_contiguous_iterator<It>::value;

template <typename It> auto raw(It it) { return thrust::raw_pointer_cast(&*it); }

template <typename C, typename K> struct order_of { static constexpr int value = -1; };
template <typename K> struct order_of<thrust::less<K>, K> { static constexpr int value = 0; };
template <typename K> struct order_of<thrust::greater<K>, K> { static constexpr int value = 1; };
template <typename K> struct order_of<thrust::less<void>, K> { static constexpr int value = 0; };
template <typename K> struct order_of<thrust::greater<void>, K> { static constexpr int value = 1; };

template <typename Op, typename T> struct is_plus : std::false_type {};
template <typename T> struct is_plus<thrust::plus<T>, T> : std::true_type {};
template <typename T> struct is_plus<thrust::plus<void>, T> : std::true_type {};
template <typename Op, typename T> struct is_equal_to : std::false_type {};
template <typename T> struct is_equal_to<thrust::equal_to<T>, T> : std::true_type {};
template <typename T> struct is_equal_to<thrust::equal_to<void>, T> : std::true_type {};

template <int N> struct is_value_size : std::integral_constant<bool, N == 1 || N == 2 || N == 4 || N == 8 || N == 16> {};

inline auto inherited(const system& s) { return thrust::cuda::par.on(s.stream); }

template <typename KeyIt, typename Compare>
constexpr bool sort_fast_v = contiguous_v<KeyIt> && is_plain_arithmetic<value_t<KeyIt>>::value &&
                             order_of<Compare, value_t<KeyIt>>::value >= 0;

template <typename KeyIt, typename ValIt, typename Compare>
void sort_pairs(system& s, KeyIt kf, KeyIt kl, ValIt vf, Compare comp, bool has_values) {
  using K = value_t<KeyIt>;
  const uint64_t n = (uint64_t)(kl - kf);
  int vb = 0;
  void* vptr = nullptr;
  if constexpr (!std::is_same<ValIt, std::nullptr_t>::value) {
    if (has_values) { vb = (int)sizeof(value_t<ValIt>); vptr = (void*)raw(vf); }
  }
  (void)comp;
  const int desc = order_of<Compare, K>::value;
  size_t bytes = 0;
  throw_on_error(tb200_radix_sort(nullptr, &bytes, nullptr, nullptr, n, dtype_of<K>(), vb, desc, 0, 8 * (int)sizeof(K),
                                  s.stream), "tb200_radix_sort");
  scratch ws(s, bytes);
  void* temp = ws.get();
  throw_on_error(tb200_radix_sort(temp, &bytes, n ? (void*)raw(kf) : nullptr, vptr, n, dtype_of<K>(), vb, desc, 0,
                                  8 * (int)sizeof(K), s.stream), "tb200_radix_sort");
  ++fast_calls();
  finish(s, temp, "tb200_radix_sort");
}

}  // namespace detail

// ---- sort / stable_sort (replaces cuda_cub::sort, stable_sort: cuda/detail/sort.h:493-532, 585-603)
template <typename It, typename Compare>
void stable_sort(system& s, It first, It last, Compare comp) {
  if constexpr (detail::sort_fast_v<It, Compare>) {
    detail::sort_pairs(s, first, last, nullptr, comp, false);
  } else {
    ++detail::forwarded_calls();
    thrust::stable_sort(detail::inherited(s), first, last, comp);
  }
}
template <typename It>
void stable_sort(system& s, It first, It last) {
  stable_sort(s, first, last, thrust::less<detail::value_t<It>>());
}
// On the radix path the reference's sort is its stable_sort (sort.h:431-484); elsewhere
// the unstable form is forwarded as such.
template <typename It, typename Compare>
void sort(system& s, It first, It last, Compare comp) {
  if constexpr (detail::sort_fast_v<It, Compare>) {
    detail::sort_pairs(s, first, last, nullptr, comp, false);
  } else {
    ++detail::forwarded_calls();
    thrust::sort(detail::inherited(s), first, last, comp);
  }
}
template <typename It>
void sort(system& s, It first, It last) {
  sort(s, first, last, thrust::less<detail::value_t<It>>());
}

// ---- sort_by_key / stable_sort_by_key (cuda/detail/sort.h:534-581, 605-623)
template <typename KeyIt, typename ValIt, typename Compare>
void stable_sort_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, Compare comp) {
  using V = detail::value_t<ValIt>;
  if constexpr (detail::sort_fast_v<KeyIt, Compare> && detail::contiguous_v<ValIt> &&
                std::is_trivially_copyable<V>::value && detail::is_value_size<(int)sizeof(V)>::value) {
    detail::sort_pairs(s, kf, kl, vf, comp, true);
  } else {
    ++detail::forwarded_calls();
    thrust::stable_sort_by_key(detail::inherited(s), kf, kl, vf, comp);
  }
}
template <typename KeyIt, typename ValIt>
void stable_sort_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf) {
  stable_sort_by_key(s, kf, kl, vf, thrust::less<detail::value_t<KeyIt>>());
}
template <typename KeyIt, typename ValIt, typename Compare>
void sort_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, Compare comp) {
  using V = detail::value_t<ValIt>;
  if constexpr (detail::sort_fast_v<KeyIt, Compare> && detail::contiguous_v<ValIt> &&
                std::is_trivially_copyable<V>::value && detail::is_value_size<(int)sizeof(V)>::value) {
    detail::sort_pairs(s, kf, kl, vf, comp, true);
  } else {
    ++detail::forwarded_calls();
    thrust::sort_by_key(detail::inherited(s), kf, kl, vf, comp);
  }
}
template <typename KeyIt, typename ValIt>
void sort_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf) {
  sort_by_key(s, kf, kl, vf, thrust::less<detail::value_t<KeyIt>>());
}

// ---- scans (cuda/detail/scan.h:213-349) ------------------------------------------------
namespace detail {
template <typename InIt, typename OutIt, typename T>
OutIt scan_fast(system& s, InIt first, InIt last, OutIt result, bool exclusive, const T* init) {
  const uint64_t n = (uint64_t)(last - first);
  size_t bytes = 0;
  throw_on_error(tb200_scan(nullptr, &bytes, nullptr, nullptr, n, dtype_of<T>(), exclusive, init, s.stream), "tb200_scan");
  scratch ws(s, bytes);
  void* temp = ws.get();
  throw_on_error(tb200_scan(temp, &bytes, n ? (const void*)raw(first) : nullptr, n ? (void*)raw(result) : nullptr, n,
                            dtype_of<T>(), exclusive, init, s.stream), "tb200_scan");
  ++fast_calls();
  finish(s, temp, "tb200_scan");
  return result + (last - first);
}
template <typename InIt, typename OutIt, typename Acc, typename Op>
constexpr bool scan_fast_v = contiguous_v<InIt> && contiguous_v<OutIt> && is_scan_type<Acc>::value &&
                             std::is_same<value_t<InIt>, Acc>::value && std::is_same<value_t<OutIt>, Acc>::value &&
                             is_plus<Op, Acc>::value;
}  // namespace detail

template <typename InIt, typename OutIt, typename Op>
OutIt inclusive_scan(system& s, InIt first, InIt last, OutIt result, Op op) {
  using T = detail::value_t<InIt>;  // accumulator = input value type (scan.h:63)
  if constexpr (detail::scan_fast_v<InIt, OutIt, T, Op>) {
    return detail::scan_fast<InIt, OutIt, T>(s, first, last, result, false, nullptr);
  } else {
    ++detail::forwarded_calls();
    return thrust::inclusive_scan(detail::inherited(s), first, last, result, op);
  }
}
template <typename InIt, typename OutIt>
OutIt inclusive_scan(system& s, InIt first, InIt last, OutIt result) {
  return inclusive_scan(s, first, last, result, thrust::plus<>{});
}
template <typename InIt, typename OutIt, typename Init, typename Op>
OutIt exclusive_scan(system& s, InIt first, InIt last, OutIt result, Init init, Op op) {
  if constexpr (detail::scan_fast_v<InIt, OutIt, Init, Op>) {  // accumulator = type of init (scan.h:142-154)
    return detail::scan_fast<InIt, OutIt, Init>(s, first, last, result, true, &init);
  } else {
    ++detail::forwarded_calls();
    return thrust::exclusive_scan(detail::inherited(s), first, last, result, init, op);
  }
}
template <typename InIt, typename OutIt, typename Init>
OutIt exclusive_scan(system& s, InIt first, InIt last, OutIt result, Init init) {
  return exclusive_scan(s, first, last, result, init, thrust::plus<>{});
}
template <typename InIt, typename OutIt>
OutIt exclusive_scan(system& s, InIt first, InIt last, OutIt result) {
  return exclusive_scan(s, first, last, result, detail::value_t<InIt>{});  // scan.h:340-349
}

// ---- scan_by_key (cuda/detail/scan_by_key.h:296-485) --------------------------------------
// Fast path: contiguous iterators, arithmetic keys, equal_to, plus, and one 4- or 8-byte
// numeric type for values, output and (exclusive) init.
namespace detail {
template <typename KeyIt, typename ValIt, typename OutIt, typename Acc, typename Pred, typename Op>
constexpr bool scan_by_key_fast_v =
    contiguous_v<KeyIt> && contiguous_v<ValIt> && contiguous_v<OutIt> && is_plain_arithmetic<value_t<KeyIt>>::value &&
    is_scan_type<Acc>::value && std::is_same<value_t<ValIt>, Acc>::value && std::is_same<value_t<OutIt>, Acc>::value &&
    is_equal_to<Pred, value_t<KeyIt>>::value && is_plus<Op, Acc>::value;
template <typename KeyIt, typename ValIt, typename OutIt, typename T>
OutIt scan_by_key_fast(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, bool exclusive, const T* init) {
  using K = value_t<KeyIt>;
  const uint64_t n = (uint64_t)(kl - kf);
  size_t bytes = 0;
  throw_on_error(tb200_scan_by_key(nullptr, &bytes, nullptr, nullptr, nullptr, n, dtype_of<K>(), dtype_of<T>(),
                                   exclusive, init, s.stream), "tb200_scan_by_key");
  scratch ws(s, bytes);
  void* temp = ws.get();
  throw_on_error(tb200_scan_by_key(temp, &bytes, n ? (const void*)raw(kf) : nullptr,
                                   n ? (const void*)raw(vf) : nullptr, n ? (void*)raw(result) : nullptr, n,
                                   dtype_of<K>(), dtype_of<T>(), exclusive, init, s.stream), "tb200_scan_by_key");
  ++fast_calls();
  finish(s, temp, "tb200_scan_by_key");
  return result + (kl - kf);
}
}  // namespace detail

template <typename KeyIt, typename ValIt, typename OutIt, typename Pred, typename Op>
OutIt inclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, Pred pred, Op op) {
  using T = detail::value_t<ValIt>;  // accumulator = value type (sequential/scan_by_key.h:52-53)
  if constexpr (detail::scan_by_key_fast_v<KeyIt, ValIt, OutIt, T, Pred, Op>) {
    return detail::scan_by_key_fast<KeyIt, ValIt, OutIt, T>(s, kf, kl, vf, result, false, nullptr);
  } else {
    ++detail::forwarded_calls();
    return thrust::inclusive_scan_by_key(detail::inherited(s), kf, kl, vf, result, pred, op);
  }
}
template <typename KeyIt, typename ValIt, typename OutIt, typename Pred>
OutIt inclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, Pred pred) {
  return inclusive_scan_by_key(s, kf, kl, vf, result, pred, thrust::plus<>{});  // scan_by_key.h:338-352
}
template <typename KeyIt, typename ValIt, typename OutIt>
OutIt inclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result) {
  return inclusive_scan_by_key(s, kf, kl, vf, result, thrust::equal_to<detail::value_t<KeyIt>>());  // :359-372
}
template <typename KeyIt, typename ValIt, typename OutIt, typename Init, typename Pred, typename Op>
OutIt exclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, Init init, Pred pred, Op op) {
  if constexpr (detail::scan_by_key_fast_v<KeyIt, ValIt, OutIt, Init, Pred, Op>) {  // accumulator = type of init
    return detail::scan_by_key_fast<KeyIt, ValIt, OutIt, Init>(s, kf, kl, vf, result, true, &init);
  } else {
    ++detail::forwarded_calls();
    return thrust::exclusive_scan_by_key(detail::inherited(s), kf, kl, vf, result, init, pred, op);
  }
}
template <typename KeyIt, typename ValIt, typename OutIt, typename Init, typename Pred>
OutIt exclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, Init init, Pred pred) {
  return exclusive_scan_by_key(s, kf, kl, vf, result, init, pred, thrust::plus<>{});  // scan_by_key.h:425-441
}
template <typename KeyIt, typename ValIt, typename OutIt, typename Init>
OutIt exclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result, Init init) {
  return exclusive_scan_by_key(s, kf, kl, vf, result, init, thrust::equal_to<detail::value_t<KeyIt>>());  // :449-463
}
template <typename KeyIt, typename ValIt, typename OutIt>
OutIt exclusive_scan_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, OutIt result) {
  return exclusive_scan_by_key(s, kf, kl, vf, result, detail::value_t<ValIt>{});  // scan_by_key.h:471-485
}

// ---- reduce (cuda/detail/reduce.h:1029-1062) ---------------------------------------------
// The accumulator and the result have the type of `init`; the fast path needs it to be the
// input's value type and the operator to be thrust::plus. Like the reference the call
// synchronises to read the result (reduce.h:984-1000), whatever the policy says.
namespace detail {
template <typename T> struct is_reduce_type
    : std::integral_constant<bool, is_plain_arithmetic<T>::value && !std::is_same<T, bool>::value> {};
template <typename InIt, typename T, typename Op>
constexpr bool reduce_fast_v = contiguous_v<InIt> && is_reduce_type<T>::value &&
                               std::is_same<value_t<InIt>, T>::value && is_plus<Op, T>::value;
template <typename InIt, typename T>
T reduce_fast(system& s, InIt first, InIt last, T init) {
  const uint64_t n = (uint64_t)(last - first);
  size_t bytes = 0;
  throw_on_error(tb200_reduce(nullptr, &bytes, nullptr, n, dtype_of<T>(), nullptr, nullptr, s.stream), "tb200_reduce");
  // the result lives in the first 256 bytes of the workspace, the library's scratch behind it
  scratch lease(s, bytes + 256);
  char* ws = lease.get();
  throw_on_error(tb200_reduce(ws + 256, &bytes, n ? (const void*)raw(first) : nullptr, n, dtype_of<T>(), &init, ws,
                              s.stream), "tb200_reduce");
  ++fast_calls();
  T result;
  throw_on_error((int)cudaMemcpyAsync(&result, ws, sizeof(T), cudaMemcpyDeviceToHost, s.stream), "tb200_reduce");
  throw_on_error((int)cudaStreamSynchronize(s.stream), "tb200_reduce");
  return result;
}
}  // namespace detail

template <typename InIt, typename T, typename Op>
T reduce(system& s, InIt first, InIt last, T init, Op op) {
  if constexpr (detail::reduce_fast_v<InIt, T, Op>) {
    return detail::reduce_fast<InIt, T>(s, first, last, init);
  } else {
    ++detail::forwarded_calls();
    return thrust::reduce(detail::inherited(s), first, last, init, op);
  }
}
template <typename InIt, typename T>
T reduce(system& s, InIt first, InIt last, T init) {
  return reduce(s, first, last, init, thrust::plus<T>());  // reduce.h:1045-1051
}
template <typename InIt>
detail::value_t<InIt> reduce(system& s, InIt first, InIt last) {
  return reduce(s, first, last, detail::value_t<InIt>(0));  // reduce.h:1057-1063
}

// ---- reduce_by_key (cuda/detail/reduce_by_key.h:1118-1200) --------------------------------
template <typename KeyIt, typename ValIt, typename KeyOut, typename ValOut, typename Pred, typename Op>
thrust::pair<KeyOut, ValOut> reduce_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, KeyOut ko, ValOut vo, Pred pred,
                                           Op op) {
  using K = detail::value_t<KeyIt>;
  using V = detail::value_t<ValIt>;
  if constexpr (detail::contiguous_v<KeyIt> && detail::contiguous_v<ValIt> && detail::contiguous_v<KeyOut> &&
                detail::contiguous_v<ValOut> && detail::is_plain_arithmetic<K>::value &&
                detail::is_scan_type<V>::value && std::is_same<detail::value_t<KeyOut>, K>::value &&
                std::is_same<detail::value_t<ValOut>, V>::value && detail::is_equal_to<Pred, K>::value &&
                detail::is_plus<Op, V>::value) {
    const uint64_t n = (uint64_t)(kl - kf);
    if (n == 0) return thrust::make_pair(ko, vo);
    size_t bytes = 0;
    detail::throw_on_error(tb200_reduce_by_key(nullptr, &bytes, nullptr, nullptr, nullptr, nullptr, nullptr, n,
                                               detail::dtype_of<K>(), detail::dtype_of<V>(), s.stream),
                           "tb200_reduce_by_key");
    detail::scratch lease(s, bytes + 256);
    char* ws = lease.get();
    auto* d_runs = reinterpret_cast<uint64_t*>(ws + ((bytes + 255) / 256) * 256);
    detail::throw_on_error(tb200_reduce_by_key(ws, &bytes, detail::raw(kf), detail::raw(vf), detail::raw(ko),
                                               detail::raw(vo), d_runs, n, detail::dtype_of<K>(),
                                               detail::dtype_of<V>(), s.stream), "tb200_reduce_by_key");
    ++detail::fast_calls();
    // the end iterators need the run count: synchronise, like the reference (reduce_by_key.h:1049-1052)
    uint64_t runs = 0;
    detail::throw_on_error((int)cudaMemcpyAsync(&runs, d_runs, sizeof(runs), cudaMemcpyDeviceToHost, s.stream),
                           "reduce_by_key: run count");
    detail::throw_on_error(tb200_temp_status(ws, s.stream), "tb200_reduce_by_key");
    return thrust::make_pair(ko + runs, vo + runs);
  } else {
    ++detail::forwarded_calls();
    return thrust::reduce_by_key(detail::inherited(s), kf, kl, vf, ko, vo, pred, op);
  }
}
template <typename KeyIt, typename ValIt, typename KeyOut, typename ValOut, typename Pred>
thrust::pair<KeyOut, ValOut> reduce_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, KeyOut ko, ValOut vo, Pred pred) {
  return reduce_by_key(s, kf, kl, vf, ko, vo, pred, thrust::plus<detail::value_t<ValIt>>());
}
template <typename KeyIt, typename ValIt, typename KeyOut, typename ValOut>
thrust::pair<KeyOut, ValOut> reduce_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, KeyOut ko, ValOut vo) {
  return reduce_by_key(s, kf, kl, vf, ko, vo, thrust::equal_to<detail::value_t<KeyIt>>());
}

// ---- unique / unique_copy / unique_by_key / unique_by_key_copy (cuda/detail/unique_by_key.h:716-905,
// cuda/detail/unique.h) --------------------------------------------------------------------------
// Fast path: contiguous iterators, arithmetic keys, thrust::equal_to, values that are trivially
// copyable and 1, 2, 4, 8 or 16 bytes wide; outputs of the inputs' value types. Like the reference
// the calls synchronise to read the count (unique_by_key.h:789-791).
namespace detail {
template <typename It> constexpr bool payload_v =
    contiguous_v<It> && std::is_trivially_copyable<value_t<It>>::value && is_value_size<(int)sizeof(value_t<It>)>::value;
template <typename KeyIt, typename Pred> constexpr bool unique_keys_fast_v =
    contiguous_v<KeyIt> && is_plain_arithmetic<value_t<KeyIt>>::value && is_equal_to<Pred, value_t<KeyIt>>::value;
template <typename A, typename B> constexpr bool same_value_v = std::is_same<value_t<A>, value_t<B>>::value;

inline uint64_t unique_by_key_raw(system& s, const void* kin, const void* vin, void* kout, void* vout, uint64_t n,
                                  int key_dtype, int val_bytes) {
  if (n == 0) return 0;
  size_t bytes = 0;
  throw_on_error(tb200_unique_by_key(nullptr, &bytes, nullptr, nullptr, nullptr, nullptr, nullptr, n, key_dtype,
                                     val_bytes, s.stream), "tb200_unique_by_key");
  scratch lease(s, bytes + 256);
  char* ws = lease.get();
  auto* d_kept = reinterpret_cast<uint64_t*>(ws + ((bytes + 255) / 256) * 256);
  throw_on_error(tb200_unique_by_key(ws, &bytes, kin, vin, kout, vout, d_kept, n, key_dtype, val_bytes, s.stream),
                 "tb200_unique_by_key");
  ++fast_calls();
  uint64_t kept = 0;
  throw_on_error((int)cudaMemcpyAsync(&kept, d_kept, sizeof(kept), cudaMemcpyDeviceToHost, s.stream), "unique: count");
  throw_on_error(tb200_temp_status(ws, s.stream), "tb200_unique_by_key");
  return kept;
}
template <typename P, typename T> struct is_identity : std::false_type {};
template <typename T> struct is_identity<thrust::identity<T>, T> : std::true_type {};
}  // namespace detail

template <typename KeyIt, typename ValIt, typename KeyOut, typename ValOut, typename Pred>
thrust::pair<KeyOut, ValOut> unique_by_key_copy(system& s, KeyIt kf, KeyIt kl, ValIt vf, KeyOut ko, ValOut vo, Pred pred) {
  if constexpr (detail::unique_keys_fast_v<KeyIt, Pred> && detail::contiguous_v<KeyOut> &&
                detail::same_value_v<KeyIt, KeyOut> && detail::payload_v<ValIt> && detail::contiguous_v<ValOut> &&
                detail::same_value_v<ValIt, ValOut>) {
    const uint64_t n = (uint64_t)(kl - kf);
    if (n == 0) return thrust::make_pair(ko, vo);
    const uint64_t kept = detail::unique_by_key_raw(s, detail::raw(kf), detail::raw(vf), detail::raw(ko), detail::raw(vo), n,
                                                    detail::dtype_of<detail::value_t<KeyIt>>(),
                                                    (int)sizeof(detail::value_t<ValIt>));
    return thrust::make_pair(ko + kept, vo + kept);
  } else {
    ++detail::forwarded_calls();
    return thrust::unique_by_key_copy(detail::inherited(s), kf, kl, vf, ko, vo, pred);
  }
}
template <typename KeyIt, typename ValIt, typename KeyOut, typename ValOut>
thrust::pair<KeyOut, ValOut> unique_by_key_copy(system& s, KeyIt kf, KeyIt kl, ValIt vf, KeyOut ko, ValOut vo) {
  return unique_by_key_copy(s, kf, kl, vf, ko, vo, thrust::equal_to<detail::value_t<KeyIt>>());  // unique_by_key.h:849-864
}
// in place: the outputs are the inputs (unique_by_key.h:871-895)
template <typename KeyIt, typename ValIt, typename Pred>
thrust::pair<KeyIt, ValIt> unique_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf, Pred pred) {
  if constexpr (detail::unique_keys_fast_v<KeyIt, Pred> && detail::payload_v<ValIt>) {
    return unique_by_key_copy(s, kf, kl, vf, kf, vf, pred);
  } else {
    ++detail::forwarded_calls();
    return thrust::unique_by_key(detail::inherited(s), kf, kl, vf, pred);
  }
}
template <typename KeyIt, typename ValIt>
thrust::pair<KeyIt, ValIt> unique_by_key(system& s, KeyIt kf, KeyIt kl, ValIt vf) {
  return unique_by_key(s, kf, kl, vf, thrust::equal_to<detail::value_t<KeyIt>>());  // unique_by_key.h:898-909
}
template <typename InIt, typename OutIt, typename Pred>
OutIt unique_copy(system& s, InIt first, InIt last, OutIt result, Pred pred) {
  if constexpr (detail::unique_keys_fast_v<InIt, Pred> && detail::contiguous_v<OutIt> && detail::same_value_v<InIt, OutIt>) {
    const uint64_t n = (uint64_t)(last - first);
    if (n == 0) return result;
    return result + detail::unique_by_key_raw(s, detail::raw(first), nullptr, detail::raw(result), nullptr, n,
                                              detail::dtype_of<detail::value_t<InIt>>(), 0);
  } else {
    ++detail::forwarded_calls();
    return thrust::unique_copy(detail::inherited(s), first, last, result, pred);
  }
}
template <typename InIt, typename OutIt>
OutIt unique_copy(system& s, InIt first, InIt last, OutIt result) {
  return unique_copy(s, first, last, result, thrust::equal_to<detail::value_t<InIt>>());
}
template <typename It, typename Pred>
It unique(system& s, It first, It last, Pred pred) {
  if constexpr (detail::unique_keys_fast_v<It, Pred>) {
    return unique_copy(s, first, last, first, pred);
  } else {
    ++detail::forwarded_calls();
    return thrust::unique(detail::inherited(s), first, last, pred);
  }
}
template <typename It>
It unique(system& s, It first, It last) {
  return unique(s, first, last, thrust::equal_to<detail::value_t<It>>());
}

// ---- copy_if (cuda/detail/copy_if.h:776-826) ------------------------------------------------
// Fast path: the stencil form with thrust::identity<Stencil> as the predicate (an element is
// copied when its stencil value is non-zero), contiguous iterators, an arithmetic stencil and
// trivially copyable elements of 1, 2, 4, 8 or 16 bytes. Any other predicate needs device code
// of the caller's and is forwarded.
template <typename InIt, typename StencilIt, typename OutIt, typename Pred>
OutIt copy_if(system& s, InIt first, InIt last, StencilIt stencil, OutIt result, Pred pred) {
  using F = detail::value_t<StencilIt>;
  if constexpr (detail::payload_v<InIt> && detail::contiguous_v<OutIt> && detail::same_value_v<InIt, OutIt> &&
                detail::contiguous_v<StencilIt> && detail::is_plain_arithmetic<F>::value &&
                detail::is_identity<Pred, F>::value) {
    const uint64_t n = (uint64_t)(last - first);
    if (n == 0) return result;
    size_t bytes = 0;
    const int eb = (int)sizeof(detail::value_t<InIt>);
    detail::throw_on_error(tb200_copy_flagged(nullptr, &bytes, nullptr, nullptr, nullptr, nullptr, n, eb,
                                              detail::dtype_of<F>(), s.stream), "tb200_copy_flagged");
    detail::scratch lease(s, bytes + 256);
    char* ws = lease.get();
    auto* d_kept = reinterpret_cast<uint64_t*>(ws + ((bytes + 255) / 256) * 256);
    detail::throw_on_error(tb200_copy_flagged(ws, &bytes, detail::raw(first), detail::raw(stencil), detail::raw(result),
                                              d_kept, n, eb, detail::dtype_of<F>(), s.stream), "tb200_copy_flagged");
    ++detail::fast_calls();
    uint64_t kept = 0;
    detail::throw_on_error((int)cudaMemcpyAsync(&kept, d_kept, sizeof(kept), cudaMemcpyDeviceToHost, s.stream),
                           "copy_if: count");
    detail::throw_on_error(tb200_temp_status(ws, s.stream), "tb200_copy_flagged");
    return result + kept;
  } else {
    ++detail::forwarded_calls();
    return thrust::copy_if(detail::inherited(s), first, last, stencil, result, pred);
  }
}
template <typename InIt, typename OutIt, typename Pred>
OutIt copy_if(system& s, InIt first, InIt last, OutIt result, Pred pred) {
  ++detail::forwarded_calls();  // the predicate reads the elements themselves: the caller's device code
  return thrust::copy_if(detail::inherited(s), first, last, result, pred);
}

// ---- asynchronous forms (thrust/async/sort.h, thrust/async/scan.h) ---------------------------
// thrust::async::sort / stable_sort / inclusive_scan / exclusive_scan reach these customization
// points by ADL on the policy (thrust/async/sort.h:60-120, thrust/async/scan.h) and get back the
// CUDA system's event type, as they do from the reference's own implementations
// (thrust/system/cuda/detail/async/sort.h:496-512, async/inclusive_scan.h, async/exclusive_scan.h:77-90).
// The work is enqueued on the event's stream — the policy's stream, or a new one if the policy
// has the default stream — and the call returns at once; the scratch stays leased until the
// event is destroyed. The device status word is not read back (no synchronisation): wait on the
// event and call the blocking form if a status is wanted.
namespace detail {
struct lease_release {
  void operator()(void* p) const { tb200_workspace_release(p); }
};
using lease_ptr = std::unique_ptr<void, lease_release>;
inline lease_ptr lease(size_t bytes, cudaStream_t stream, char** aligned) {
  void* raw = nullptr;
  const int rc = tb200_workspace_acquire(bytes + 256, stream, &raw);
  if (rc == (int)cudaErrorMemoryAllocation) throw std::bad_alloc();
  throw_on_error(rc, "tb200_workspace_acquire");
  *aligned = reinterpret_cast<char*>((reinterpret_cast<std::uintptr_t>(raw) + 255) / 256 * 256);
  return lease_ptr(raw);
}
// The event of an asynchronous call: keeps `keep` alive and names the stream the work goes to.
inline thrust::system::cuda::unique_eager_event async_event(const system& s, lease_ptr keep) {
  namespace cd = thrust::system::cuda::detail;
  if (s.stream != nullptr)
    return cd::make_dependent_event(std::make_tuple(std::move(keep), cd::unique_stream(cd::nonowning, s.stream)));
  return cd::make_dependent_event(std::make_tuple(std::move(keep)));
}
}  // namespace detail

template <typename It, typename Sentinel, typename Compare>
auto async_stable_sort(system& s, It first, Sentinel last, Compare comp) {
  if constexpr (detail::sort_fast_v<It, Compare> && std::is_same<It, Sentinel>::value) {
    using K = detail::value_t<It>;
    const uint64_t n = (uint64_t)(last - first);
    size_t bytes = 0;
    detail::throw_on_error(tb200_radix_sort(nullptr, &bytes, nullptr, nullptr, n, detail::dtype_of<K>(), 0,
                                            detail::order_of<Compare, K>::value, 0, 8 * (int)sizeof(K), nullptr),
                           "tb200_radix_sort");
    // the lease is taken for the legacy stream's pool when the event brings its own stream: its
    // first use is ordered by the event, and it is released only when the event dies
    char* temp = nullptr;
    auto keep = detail::lease(bytes, s.stream, &temp);
    auto e = detail::async_event(s, std::move(keep));
    detail::throw_on_error(tb200_radix_sort(temp, &bytes, n ? (void*)detail::raw(first) : nullptr, nullptr, n,
                                            detail::dtype_of<K>(), 0, detail::order_of<Compare, K>::value, 0,
                                            8 * (int)sizeof(K), e.stream().native_handle()), "tb200_radix_sort");
    ++detail::fast_calls();
    (void)comp;
    return e;
  } else {
    ++detail::forwarded_calls();
    auto inherited = detail::inherited(s);
    return thrust::cuda_cub::async_stable_sort(inherited, first, last, comp);
  }
}

namespace detail {
template <typename InIt, typename OutIt, typename T>
auto async_scan_fast(system& s, InIt first, InIt last, OutIt out, bool exclusive, const T* init) {
  const uint64_t n = (uint64_t)(last - first);
  size_t bytes = 0;
  throw_on_error(tb200_scan(nullptr, &bytes, nullptr, nullptr, n, dtype_of<T>(), exclusive, init, nullptr), "tb200_scan");
  char* temp = nullptr;
  auto keep = lease(bytes, s.stream, &temp);
  auto e = async_event(s, std::move(keep));
  throw_on_error(tb200_scan(temp, &bytes, n ? (const void*)raw(first) : nullptr, n ? (void*)raw(out) : nullptr, n,
                            dtype_of<T>(), exclusive, init, e.stream().native_handle()), "tb200_scan");
  ++fast_calls();
  return e;
}
}  // namespace detail

template <typename InIt, typename Sentinel, typename OutIt, typename Op>
auto async_inclusive_scan(system& s, InIt first, Sentinel last, OutIt out, Op op) {
  using T = detail::value_t<InIt>;
  if constexpr (detail::scan_fast_v<InIt, OutIt, T, Op> && std::is_same<InIt, Sentinel>::value) {
    return detail::async_scan_fast<InIt, OutIt, T>(s, first, last, out, false, nullptr);
  } else {
    ++detail::forwarded_calls();
    auto inherited = detail::inherited(s);
    return thrust::cuda_cub::async_inclusive_scan(inherited, first, last, out, op);
  }
}
template <typename InIt, typename Sentinel, typename OutIt, typename Init, typename Op>
auto async_exclusive_scan(system& s, InIt first, Sentinel last, OutIt out, Init init, Op op) {
  if constexpr (detail::scan_fast_v<InIt, OutIt, Init, Op> && std::is_same<InIt, Sentinel>::value) {
    return detail::async_scan_fast<InIt, OutIt, Init>(s, first, last, out, true, &init);
  } else {
    ++detail::forwarded_calls();
    auto inherited = detail::inherited(s);
    return thrust::cuda_cub::async_exclusive_scan(inherited, first, last, out, init, op);
  }
}

}  // namespace thrust_b200
