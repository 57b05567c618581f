// Boundary tests of thrust_b200::system: the thrust:: algorithms, called with the
// custom policy (or through iterators retagged with it), must reach the sm_100a path
// for arithmetic data and the inherited CUDA path for everything else, and must give
// the results of the host (CPP) system — the same device==host comparison the
// reference's unit tests make (testing/sort.cu:80-90, scan.cu:379-415,
// reduce_by_key.cu:115-156). Known-answer vectors are the reference's own
// (testing/sort.cu:42-62, sort_by_key.cu:44-70, scan.cu:44-104, reduce_by_key.cu:15-112).
#include <thrust/async/scan.h>
#include <thrust/async/sort.h>
#include <thrust/device_vector.h>
#include <thrust/host_vector.h>
#include <thrust/iterator/counting_iterator.h>
#include <thrust/iterator/retag.h>
#include <thrust/sequence.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <map>
#include <thread>
#include <numeric>
#include <cstdlib>
#include <random>
#include <vector>

#include "thrust_b200/system.h"

static int g_failed = 0, g_checks = 0;
static char g_ctx[128] = "";
#define CHECK(cond)                                                             \
  do {                                                                          \
    ++g_checks;                                                                 \
    if (!(cond)) { ++g_failed; std::printf("FAIL %s:%d  %s   [%s]\n", __FILE__, __LINE__, #cond, g_ctx); } \
  } while (0)

namespace tb = thrust_b200;
static unsigned long long fast() { return tb::detail::fast_calls().load(); }
static unsigned long long fwd() { return tb::detail::forwarded_calls().load(); }

template <typename T>
thrust::host_vector<T> random_vec(size_t n, unsigned seed, long long lo, long long hi) {
  std::mt19937_64 rng(seed);
  thrust::host_vector<T> h(n);
  for (size_t i = 0; i < n; ++i) h[i] = (T)(lo + (long long)(rng() % (unsigned long long)(hi - lo + 1)));
  return h;
}

// Host-side expectation for the sorts: std::stable_sort (the toolkit's own host radix sort
// is not used as the comparator; for int keys it orders negative values after positive ones).
template <typename T, typename Cmp>
void host_stable_sort_by_key(thrust::host_vector<T>& k, thrust::host_vector<unsigned>* v, Cmp cmp) {
  std::vector<size_t> idx(k.size());
  std::iota(idx.begin(), idx.end(), (size_t)0);
  std::stable_sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return cmp(k[a], k[b]); });
  thrust::host_vector<T> k2(k.size());
  thrust::host_vector<unsigned> v2(k.size());
  for (size_t i = 0; i < idx.size(); ++i) { k2[i] = k[idx[i]]; if (v) v2[i] = (*v)[idx[i]]; }
  k = k2;
  if (v) *v = v2;
}

template <typename T> struct less_div_10 {
  __host__ __device__ bool operator()(const T& a, const T& b) const { return (int)a / 10 < (int)b / 10; }
};

template <typename T>
void test_sort_type(size_t n, long long lo, long long hi) {
  std::snprintf(g_ctx, sizeof g_ctx, "sort %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<T> h = random_vec<T>(n, 17 + (unsigned)n, lo, hi);
  thrust::device_vector<T> d = h;
  const auto f0 = fast();
  thrust::sort(tb::par, d.begin(), d.end());
  CHECK(fast() == f0 + 1);
  host_stable_sort_by_key(h, nullptr, std::less<T>());
  CHECK(thrust::host_vector<T>(d) == h);

  h = random_vec<T>(n, 18 + (unsigned)n, lo, hi);
  d = h;
  thrust::stable_sort(tb::par, d.begin(), d.end(), thrust::greater<T>());
  host_stable_sort_by_key(h, nullptr, std::greater<T>());
  CHECK(thrust::host_vector<T>(d) == h);

  // stability is observable: narrow keys, independent values
  thrust::host_vector<T> hk = random_vec<T>(n, 19 + (unsigned)n, lo / 64, hi / 64);
  thrust::host_vector<unsigned> hv = random_vec<unsigned>(n, 20, 0, 1 << 30);
  thrust::device_vector<T> dk = hk;
  thrust::device_vector<unsigned> dv = hv;
  thrust::stable_sort_by_key(tb::par, dk.begin(), dk.end(), dv.begin());
  host_stable_sort_by_key(hk, &hv, std::less<T>());
  CHECK(thrust::host_vector<T>(dk) == hk);
  CHECK(thrust::host_vector<unsigned>(dv) == hv);
  dk = hk = random_vec<T>(n, 21 + (unsigned)n, lo / 64, hi / 64);
  dv = hv = random_vec<unsigned>(n, 22, 0, 1 << 30);
  thrust::sort_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), thrust::greater<T>());
  host_stable_sort_by_key(hk, &hv, std::greater<T>());
  CHECK(thrust::host_vector<T>(dk) == hk);
  CHECK(thrust::host_vector<unsigned>(dv) == hv);
}

template <typename T>
void test_scan_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "scan %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<T> h = random_vec<T>(n, 31 + (unsigned)n, -1000, 1000);
  thrust::device_vector<T> d = h, out(n);
  thrust::host_vector<T> hout(n);
  const auto f0 = fast();
  auto e = thrust::inclusive_scan(tb::par, d.begin(), d.end(), out.begin());
  CHECK(e == out.end());
  CHECK(fast() == f0 + 1);
  thrust::inclusive_scan(thrust::host, h.begin(), h.end(), hout.begin());
  CHECK(thrust::host_vector<T>(out) == hout);
  thrust::exclusive_scan(tb::par, d.begin(), d.end(), out.begin());
  thrust::exclusive_scan(thrust::host, h.begin(), h.end(), hout.begin());
  CHECK(thrust::host_vector<T>(out) == hout);
  thrust::exclusive_scan(tb::par, d.begin(), d.end(), out.begin(), (T)11);
  thrust::exclusive_scan(thrust::host, h.begin(), h.end(), hout.begin(), (T)11);
  CHECK(thrust::host_vector<T>(out) == hout);
  thrust::exclusive_scan(tb::par, d.begin(), d.end(), out.begin(), (T)11, thrust::plus<T>());
  CHECK(thrust::host_vector<T>(out) == hout);
  CHECK(fast() == f0 + 4);
  // in place
  thrust::inclusive_scan(tb::par, d.begin(), d.end(), d.begin());
  thrust::inclusive_scan(thrust::host, h.begin(), h.end(), h.begin());
  CHECK(thrust::host_vector<T>(d) == h);
}

template <typename K, typename V>
void test_scan_by_key_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "scan_by_key %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<K> hk(n);
  std::mt19937 rng(53 + (unsigned)n);
  K cur = 0;
  for (size_t i = 0; i < n; ++i) { if (rng() % 5 == 0) cur = (K)(cur + 1); hk[i] = cur; }
  thrust::host_vector<V> hv = random_vec<V>(n, 59, 0, 1000), hout(n);
  thrust::device_vector<K> dk = hk;
  thrust::device_vector<V> dv = hv, out(n);
  const auto f0 = fast();
  auto e = thrust::inclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin());
  CHECK(e == out.end());
  thrust::inclusive_scan_by_key(thrust::host, hk.begin(), hk.end(), hv.begin(), hout.begin());
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::inclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin(), thrust::equal_to<K>());
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::inclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin(), thrust::equal_to<K>(),
                                thrust::plus<V>());
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::exclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin());
  thrust::exclusive_scan_by_key(thrust::host, hk.begin(), hk.end(), hv.begin(), hout.begin());
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::exclusive_scan_by_key(thrust::host, hk.begin(), hk.end(), hv.begin(), hout.begin(), (V)11);
  thrust::exclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin(), (V)11);
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::exclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin(), (V)11, thrust::equal_to<K>());
  CHECK(thrust::host_vector<V>(out) == hout);
  thrust::exclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), out.begin(), (V)11, thrust::equal_to<K>(),
                                thrust::plus<V>());
  CHECK(thrust::host_vector<V>(out) == hout);
  CHECK(fast() == f0 + 7);
  // in place on the values
  thrust::inclusive_scan_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), dv.begin());
  thrust::inclusive_scan_by_key(thrust::host, hk.begin(), hk.end(), hv.begin(), hv.begin());
  CHECK(thrust::host_vector<V>(dv) == hv);
}

template <typename T>
void test_reduce_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "reduce %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<T> h = random_vec<T>(n, 37 + (unsigned)n, -1000, 1000);
  thrust::device_vector<T> d = h;
  const auto f0 = fast();
  // all three arities (the CUDA system forwards the short forms with qualified calls,
  // thrust/system/cuda/detail/reduce.h:1045-1063)
  CHECK(thrust::reduce(tb::par, d.begin(), d.end()) == thrust::reduce(thrust::host, h.begin(), h.end()));
  CHECK(thrust::reduce(tb::par, d.begin(), d.end(), (T)13) == thrust::reduce(thrust::host, h.begin(), h.end(), (T)13));
  CHECK(thrust::reduce(tb::par, d.begin(), d.end(), (T)13, thrust::plus<T>()) ==
        thrust::reduce(thrust::host, h.begin(), h.end(), (T)13));
  CHECK(fast() == f0 + 3);
}

template <typename K, typename V>
void test_rbk_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "rbk %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<K> hk(n);
  std::mt19937 rng(41 + (unsigned)n);
  K cur = 0;
  for (size_t i = 0; i < n; ++i) { if (rng() % 3 == 0) cur = (K)(cur + 1); hk[i] = cur; }
  thrust::host_vector<V> hv = random_vec<V>(n, 43, 0, 1000);
  thrust::device_vector<K> dk = hk, dko(n);
  thrust::device_vector<V> dv = hv, dvo(n);
  thrust::host_vector<K> hko(n);
  thrust::host_vector<V> hvo(n);
  const auto f0 = fast();
  auto de = thrust::reduce_by_key(tb::par, dk.begin(), dk.end(), dv.begin(), dko.begin(), dvo.begin());
  CHECK(fast() == f0 + (n ? 1 : 0));
  auto he = thrust::reduce_by_key(thrust::host, hk.begin(), hk.end(), hv.begin(), hko.begin(), hvo.begin());
  const size_t runs = he.first - hko.begin();
  CHECK((size_t)(de.first - dko.begin()) == runs);
  CHECK((size_t)(de.second - dvo.begin()) == runs);
  dko.resize(runs); dvo.resize(runs); hko.resize(runs); hvo.resize(runs);
  CHECK(thrust::host_vector<K>(dko) == hko);
  CHECK(thrust::host_vector<V>(dvo) == hvo);
}

template <typename K, typename V>
void test_unique_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "unique %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<K> hk(n);
  std::mt19937 rng(51 + (unsigned)n);
  K cur = 0;
  for (size_t i = 0; i < n; ++i) { if (rng() % 3 == 0) cur = (K)(cur + 1); hk[i] = cur; }
  thrust::host_vector<V> hv = random_vec<V>(n, 53, 0, 100);
  thrust::device_vector<K> dk = hk, dko(n);
  thrust::device_vector<V> dv = hv, dvo(n);
  thrust::host_vector<K> hko(n);
  thrust::host_vector<V> hvo(n);
  const auto f0 = fast();
  auto de = thrust::unique_by_key_copy(tb::par, dk.begin(), dk.end(), dv.begin(), dko.begin(), dvo.begin());
  CHECK(fast() == f0 + (n ? 1 : 0));
  auto he = thrust::unique_by_key_copy(thrust::host, hk.begin(), hk.end(), hv.begin(), hko.begin(), hvo.begin());
  const size_t kept = he.first - hko.begin();
  CHECK((size_t)(de.first - dko.begin()) == kept);
  CHECK((size_t)(de.second - dvo.begin()) == kept);
  hko.resize(kept); hvo.resize(kept);
  CHECK(thrust::host_vector<K>(dko.begin(), dko.begin() + kept) == hko);
  CHECK(thrust::host_vector<V>(dvo.begin(), dvo.begin() + kept) == hvo);
  // keys only, copying and in place
  auto ue = thrust::unique_copy(tb::par, dk.begin(), dk.end(), dko.begin());
  CHECK((size_t)(ue - dko.begin()) == kept);
  CHECK(thrust::host_vector<K>(dko.begin(), dko.begin() + kept) == hko);
  thrust::device_vector<K> dk2 = dk;
  auto ie = thrust::unique(tb::par, dk2.begin(), dk2.end());
  CHECK((size_t)(ie - dk2.begin()) == kept);
  CHECK(thrust::host_vector<K>(dk2.begin(), dk2.begin() + kept) == hko);
  // in place by key
  auto pe = thrust::unique_by_key(tb::par, dk.begin(), dk.end(), dv.begin());
  CHECK((size_t)(pe.first - dk.begin()) == kept && (size_t)(pe.second - dv.begin()) == kept);
  CHECK(thrust::host_vector<K>(dk.begin(), dk.begin() + kept) == hko);
  CHECK(thrust::host_vector<V>(dv.begin(), dv.begin() + kept) == hvo);
}

template <typename T, typename F>
void test_copy_if_type(size_t n) {
  std::snprintf(g_ctx, sizeof g_ctx, "copy_if %s n=%zu", __PRETTY_FUNCTION__, n);
  thrust::host_vector<T> h = random_vec<T>(n, 61 + (unsigned)n, 0, 100);
  thrust::host_vector<F> hs = random_vec<F>(n, 62, 0, 2);
  thrust::device_vector<T> d = h, dout(n);
  thrust::device_vector<F> ds = hs;
  thrust::host_vector<T> hout(n);
  const auto f0 = fast();
  auto de = thrust::copy_if(tb::par, d.begin(), d.end(), ds.begin(), dout.begin(), thrust::identity<F>());
  CHECK(fast() == f0 + (n ? 1 : 0));
  auto he = thrust::copy_if(thrust::host, h.begin(), h.end(), hs.begin(), hout.begin(), thrust::identity<F>());
  const size_t kept = he - hout.begin();
  CHECK((size_t)(de - dout.begin()) == kept);
  hout.resize(kept);
  CHECK(thrust::host_vector<T>(dout.begin(), dout.begin() + kept) == hout);
}

template <typename T> struct is_even_pred {
  __host__ __device__ bool operator()(const T& x) const { return ((int)x & 1) == 0; }
};

// A caching allocator in the style of examples/cuda/custom_temporary_allocation.cu: blocks are
// kept and reused by size; `mallocs` counts the cudaMalloc calls it had to make.
struct caching_allocator {
  typedef char value_type;
  std::multimap<std::ptrdiff_t, char*> free_blocks;
  std::map<char*, std::ptrdiff_t> live;
  int mallocs = 0, allocations = 0, deallocations = 0;
  char* allocate(std::ptrdiff_t bytes) {
    ++allocations;
    char* p = nullptr;
    auto it = free_blocks.lower_bound(bytes);
    if (it != free_blocks.end()) { p = it->second; bytes = it->first; free_blocks.erase(it); }
    else { ++mallocs; if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) throw std::bad_alloc(); }
    live[p] = bytes;
    return p;
  }
  void deallocate(char* p, size_t) {
    ++deallocations;
    auto it = live.find(p);
    free_blocks.insert(std::make_pair(it->second, p));
    live.erase(it);
  }
  ~caching_allocator() {
    for (auto& b : free_blocks) cudaFree(b.second);
    for (auto& b : live) cudaFree(b.first);
  }
};

int main() {
  // ---- known answers -------------------------------------------------------------------
  {
    const int raw[7] = {1, 3, 6, 5, 2, 0, 4};
    thrust::device_vector<int> k(raw, raw + 7);
    thrust::sort(tb::par, k.begin(), k.end());
    for (int i = 0; i < 7; ++i) CHECK(k[i] == i);
    thrust::device_vector<int> k2(raw, raw + 7), v2(7);
    thrust::sequence(v2.begin(), v2.end());
    thrust::sort_by_key(tb::par, k2.begin(), k2.end(), v2.begin());
    const int want_v[7] = {5, 0, 4, 1, 6, 3, 2};
    for (int i = 0; i < 7; ++i) { CHECK(k2[i] == i); CHECK(v2[i] == want_v[i]); }
  }
  {
    const int raw[5] = {1, 3, -2, 4, -5};
    thrust::device_vector<int> in(raw, raw + 5), out(5);
    thrust::inclusive_scan(tb::par, in.begin(), in.end(), out.begin());
    const int w1[5] = {1, 4, 2, 6, 1};
    for (int i = 0; i < 5; ++i) CHECK(out[i] == w1[i]);
    thrust::exclusive_scan(tb::par, in.begin(), in.end(), out.begin());
    const int w2[5] = {0, 1, 4, 2, 6};
    for (int i = 0; i < 5; ++i) CHECK(out[i] == w2[i]);
    thrust::exclusive_scan(tb::par, in.begin(), in.end(), out.begin(), 3);
    const int w3[5] = {3, 4, 7, 5, 9};
    for (int i = 0; i < 5; ++i) CHECK(out[i] == w3[i]);
    thrust::inclusive_scan(tb::par, in.begin(), in.end(), in.begin());  // in place
    for (int i = 0; i < 5; ++i) CHECK(in[i] == w1[i]);
  }
  {
    const int rk[7] = {0, 1, 1, 1, 2, 3, 3}, rv[7] = {1, 2, 3, 4, 5, 6, 7};  // testing/scan_by_key.inclusive.cu:12-60
    thrust::device_vector<int> k(rk, rk + 7), v(rv, rv + 7), o(7);
    thrust::inclusive_scan_by_key(tb::par, k.begin(), k.end(), v.begin(), o.begin());
    const int w1[7] = {1, 2, 5, 9, 5, 6, 13};
    for (int i = 0; i < 7; ++i) CHECK(o[i] == w1[i]);
    thrust::exclusive_scan_by_key(tb::par, k.begin(), k.end(), v.begin(), o.begin());
    const int w2[7] = {0, 0, 2, 5, 0, 0, 6};
    for (int i = 0; i < 7; ++i) CHECK(o[i] == w2[i]);
    thrust::exclusive_scan_by_key(tb::par, k.begin(), k.end(), v.begin(), o.begin(), 10);
    const int w3[7] = {10, 10, 12, 15, 10, 10, 16};
    for (int i = 0; i < 7; ++i) CHECK(o[i] == w3[i]);
    // multiplies is not plus: forwarded, same answers as the reference's test
    const auto w0 = fwd();
    thrust::inclusive_scan_by_key(tb::par, k.begin(), k.end(), v.begin(), o.begin(), thrust::equal_to<int>(),
                                  thrust::multiplies<int>());
    const int w4[7] = {1, 2, 6, 24, 5, 6, 42};
    for (int i = 0; i < 7; ++i) CHECK(o[i] == w4[i]);
    thrust::exclusive_scan_by_key(tb::par, k.begin(), k.end(), v.begin(), o.begin(), 10, thrust::equal_to<int>(),
                                  thrust::multiplies<int>());
    const int w5[7] = {10, 10, 20, 60, 10, 10, 60};
    for (int i = 0; i < 7; ++i) CHECK(o[i] == w5[i]);
    CHECK(fwd() == w0 + 2);
  }
  {
    const int raw[3] = {1, -2, 3};  // testing/reduce.cu:26-38
    thrust::device_vector<int> v(raw, raw + 3);
    CHECK(thrust::reduce(tb::par, v.begin(), v.end()) == 2);
    CHECK(thrust::reduce(tb::par, v.begin(), v.end(), 10) == 12);
  }
  {
    const int rk[9] = {11, 11, 21, 20, 21, 21, 21, 37, 37};
    thrust::device_vector<int> k(rk, rk + 9), v(9), ko(9), vo(9);
    thrust::sequence(v.begin(), v.end());
    auto e = thrust::reduce_by_key(tb::par, k.begin(), k.end(), v.begin(), ko.begin(), vo.begin());
    CHECK(e.first - ko.begin() == 5);
    CHECK(e.second - vo.begin() == 5);
    const int wk[5] = {11, 21, 20, 21, 37}, wv[5] = {1, 2, 3, 15, 15};
    for (int i = 0; i < 5; ++i) { CHECK(ko[i] == wk[i]); CHECK(vo[i] == wv[i]); }
    e = thrust::reduce_by_key(tb::par, k.begin(), k.end(), v.begin(), ko.begin(), vo.begin(),
                              thrust::equal_to<int>(), thrust::plus<int>());
    CHECK(e.first - ko.begin() == 5);
    for (int i = 0; i < 5; ++i) { CHECK(ko[i] == wk[i]); CHECK(vo[i] == wv[i]); }
  }

  {
    // testing/unique_by_key.cu:127-207 (basic test and a predicate that is forwarded)
    const int rk[9] = {11, 11, 21, 20, 21, 21, 21, 37, 37};
    thrust::device_vector<int> k(rk, rk + 9), v(9);
    thrust::sequence(v.begin(), v.end());
    auto e = thrust::unique_by_key(tb::par, k.begin(), k.end(), v.begin());
    CHECK(e.first - k.begin() == 5 && e.second - v.begin() == 5);
    const int wk[5] = {11, 21, 20, 21, 37}, wv[5] = {0, 2, 3, 4, 7};
    for (int i = 0; i < 5; ++i) { CHECK(k[i] == wk[i]); CHECK(v[i] == wv[i]); }
    thrust::device_vector<int> k2(rk, rk + 9), v2(9), ko(9), vo(9);
    thrust::sequence(v2.begin(), v2.end());
    auto e2 = thrust::unique_by_key_copy(tb::par, k2.begin(), k2.end(), v2.begin(), ko.begin(), vo.begin());
    CHECK(e2.first - ko.begin() == 5 && e2.second - vo.begin() == 5);
    for (int i = 0; i < 5; ++i) { CHECK(ko[i] == wk[i]); CHECK(vo[i] == wv[i]); }
    const auto w0 = fwd();
    auto e3 = thrust::unique_by_key_copy(tb::par, k2.begin(), k2.end(), v2.begin(), ko.begin(), vo.begin(),
                                         [] __host__ __device__(int a, int b) { return a / 10 == b / 10; });
    CHECK(fwd() == w0 + 1);
    CHECK(e3.first - ko.begin() == 3);
    CHECK(ko[0] == 11 && ko[1] == 21 && ko[2] == 37 && vo[0] == 0 && vo[1] == 2 && vo[2] == 7);
    // copy_if: a predicate on the stencil other than identity, and the form without a stencil, are forwarded
    thrust::device_vector<int> out(9);
    auto c1 = thrust::copy_if(tb::par, v2.begin(), v2.end(), k2.begin(), out.begin(), is_even_pred<int>());
    CHECK(c1 - out.begin() == 1 && out[0] == 3);
    auto c2 = thrust::copy_if(tb::par, v2.begin(), v2.end(), out.begin(), is_even_pred<int>());
    CHECK(c2 - out.begin() == 5 && out[4] == 8);
    CHECK(fwd() == w0 + 3);
  }

  // ---- device == host over types and sizes ---------------------------------------------------
  for (size_t n : {(size_t)0, (size_t)1, (size_t)33, (size_t)10027, (size_t)300007}) {
    test_sort_type<signed char>(n, -128, 127);
    test_sort_type<unsigned short>(n, 0, 65535);
    test_sort_type<int>(n, -2000000000LL, 2000000000LL);
    test_sort_type<unsigned int>(n, 0, 4000000000LL);
    test_sort_type<long long>(n, -(1LL << 60), 1LL << 60);
    test_sort_type<unsigned long long>(n, 0, 1LL << 62);
    test_sort_type<float>(n, -100000, 100000);
    test_sort_type<double>(n, -100000, 100000);
    test_scan_type<int>(n);
    test_scan_type<unsigned int>(n);
    test_scan_type<long long>(n);
    test_scan_by_key_type<int, int>(n);
    test_scan_by_key_type<unsigned char, long long>(n);
    test_scan_by_key_type<long long, unsigned int>(n);
    test_reduce_type<signed char>(n);
    test_reduce_type<unsigned short>(n);
    test_reduce_type<int>(n);
    test_reduce_type<unsigned long long>(n);
    test_rbk_type<int, unsigned int>(n);
    test_rbk_type<unsigned char, long long>(n);
    test_rbk_type<long long, int>(n);
    test_unique_type<int, unsigned int>(n);
    test_unique_type<unsigned char, long long>(n);
    test_unique_type<long long, short>(n);
    test_unique_type<float, unsigned char>(n);
    test_copy_if_type<int, unsigned char>(n);
    test_copy_if_type<long long, int>(n);
    test_copy_if_type<short, bool>(n);
  }

  // ---- everything else is forwarded to the inherited CUDA path and still correct --------------
  {
    thrust::host_vector<int> h = random_vec<int>(5000, 7, 0, 999);
    thrust::device_vector<int> d = h;
    const auto w0 = fwd(), f0 = fast();
    thrust::stable_sort(tb::par, d.begin(), d.end(), less_div_10<int>());
    thrust::stable_sort(thrust::host, h.begin(), h.end(), less_div_10<int>());
    CHECK(fwd() == w0 + 1 && fast() == f0);
    CHECK(thrust::host_vector<int>(d) == h);
    // a max-scan is not plus
    thrust::device_vector<int> out(5000);
    thrust::host_vector<int> hout(5000);
    thrust::inclusive_scan(tb::par, d.begin(), d.end(), out.begin(), thrust::maximum<int>());
    thrust::inclusive_scan(thrust::host, h.begin(), h.end(), hout.begin(), thrust::maximum<int>());
    CHECK(fwd() == w0 + 2);
    CHECK(thrust::host_vector<int>(out) == hout);
    // a counting iterator is not contiguous
    thrust::inclusive_scan(tb::par, thrust::counting_iterator<int>(0), thrust::counting_iterator<int>(5000), out.begin());
    CHECK(fwd() == w0 + 3);
    CHECK(out[4999] == 4999 * 5000 / 2);
    // mixed types: the accumulator is the init's type (testing/scan.cu:250-320)
    thrust::device_vector<float> fin(4, 1.5f);
    thrust::device_vector<int> iout(4);
    thrust::exclusive_scan(tb::par, fin.begin(), fin.end(), iout.begin(), (int)0);
    CHECK(fwd() == w0 + 4);
    CHECK(iout[0] == 0 && iout[1] == 1 && iout[2] == 2 && iout[3] == 3);
    // reduce: float input with an int accumulator, and int input with a float one
    // (testing/reduce.cu:99-119), then an operator that is not plus
    thrust::device_vector<float> fr(4);
    fr[0] = 1.5f; fr[1] = 2.5f; fr[2] = 3.5f; fr[3] = 4.5f;
    thrust::device_vector<int> ir(4);
    ir[0] = 1; ir[1] = 2; ir[2] = 3; ir[3] = 4;
    CHECK(thrust::reduce(tb::par, fr.begin(), fr.end(), (int)0) == 10);
    CHECK(thrust::reduce(tb::par, ir.begin(), ir.end(), 0.5f) == 10.5f);
    CHECK(thrust::reduce(tb::par, ir.begin(), ir.end(), 0, thrust::maximum<int>()) == 4);
    CHECK(fwd() == w0 + 7);
  }

  // ---- dispatch by iterator tag, streams, nosync ---------------------------------------------
  {
    thrust::device_vector<int> d = random_vec<int>(4096, 9, -5000, 5000);
    const auto f0 = fast();
    thrust::sort(thrust::retag<tb::system>(d.begin()), thrust::retag<tb::system>(d.end()));
    CHECK(fast() == f0 + 1);
    CHECK(thrust::is_sorted(d.begin(), d.end()));

    cudaStream_t s;
    cudaStreamCreate(&s);
    thrust::device_vector<long long> a = random_vec<long long>(100000, 10, -1000, 1000), b(100000);
    thrust::host_vector<long long> ha = a, hb(100000);
    thrust::inclusive_scan(tb::par_nosync.on(s), a.begin(), a.end(), b.begin());
    cudaStreamSynchronize(s);
    thrust::inclusive_scan(thrust::host, ha.begin(), ha.end(), hb.begin());
    CHECK(thrust::host_vector<long long>(b) == hb);
    thrust::sort(tb::par.on(s), a.begin(), a.end());
    std::sort(ha.begin(), ha.end());
    CHECK(thrust::host_vector<long long>(a) == ha);
    // raw device pointers work too
    int* raw = thrust::raw_pointer_cast(d.data());
    thrust::sort(tb::par.on(s), raw, raw + d.size(), thrust::greater<int>());
    CHECK(thrust::is_sorted(d.begin(), d.end(), thrust::greater<int>()));
    cudaStreamDestroy(s);
  }

  // ---- scratch: the pool allocates nothing in steady state; par(alloc) uses the caller's allocator
  {
    std::snprintf(g_ctx, sizeof g_ctx, "scratch");
    thrust::device_vector<unsigned long long> k = random_vec<unsigned long long>(200000, 5, 0, 1LL << 40);
    thrust::device_vector<unsigned> v(200000);
    thrust::device_vector<int> a = random_vec<int>(200000, 6, -100, 100), b(200000);
    auto step = [&](tb::system pol) {
      thrust::sort_by_key(pol, k.begin(), k.end(), v.begin());
      thrust::inclusive_scan(pol, a.begin(), a.end(), b.begin());
      (void)thrust::reduce(pol, a.begin(), a.end());
      (void)thrust::unique_copy(pol, a.begin(), a.end(), b.begin());
    };
    step(tb::par);  // warm-up: the pool grows to what these calls need
    uint64_t allocs0 = 0, allocs1 = 0, held = 0;
    tb200_workspace_stats(&allocs0, &held);
    CHECK(held > 0);
    for (int i = 0; i < 100; ++i) step(tb::par);
    tb200_workspace_stats(&allocs1, &held);
    CHECK(allocs1 == allocs0);  // 400 steady-state calls, no device allocation

    caching_allocator alloc;
    const auto f0 = fast();
    step(tb::par(alloc));
    const int warm_mallocs = alloc.mallocs;
    CHECK(warm_mallocs >= 1 && alloc.allocations == 4 && alloc.deallocations == 4);
    cudaStream_t s;
    cudaStreamCreate(&s);
    for (int i = 0; i < 100; ++i) step(tb::par(alloc).on(s));
    CHECK(alloc.mallocs == warm_mallocs);  // every later call was served from the allocator's cache
    CHECK(alloc.allocations == 404 && alloc.deallocations == 404 && alloc.live.empty());
    CHECK(fast() == f0 + 404);
    tb200_workspace_stats(&allocs1, &held);
    CHECK(allocs1 == allocs0);  // the pool was not touched by the allocator-aware calls
    cudaStreamDestroy(s);
    CHECK(thrust::is_sorted(k.begin(), k.end()));
  }

  // ---- asynchronous forms: thrust::async::sort / inclusive_scan / exclusive_scan return events ---------
  {
    std::snprintf(g_ctx, sizeof g_ctx, "async");
    thrust::host_vector<int> h = random_vec<int>(300007, 77, -1000000, 1000000);
    thrust::device_vector<int> d = h, out(h.size());
    cudaStream_t s;
    cudaStreamCreate(&s);
    const auto f0 = fast();
    {
      auto e = thrust::async::sort(tb::par.on(s), d.begin(), d.end());
      CHECK(fast() == f0 + 1);
      e.wait();
    }
    std::sort(h.begin(), h.end());
    CHECK(thrust::host_vector<int>(d) == h);
    {
      auto e = thrust::async::inclusive_scan(tb::par.on(s), d.begin(), d.end(), out.begin());
      e.wait();
    }
    thrust::host_vector<int> hs(h.size());
    std::partial_sum(h.begin(), h.end(), hs.begin());
    CHECK(thrust::host_vector<int>(out) == hs);
    {
      auto e = thrust::async::exclusive_scan(tb::par, d.begin(), d.end(), out.begin(), 5);  // default stream: the event brings its own
      e.wait();
    }
    CHECK(out[0] == 5 && out[1] == 5 + h[0] && out[h.size() - 1] == 5 + hs[h.size() - 2]);
    {
      auto e = thrust::async::stable_sort(tb::par.on(s), d.begin(), d.end(), thrust::greater<int>());
      e.wait();
    }
    CHECK(thrust::is_sorted(d.begin(), d.end(), thrust::greater<int>()));
    CHECK(fast() == f0 + 4);
    // a comparator of the caller's is forwarded to the inherited asynchronous sort
    const auto w0 = fwd();
    {
      auto e = thrust::async::sort(tb::par.on(s), d.begin(), d.end(), less_div_10<int>());
      e.wait();
    }
    CHECK(fwd() == w0 + 1);
    CHECK(thrust::is_sorted(d.begin(), d.end(), less_div_10<int>()));
    cudaStreamDestroy(s);
  }

  // ---- two host threads on the default stream: every call holds its own scratch -----------------
  {
    std::snprintf(g_ctx, sizeof g_ctx, "threads");
    std::atomic<int> bad{0};
    auto worker = [&](unsigned seed, size_t n) {
      for (int rep = 0; rep < 20; ++rep) {
        thrust::host_vector<int> h = random_vec<int>(n, seed + (unsigned)rep, -1000000, 1000000);
        thrust::device_vector<int> d = h;
        thrust::sort(tb::par, d.begin(), d.end());
        std::sort(h.begin(), h.end());
        if (!(thrust::host_vector<int>(d) == h)) ++bad;
        thrust::device_vector<int> out(n);
        thrust::inclusive_scan(tb::par, d.begin(), d.end(), out.begin());
        thrust::host_vector<int> hs(n);
        std::partial_sum(h.begin(), h.end(), hs.begin());
        if (!(thrust::host_vector<int>(out) == hs)) ++bad;
      }
    };
    std::thread t1(worker, 100u, (size_t)300007), t2(worker, 200u, (size_t)5000011);  // the second keeps growing the pool
    t1.join();
    t2.join();
    CHECK(bad.load() == 0);
  }

  CHECK(cudaGetLastError() == cudaSuccess);
  tb200_workspace_release_all();
  std::printf("%s: %d checks, %d failed (fast-path calls %llu, forwarded %llu)\n", g_failed ? "FAILED" : "PASSED",
              g_checks, g_failed, fast(), fwd());
  return g_failed ? 1 : 0;
}
