// TEST INFRASTRUCTURE — not part of the product.
//
// C-ABI shim around the *unmodified* reference Thrust headers, compiled against
// the reference's own CPU device systems (THRUST_DEVICE_SYSTEM = OMP or CPP).
// It is built by oracle/Makefile into oracle/_ref/libthrust_ref_{omp,cpp}.so and
// is used (a) to validate the plain-C restatement in oracle/oracle.c, (b) as the
// parity checker in tests, and (c) as the timed CPU baseline of bench.py.
//
// Every entry point calls the public thrust:: algorithm with thrust::device, so
// the call stack is the reference's own:
//   sort            thrust/detail/sort.inl:30-38 -> generic/sort.inl:40-63 ->
//                   omp/detail/sort.inl:100-171 (OMP) or sequential/sort.inl:158-180 (CPP)
//   scan            thrust/detail/scan.inl:36-111 -> sequential/scan.h:39-116
//   reduce_by_key   generic/reduce_by_key.inl:67-132 (OMP), sequential/reduce_by_key.h:34-96 (CPP)
//   histogram       the recipe of examples/histogram.cu:60-101
//   unique_by_key   thrust/detail/unique.inl -> generic/unique_by_key.inl (OMP), sequential/unique_by_key.h:38-90 (CPP)
//   copy_if         thrust/detail/copy_if.inl -> generic/copy_if.inl (OMP), sequential/copy_if.h:38-67 (CPP)
#include <thrust/execution_policy.h>
#include <thrust/sort.h>
#include <thrust/scan.h>
#include <thrust/reduce.h>
#include <thrust/binary_search.h>
#include <thrust/adjacent_difference.h>
#include <thrust/functional.h>
#include <thrust/unique.h>
#include <thrust/copy.h>
#include <thrust/version.h>

#include <cstdint>
#include <cstddef>
#if defined(_OPENMP)
#include <omp.h>
#endif

// dtype codes shared with include/thrust_b200.h (kept numerically identical).
enum { DT_I8 = 0, DT_U8, DT_I16, DT_U16, DT_I32, DT_U32, DT_I64, DT_U64, DT_F32, DT_F64, DT_BOOL };

struct v16 { uint64_t a, b; };

template <typename K, typename V>
static int64_t ubk_kv(const void* kin, const void* vin, void* kout, void* vout, uint64_t n) {
  const K* k = static_cast<const K*>(kin);
  const V* v = static_cast<const V*>(vin);
  K* ko = static_cast<K*>(kout);
  V* vo = static_cast<V*>(vout);
  if (kin == kout) {  // the in-place form
    thrust::pair<K*, V*> e = thrust::unique_by_key(thrust::device, ko, ko + n, vo);
    return static_cast<int64_t>(e.first - ko);
  }
  thrust::pair<K*, V*> e = thrust::unique_by_key_copy(thrust::device, k, k + n, v, ko, vo);
  return static_cast<int64_t>(e.first - ko);
}
template <typename K>
static int64_t ubk_k(const void* kin, const void* vin, void* kout, void* vout, uint64_t n, int val_bytes) {
  switch (val_bytes) {
    case 0: {
      const K* k = static_cast<const K*>(kin);
      K* ko = static_cast<K*>(kout);
      if (kin == kout) return static_cast<int64_t>(thrust::unique(thrust::device, ko, ko + n) - ko);
      return static_cast<int64_t>(thrust::unique_copy(thrust::device, k, k + n, ko) - ko);
    }
    case 1: return ubk_kv<K, uint8_t>(kin, vin, kout, vout, n);
    case 2: return ubk_kv<K, uint16_t>(kin, vin, kout, vout, n);
    case 4: return ubk_kv<K, uint32_t>(kin, vin, kout, vout, n);
    case 8: return ubk_kv<K, uint64_t>(kin, vin, kout, vout, n);
    default: return -1;
  }
}
template <typename F, typename T>
static int64_t cpf_ft(const void* in, const void* flags, void* out, uint64_t n) {
  const T* d = static_cast<const T*>(in);
  const F* f = static_cast<const F*>(flags);
  T* o = static_cast<T*>(out);
  return static_cast<int64_t>(thrust::copy_if(thrust::device, d, d + n, f, o, thrust::identity<F>()) - o);
}
template <typename F>
static int64_t cpf_f(const void* in, const void* flags, void* out, uint64_t n, int elem_bytes) {
  switch (elem_bytes) {
    case 1: return cpf_ft<F, uint8_t>(in, flags, out, n);
    case 2: return cpf_ft<F, uint16_t>(in, flags, out, n);
    case 4: return cpf_ft<F, uint32_t>(in, flags, out, n);
    case 8: return cpf_ft<F, uint64_t>(in, flags, out, n);
    default: return -1;
  }
}

template <typename K>
static int sort_keys(void* keys, uint64_t n, int descending) {
  K* k = static_cast<K*>(keys);
  if (descending) thrust::sort(thrust::device, k, k + n, thrust::greater<K>());
  else            thrust::sort(thrust::device, k, k + n);
  return 0;
}

template <typename K, typename V>
static int sort_pairs_kv(void* keys, void* vals, uint64_t n, int descending) {
  K* k = static_cast<K*>(keys);
  V* v = static_cast<V*>(vals);
  if (descending) thrust::stable_sort_by_key(thrust::device, k, k + n, v, thrust::greater<K>());
  else            thrust::stable_sort_by_key(thrust::device, k, k + n, v);
  return 0;
}

template <typename K>
static int sort_pairs_k(void* keys, void* vals, uint64_t n, int val_bytes, int descending) {
  switch (val_bytes) {
    case 1: return sort_pairs_kv<K, uint8_t >(keys, vals, n, descending);
    case 2: return sort_pairs_kv<K, uint16_t>(keys, vals, n, descending);
    case 4: return sort_pairs_kv<K, uint32_t>(keys, vals, n, descending);
    case 8: return sort_pairs_kv<K, uint64_t>(keys, vals, n, descending);
    default: return -1;
  }
}

#define DISPATCH_KEY(DT, CALL)                                  \
  switch (DT) {                                                 \
    case DT_I8:  { typedef signed char   K; return CALL; }      \
    case DT_U8:  { typedef unsigned char K; return CALL; }      \
    case DT_I16: { typedef short         K; return CALL; }      \
    case DT_U16: { typedef unsigned short K; return CALL; }     \
    case DT_I32: { typedef int           K; return CALL; }      \
    case DT_U32: { typedef unsigned int  K; return CALL; }      \
    case DT_I64: { typedef long long     K; return CALL; }      \
    case DT_U64: { typedef unsigned long long K; return CALL; } \
    case DT_F32: { typedef float         K; return CALL; }      \
    case DT_F64: { typedef double        K; return CALL; }      \
    case DT_BOOL:{ typedef bool          K; return CALL; }      \
    default: return -1;                                         \
  }

#define DISPATCH_NUM(DT, CALL)                                  \
  switch (DT) {                                                 \
    case DT_I32: { typedef int           T; return CALL; }      \
    case DT_U32: { typedef unsigned int  T; return CALL; }      \
    case DT_I64: { typedef long long     T; return CALL; }      \
    case DT_U64: { typedef unsigned long long T; return CALL; } \
    case DT_F32: { typedef float         T; return CALL; }      \
    case DT_F64: { typedef double        T; return CALL; }      \
    default: return -1;                                         \
  }

template <typename K>
static int reduce_t(const void* in, uint64_t n, const void* init, void* out) {
  const K* i = static_cast<const K*>(in);
  *static_cast<K*>(out) = init ? thrust::reduce(thrust::device, i, i + n, *static_cast<const K*>(init))
                               : thrust::reduce(thrust::device, i, i + n);
  return 0;
}

template <typename K, typename V>
static int sbk_t(const void* kin, const void* vin, void* vout, uint64_t n, int exclusive, const void* init) {
  const K* k = static_cast<const K*>(kin);
  const V* v = static_cast<const V*>(vin);
  V* o = static_cast<V*>(vout);
  if (!exclusive)      thrust::inclusive_scan_by_key(thrust::device, k, k + n, v, o);
  else if (init)       thrust::exclusive_scan_by_key(thrust::device, k, k + n, v, o, *static_cast<const V*>(init));
  else                 thrust::exclusive_scan_by_key(thrust::device, k, k + n, v, o);
  return 0;
}
template <typename K>
static int sbk_k(const void* kin, const void* vin, void* vout, uint64_t n, int val_dtype, int exclusive,
                 const void* init) {
  switch (val_dtype) {
    case DT_I32: return sbk_t<K, int>(kin, vin, vout, n, exclusive, init);
    case DT_U32: return sbk_t<K, unsigned int>(kin, vin, vout, n, exclusive, init);
    case DT_I64: return sbk_t<K, long long>(kin, vin, vout, n, exclusive, init);
    case DT_U64: return sbk_t<K, unsigned long long>(kin, vin, vout, n, exclusive, init);
    case DT_F32: return sbk_t<K, float>(kin, vin, vout, n, exclusive, init);
    case DT_F64: return sbk_t<K, double>(kin, vin, vout, n, exclusive, init);
    default: return -1;
  }
}

template <typename T>
static int scan_t(const void* in, void* out, uint64_t n, int exclusive, const void* init) {
  const T* i = static_cast<const T*>(in);
  T* o = static_cast<T*>(out);
  if (!exclusive)      thrust::inclusive_scan(thrust::device, i, i + n, o);
  else if (init)       thrust::exclusive_scan(thrust::device, i, i + n, o, *static_cast<const T*>(init));
  else                 thrust::exclusive_scan(thrust::device, i, i + n, o);
  return 0;
}

template <typename K, typename V>
static int64_t rbk_kv(const void* kin, const void* vin, void* kout, void* vout, uint64_t n) {
  const K* k = static_cast<const K*>(kin);
  const V* v = static_cast<const V*>(vin);
  K* ko = static_cast<K*>(kout);
  V* vo = static_cast<V*>(vout);
  thrust::pair<K*, V*> e = thrust::reduce_by_key(thrust::device, k, k + n, v, ko, vo);
  return static_cast<int64_t>(e.first - ko);
}

template <typename K>
static int64_t rbk_k(const void* kin, const void* vin, void* kout, void* vout, uint64_t n, int vdt) {
  switch (vdt) {
    case DT_I32: return rbk_kv<K, int>(kin, vin, kout, vout, n);
    case DT_U32: return rbk_kv<K, unsigned int>(kin, vin, kout, vout, n);
    case DT_I64: return rbk_kv<K, long long>(kin, vin, kout, vout, n);
    case DT_U64: return rbk_kv<K, unsigned long long>(kin, vin, kout, vout, n);
    case DT_F32: return rbk_kv<K, float>(kin, vin, kout, vout, n);
    case DT_F64: return rbk_kv<K, double>(kin, vin, kout, vout, n);
    default: return -1;
  }
}

template <typename T>
static int hist_t(void* data, uint64_t n, const void* bin_values, uint32_t num_bins, uint32_t* counts) {
  T* d = static_cast<T*>(data);
  const T* b = static_cast<const T*>(bin_values);
  thrust::sort(thrust::device, d, d + n);
  thrust::upper_bound(thrust::device, d, d + n, b, b + num_bins, counts);
  thrust::adjacent_difference(thrust::device, counts, counts + num_bins, counts);
  return 0;
}

extern "C" {

int ref_thrust_version(void) { return THRUST_VERSION; }

int ref_device_system(void) { return THRUST_DEVICE_SYSTEM; }

// Launchers that start one process per GPU export OMP_NUM_THREADS=1; the timed baseline asks
// for the host's cores explicitly.
void ref_set_num_threads(int n) {
#if defined(_OPENMP)
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int ref_num_threads(void) {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// thrust::sort(first, last [, greater<K>()]) on n keys, in place.
int ref_sort(void* keys, uint64_t n, int key_dtype, int descending) {
  DISPATCH_KEY(key_dtype, sort_keys<K>(keys, n, descending));
}

// thrust::stable_sort_by_key(first, last, values [, greater<K>()]), in place.
int ref_sort_by_key(void* keys, void* vals, uint64_t n, int key_dtype, int val_bytes, int descending) {
  DISPATCH_KEY(key_dtype, sort_pairs_k<K>(keys, vals, n, val_bytes, descending));
}

// thrust::inclusive_scan / exclusive_scan with plus; init == NULL means the
// 4-argument exclusive_scan (init = value_type{}).
int ref_scan(const void* in, void* out, uint64_t n, int dtype, int exclusive, const void* init) {
  DISPATCH_NUM(dtype, scan_t<T>(in, out, n, exclusive, init));
}

// thrust::reduce(first, last, init) with plus; init == NULL means the 2-argument form
// (init = value_type(0)).
int ref_reduce(const void* in, uint64_t n, int dtype, const void* init, void* out) {
  if (dtype == DT_BOOL) return -1;
  DISPATCH_KEY(dtype, reduce_t<K>(in, n, init, out));
}

// thrust::inclusive_scan_by_key / exclusive_scan_by_key (equal_to, plus); init == NULL means
// the form without init (0).
int ref_scan_by_key(const void* kin, const void* vin, void* vout, uint64_t n, int key_dtype, int val_dtype,
                    int exclusive, const void* init) {
  DISPATCH_KEY(key_dtype, sbk_k<K>(kin, vin, vout, n, val_dtype, exclusive, init));
}

// thrust::reduce_by_key(keys, keys+n, vals, keys_out, vals_out) (equal_to, plus).
// Returns the number of runs written, or -1 for an unsupported type.
int64_t ref_reduce_by_key(const void* kin, const void* vin, void* kout, void* vout, uint64_t n,
                          int key_dtype, int val_dtype) {
  switch (key_dtype) {
    case DT_I8:  return rbk_k<signed char>(kin, vin, kout, vout, n, val_dtype);
    case DT_U8:  return rbk_k<unsigned char>(kin, vin, kout, vout, n, val_dtype);
    case DT_I16: return rbk_k<short>(kin, vin, kout, vout, n, val_dtype);
    case DT_U16: return rbk_k<unsigned short>(kin, vin, kout, vout, n, val_dtype);
    case DT_I32: return rbk_k<int>(kin, vin, kout, vout, n, val_dtype);
    case DT_U32: return rbk_k<unsigned int>(kin, vin, kout, vout, n, val_dtype);
    case DT_I64: return rbk_k<long long>(kin, vin, kout, vout, n, val_dtype);
    case DT_U64: return rbk_k<unsigned long long>(kin, vin, kout, vout, n, val_dtype);
    case DT_F32: return rbk_k<float>(kin, vin, kout, vout, n, val_dtype);
    case DT_F64: return rbk_k<double>(kin, vin, kout, vout, n, val_dtype);
    default: return -1;
  }
}

// thrust::unique_by_key_copy / unique_by_key (in place when kin == kout) / unique_copy / unique
// (val_bytes == 0) with equal_to. Returns the number of elements kept, or -1.
int64_t ref_unique_by_key(const void* kin, const void* vin, void* kout, void* vout, uint64_t n, int key_dtype,
                          int val_bytes) {
  DISPATCH_KEY(key_dtype, ubk_k<K>(kin, vin, kout, vout, n, val_bytes));
}

// thrust::copy_if(first, last, stencil, result, thrust::identity<Flag>()). Returns the count, or -1.
int64_t ref_copy_flagged(const void* in, const void* flags, void* out, uint64_t n, int elem_bytes, int flag_dtype) {
  DISPATCH_KEY(flag_dtype, cpf_f<K>(in, flags, out, n, elem_bytes));
}

// Dense histogram by the sort + upper_bound + adjacent_difference recipe
// (examples/histogram.cu:60-101). `data` is sorted in place; `bin_values` holds
// num_bins ascending search values of the same type (the example uses
// counting_iterator 0..num_bins-1); counts[b] = number of elements x with
// bin_values[b-1] < x <= bin_values[b] (x <= bin_values[0] for b == 0).
int ref_histogram(void* data, uint64_t n, int dtype, const void* bin_values, uint32_t num_bins,
                  uint32_t* counts) {
  DISPATCH_NUM(dtype, hist_t<T>(data, n, bin_values, num_bins, counts));
}

}  // extern "C"
