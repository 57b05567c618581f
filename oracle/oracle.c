/* TEST INFRASTRUCTURE — not part of the product, never linked or called by it.
 *
 * Plain-C, single-threaded restatement of the reference's CPU algorithms for the
 * sort / scan / reduce_by_key / sort-based-histogram path. Only tests/,
 * __graft_entry__.smoke() and the cpu_baseline leg of bench.py may load it.
 *
 * Parity pin: tests/test_oracle.py checks every function here against (a) the
 * known-answer vectors of the reference's own unit tests (tests/golden/) and
 * (b) the unmodified reference headers compiled as oracle/_ref (ref_shim.cpp),
 * on seeded random inputs of every supported type.
 *
 * Reference files restated (paths inside the reference project):
 *   key encoders      thrust/system/detail/sequential/stable_radix_sort.inl:43-141
 *   LSD radix sort    thrust/system/detail/sequential/stable_radix_sort.inl:224-339
 *   greater<T>        thrust/system/detail/sequential/sort.inl:54-104
 *   scans             thrust/system/detail/sequential/scan.h:39-116
 *   reduce            thrust/system/detail/sequential/reduce.h:43-62
 *   reduce_by_key     thrust/system/detail/sequential/reduce_by_key.h:34-96
 *   scan_by_key       thrust/system/detail/sequential/scan_by_key.h:34-146
 *   histogram         examples/histogram.cu:60-101 (+ generic/binary_search.inl:95-133)
 *   unique_by_key     thrust/system/detail/sequential/unique_by_key.h:38-90
 *   copy_if (stencil) thrust/system/detail/sequential/copy_if.h:38-67
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

enum { DT_I8 = 0, DT_U8, DT_I16, DT_U16, DT_I32, DT_U32, DT_I64, DT_U64, DT_F32, DT_F64, DT_BOOL };

static int dtype_bytes(int dt) {
  switch (dt) {
    case DT_I8: case DT_U8: case DT_BOOL: return 1;
    case DT_I16: case DT_U16: return 2;
    case DT_I32: case DT_U32: case DT_F32: return 4;
    case DT_I64: case DT_U64: case DT_F64: return 8;
    default: return 0;
  }
}

/* RadixEncoder<T> (stable_radix_sort.inl:43-141): unsigned and bool keys are used
 * as they are; signed integers flip the sign bit; float/double flip every bit of
 * a negative value and only the sign bit of a non-negative one. The result is an
 * unsigned integer whose natural order is the key order (a bitwise total order
 * for floating point: -0.0 sorts before +0.0, NaNs sort by payload). */
static uint64_t encode_key(const void* p, int dt) {
  switch (dt) {
    case DT_U8: case DT_BOOL: return *(const uint8_t*)p;
    case DT_I8:  return (uint8_t)(*(const uint8_t*)p ^ 0x80u);
    case DT_U16: return *(const uint16_t*)p;
    case DT_I16: return (uint16_t)(*(const uint16_t*)p ^ 0x8000u);
    case DT_U32: return *(const uint32_t*)p;
    case DT_I32: return *(const uint32_t*)p ^ 0x80000000u;
    case DT_U64: return *(const uint64_t*)p;
    case DT_I64: return *(const uint64_t*)p ^ 0x8000000000000000ull;
    case DT_F32: {
      uint32_t i = *(const uint32_t*)p;
      uint32_t mask = (uint32_t)(-(int32_t)(i >> 31)) | 0x80000000u;
      return i ^ mask;
    }
    case DT_F64: {
      uint64_t i = *(const uint64_t*)p;
      uint64_t mask = (uint64_t)(-(int64_t)(i >> 63)) | 0x8000000000000000ull;
      return i ^ mask;
    }
    default: return 0;
  }
}

static void reverse_bytes_array(void* base, uint64_t n, int width) {
  unsigned char* a = (unsigned char*)base;
  unsigned char tmp[16];
  if (n < 2) return;
  for (uint64_t i = 0, j = n - 1; i < j; ++i, --j) {
    memcpy(tmp, a + i * width, (size_t)width);
    memcpy(a + i * width, a + j * width, (size_t)width);
    memcpy(a + j * width, tmp, (size_t)width);
  }
}

/* radix_sort<8, HasValues> (stable_radix_sort.inl:224-339): one upfront sweep
 * builds the histogram of every digit position; each histogram is turned into
 * exclusive offsets; a pass whose histogram has one bin holding all N keys is
 * skipped; every other pass is a stable scatter between two ping-pong buffers;
 * a final copy brings the result back if it ended in the second buffer.
 * The reference picks 3, 4 or 8 radix bits by N; a stable LSD sort gives the
 * same output for any digit width, so 8 bits is used throughout. */
static int radix_sort_ascending(void* keys, void* vals, uint64_t n, int dt, int vbytes) {
  const int kbytes = dtype_bytes(dt);
  if (kbytes == 0) return -1;
  if (n < 2) return 0;
  const int passes = kbytes;
  uint64_t (*hist)[256] = calloc((size_t)passes, sizeof *hist);
  unsigned char* k1 = (unsigned char*)keys;
  unsigned char* v1 = (unsigned char*)vals;
  unsigned char* k2 = malloc((size_t)n * kbytes);
  unsigned char* v2 = vals ? malloc((size_t)n * vbytes) : NULL;
  uint64_t* enc = malloc((size_t)n * sizeof(uint64_t));
  uint64_t* enc2 = malloc((size_t)n * sizeof(uint64_t));
  if (!hist || !k2 || (vals && !v2) || !enc || !enc2) { free(hist); free(k2); free(v2); free(enc); free(enc2); return -2; }

  for (uint64_t i = 0; i < n; ++i) {
    uint64_t x = encode_key(k1 + i * kbytes, dt);
    enc[i] = x;
    for (int j = 0; j < passes; ++j) hist[j][(x >> (8 * j)) & 0xff]++;
  }
  int skip[8] = {0};
  for (int j = 0; j < passes; ++j) {
    uint64_t sum = 0;
    for (int b = 0; b < 256; ++b) {
      uint64_t c = hist[j][b];
      if (c == n) skip[j] = 1;
      hist[j][b] = sum;
      sum += c;
    }
  }
  int flip = 0;
  for (int j = 0; j < passes; ++j) {
    if (skip[j]) continue;
    unsigned char *ks = flip ? k2 : k1, *kd = flip ? k1 : k2;
    unsigned char *vs = flip ? v2 : v1, *vd = flip ? v1 : v2;
    uint64_t *es = flip ? enc2 : enc, *ed = flip ? enc : enc2;
    for (uint64_t i = 0; i < n; ++i) {
      uint64_t pos = hist[j][(es[i] >> (8 * j)) & 0xff]++;
      memcpy(kd + pos * kbytes, ks + i * kbytes, (size_t)kbytes);
      ed[pos] = es[i];
      if (vals) memcpy(vd + pos * vbytes, vs + i * vbytes, (size_t)vbytes);
    }
    flip = !flip;
  }
  if (flip) {
    memcpy(k1, k2, (size_t)n * kbytes);
    if (vals) memcpy(v1, v2, (size_t)n * vbytes);
  }
  free(hist); free(k2); free(v2); free(enc); free(enc2);
  return 0;
}

/* thrust::sort / stable_sort on arithmetic keys with less<T> (descending == 0)
 * or greater<T> (descending != 0): sort ascending, then reverse (sort.inl:54-71). */
int oracle_sort(void* keys, uint64_t n, int key_dtype, int descending) {
  int rc = radix_sort_ascending(keys, NULL, n, key_dtype, 0);
  if (rc) return rc;
  if (descending) reverse_bytes_array(keys, n, dtype_bytes(key_dtype));
  return 0;
}

/* thrust::sort_by_key / stable_sort_by_key. greater<T>: reverse keys and values,
 * sort ascending, reverse both again, which keeps equal keys in input order in
 * the descending output (sort.inl:74-104). */
int oracle_sort_by_key(void* keys, void* vals, uint64_t n, int key_dtype, int val_bytes, int descending) {
  const int kb = dtype_bytes(key_dtype);
  if (kb == 0 || val_bytes < 1 || val_bytes > 16) return -1;
  if (descending) { reverse_bytes_array(keys, n, kb); reverse_bytes_array(vals, n, val_bytes); }
  int rc = radix_sort_ascending(keys, vals, n, key_dtype, val_bytes);
  if (rc) return rc;
  if (descending) { reverse_bytes_array(keys, n, kb); reverse_bytes_array(vals, n, val_bytes); }
  return 0;
}

/* inclusive_scan: accumulator has the input's value type, strictly left to right
 * (scan.h:39-73). exclusive_scan: accumulator has the type of init, the input
 * element is read before the output is written so in == out works (scan.h:76-116).
 * init == NULL stands for value_type{} (generic/scan.inl:51-63). */
#define SCAN_BODY(T)                                                        \
  do {                                                                      \
    const T* a = (const T*)in; T* o = (T*)out;                              \
    if (n == 0) return 0;                                                   \
    if (!exclusive) {                                                       \
      T sum = a[0]; o[0] = sum;                                             \
      for (uint64_t i = 1; i < n; ++i) { sum = (T)(sum + a[i]); o[i] = sum; } \
    } else {                                                                \
      T sum = init ? *(const T*)init : (T)0;                                \
      for (uint64_t i = 0; i < n; ++i) { T tmp = a[i]; o[i] = sum; sum = (T)(sum + tmp); } \
    }                                                                       \
    return 0;                                                               \
  } while (0)

int oracle_scan(const void* in, void* out, uint64_t n, int dtype, int exclusive, const void* init) {
  switch (dtype) {
    case DT_I32: case DT_U32: SCAN_BODY(uint32_t);   /* two's-complement wrap == unsigned add */
    case DT_I64: case DT_U64: SCAN_BODY(uint64_t);
    case DT_F32: SCAN_BODY(float);
    case DT_F64: SCAN_BODY(double);
    default: return -1;
  }
}

/* reduce with plus (sequential/reduce.h:43-62): the accumulator starts as init, has its
 * type, and adds the elements left to right. The narrow integer types add in int and
 * convert back after every step, which is addition modulo 2^width. init == NULL is 0. */
#define REDUCE_BODY(T)                                                      \
  do {                                                                      \
    const T* a = (const T*)in;                                              \
    T sum = init ? *(const T*)init : (T)0;                                  \
    for (uint64_t i = 0; i < n; ++i) sum = (T)(sum + a[i]);                 \
    *(T*)out = sum;                                                         \
    return 0;                                                               \
  } while (0)

int oracle_reduce(const void* in, uint64_t n, int dtype, const void* init, void* out) {
  switch (dtype) {
    case DT_I8: case DT_U8: REDUCE_BODY(uint8_t);   /* two's-complement wrap == unsigned add */
    case DT_I16: case DT_U16: REDUCE_BODY(uint16_t);
    case DT_I32: case DT_U32: REDUCE_BODY(uint32_t);
    case DT_I64: case DT_U64: REDUCE_BODY(uint64_t);
    case DT_F32: REDUCE_BODY(float);
    case DT_F64: REDUCE_BODY(double);
    default: return -1;
  }
}

/* reduce_by_key with equal_to / plus (reduce_by_key.h:34-96): a run's key is its
 * FIRST key, every later key is compared with that first key, the accumulator has
 * the values' type and adds left to right. Returns the number of runs. */
#define RBK_BODY(KT, VT, EQ)                                                \
  do {                                                                      \
    const KT* k = (const KT*)kin; const VT* v = (const VT*)vin;             \
    KT* ko = (KT*)kout; VT* vo = (VT*)vout;                                 \
    if (n == 0) return 0;                                                   \
    int64_t r = 0; KT tk = k[0]; VT tv = v[0];                              \
    for (uint64_t i = 1; i < n; ++i) {                                      \
      if (EQ(tk, k[i])) tv = (VT)(tv + v[i]);                               \
      else { ko[r] = tk; vo[r] = tv; ++r; tk = k[i]; tv = v[i]; }           \
    }                                                                       \
    ko[r] = tk; vo[r] = tv; ++r;                                            \
    return r;                                                               \
  } while (0)
#define EQ_PLAIN(a, b) ((a) == (b))

#define RBK_VALS(KT)                                                        \
  switch (val_dtype) {                                                      \
    case DT_I32: case DT_U32: RBK_BODY(KT, uint32_t, EQ_PLAIN);             \
    case DT_I64: case DT_U64: RBK_BODY(KT, uint64_t, EQ_PLAIN);             \
    case DT_F32: RBK_BODY(KT, float, EQ_PLAIN);                             \
    case DT_F64: RBK_BODY(KT, double, EQ_PLAIN);                            \
    default: return -1;                                                     \
  }

/* inclusive / exclusive scan_by_key with equal_to / plus (scan_by_key.h:34-146): consecutive
 * keys are compared; the inclusive accumulator has the values' type; the exclusive one starts
 * every run at init and adds left to right ((init + v0) + v1 ...). init == NULL is 0. */
#define SBK_BODY(KT, VT)                                                    \
  do {                                                                      \
    const KT* k = (const KT*)kin; const VT* v = (const VT*)vin;             \
    VT* o = (VT*)vout;                                                      \
    const VT ini = init ? *(const VT*)init : (VT)0;                         \
    if (n == 0) return 0;                                                   \
    if (!exclusive) {                                                       \
      VT pv = v[0]; o[0] = pv;                                              \
      for (uint64_t i = 1; i < n; ++i) {                                    \
        const VT x = v[i];                                                  \
        pv = (k[i - 1] == k[i]) ? (VT)(pv + x) : x;                         \
        o[i] = pv;                                                          \
      }                                                                     \
    } else {                                                                \
      VT next = ini;                                                        \
      for (uint64_t i = 0; i < n; ++i) {                                    \
        const VT x = v[i];                                                  \
        if (i > 0 && !(k[i - 1] == k[i])) next = ini;                       \
        o[i] = next;                                                        \
        next = (VT)(next + x);                                              \
      }                                                                     \
    }                                                                       \
    return 0;                                                               \
  } while (0)

#define SBK_VALS(KT)                                                        \
  switch (val_dtype) {                                                      \
    case DT_I32: case DT_U32: SBK_BODY(KT, uint32_t);                       \
    case DT_I64: case DT_U64: SBK_BODY(KT, uint64_t);                       \
    case DT_F32: SBK_BODY(KT, float);                                       \
    case DT_F64: SBK_BODY(KT, double);                                      \
    default: return -1;                                                     \
  }

int oracle_scan_by_key(const void* kin, const void* vin, void* vout, uint64_t n, int key_dtype, int val_dtype,
                       int exclusive, const void* init) {
  switch (key_dtype) {
    case DT_I8: case DT_U8: case DT_BOOL: SBK_VALS(uint8_t);
    case DT_I16: case DT_U16: SBK_VALS(uint16_t);
    case DT_I32: case DT_U32: SBK_VALS(uint32_t);
    case DT_I64: case DT_U64: SBK_VALS(uint64_t);
    case DT_F32: SBK_VALS(float);
    case DT_F64: SBK_VALS(double);
    default: return -1;
  }
}

int64_t oracle_reduce_by_key(const void* kin, const void* vin, void* kout, void* vout, uint64_t n,
                             int key_dtype, int val_dtype) {
  switch (key_dtype) {
    case DT_I8: case DT_U8: case DT_BOOL: RBK_VALS(uint8_t);
    case DT_I16: case DT_U16: RBK_VALS(uint16_t);
    case DT_I32: case DT_U32: RBK_VALS(uint32_t);
    case DT_I64: case DT_U64: RBK_VALS(uint64_t);
    case DT_F32: RBK_VALS(float);     /* IEEE ==: -0.0 equals +0.0, NaN equals nothing */
    case DT_F64: RBK_VALS(double);
    default: return -1;
  }
}

/* Dense histogram recipe (examples/histogram.cu:60-101): sort the data, take
 * upper_bound of every bin value in the sorted data (the cumulative histogram;
 * upper_bound compares with operator<, generic/binary_search.inl:95-133), then
 * adjacent_difference in place. `data` is left sorted. */
#define HIST_BODY(T)                                                        \
  do {                                                                      \
    const T* d = (const T*)data; const T* b = (const T*)bin_values;         \
    for (uint32_t j = 0; j < num_bins; ++j) {                               \
      uint64_t lo = 0, hi = n;                                              \
      while (lo < hi) { uint64_t mid = lo + (hi - lo) / 2;                  \
        if (b[j] < d[mid]) hi = mid; else lo = mid + 1; }                   \
      counts[j] = (uint32_t)lo;                                             \
    }                                                                       \
  } while (0)

int oracle_histogram(void* data, uint64_t n, int dtype, const void* bin_values, uint32_t num_bins,
                     uint32_t* counts) {
  int rc = oracle_sort(data, n, dtype, 0);
  if (rc) return rc;
  switch (dtype) {
    case DT_I32: HIST_BODY(int32_t); break;
    case DT_U32: HIST_BODY(uint32_t); break;
    case DT_I64: HIST_BODY(int64_t); break;
    case DT_U64: HIST_BODY(uint64_t); break;
    case DT_F32: HIST_BODY(float); break;
    case DT_F64: HIST_BODY(double); break;
    default: return -1;
  }
  for (uint32_t j = num_bins; j-- > 1;) counts[j] -= counts[j - 1];
  return 0;
}

/* unique_by_key_copy with equal_to (unique_by_key.h:38-90): the first (key, value) pair of every
 * run is kept; every later key is compared with the KEPT key of the run (temp_key), not with its
 * neighbour. Values are opaque (val_bytes 0 = the keys-only form, thrust::unique). The outputs
 * may be the inputs (the reference's in-place form is this same loop). Returns the pairs kept. */
#define UBK_BODY(KT)                                                        \
  do {                                                                      \
    const KT* k = (const KT*)kin; KT* ko = (KT*)kout;                       \
    const unsigned char* v = (const unsigned char*)vin;                     \
    unsigned char* vo = (unsigned char*)vout;                               \
    unsigned char tv[16];                                                   \
    if (n == 0) return 0;                                                   \
    int64_t r = 0; KT tk = k[0];                                            \
    if (val_bytes) memcpy(tv, v, (size_t)val_bytes);                        \
    for (uint64_t i = 1; i < n; ++i) {                                      \
      const KT key = k[i];                                                  \
      unsigned char val[16];                                                \
      if (val_bytes) memcpy(val, v + i * (uint64_t)val_bytes, (size_t)val_bytes); \
      if (!(tk == key)) {                                                   \
        ko[r] = tk;                                                         \
        if (val_bytes) memcpy(vo + (uint64_t)r * val_bytes, tv, (size_t)val_bytes); \
        ++r; tk = key;                                                      \
        if (val_bytes) memcpy(tv, val, (size_t)val_bytes);                  \
      }                                                                     \
    }                                                                       \
    ko[r] = tk;                                                             \
    if (val_bytes) memcpy(vo + (uint64_t)r * val_bytes, tv, (size_t)val_bytes); \
    return r + 1;                                                           \
  } while (0)

int64_t oracle_unique_by_key(const void* kin, const void* vin, void* kout, void* vout, uint64_t n, int key_dtype,
                             int val_bytes) {
  if (val_bytes < 0 || val_bytes > 16) return -1;
  switch (key_dtype) {
    case DT_I8: case DT_U8: case DT_BOOL: UBK_BODY(uint8_t);
    case DT_I16: case DT_U16: UBK_BODY(uint16_t);
    case DT_I32: case DT_U32: UBK_BODY(uint32_t);
    case DT_I64: case DT_U64: UBK_BODY(uint64_t);
    case DT_F32: UBK_BODY(float);     /* IEEE ==: -0.0 equals +0.0, NaN equals nothing */
    case DT_F64: UBK_BODY(double);
    default: return -1;
  }
}

/* copy_if(first, last, stencil, result, identity) (copy_if.h:38-67): element i is copied when
 * its stencil value converts to true, i.e. is non-zero. Elements are opaque. Returns the count. */
#define CPF_BODY(FT)                                                        \
  do {                                                                      \
    const FT* f = (const FT*)flags;                                         \
    const unsigned char* d = (const unsigned char*)in;                      \
    unsigned char* o = (unsigned char*)out;                                 \
    int64_t r = 0;                                                          \
    for (uint64_t i = 0; i < n; ++i)                                        \
      if (f[i] != (FT)0) { memcpy(o + (uint64_t)r * elem_bytes, d + i * (uint64_t)elem_bytes, (size_t)elem_bytes); ++r; } \
    return r;                                                               \
  } while (0)

int64_t oracle_copy_flagged(const void* in, const void* flags, void* out, uint64_t n, int elem_bytes, int flag_dtype) {
  if (elem_bytes < 1 || elem_bytes > 16) return -1;
  switch (flag_dtype) {
    case DT_I8: case DT_U8: case DT_BOOL: CPF_BODY(uint8_t);
    case DT_I16: case DT_U16: CPF_BODY(uint16_t);
    case DT_I32: case DT_U32: CPF_BODY(uint32_t);
    case DT_I64: case DT_U64: CPF_BODY(uint64_t);
    case DT_F32: CPF_BODY(float);
    case DT_F64: CPF_BODY(double);
    default: return -1;
  }
}
