// Stream compaction on the by-key streaming skeleton (seg_stream.cuh): unique_by_key /
// unique (the first element of every run of equal consecutive keys) and the copy of flagged
// elements (copy_if with a stencil). One pass: flags, a look-back chain over the per-tile
// counts, and a compacting scatter of the selected elements in input order.
//
// Values are opaque payloads of 1, 2, 4, 8 or 16 bytes; keys compare with == (integers by
// bit pattern, floating point with IEEE equality, like thrust::equal_to).
#include "common.cuh"
#include "seg_stream.cuh"

namespace tb200 {
namespace {

template <int MODE, typename K, typename V>
int launch_select(void* d_temp, size_t* temp_bytes, const void* kin, const void* vin, void* kout, void* vout,
                  uint64_t* d_num_out, uint64_t n, cudaStream_t stream, int trace_kind) {
  constexpr bool kHasVals = seg::Shape<K, V>::kHasVals;
  const size_t need = seg::scratch_bytes<K, V>(n);
  if (d_temp == nullptr) {
    *temp_bytes = need;
    return TB200_OK;
  }
  if (*temp_bytes < need) return TB200_ERR_TEMP_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(d_temp) % 256) return TB200_ERR_INVALID_ARGUMENT;
  if (d_num_out == nullptr || reinterpret_cast<uintptr_t>(d_num_out) % 8) return TB200_ERR_INVALID_ARGUMENT;
  TB200_CUDA_TRY(cudaMemsetAsync(d_temp, 0, need, stream));
  TB200_CUDA_TRY(cudaMemsetAsync(d_num_out, 0, sizeof(uint64_t), stream));
  if (n == 0) return TB200_OK;
  if (!kin || (kHasVals && (!vin || !vout)) || (MODE == seg::kUniqueByKey && !kout)) return TB200_ERR_INVALID_ARGUMENT;
  uintptr_t bits = reinterpret_cast<uintptr_t>(kin);
  if (kHasVals) bits |= reinterpret_cast<uintptr_t>(vin);
  const bool bulk = bits % 16 == 0;
  // unique / unique_by_key may run in place (thrust::unique_by_key is unique_by_key_copy onto its own input)
  auto overlap = [n](const void* in, const void* out, size_t elem) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(in), b = reinterpret_cast<uintptr_t>(out), len = (uintptr_t)n * elem;
    return in && out && a < b + len && b < a + len;
  };
  const bool inplace = (MODE == seg::kUniqueByKey && overlap(kin, kout, sizeof(K))) ||
                       (kHasVals && overlap(vin, vout, seg::Shape<K, V>::kValSize));
  const int rc = seg::launch<MODE, K, V>(static_cast<const K*>(kin), static_cast<const V*>(vin), static_cast<K*>(kout),
                                         static_cast<V*>(vout), reinterpret_cast<unsigned long long*>(d_num_out), n,
                                         V{}, bulk, d_temp, stream, inplace);
  trace_mark(stream, trace_kind);
  return rc;
}

template <int MODE, typename K>
int select_vals(int val_bytes, void* d_temp, size_t* temp_bytes, const void* kin, const void* vin, void* kout,
                void* vout, uint64_t* d_num_out, uint64_t n, cudaStream_t stream, int trace_kind) {
#define TB200_SEL(V) \
  return launch_select<MODE, K, V>(d_temp, temp_bytes, kin, vin, kout, vout, d_num_out, n, stream, trace_kind)
  switch (val_bytes) {
    case 0:
      if constexpr (MODE == seg::kUniqueByKey) TB200_SEL(seg::NoVal);
      else return TB200_ERR_UNSUPPORTED;
    case 1: TB200_SEL(seg::Blob<1>::type);
    case 2: TB200_SEL(seg::Blob<2>::type);
    case 4: TB200_SEL(seg::Blob<4>::type);
    case 8: TB200_SEL(seg::Blob<8>::type);
    case 16: TB200_SEL(seg::Blob<16>::type);
    default: return TB200_ERR_UNSUPPORTED;
  }
#undef TB200_SEL
}

template <int MODE>
int select_keys(int key_dtype, int val_bytes, void* d_temp, size_t* temp_bytes, const void* kin, const void* vin,
                void* kout, void* vout, uint64_t* d_num_out, uint64_t n, cudaStream_t stream, int trace_kind) {
#define TB200_SEL(K) \
  return select_vals<MODE, K>(val_bytes, d_temp, temp_bytes, kin, vin, kout, vout, d_num_out, n, stream, trace_kind)
  switch (key_dtype) {
    case TB200_I8: case TB200_U8: case TB200_BOOL: TB200_SEL(uint8_t);
    case TB200_I16: case TB200_U16: TB200_SEL(uint16_t);
    case TB200_I32: case TB200_U32: TB200_SEL(uint32_t);
    case TB200_I64: case TB200_U64: TB200_SEL(unsigned long long);
    case TB200_F32: TB200_SEL(float);
    case TB200_F64: TB200_SEL(double);
    default: return TB200_ERR_UNSUPPORTED;
  }
#undef TB200_SEL
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_unique_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys_in, const void* d_vals_in,
                                   void* d_keys_out, void* d_vals_out, uint64_t* d_num_out, uint64_t n, int key_dtype,
                                   int val_bytes, tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  return select_keys<seg::kUniqueByKey>(key_dtype, val_bytes, d_temp, temp_bytes, d_keys_in, d_vals_in, d_keys_out,
                                        d_vals_out, d_num_out, n, stream, kTraceUniqueByKey);
}

extern "C" int tb200_copy_flagged(void* d_temp, size_t* temp_bytes, const void* d_in, const void* d_flags, void* d_out,
                                  uint64_t* d_num_out, uint64_t n, int elem_bytes, int flag_dtype,
                                  tb200_stream_t stream) {
  using namespace tb200;
  if (temp_bytes == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  return select_keys<seg::kCopyFlagged>(flag_dtype, elem_bytes, d_temp, temp_bytes, d_flags, d_in, nullptr, d_out,
                                        d_num_out, n, stream, kTraceCopyFlagged);
}
