// Host-side runtime of the C ABI: status read-back, error strings, the workspace
// pool and the host-buffer entry points (stage in, run the device path, copy out).
#include "common.cuh"

#include <map>
#include <mutex>
#include <utility>
#include <vector>

namespace tb200 {
namespace {

// Workspace pool: blocks are leased per call. A lease is taken from the free blocks of its
// (device, stream) — so a block is only ever reused by work that is ordered after its previous
// use on that stream — and two host threads that share a stream simply hold different blocks.
struct PoolBlock {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool leased = false;
};
struct PoolKeyed {
  std::vector<PoolBlock> blocks;
};
std::mutex g_pool_mutex;
std::map<std::pair<int, cudaStream_t>, PoolKeyed> g_pool;
std::map<void*, std::pair<int, cudaStream_t>> g_pool_owner;  // leased block -> its (device, stream)
unsigned long long g_pool_mallocs = 0;  // cudaMalloc calls made by the pool since load
unsigned long long g_pool_bytes = 0;    // bytes the pool holds now

// The host-buffer forms carve their staging arrays and the algorithm scratch out of ONE lease.
struct Lease {  // returns the block to the pool when the host-buffer call leaves
  void* ptr = nullptr;
  ~Lease() { tb200_workspace_release(ptr); }
};

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  void* take(size_t bytes) {
    void* r = base ? base + off : nullptr;
    off += align_up(bytes, 256);
    return r;
  }
};

thread_local bool t_trace_on = false;
thread_local std::vector<cudaEvent_t> t_trace_events;
thread_local std::vector<int> t_trace_kinds;

}  // namespace

void trace_mark(cudaStream_t stream, int kind) {
  if (!t_trace_on) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, stream);
  t_trace_events.push_back(e);
  t_trace_kinds.push_back(kind);
}

}  // namespace tb200

extern "C" int tb200_trace_begin(tb200_stream_t stream) {
  using namespace tb200;
  for (cudaEvent_t e : t_trace_events) cudaEventDestroy(e);
  t_trace_events.clear();
  t_trace_kinds.clear();
  t_trace_on = true;
  trace_mark(stream, kTraceOther);
  return TB200_OK;
}

extern "C" int tb200_trace_end(float* ms, int* kinds, int capacity) {
  using namespace tb200;
  t_trace_on = false;
  if (t_trace_events.empty()) return 0;
  cudaError_t err = cudaEventSynchronize(t_trace_events.back());
  if (err != cudaSuccess) return -(int)err;
  const int launches = (int)t_trace_events.size() - 1;
  for (int i = 0; i < launches && i < capacity; ++i) {
    cudaEventElapsedTime(&ms[i], t_trace_events[i], t_trace_events[i + 1]);
    if (kinds) kinds[i] = t_trace_kinds[i + 1];
  }
  for (cudaEvent_t e : t_trace_events) cudaEventDestroy(e);
  t_trace_events.clear();
  return launches;
}

extern "C" int tb200_version(void) { return 100; }

extern "C" const char* tb200_error_string(int code) {
  switch (code) {
    case TB200_OK: return "success";
    case TB200_ERR_UNSUPPORTED: return "tb200: unsupported type or size";
    case TB200_ERR_INVALID_ARGUMENT: return "tb200: invalid argument";
    case TB200_ERR_TEMP_TOO_SMALL: return "tb200: temporary storage too small";
    case TB200_ERR_WAIT_TIMEOUT: return "tb200: bounded look-back wait ran out";
    case TB200_ERR_OVERFLOW: return "tb200: fixed-capacity buffer overflow";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "tb200: unknown error";
  }
}

extern "C" int tb200_temp_status(const void* d_temp, tb200_stream_t stream) {
  if (d_temp == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  int st = 0;
  TB200_CUDA_TRY(cudaMemcpyAsync(&st, d_temp, sizeof(int), cudaMemcpyDeviceToHost, stream));
  TB200_CUDA_TRY(cudaStreamSynchronize(stream));
  return st;
}

extern "C" int tb200_workspace_acquire(size_t bytes, tb200_stream_t stream, void** d_ptr) {
  using namespace tb200;
  if (d_ptr == nullptr) return TB200_ERR_INVALID_ARGUMENT;
  *d_ptr = nullptr;
  int dev = 0;
  TB200_CUDA_TRY(cudaGetDevice(&dev));
  const auto key = std::make_pair(dev, (cudaStream_t)stream);
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  PoolKeyed& k = g_pool[key];
  // smallest free block that is large enough
  PoolBlock* best = nullptr;
  for (PoolBlock& b : k.blocks)
    if (!b.leased && b.bytes >= bytes && (best == nullptr || b.bytes < best->bytes)) best = &b;
  if (best == nullptr) {
    // none fits: the free blocks of this (device, stream) are all too small, so give them back
    // first (cudaFree waits for the work that still uses them) and allocate one that fits
    for (size_t i = 0; i < k.blocks.size();) {
      if (!k.blocks[i].leased) {
        TB200_CUDA_TRY(cudaFree(k.blocks[i].ptr));
        g_pool_bytes -= k.blocks[i].bytes;
        k.blocks.erase(k.blocks.begin() + (long)i);
      } else {
        ++i;
      }
    }
    PoolBlock nb;
    nb.bytes = align_up(bytes + bytes / 16, (size_t)2 << 20);
    const cudaError_t err = cudaMalloc(&nb.ptr, nb.bytes);
    if (err != cudaSuccess) {
      (void)cudaGetLastError();  // clear the sticky allocation error, as the reference does
      return (int)err;
    }
    ++g_pool_mallocs;
    g_pool_bytes += nb.bytes;
    k.blocks.push_back(nb);
    best = &k.blocks.back();
  }
  best->leased = true;
  g_pool_owner[best->ptr] = key;
  *d_ptr = best->ptr;
  return TB200_OK;
}

extern "C" int tb200_workspace_release(void* d_ptr) {
  using namespace tb200;
  if (d_ptr == nullptr) return TB200_OK;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  auto owner = g_pool_owner.find(d_ptr);
  if (owner == g_pool_owner.end()) return TB200_ERR_INVALID_ARGUMENT;
  for (PoolBlock& b : g_pool[owner->second].blocks)
    if (b.ptr == d_ptr) b.leased = false;
  g_pool_owner.erase(owner);
  return TB200_OK;
}

extern "C" int tb200_workspace_stats(uint64_t* device_allocations, uint64_t* bytes_held) {
  using namespace tb200;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  if (device_allocations) *device_allocations = g_pool_mallocs;
  if (bytes_held) *bytes_held = g_pool_bytes;
  return TB200_OK;
}

extern "C" int tb200_workspace_release_all(void) {
  using namespace tb200;
  std::lock_guard<std::mutex> lock(g_pool_mutex);
  int rc = TB200_OK;
  int cur = 0;
  cudaGetDevice(&cur);
  for (auto& kv : g_pool) {
    for (PoolBlock& b : kv.second.blocks) {
      cudaSetDevice(kv.first.first);
      const cudaError_t e = cudaFree(b.ptr);
      if (e != cudaSuccess) rc = (int)e;
    }
  }
  g_pool.clear();
  g_pool_owner.clear();
  g_pool_bytes = 0;
  cudaSetDevice(cur);
  return rc;
}

extern "C" int tb200_scan_host(const void* h_in, void* h_out, uint64_t n, int dtype, int exclusive,
                               const void* h_init, tb200_stream_t stream) {
  using namespace tb200;
  const int eb = dtype_bytes(dtype);
  if (eb == 0) return TB200_ERR_UNSUPPORTED;
  if (n == 0) return TB200_OK;
  if (!h_in || !h_out) return TB200_ERR_INVALID_ARGUMENT;
  size_t temp_bytes = 0;
  int rc = tb200_scan(nullptr, &temp_bytes, nullptr, nullptr, n, dtype, exclusive, h_init, stream);
  if (rc) return rc;
  Carver size(nullptr);
  size.take(temp_bytes);
  size.take((size_t)n * eb);
  Lease lease;
  rc = tb200_workspace_acquire(size.off, stream, &lease.ptr);
  if (rc) return rc;
  Carver c(lease.ptr);
  void* d_temp = c.take(temp_bytes);
  void* d_data = c.take((size_t)n * eb);
  TB200_CUDA_TRY(cudaMemcpyAsync(d_data, h_in, (size_t)n * eb, cudaMemcpyHostToDevice, stream));
  rc = tb200_scan(d_temp, &temp_bytes, d_data, d_data, n, dtype, exclusive, h_init, stream);
  if (rc) return rc;
  TB200_CUDA_TRY(cudaMemcpyAsync(h_out, d_data, (size_t)n * eb, cudaMemcpyDeviceToHost, stream));
  return tb200_temp_status(d_temp, stream);
}

extern "C" int tb200_radix_sort_host(void* h_keys, void* h_vals, uint64_t n, int key_dtype, int val_bytes,
                                     int descending, tb200_stream_t stream) {
  using namespace tb200;
  const int kb = dtype_bytes(key_dtype);
  if (kb == 0) return TB200_ERR_UNSUPPORTED;
  if (n == 0) return TB200_OK;
  if (!h_keys || (val_bytes && !h_vals)) return TB200_ERR_INVALID_ARGUMENT;
  size_t temp_bytes = 0;
  int rc = tb200_radix_sort(nullptr, &temp_bytes, nullptr, nullptr, n, key_dtype, val_bytes, descending, 0,
                            8 * kb, stream);
  if (rc) return rc;
  Carver size(nullptr);
  size.take(temp_bytes);
  size.take((size_t)n * kb);
  size.take((size_t)n * val_bytes);
  Lease lease;
  rc = tb200_workspace_acquire(size.off, stream, &lease.ptr);
  if (rc) return rc;
  Carver c(lease.ptr);
  void* d_temp = c.take(temp_bytes);
  void* d_keys = c.take((size_t)n * kb);
  void* d_vals = c.take((size_t)n * val_bytes);
  TB200_CUDA_TRY(cudaMemcpyAsync(d_keys, h_keys, (size_t)n * kb, cudaMemcpyHostToDevice, stream));
  if (val_bytes)
    TB200_CUDA_TRY(cudaMemcpyAsync(d_vals, h_vals, (size_t)n * val_bytes, cudaMemcpyHostToDevice, stream));
  rc = tb200_radix_sort(d_temp, &temp_bytes, d_keys, val_bytes ? d_vals : nullptr, n, key_dtype, val_bytes,
                        descending, 0, 8 * kb, stream);
  if (rc) return rc;
  TB200_CUDA_TRY(cudaMemcpyAsync(h_keys, d_keys, (size_t)n * kb, cudaMemcpyDeviceToHost, stream));
  if (val_bytes)
    TB200_CUDA_TRY(cudaMemcpyAsync(h_vals, d_vals, (size_t)n * val_bytes, cudaMemcpyDeviceToHost, stream));
  return tb200_temp_status(d_temp, stream);
}

extern "C" int tb200_reduce_by_key_host(const void* h_keys_in, const void* h_vals_in, void* h_keys_out,
                                        void* h_vals_out, uint64_t* h_num_runs, uint64_t n, int key_dtype,
                                        int val_dtype, tb200_stream_t stream) {
  using namespace tb200;
  const int kb = dtype_bytes(key_dtype), vb = dtype_bytes(val_dtype);
  if (kb == 0 || vb == 0) return TB200_ERR_UNSUPPORTED;
  if (!h_num_runs) return TB200_ERR_INVALID_ARGUMENT;
  *h_num_runs = 0;
  if (n == 0) return TB200_OK;
  if (!h_keys_in || !h_vals_in || !h_keys_out || !h_vals_out) return TB200_ERR_INVALID_ARGUMENT;
  size_t temp_bytes = 0;
  int rc = tb200_reduce_by_key(nullptr, &temp_bytes, nullptr, nullptr, nullptr, nullptr, nullptr, n,
                               key_dtype, val_dtype, stream);
  if (rc) return rc;
  Carver size(nullptr);
  size.take(temp_bytes);
  size.take(256);
  for (int i = 0; i < 2; ++i) { size.take((size_t)n * kb); size.take((size_t)n * vb); }
  Lease lease;
  rc = tb200_workspace_acquire(size.off, stream, &lease.ptr);
  if (rc) return rc;
  Carver c(lease.ptr);
  void* d_temp = c.take(temp_bytes);
  auto* d_runs = static_cast<uint64_t*>(c.take(256));
  void* d_kin = c.take((size_t)n * kb);
  void* d_vin = c.take((size_t)n * vb);
  void* d_kout = c.take((size_t)n * kb);
  void* d_vout = c.take((size_t)n * vb);
  TB200_CUDA_TRY(cudaMemcpyAsync(d_kin, h_keys_in, (size_t)n * kb, cudaMemcpyHostToDevice, stream));
  TB200_CUDA_TRY(cudaMemcpyAsync(d_vin, h_vals_in, (size_t)n * vb, cudaMemcpyHostToDevice, stream));
  rc = tb200_reduce_by_key(d_temp, &temp_bytes, d_kin, d_vin, d_kout, d_vout, d_runs, n, key_dtype,
                           val_dtype, stream);
  if (rc) return rc;
  uint64_t runs = 0;
  TB200_CUDA_TRY(cudaMemcpyAsync(&runs, d_runs, sizeof(runs), cudaMemcpyDeviceToHost, stream));
  TB200_CUDA_TRY(cudaStreamSynchronize(stream));
  TB200_CUDA_TRY(cudaMemcpyAsync(h_keys_out, d_kout, (size_t)runs * kb, cudaMemcpyDeviceToHost, stream));
  TB200_CUDA_TRY(cudaMemcpyAsync(h_vals_out, d_vout, (size_t)runs * vb, cudaMemcpyDeviceToHost, stream));
  *h_num_runs = runs;
  return tb200_temp_status(d_temp, stream);
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded-wait convention: a kernel polls a flag that nothing sets, with
// the same loop shape the look-back chains use, gives up after `limit_polls` polls and
// reports TB200_ERR_WAIT_TIMEOUT through a status word — the context stays usable.
// ---------------------------------------------------------------------------------------
namespace tb200 {
namespace {
__global__ void selftest_wait_kernel(const unsigned* flag, unsigned limit_polls, int* status) {
  unsigned polls = 0;
  while (ld_relaxed_u32(flag) == 0u) {
    backoff(++polls);
    if (polls >= limit_polls) {
      atomicExch(status, (int)TB200_ERR_WAIT_TIMEOUT);
      break;
    }
  }
}
}  // namespace
}  // namespace tb200

extern "C" int tb200_selftest_wait_timeout(uint32_t limit_polls, tb200_stream_t stream) {
  using namespace tb200;
  if (limit_polls == 0 || limit_polls > (1u << 20)) return TB200_ERR_INVALID_ARGUMENT;
  Lease lease;
  int rc = tb200_workspace_acquire(512, stream, &lease.ptr);
  if (rc) return rc;
  void* ws = lease.ptr;
  TB200_CUDA_TRY(cudaMemsetAsync(ws, 0, 512, stream));
  int* status = static_cast<int*>(ws);
  const unsigned* flag = reinterpret_cast<const unsigned*>(static_cast<char*>(ws) + 256);
  selftest_wait_kernel<<<1, 32, 0, stream>>>(flag, limit_polls, status);
  TB200_CUDA_TRY(cudaGetLastError());
  return tb200_temp_status(ws, stream);
}
