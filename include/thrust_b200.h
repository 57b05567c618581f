/* thrust_b200 — C ABI of the B200 (sm_100a) sort / scan / reduce_by_key path.
 *
 * This is the boundary a Thrust custom system (include/thrust_b200/system.h) binds
 * to. Every entry point replaces one dispatch of the reference's CUDA system
 * (file:line below are paths inside the reference project, Thrust 2.2.0).
 *
 * Conventions
 *  - All data pointers are DEVICE pointers unless a parameter is named h_*.
 *  - Scratch follows the two-phase convention the reference uses around its device
 *    library calls (thrust/system/cuda/detail/sort.h:330-365, scan.h:80-118,
 *    reduce_by_key.h:999-1047): call with d_temp == NULL to get *temp_bytes, then
 *    call again with a buffer of at least that size (256-byte aligned).
 *  - Work is enqueued on `stream` and the call returns without synchronising.
 *    Kernels never trap or spin forever: a wait that runs out records a status
 *    word in d_temp, read back with tb200_temp_status() after the stream is idle.
 *  - Return value: 0 = success, > 0 = a cudaError_t, < 0 = one of tb200_error.
 *  - Re-entrant: no global mutable state except the optional workspace pool
 *    (mutex protected, leases per call). Calls that share d_temp must be stream-ordered.
 */
#ifndef THRUST_B200_H_
#define THRUST_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tb200_stream_t; /* same type as cudaStream_t */

typedef enum tb200_dtype {
  TB200_I8 = 0, TB200_U8 = 1, TB200_I16 = 2, TB200_U16 = 3, TB200_I32 = 4, TB200_U32 = 5,
  TB200_I64 = 6, TB200_U64 = 7, TB200_F32 = 8, TB200_F64 = 9, TB200_BOOL = 10
} tb200_dtype;

typedef enum tb200_error {
  TB200_OK = 0,
  TB200_ERR_UNSUPPORTED = -1,      /* type / size combination has no kernel            */
  TB200_ERR_INVALID_ARGUMENT = -2, /* NULL pointer, bad bit range, misaligned temp ... */
  TB200_ERR_TEMP_TOO_SMALL = -3,   /* *temp_bytes below what the size query returned   */
  TB200_ERR_WAIT_TIMEOUT = -4,     /* a bounded look-back wait ran out (device status) */
  TB200_ERR_OVERFLOW = -5          /* a fixed-capacity buffer would have overflowed    */
} tb200_error;

/* Library version (major*10000 + minor*100 + patch) and a static description string. */
int tb200_version(void);
const char* tb200_error_string(int code);

/* ---- radix sort ---------------------------------------------------------------------
 * Stable LSD radix sort of n arithmetic keys, in place, optionally carrying one value
 * array (val_bytes in {0,1,2,4,8,16}; 0 = keys only, d_vals ignored). Order: the
 * reference's key encoding (sequential/stable_radix_sort.inl:43-141): integers by value,
 * floating point by the bitwise total order (-0.0 before +0.0, NaNs by payload).
 * descending != 0 gives thrust::greater<Key> with equal keys kept in input order
 * (sequential/sort.inl:74-104). Only key bits [begin_bit, end_bit) are compared
 * (0 and 8*sizeof(key) sort whole keys, which is what Thrust does).
 * Replaces: thrust::cuda_cub::__radix_sort::radix_sort and the four
 * cub::DeviceRadixSort calls behind sort / stable_sort / sort_by_key / stable_sort_by_key
 * (thrust/system/cuda/detail/sort.h:209-380, 493-623). n is 64-bit (the reference
 * narrows it to int, sort.h:228). */
int tb200_radix_sort(void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n,
                     int key_dtype, int val_bytes, int descending, int begin_bit, int end_bit,
                     tb200_stream_t stream);

/* ---- stable multi-way partition -------------------------------------------------------
 * Scatters n (key, value) pairs into num_splitters + 1 contiguous buckets of d_keys_out /
 * d_vals_out, keeping input order inside a bucket: bucket b holds the keys in
 * (splitter[b-1], splitter[b]] (unsigned comparison; splitters ascending, at most 255).
 * d_counts (device, num_splitters + 1 x uint64) receives the bucket sizes. key_dtype U32 or
 * U64, val_bytes 0, 4 or 8; outputs must not overlap inputs. One onesweep pass whose digit
 * is the bucket id. It is the partition step of the sharded sample sort; the reference's
 * closest algorithm is the two-way thrust::stable_partition (cuda/detail/partition.h:138),
 * it has no multi-way form. */
int tb200_partition(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                    void* d_keys_out, void* d_vals_out, uint64_t n, int key_dtype, int val_bytes,
                    const void* d_splitters, uint32_t num_splitters, uint64_t* d_counts,
                    tb200_stream_t stream);

/* The two halves of tb200_partition, for callers that place the buckets themselves.
 * tb200_partition_count writes the bucket sizes to d_counts (it reads the keys once);
 * tb200_partition_scatter, called once afterwards with the same scratch, keys and splitters,
 * moves bucket b to h_bucket_keys[b] / h_bucket_vals[b]: HOST arrays of num_splitters + 1
 * device pointers to each bucket's first element. The buckets may lie in different
 * allocations, including memory of another GPU mapped into this process (the partition then
 * stores straight across NVLink: the push form of the sharded sort's exchange, where bucket
 * b is rank b's share and its pointer is rank b's receive buffer plus what lower ranks send
 * there). Plain stores only; no counterpart in the reference. */
int tb200_partition_count(void* d_temp, size_t* temp_bytes, const void* d_keys, uint64_t n, int key_dtype,
                          int val_bytes, const void* d_splitters, uint32_t num_splitters, uint64_t* d_counts,
                          tb200_stream_t stream);
int tb200_partition_scatter(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals, uint64_t n,
                            int key_dtype, int val_bytes, const void* d_splitters, uint32_t num_splitters,
                            void* const* h_bucket_keys, void* const* h_bucket_vals, tb200_stream_t stream);

/* The same three with (key, index) PAIRS as the thing that is compared: splitter i is the pair
 * (d_splitters[i], d_splitter_index[i]), element g of the input is the pair (key, index_base + g),
 * pairs compare by key first, then by index, and bucket b holds the pairs in (splitter[b-1],
 * splitter[b]]. Equal keys can then be divided between buckets, in input order: the sharded sort
 * uses this (index = position in the global sequence) when a few keys make up most of the
 * input and all copies of one key would not fit one rank. d_splitter_index == NULL is the plain
 * form. No counterpart in the reference. */
int tb200_partition_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                         void* d_keys_out, void* d_vals_out, uint64_t n, int key_dtype, int val_bytes,
                         const void* d_splitters, const uint64_t* d_splitter_index, uint32_t num_splitters,
                         uint64_t index_base, uint64_t* d_counts, tb200_stream_t stream);
int tb200_partition_count_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, uint64_t n, int key_dtype,
                               int val_bytes, const void* d_splitters, const uint64_t* d_splitter_index,
                               uint32_t num_splitters, uint64_t index_base, uint64_t* d_counts,
                               tb200_stream_t stream);
int tb200_partition_scatter_ties(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals,
                                 uint64_t n, int key_dtype, int val_bytes, const void* d_splitters,
                                 const uint64_t* d_splitter_index, uint32_t num_splitters, uint64_t index_base,
                                 void* const* h_bucket_keys, void* const* h_bucket_vals, tb200_stream_t stream);

/* ---- segment gather (exchange step of the sharded sort) ---------------------------------
 * Concatenates num_segments (at most 16) source ranges into d_dst, in order: segment s is
 * h_count[s] elements of elem_bytes (4, 8 or 16) starting h_src_offset[s] elements into
 * h_src[s]. The three arrays are HOST arrays; the source pointers are device pointers and may
 * be peer mappings of other GPUs' memory (the caller establishes the mapping and the
 * ordering against the peers' writes). One kernel of plain loads and stores: each GPU pulls
 * its runs over NVLink itself instead of calling a collective. Its CTAs work on all segments
 * at once, starting `rotate` segments in (pass the caller's rank), so that neither one
 * source GPU nor one link is read by everyone at the same time. No counterpart in the
 * reference (it has no multi-GPU code).
 * d_sort_temp (may be NULL; 8-byte elements only): scratch of a uint64 sort prepared with
 * tb200_radix_sort_begin — the kernel then also counts the digits of every key it moves, so
 * that tb200_radix_sort_finish can skip the sort's own histogram pass over the data. */
int tb200_gather_segments(void* d_dst, const void* const* h_src, const uint64_t* h_src_offset,
                          const uint64_t* h_count, uint32_t num_segments, int elem_bytes,
                          uint32_t rotate, void* d_sort_temp, tb200_stream_t stream);

/* tb200_radix_sort in two halves for whole uint64 keys (ascending): _begin clears the scratch,
 * the caller accumulates the histograms of the n keys through tb200_gather_segments(...,
 * d_sort_temp, ...), _finish runs the passes. Same scratch size and result as tb200_radix_sort. */
int tb200_radix_sort_begin(void* d_temp, size_t* temp_bytes, uint64_t n, int key_dtype, int val_bytes,
                           tb200_stream_t stream);
int tb200_radix_sort_finish(void* d_temp, size_t* temp_bytes, void* d_keys, void* d_vals, uint64_t n,
                            int key_dtype, int val_bytes, tb200_stream_t stream);

/* ---- scan ---------------------------------------------------------------------------
 * Prefix sum with plus over n elements of dtype in {I32,U32,I64,U64,F32,F64}; accumulator
 * type == element type. exclusive == 0: inclusive_scan. exclusive != 0: exclusive_scan.
 * Both are seeded with *h_init (a HOST pointer to one element; NULL = value-initialised zero):
 * out[i] = init + in[0] + ... + in[i] or init + in[0] + ... + in[i-1]. (A seeded inclusive
 * scan is what a shard of a distributed scan runs: the seed is the sum of the shards in front.)
 * d_out may equal d_in (exactly in place); no other overlap.
 * Replaces: cuda_cub::detail::inclusive_scan_n_impl / exclusive_scan_n_impl and their
 * cub::DispatchScan calls (thrust/system/cuda/detail/scan.h:50-125, 127-204). */
int tb200_scan(void* d_temp, size_t* temp_bytes, const void* d_in, void* d_out, uint64_t n,
               int dtype, int exclusive, const void* h_init, tb200_stream_t stream);

/* tb200_scan without any allocation — no counterpart in the reference (its scan always
 * allocates scratch through the policy, thrust/system/cuda/detail/scan.h:96-104).
 * For callers that must not allocate device memory around the call: code that runs while
 * another component owns the allocator (a framework's caching pool, a fixed arena sized at
 * start-up), latency-critical loops where cudaMalloc's device-wide synchronisation is not
 * acceptable, and processes near their memory limit where a late allocation could fail.
 * The look-back descriptors live in a device array inside the library (about 2 MiB on every
 * GPU that loads it, held until the process exits), so the caller passes only input and
 * output. Limits: n <= 2^31 elements for 4-byte types, n <= 2^29 for 8-byte types (both
 * inclusive); larger n returns TB200_ERR_OVERFLOW before anything is enqueued (use
 * tb200_scan). The first call on each device looks up the
 * array's device address; make that first call outside any stream capture. All calls on a
 * device share the one array (each call clears what it needs on `stream` first), so calls
 * that can overlap on the GPU — different streams without ordering — race; keep them
 * stream-ordered. Makes no cudaMalloc / cudaFree and calls no allocating library routine. */
int tb200_scan_static(const void* d_in, void* d_out, uint64_t n, int dtype, int exclusive,
                      const void* h_init, tb200_stream_t stream);
/* Device status word of the last tb200_scan_static call on the current device (0 or a
 * tb200_error such as TB200_ERR_WAIT_TIMEOUT): tb200_temp_status for the library's own array,
 * which the caller cannot name. Synchronises `stream`. No counterpart in the reference. */
int tb200_scan_static_status(tb200_stream_t stream);

/* ---- reduce_by_key ------------------------------------------------------------------
 * Runs of consecutive equal keys (thrust::equal_to<Key>) are reduced with plus over the
 * values' own type. Emits, per run, its FIRST key (thrust/reduce.h:347) and the sum, and
 * writes the run count to *d_num_runs (device, 8-byte aligned). Key types: any
 * tb200_dtype; value dtype in {I32,U32,I64,U64,F32,F64}. Outputs must not overlap inputs.
 * Replaces: cuda_cub::__reduce_by_key::reduce_by_key_dispatch / doit_step and the
 * InitAgent + ReduceByKeyAgent kernels (thrust/system/cuda/detail/reduce_by_key.h:81-1058).
 * Unlike the reference (reduce_by_key.h:1049-1052) the call itself does not synchronise;
 * the caller reads *d_num_runs when it needs the end iterators. */
int tb200_reduce_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys_in,
                        const void* d_vals_in, void* d_keys_out, void* d_vals_out,
                        uint64_t* d_num_runs, uint64_t n, int key_dtype, int val_dtype,
                        tb200_stream_t stream);

/* ---- scan_by_key ----------------------------------------------------------------------
 * Segmented prefix sums with thrust::equal_to on consecutive keys and thrust::plus:
 * out[i] = sum of the elements of i's run up to and including i (exclusive == 0), or
 * init + the sum of those before i (exclusive != 0: every run restarts at init; h_init is a
 * HOST pointer to one value, NULL = 0). Keys: any dtype code (integers by bit pattern,
 * floating point with IEEE ==); values: 4- or 8-byte integers, F32, F64. d_vals_out may be
 * d_vals_in. Integer sums are exact (they wrap); floating-point sums are formed in scan-tree
 * order. Replaces thrust::cuda_cub::detail::{inclusive,exclusive}_scan_by_key_n and their
 * cub::DispatchScanByKey (thrust/system/cuda/detail/scan_by_key.h:96-290); semantics of
 * thrust/system/detail/sequential/scan_by_key.h:34-146. */
int tb200_scan_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys, const void* d_vals_in,
                      void* d_vals_out, uint64_t n, int key_dtype, int val_dtype, int exclusive,
                      const void* h_init, tb200_stream_t stream);

/* ---- unique_by_key / unique ------------------------------------------------------------
 * Keeps the FIRST (key, value) pair of every run of consecutive equal keys (thrust::equal_to:
 * integers by bit pattern, floating point with IEEE ==), in input order, and writes the number
 * of pairs kept to *d_num_out (device, 8-byte aligned). Keys: any dtype code; values: opaque
 * payloads of val_bytes in {1,2,4,8,16}, or val_bytes == 0 for the keys-only form
 * (thrust::unique / unique_copy; d_vals_in and d_vals_out ignored). The outputs may be the
 * inputs themselves (d_keys_out == d_keys_in and d_vals_out == d_vals_in: the in-place forms
 * thrust::unique_by_key / thrust::unique); no other overlap.
 * Replaces thrust::cuda_cub::unique_by_key_copy / unique_by_key and the UniqueByKeyAgent
 * behind them (thrust/system/cuda/detail/unique_by_key.h:190-590, 716-905); semantics of
 * thrust/system/detail/sequential/unique_by_key.h:38-90. */
int tb200_unique_by_key(void* d_temp, size_t* temp_bytes, const void* d_keys_in, const void* d_vals_in,
                        void* d_keys_out, void* d_vals_out, uint64_t* d_num_out, uint64_t n, int key_dtype,
                        int val_bytes, tb200_stream_t stream);

/* ---- copy of flagged elements (copy_if with a stencil) -----------------------------------
 * d_out receives, in input order, every element d_in[i] (opaque, elem_bytes in {1,2,4,8,16})
 * whose flag d_flags[i] (any dtype code) is non-zero; *d_num_out (device, 8-byte aligned)
 * the number copied. This is thrust::copy_if(first, last, stencil, result,
 * thrust::identity<Flag>()). Output must not overlap the inputs.
 * Replaces thrust::cuda_cub::__copy_if::copy_if and its CopyIfAgent
 * (thrust/system/cuda/detail/copy_if.h:161-570, 699-826); semantics of
 * thrust/system/detail/sequential/copy_if.h:38-67. */
int tb200_copy_flagged(void* d_temp, size_t* temp_bytes, const void* d_in, const void* d_flags, void* d_out,
                       uint64_t* d_num_out, uint64_t n, int elem_bytes, int flag_dtype, tb200_stream_t stream);

/* ---- reduce ---------------------------------------------------------------------------
 * *d_out = init + in[0] + ... + in[n-1] with thrust::plus in the element type (integer sums
 * wrap; dtype: any integer or floating-point code, not BOOL). h_init is a HOST pointer to
 * one element, NULL = 0; d_out is a device pointer to one element; n = 0 gives init. The
 * sum is reproducible from run to run on one device; for floating point it differs from the
 * left-to-right order of the reference's CPU systems (sequential/reduce.h:43-62) by rounding
 * only. Replaces thrust::cuda_cub::detail::reduce_n_impl and its cub::DeviceReduce::Reduce
 * (thrust/system/cuda/detail/reduce.h:930-1000, entry points reduce.h:1029-1062). */
int tb200_reduce(void* d_temp, size_t* temp_bytes, const void* d_in, uint64_t n, int dtype, const void* h_init,
                 void* d_out, tb200_stream_t stream);

/* ---- sort-based histogram -----------------------------------------------------------
 * Second half of the dense-histogram recipe (examples/histogram.cu:84-97): given SORTED
 * data (dtype in {I32,U32,I64,U64,F32,F64}) and num_bins ascending bin values of the same
 * type, counts[b] = upper_bound(data, bin[b]) - upper_bound(data, bin[b-1]) with
 * operator< (so -0.0 == +0.0 here), counts[0] = upper_bound(data, bin[0]).
 * Replaces: the vectorised thrust::upper_bound (generic/binary_search.inl:95-133 over
 * cuda/detail/parallel_for.h:68-147) followed by thrust::adjacent_difference
 * (cuda/detail/adjacent_difference.h:176-229), fused into one kernel. No scratch. */
int tb200_histogram_sorted(const void* d_sorted, uint64_t n, int dtype, const void* d_bin_values,
                           uint32_t num_bins, uint32_t* d_counts, tb200_stream_t stream);

/* Status word of the last call that used d_temp: 0 or a tb200_error. Synchronises the
 * stream (one 4-byte copy). Mirrors the reference's end-of-call synchronize + error check
 * (thrust/system/cuda/detail/util.h:113-140, 251-299). */
int tb200_temp_status(const void* d_temp, tb200_stream_t stream);

/* Self-test of the bounded-wait convention every kernel here follows: launches one warp that
 * polls a flag nothing ever sets, for at most limit_polls polls (1 .. 2^20), and returns the
 * device status it reports — TB200_ERR_WAIT_TIMEOUT — after which the context is still
 * usable. (The reference's device code prints and traps on errors, util.h:202-205.) */
int tb200_selftest_wait_timeout(uint32_t limit_polls, tb200_stream_t stream);

/* ---- launch tracing -------------------------------------------------------------------
 * Plays the role of the reference's THRUST_DEBUG_SYNC launch log
 * (thrust/system/cuda/detail/core/agent_launcher.h:501-560) without a sync per launch:
 * between tb200_trace_begin and tb200_trace_end every kernel this library launches from
 * the calling thread is followed by an event record on its stream. tb200_trace_end
 * synchronises, writes the device time of launch i (milliseconds) to ms[i] and what it was
 * to kinds[i] (may be NULL) for i < capacity and returns the number of launches (negative:
 * -cudaError_t). kinds: 1 sort histogram, 2 radix pass, 3 sort copy-back, 4 scan,
 * 5 reduce_by_key, 6 histogram of sorted data, 7 partition histogram, 8 partition pass,
 * 9 reduce, 10 scan_by_key, 11 unique_by_key, 12 copy of flagged elements. */
int tb200_trace_begin(tb200_stream_t stream);
int tb200_trace_end(float* ms, int* kinds, int capacity);

/* ---- workspace pool -----------------------------------------------------------------
 * The reference allocates and frees scratch with cudaMalloc/cudaFree inside every call
 * (thrust/system/cuda/detail/malloc_and_free.h:53-118). The pool keeps device blocks per
 * (device, stream) and LEASES them per call, so steady-state calls allocate nothing and calls
 * from several host threads, on one stream or on many, never share a block.
 * tb200_workspace_acquire leases a block of at least `bytes`; tb200_workspace_release gives it
 * back once the caller has ENQUEUED its last use (the block is only handed to later work on the
 * same stream, which runs after it). tb200_workspace_stats reports how many device allocations
 * the pool has made since the library was loaded and how many bytes it holds;
 * tb200_workspace_release_all frees everything (no lease may be outstanding). */
int tb200_workspace_acquire(size_t bytes, tb200_stream_t stream, void** d_ptr);
int tb200_workspace_release(void* d_ptr);
int tb200_workspace_stats(uint64_t* device_allocations, uint64_t* bytes_held);
int tb200_workspace_release_all(void);

/* ---- host-buffer forms --------------------------------------------------------------
 * The reference's flagship use is host vector -> device -> sort -> host (README.md:42-54;
 * copies via thrust/system/cuda/detail/internal/copy_cross_system.h:51-113). These take
 * HOST pointers (pinned for full speed), stage through pool workspace on the current
 * device, run the device path above and copy the result back, synchronising before
 * return. */
int tb200_radix_sort_host(void* h_keys, void* h_vals, uint64_t n, int key_dtype, int val_bytes,
                          int descending, tb200_stream_t stream);
int tb200_scan_host(const void* h_in, void* h_out, uint64_t n, int dtype, int exclusive,
                    const void* h_init, tb200_stream_t stream);
int tb200_reduce_by_key_host(const void* h_keys_in, const void* h_vals_in, void* h_keys_out,
                             void* h_vals_out, uint64_t* h_num_runs, uint64_t n, int key_dtype,
                             int val_dtype, tb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* THRUST_B200_H_ */
