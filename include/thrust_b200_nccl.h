/* thrust_b200_nccl.h — the sharded sort behind one C entry point (libthrust_b200_nccl.so).
 *
 * One process per GPU, an NCCL communicator over the ranks. The library owns the whole step:
 * regular sample, all-gather, splitters, bucket counts, the count matrix, the exchange and the
 * final local sort; the kernels are those of libthrust_b200.so. It links NCCL, which is why it is
 * a library of its own: applications that sort on one GPU never load NCCL.
 *
 * The reference has no multi-GPU code. The result is the single-process
 * thrust::stable_sort_by_key (thrust/sort.h:1016-1094) of the concatenation of the shards in
 * rank order, cut into nranks consecutive slices.
 */
#ifndef THRUST_B200_NCCL_H_
#define THRUST_B200_NCCL_H_

#include "thrust_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

struct ncclComm;
typedef struct ncclComm* tb200_nccl_comm_t; /* an ncclComm_t (nccl.h) */

/* Stable sort_by_key of (uint64 key, 4-byte value) pairs sharded over the ranks of `comm`.
 * This rank passes its shard, n pairs in d_keys / d_vals (the shards of ranks 0, 1, ... form the
 * global sequence in that order; they may differ in length). On return d_keys_out / d_vals_out
 * (room for `capacity` pairs) hold this rank's slice of the globally sorted sequence and
 * *h_count_out its length; equal keys keep their global input order. d_keys / d_vals are left
 * unchanged.
 *
 * Scratch: two-phase like every entry point (d_temp == NULL writes *temp_bytes for this n,
 * capacity, nranks and exchange form). All ranks must pass the same capacity and the same
 * exchange form.
 *
 * Exchange: with peer_keys == NULL the partitioned buckets travel through ncclSend / ncclRecv.
 * Otherwise peer_keys / peer_vals are HOST arrays of nranks device pointers: rank b's d_keys_out
 * / d_vals_out as mapped into THIS process (entry [rank] is this rank's own buffer), and the
 * partition pass stores every bucket straight into its destination over NVLink (plain stores,
 * no multicast); the caller establishes the mappings (cudaIpc, cuMemMap, symmetric memory) and
 * must not touch the output buffers of any rank while the call runs.
 *
 * The call synchronises `stream` (the count matrix is read on the host). Returns TB200_OK, a
 * cudaError_t value, a tb200_error, TB200_ERR_OVERFLOW on EVERY rank when some rank would
 * receive more than `capacity` pairs (nothing has been exchanged then), or TB200_ERR_NCCL. */
#define TB200_ERR_NCCL (-6)
int tb200_sample_sort(tb200_nccl_comm_t comm, int rank, int nranks, void* d_temp, size_t* temp_bytes,
                      const void* d_keys, const void* d_vals, uint64_t n, void* d_keys_out, void* d_vals_out,
                      uint64_t capacity, void* const* peer_keys, void* const* peer_vals, uint64_t* h_count_out,
                      tb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* THRUST_B200_NCCL_H_ */
