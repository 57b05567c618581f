/* Counter-based synthetic inputs for the tests and benchmarks of thrust_b200.
 *
 * Element i of every stream is a pure function of (seed, i), so any rank, the host
 * and the device produce identical data and a checker can regenerate a key from its
 * global index. These stand in for the reference's own hash-generated benchmark inputs
 * (internal/benchmark/random.h:6-92) with the value distributions of this repository's
 * benchmark configurations. Not part of the algorithm ABI: these live in libtb200_datagen.so,
 * which only the tests and bench.py load.
 */
#ifndef THRUST_B200_DATAGEN_H_
#define THRUST_B200_DATAGEN_H_

#include "../../include/thrust_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tb200_gen_kind {
  TB200_GEN_BITS_U32 = 0,      /* uint32: low 32 bits of hash(seed, i) (as int32: uniform over its range) */
  TB200_GEN_BITS_U64 = 1,      /* uint64: hash(seed, i)                                                  */
  TB200_GEN_INDEX_U32 = 2,     /* uint32: (uint32)i                                                      */
  TB200_GEN_UNIFORM_F32 = 3,   /* float : aux = {lo, hi} (2 floats, host pointer): uniform in [lo, hi)   */
  TB200_GEN_UNIFORM_I64 = 4,   /* int64 : aux = {lo, hi} (2 int64, host pointer): uniform in [lo, hi]    */
  TB200_GEN_HEAD_FLAGS_I32 = 5,/* int32 : 1 with probability 1/aux[0] (uint32, host pointer), else 0; i==0 -> 1 */
  TB200_GEN_AND3_F32 = 6,      /* float : bitwise AND of three independent words, NaN patterns redrawn   */
  TB200_GEN_ZIPF_RANK_U32 = 7  /* uint32: rank r in [0, aux_len) drawn by inverse CDF; aux = cdf[aux_len]
                                  (doubles, ascending, last == 1) in the same memory space as `out`     */
} tb200_gen_kind;

/* Writes elements first_index .. first_index+n-1 of stream (kind, seed) to out.
 * on_device != 0: out is a device pointer, work is enqueued on stream.
 * on_device == 0: out is a host pointer, filled by the calling thread's OpenMP team. */
int tb200_datagen(void* out, uint64_t n, uint64_t first_index, int kind, uint64_t seed, const void* aux,
                  uint32_t aux_len, int on_device, tb200_stream_t stream);

/* Reference-free check of one sorted shard of (key = hash(seed, g), value = (uint32)g) pairs
 * drawn from global indices g in [0, total). d_result4 (device, 4 x uint64) receives:
 * [0] order violations (key[j-1] > key[j], or equal keys whose global indices do not increase),
 * [1] pairs whose key is not the hash of any index congruent to the value mod 2^32,
 * [2] the sum of the recovered global indices mod 2^64, [3] the number of pairs checked.
 * Zero violations on every shard, ordered shard boundaries and [3] summing to `total`
 * imply that the output is THE stable sort of the input. */
int tb200_check_hashed_pairs(const void* d_keys, const void* d_vals, uint64_t n, uint64_t seed, uint64_t total,
                             uint64_t* d_result4, tb200_stream_t stream);

/* hash(seed, i) itself, for checkers. */
uint64_t tb200_datagen_hash(uint64_t seed, uint64_t i);

#ifdef __cplusplus
}
#endif
#endif
