#include "common.cuh"
extern "C" int tb200_radix_sort(void*, size_t*, void*, void*, uint64_t, int, int, int, int, int, tb200_stream_t) { return TB200_ERR_UNSUPPORTED; }
