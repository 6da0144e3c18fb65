// Allocation-free sort entry point.
//
// This entry point has no counterpart in the reference: it exists for callers of this library that must
// not allocate device memory at the time of the call, for example code that runs between the capture and
// the replay of its own resource plan, real-time render loops that pre-size everything at start-up, or
// hosts embedding the library under a fixed memory budget where a cudaMalloc may fail or stall. Such a
// caller still owns the inputs and outputs (keys, values, tile ranges, the counter block); what it cannot
// provide is the sort's scratch space (ping-pong buffers and digit histograms), so that lives in a
// fixed-size array inside the library's device image.
//
// Limits and rules:
//  * at most RGS_NOALLOC_MAX_PAIRS (key, value) pairs of capacity per call; a larger capacity is refused
//    with RGS_NOALLOC_ERR_TOO_LARGE and the text returned by rgs_cuda_noalloc_last_error();
//  * the scratch array (about 12.3 MB) is part of the library image: every GPU on which the library is
//    loaded holds it until the process exits;
//  * the first call on a device looks up the device address of the array (cudaGetSymbolAddress, with that
//    device current). With the CUDA runtime's lazy module loading that first call may also be the moment at
//    which the runtime loads the library's device image (and with it the scratch array) onto the device, which
//    takes device memory once; every later call leaves the amount of free device memory unchanged. Make that
//    first call at start-up, before any stream capture on that device;
//  * all calls on a device share the one array and it keeps the previous call's contents. The sort
//    overwrites every word it later reads, so nothing has to be cleared, but two calls that overlap on
//    the GPU (different streams, no dependency) race on it: serialise them;
//  * no cudaMalloc, cudaFree or other allocating routine is called, here or in what it launches.
#pragma once
#include <stdint.h>

#define RGS_NOALLOC_MAX_PAIRS (1 << 20)
#define RGS_NOALLOC_ERR_TOO_LARGE 40
#define RGS_NOALLOC_ERR_SYMBOL 41

#ifdef __cplusplus
extern "C" {
#endif

// Same contract as rgs_cuda_sort_ranges (sort (key, value) pairs by bits [0, 32 + ceil(log2 num_tiles)),
// sorted values end up in `vals`, per-tile [start,end) in `ranges`; the pair count is read from
// counters[RGS_CNT_INST] on the device) but without the caller-provided scratch buffers.
// cap_pairs is the capacity of `keys` / `vals` and must not exceed RGS_NOALLOC_MAX_PAIRS.
int rgs_cuda_sort_ranges_noalloc(uint64_t* keys, uint32_t* vals, int64_t cap_pairs, const int32_t* counters,
                                 int64_t num_tiles, int32_t* ranges, void* stream);

// Text of the last error this entry point reported to the calling thread ("" when none). The buffer belongs to
// the calling thread: it is not rewritten by errors that other threads run into.
const char* rgs_cuda_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
