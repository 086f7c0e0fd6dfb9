// rs_unique_keys_noalloc: device-side unique() of a key batch for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library.
//
// Who needs it.  rs_unique_keys wants two scratch arrays from its caller.  Some callers have no way
// to get device memory at the moment they need the result: a serving process whose whole HBM budget
// was handed to another allocator at start-up, a plug-in that runs under a host framework which
// forbids driver allocations from its worker threads, or a latency-critical path that cannot accept
// the implicit device-wide synchronisation of cudaMalloc / cudaFree.  For them the scratch lives in a
// fixed array inside the library's own device image.
//
// Cost and limit.  The array is RS_UNIQUE_NOALLOC_MAX_KEYS * 2 hash slots * 12 bytes = 3 MiB.  It is
// part of the loaded module, so EVERY GPU on which this library is loaded holds those 3 MiB until the
// process exits, whether or not the function is ever called.  Batches larger than
// RS_UNIQUE_NOALLOC_MAX_KEYS keys are rejected with RS_ERR_CAPACITY and a message; nothing is
// truncated silently.
//
// Rules of use.
//   * Inputs and outputs are still the caller's: keys[n], unique_out[n], inverse[n] (optional),
//     count (one int) and the optional status word, all device pointers on the current device.
//   * The function calls no cudaMalloc, no cudaFree and no allocating library routine.
//   * The first call on each device looks up the device address of the array (cudaGetSymbolAddress,
//     with that device current) and remembers it.  Make that first call outside any stream capture.
//   * All calls on one device share the one array, and it keeps whatever the previous call left in
//     it.  Every call therefore clears the slots it is going to use before it hashes into them, on
//     the caller's stream.  Two calls whose kernels can overlap on the GPU (different streams without
//     an ordering between them, or different host threads) race on the array and give wrong results:
//     order them.
//   * Keys are 64-bit patterns.  Two of them are reserved for the hash slots themselves: -1 (empty) and -2
//     (tombstone), read as signed values.  Such a key takes no output position: inverse[i] = -1, it is not
//     counted, and RS_DEV_BAD_ARG is ORed into the status word.  Map padding ids to something else first.
//   * The order of unique_out is arbitrary (first hash-slot claimer wins), as for rs_unique_keys;
//     unique_out[inverse[i]] == keys[i] holds for every i
//     whose key is not reserved.
#pragma once
#include <cuda_runtime.h>

#define RS_UNIQUE_NOALLOC_MAX_KEYS (1 << 17)

extern "C" int rs_unique_keys_noalloc(const long long* keys, long long n, long long* unique_out, int* inverse, int* count,
                                      unsigned long long* status, cudaStream_t stream);
