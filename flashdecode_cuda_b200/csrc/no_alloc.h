// Entry point that allocates nothing.  It has no counterpart in
// davidjoyme/flashdecode-cuda, whose binding allocates its outputs and scratch
// tensors on every call (kernels/bindings.cpp:135-150).
//
// Who it is for: callers that may not, or cannot, obtain device memory at the
// moment they need a token chosen.  Examples: a host thread with a latency
// bound, for which cudaMalloc is off limits because it may take the driver's
// allocation locks and synchronise the device; a process whose device memory
// has been handed over in full to another allocator (a serving process that
// gave everything left to its KV cache has nothing to give a helper); code
// that runs inside someone else's callback or plugin interface whose contract
// forbids allocation.  fd_sample (sampling.cu) needs the caller to bring
// scratch memory for large vocabularies; this variant brings its own.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of fd_sample_no_alloc.  The scratch array they imply
// (2 * FD_NO_ALLOC_MAX_ROWS * FD_NO_ALLOC_MAX_CHUNKS 4-byte words = 128 KB)
// is part of the library image: every GPU that loads the library holds it
// until the process exits, whether or not the entry point is ever called.
#define FD_NO_ALLOC_MAX_ROWS 256          // rows of logits per call
#define FD_NO_ALLOC_MAX_CHUNKS 64         // 4096-entry chunks per row: vocabularies up to 262,144

// Same result as fd_sample for the same arguments: out[i] = argmax of row i
// (temperature null or <= 0; the lowest index wins a tie) or a Gumbel-max draw
// from softmax(logits[i] / temperature[i]) keyed by (seed, request[i], step[i]).
// The caller passes inputs and outputs only; the per-chunk winners that the two
// kernels hand to each other live in a static device array of this library.
//
// * It calls no cudaMalloc, cudaFree or other allocating routine.
// * It returns 0, or a negative code with the text in fd_last_error():
//   more than FD_NO_ALLOC_MAX_ROWS rows or a vocabulary beyond
//   FD_NO_ALLOC_MAX_CHUNKS * 4096 entries are refused, nothing is launched.
// * The first call on each device looks up the array's device address (with
//   that device current) and remembers it; make that first call during set-up,
//   before any stream capture begins.
// * All calls on a device share the one array.  It keeps whatever the last
//   call left, which is harmless: every word that the second kernel reads has
//   been written by the first kernel of the same call, so nothing has to start
//   at zero and nothing is cleared.  Two calls whose kernels can overlap on the
//   GPU (different streams without an ordering between them, or different host
//   threads on different streams) race on the array and may return wrong
//   tokens: keep calls on one stream, or order the streams with events.
int fd_sample_no_alloc(const float* logits, int n, int V, const float* temperature,
                       const long long* request, const int* step, unsigned long long seed, int* out,
                       cudaStream_t stream);

#ifdef __cplusplus
}
#endif
