// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library that run where cudaMalloc is not an option: code that is already inside a CUDA-graph
// capture or holds a fixed, pre-sized memory budget, host threads that must not take the
// allocator's locks (a real-time or signal-handling path), and processes whose device memory is
// fully handed to another allocator.  Such a caller still owns its inputs and outputs; what it
// cannot provide is the scratch memory in which the split-key decode kernel keeps its partial
// results.  Here that scratch is a fixed array inside the library.
//
// vob_attention_decode_noalloc() computes exactly what vob_attention_decode() computes (same
// kernels, same arguments, minus the scratch pointer) and differs only in where the partial
// results live:
//   * The scratch is a file-scope `static __device__` array of
//     VOB_DECODE_NOALLOC_MAX_FLOATS floats (8 MiB).  Every GPU on which this library is loaded
//     holds that much memory until the process exits.
//   * A launch needs num_requests * nh * num_splits * (head size + 1) floats (nothing with one
//     split).  A launch that needs more than the array holds is refused with
//     VOB_NOALLOC_TOO_LARGE before anything runs; vob_attention_decode_noalloc_error() gives the
//     text for a code.
//   * The first call on each device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside any stream capture.
//   * At EVERY call the current device must be the one that owns `stream` and all the buffers:
//     the array that is used is the current device's, whatever device the pointers belong to.
//   * Host threads may call it at the same time (the look-up of the address may then happen twice,
//     with the same result); what they launch is subject to the rule on overlapping calls below.
//   * Arguments are checked before anything else: a call that is refused has looked up nothing
//     and launched nothing.
//   * The function calls no cudaMalloc, cudaFree or allocating library routine.
//   * All calls share the one array, and it keeps what the previous call left in it.  The kernels
//     overwrite every entry they later read, so nothing needs clearing between calls; but two calls
//     whose kernels overlap on the GPU (different streams, no ordering between them) race on it.
//     Order such calls, or use vob_attention_decode() with scratch memory of your own.
#pragma once
#include <cuda_runtime.h>

#define VOB_DECODE_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)
#define VOB_NOALLOC_TOO_LARGE 2003
#define VOB_NOALLOC_NO_DEVICE 2004

extern "C" {
// Arguments as vob_attention_decode(), without `scratch`.  Returns 0, a cudaError_t value, or one of the
// codes above.
int vob_attention_decode_noalloc(const void* q, long q_stride, void* out, const void* kcache, const void* vcache,
                                 const int* block_tables, int table_stride, const int* cu_q, const int* context_lens,
                                 int num_requests, int nh, int kvh, int block_size, int window, float scale,
                                 long num_pages, int num_splits, int* err, cudaStream_t stream);
// Floats of the built-in scratch array.
long vob_attention_decode_noalloc_max_floats(void);
// Text for a code returned by vob_attention_decode_noalloc().
const char* vob_attention_decode_noalloc_error(int code);
}
