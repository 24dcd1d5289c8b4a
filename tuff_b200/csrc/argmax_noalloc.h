// tuff_argmax_noalloc: greedy token choice for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (niihelium/tuff allocates all of its
// device buffers itself at start-up).  It exists for hosts that embed this library into a
// process whose device memory is already spoken for: a serving process that handed the whole
// GPU to its own arena at start, a plug-in that runs under a memory budget it does not own, or
// a latency-critical loop in which cudaMalloc (which synchronises the device) may never be
// reached.  Such callers pass their own input and output buffers; the kernel's working memory
// is a fixed array inside the library.
//
// Rules for callers:
//   * at most TUFF_ARGMAX_NOALLOC_MAX_ROWS rows per call; more is refused with
//     TUFF_ARGMAX_NOALLOC_E_ROWS and nothing is launched;
//   * the first call on a device looks up the device address of the library's working array
//     (cudaGetSymbolAddress) and keeps it; make that first call outside of any stream capture;
//   * every call on a device uses the same working array: calls that may overlap on the GPU
//     (different streams without ordering) race and give wrong answers; order them;
//   * every GPU that loads the library holds the array (about 66 KB) until the process exits.
#pragma once
#include <cuda_runtime.h>

#define TUFF_ARGMAX_NOALLOC_MAX_ROWS 256
#define TUFF_ARGMAX_NOALLOC_E_ROWS (-3)     // more rows than the working array serves
#define TUFF_ARGMAX_NOALLOC_E_ARG (-6)      // a null pointer or an empty vocabulary

#ifdef __cplusplus
extern "C" {
#endif

// out[r] = index of the first maximum of logits[r, 0..V) for r < n_rows; logits fp32, row-major,
// on the current device; out int32 on the device.  Returns 0, a cudaError_t, or one of the
// TUFF_ARGMAX_NOALLOC_E_* codes.  Calls no cudaMalloc, cudaFree or other allocating routine.
int tuff_argmax_noalloc(const float* logits, int n_rows, int V, int* out, cudaStream_t stream);

// The largest n_rows a call may pass.
int tuff_argmax_noalloc_max_rows(void);

// A sentence for a return code of tuff_argmax_noalloc.
const char* tuff_argmax_noalloc_message(int code);

#ifdef __cplusplus
}
#endif
