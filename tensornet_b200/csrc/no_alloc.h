// tn_unique_assign_static: the batch dedup (unique_assign, unique.cu) for callers that must not
// allocate device memory.  This entry point has no counterpart in the reference.
//
// Who needs it: code that runs where cudaMalloc is unavailable or forbidden - a serving process
// whose memory was carved up at start-up and handed out completely, a host thread that may run
// while another thread is capturing a CUDA graph (an allocation there would invalidate the
// capture), or a plug-in called from a framework that owns the allocator.  Such callers bring
// their input and output buffers; the open-addressing scratch the dedup needs lives in a fixed
// array inside this library instead of being allocated per call.
//
// Contract
//   * n <= TN_UNIQUE_STATIC_MAX_IDS ids per call, otherwise the call is rejected (returns
//     TN_NOALLOC_TOO_LARGE, nothing is launched).  `uniq`, `show`, `click` need room for
//     min(n, uniq_cap) entries; more distinct signs than `uniq_cap` sets the device error word
//     reported by tn_unique_assign_static_status().
//   * The scratch (1.5 MiB + 64 B) is a file-scope __device__ array: every GPU that loads the
//     library holds it until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per
//     device, with that device current).  Make that first call outside any stream capture.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any path.
//   * All calls on one device share the scratch.  Each call re-initialises what it needs at its
//     start, so earlier contents never leak into a result; calls whose kernels overlap on the GPU
//     (different streams, no ordering between them) race on it and produce garbage.  Serialise them.
#pragma once
#include <cuda_runtime.h>

#define TN_UNIQUE_STATIC_MAX_IDS 65536

#define TN_NOALLOC_OK 0
#define TN_NOALLOC_TOO_LARGE 1
#define TN_NOALLOC_BAD_ARGUMENT 2
#define TN_NOALLOC_CUDA_ERROR 3

#ifdef __cplusplus
extern "C" {
#endif

// ids      [n]        int64 signs (device)
// labels   [n]        optional fp32 click labels (device) or NULL
// uniq     [uniq_cap] out: distinct signs, index = virtual index
// inverse  [n]        out: virtual index of every id
// show     [uniq_cap] out (optional, may be NULL): occurrences per distinct sign
// click    [uniq_cap] out (optional, may be NULL): sum of labels per distinct sign
// count    [1]        out: number of distinct signs
// Returns TN_NOALLOC_OK or an error code; tn_unique_assign_static_error() gives the text.
int tn_unique_assign_static(const long long* ids, int n, const float* labels, unsigned long long* uniq, int uniq_cap,
                            int* inverse, float* show, float* click, int* count, cudaStream_t stream);

// Text of the last error returned on this thread ("" when none).
const char* tn_unique_assign_static_error(void);

// Copies the four device error words of the last call on the current device to `host_out`
// (synchronises `stream`); word 0 is zero when the call was clean.
int tn_unique_assign_static_status(int* host_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
