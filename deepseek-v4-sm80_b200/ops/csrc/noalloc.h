// dsv4_indexer_select_noalloc: indexer top-k selection for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a host thread inside a real-time serving loop that
// may not take the allocator's locks or trigger an implicit device synchronisation, a plugin running under a host
// framework that owns all device memory and hands out fixed buffers only, or a process whose memory budget was fixed
// at start-up.  The regular path (dsv4_indexer_logits followed by dsv4_topk) needs a caller-supplied fp32 logits
// workspace of t x width elements, which such callers would otherwise have to allocate per shape.
//
// What it does: the same two kernels, but the logits workspace is a file-scope device array inside the library
// (4 MiB, i.e. DSV4_NOALLOC_MAX_ELEMS floats), resident on every GPU that loads the library until the process exits.
// Inputs and outputs are still passed by the caller.  The function performs no cudaMalloc / cudaFree and calls no
// allocating library routine.
//
// Rules for callers:
//   * t * width must not exceed DSV4_NOALLOC_MAX_ELEMS; larger requests are rejected (return code 460) and
//     dsv4_noalloc_last_error() describes the limit.  width is the logits row length (a multiple of 64 covering
//     the longest compressed history of the batch, max(pos)/4 + 1 rounded up).
//   * The first call on each device looks up the workspace's device address (cudaGetSymbolAddress) with that device
//     current; make that first call outside any stream capture.
//   * All calls share the one workspace, which keeps the previous call's contents.  The kernels overwrite every
//     element they later read, so nothing needs clearing, but two calls that overlap on the GPU (different streams,
//     or the same stream from two threads without ordering) race on it: serialise them.
#pragma once
#include <cuda_runtime.h>

#define DSV4_NOALLOC_MAX_ELEMS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// qc [t, heads, 128] e4m3 codes, wf [t, heads] fp32 folded head weights, kvals / kscale the paged indexer cache,
// slots / pos [t] int32, page_table [*, ld_pt] int32 token locations, ps the page size.
// Outputs: idx [t, k] int32 (selected compressed indices in ascending order, -1 padded), out_len [t] int32.
// Returns 0 on success, 460 when t * width exceeds DSV4_NOALLOC_MAX_ELEMS, 461 when the workspace address cannot be
// resolved, otherwise the code of the failing launch.
int dsv4_indexer_select_noalloc(const void* qc, const float* wf, const void* kvals, const float* kscale,
                                const int* slots, const int* pos, const int* page_table, int ld_pt, int ps, int width,
                                int t, int heads, int d, int* idx, int* out_len, int k, cudaStream_t stream);

// Human-readable description of the last non-zero return of the function above on this host thread ("" if none).
const char* dsv4_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
