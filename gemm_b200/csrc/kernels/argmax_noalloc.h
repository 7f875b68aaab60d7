// gb_argmax_noalloc: greedy arg-max over wide logit rows for callers that must not allocate device memory.
// This entry point has no counterpart in the reference project; it exists for embedders of this library.
//
// Who needs it: code that calls into the library from a place where the CUDA allocator is off limits — a
// real-time or serving loop that has handed all device memory to its own pool, a plug-in running under
// another framework's memory manager, or a host thread that is not allowed to take the allocator's locks.
// The regular two-stage arg-max (gb_argmax2) needs a scratch buffer of partial results that its caller
// allocates; here that scratch is a fixed array inside the library image itself, so the call allocates
// nothing: no cudaMalloc / cudaFree and no allocating library routine is reached.  Inputs and outputs are
// still the caller's buffers.
//
// Limits and rules:
//   * rows <= GB_ARGMAX_NOALLOC_MAX_ROWS (1024).  Larger batches are refused with an error message
//     (gb_last_error()), nothing is launched.  The scratch array takes 512 KiB of device memory on every GPU
//     that loads the library, until the process exits.
//   * The first call on a device looks up the device address of the scratch array (with that device current)
//     and caches it; make that first call outside of any stream capture.  Later calls only launch kernels.
//   * All calls on one device share the one scratch array.  Every entry a call reads it has written itself
//     first, so stale contents of earlier calls are harmless and nothing needs clearing — but two calls
//     whose kernels overlap in time on the same device (different streams, no ordering) race on it.
//     Serialise them on one stream or order them with events.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GB_ARGMAX_NOALLOC_MAX_ROWS 1024

// logits: [rows, ld] elements (dtype 0 = float32, 1 = bfloat16), device memory.
// out_idx: int32 [rows] (winning column + idx_offset; ties resolve to the lowest column), device memory.
// out_val: float32 [rows] or NULL.
// Returns 0 on success, -1 on error (message in gb_last_error()).
int gb_argmax_noalloc(const void* logits, int* out_idx, float* out_val, int rows, int vocab, long ld, int dtype, int idx_offset,
                      cudaStream_t stream);

#ifdef __cplusplus
}
#endif
