// Greedy token selection for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Coheryn/coheryn-ai-studio picks
// tokens on the CPU); it exists for hosts of this library that cannot call cudaMalloc at
// the moment they need a token:
//   * a serving process that has already handed every free byte of the GPU to its cache
//     pool, so that a later allocation may simply fail;
//   * a latency-critical loop in which the implicit device synchronisation of cudaMalloc
//     and cudaFree is not acceptable;
//   * plain C or C++ callers that have no caching allocator of their own to draw the
//     piece buffers of the ordinary entry point (coheryn_argmax) from.
//
// coheryn_argmax_static does the same two-stage reduction as coheryn_argmax (pieces of 4096
// logits, then the pick among the pieces; ties go to the lowest id) and gives bit-identical
// results, but keeps its piece buffers in a fixed array inside the library's device image.
//
// Limit: rows * ceil(vocab / 4096) <= COHERYN_ARGMAX_STATIC_SLOTS (65,536 slots of 8 bytes =
// 512 KiB, e.g. 256 rows of a 1,048,576-entry vocabulary, or 1,724 rows of 151,936), and at most
// 65,535 rows per call whatever the vocabulary (each row is one row of the launch grid).  Larger
// requests are refused with an error; nothing is launched.  Every GPU that loads the library
// holds the 512 KiB until the process exits.
//
// Set-up: the first call on a device looks the array's address up (cudaGetSymbolAddress with
// that device current) and remembers it; make that first call before any stream capture.
// No call allocates or frees memory, by the CUDA runtime or otherwise.
//
// Sharing: all calls on a device use the one array.  It keeps the previous call's contents;
// nothing in it has to start at zero, because every slot a call reads was written by that
// same call.  Two calls whose kernels overlap on the GPU (different streams, no ordering
// between them) race on the array and both results are undefined: order them.
#pragma once
#include <cuda_runtime.h>

#define COHERYN_ARGMAX_STATIC_SLOTS 65536

#ifdef __cplusplus
extern "C" {
#endif

// logits: float32 [rows, vocab] on the device with row stride `stride` (elements);
// out: int32 [rows] on the device; status: one int32 on the device that is set to 2 when a
// logit is not finite.  Returns 0 on success; otherwise coheryn_last_error() tells why.
int coheryn_argmax_static(const float* logits, long stride, int rows, int vocab, int* out, int* status,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
