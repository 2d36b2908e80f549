// Token sampling for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project: there the device sampler always
// receives a rows x vocab work buffer from its allocator.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a plugin called from inside another
// runtime's memory plan, a latency-critical serving loop that has handed the whole device to a pool it
// does not own, a host that forbids allocation after start-up so that its memory budget stays fixed.
// Such a caller can still pass its own logits, parameters and output, but has nowhere to get the
// sampler's scratch (one 32-bit weight per logit per row).  Here that scratch is a fixed array inside
// the library image instead.
//
// Limits and rules:
//   * at most 4 rows per call and a vocabulary of at most 262144 entries; anything larger, or a row stride
//     `ld` shorter than the vocabulary, is refused with -3 and nothing is launched.  The array takes 4 MiB on
//     every GPU that loads the library, for the life of the process.
//   * the call allocates nothing: no cudaMalloc / cudaFree and no allocating library routine.  The first
//     call on each device looks up the array's device address (with that device current); make that first
//     call outside any stream capture.  The address used is that of the device that is current at the call,
//     so `stream` must belong to the current device.
//   * every call uses the same array.  The kernel rewrites each weight it later reads, so nothing needs
//     clearing between calls, but two calls that run at the same time on one GPU (different streams)
//     would overwrite each other's weights: issue them one after the other.
//   * arguments and results are those of ogb_sample_bf16 without the `work` pointer: bf16 logits
//     [rows, ld], per-row temperature / top_k / top_p / min_p / uniform draw, int32 tokens out.  Returns 0,
//     a negative argument code, or a cudaError_t.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int ogb_sample_bf16_no_alloc(const void* logits, int* out_tokens, const float* temperature, const int* top_k,
                             const float* top_p, const float* min_p, const float* uniform, int rows, int vocab, int ld,
                             void* stream);

#ifdef __cplusplus
}
#endif
