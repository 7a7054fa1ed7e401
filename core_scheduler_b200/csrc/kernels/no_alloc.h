// SPDX-License-Identifier: Apache-2.0
// C entry point that never allocates. It has no counterpart in the reference project.
//
// Who needs it: code that drives this library from a place where device allocation is not
// an option -- a real-time or embedded-style host loop that reserved all of its memory at
// start-up, a plugin loaded into a process whose allocator it does not own, a caller inside
// a region where a cudaMalloc (an implicit device synchronisation) would stall other streams,
// or a plain C / ctypes client that has no torch allocator at all. Such callers own their
// input and output buffers already; what they cannot supply conveniently is the scratch
// memory some kernels need.
//
// cs_layernorm_backward_noalloc() is the LayerNorm backward pass (dx, dgamma, dbeta in a
// single sweep over dy and x) with its partial-sum scratch taken from a fixed array that is
// part of the library image instead of from an allocator.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch: rows may be anything, the normalised width is capped.
// The array holds CS_NOALLOC_LN_PARTS * 2 * CS_NOALLOC_LN_MAX_D floats (about 2.3 MiB) and
// stays resident on every GPU that loads the library until the process exits.
#define CS_NOALLOC_LN_MAX_D 2048
#define CS_NOALLOC_LN_PARTS 148

// LayerNorm backward over the last dimension `d` for `rows` rows.
//   dy, x, grad_residual, dx : bf16 [rows, d] device pointers (grad_residual may be NULL;
//                              when given it is added to dx)
//   gamma                    : fp32 [d]
//   mean, rstd               : fp32 [rows] as produced by the forward pass
//   dgamma, dbeta            : fp32 [d]; accumulate != 0 adds to their current contents
//   stream                   : cudaStream_t (NULL = default stream)
// Returns 0 on success, -1 when d is not a multiple of 8 or exceeds CS_NOALLOC_LN_MAX_D,
// -2 for a NULL required pointer or negative rows, otherwise a cudaError_t value.
//
// The call performs no cudaMalloc/cudaFree and calls no allocating library routine. The first
// call on each device resolves the device address of the scratch array (a one-time set-up with
// that device current). The first call on each device for each width class (d up to 512, 768,
// 1024, 1280, 2048) also loads that kernel variant and, for d above about 1360, raises its
// shared-memory limit. Make those first calls outside of any stream capture, e.g. one warm-up
// call per width you will use.
// All calls share the one scratch array: each call fully rewrites the part it reads, so nothing
// has to be cleared between calls, but two calls that overlap on the GPU (different streams, or
// different host threads without ordering) race on it. Serialise them on one stream.
int cs_layernorm_backward_noalloc(const void *dy, const void *x, const float *gamma, const float *mean,
                                  const float *rstd, const void *grad_residual, void *dx, float *dgamma, float *dbeta,
                                  int accumulate, int64_t rows, int64_t d, void *stream);

#ifdef __cplusplus
}
#endif
