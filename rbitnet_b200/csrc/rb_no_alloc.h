// Entry points of the kernel library that allocate nothing.
//
// This header has no counterpart in azerothl/Rbitnet: the reference is a CPU program and has
// no device memory to manage.  It exists for callers of this library that cannot call
// cudaMalloc themselves and cannot let a library do it for them: code that runs inside a
// memory budget fixed at start-up, plug-ins of a host program that owns the allocator, and
// real-time loops in which an allocation (which may synchronise the device) is not allowed.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the static decode entry point can serve, in float32 values.  The array of
// this size (8 MiB) lives in the library image: every GPU that loads the library holds it
// until the process exits.
#define RB_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Split-key decode attention (the same kernels as rb_attention_decode) whose scratch for the
// partial results is a static device array inside the library instead of caller memory.
//
//   out [B, H*D] bfloat16, q [B, H, D] bfloat16, one token per sequence; keys and values in the
//   paged cache; the caller passes all inputs and the output.
//
// With n_splits > 1 it needs B*H*n_splits*(D+2) <= RB_STATIC_SCRATCH_FLOATS, else it returns -1
// with a message in rb_last_error(); with n_splits == 1 no scratch is used and any size goes.
// It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Set-up happens inside the first calls: the first call on a device looks up the array's device
// address (cudaGetSymbolAddress, with that device current), and the first call on a device for
// each head size sets that kernel's shared-memory attribute.  Make one call per device and head
// size you will use before any stream capture on that device.
//
// All calls share the one array and it keeps the last call's contents.  Nothing in it has to
// start at zero: each call writes every partial it later reads.  Two calls that overlap on
// the GPU (different streams, or graphs replayed concurrently) race on the array: order them.
int rb_attention_decode_static(void* out, const void* q, const void* cache_k, const void* cache_v,
                               const int* page_table, int max_pages, int page_size, const int* tok_pos,
                               const int* tok_slot, int B, int H, int Kh, int D, float scale, int window,
                               int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
