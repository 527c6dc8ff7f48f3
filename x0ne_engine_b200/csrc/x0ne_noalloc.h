// Declaration of the one entry point of this library that allocates nothing.
//
// This entry point has no counterpart in the reference project: it exists for users of this
// library, not for parity.
//
// Who needs it.  Some callers cannot allocate device memory at the moment they want attention
// computed: a host runtime that took all of the device's memory into one arena at start-up and
// froze it; code that runs inside someone else's memory budget and may not grow it; a serving
// loop that must not pay the device-wide synchronisation that cudaMalloc and cudaFree imply.  The
// ordinary decode-attention entry point (x0ne_attention_decode_bf16) leaves the scratch buffer
// for its split partial results to the caller, which in practice means an allocation by whoever
// calls it.  This variant carries that scratch inside the library instead.
//
// What it costs.  The scratch is a fixed array of X0NE_NOALLOC_SCRATCH_BYTES bytes in device
// memory that every GPU which loads the library keeps until the process exits, used or not.
// Sizes whose partial results do not fit are refused with an error; nothing is ever allocated.
//
// Rules for callers.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress)
//     and sets the kernel's shared-memory attribute for that device.  Make that first call, with
//     the device current, before any stream capture you intend to do, and from one host thread:
//     the look-up is not locked (two threads racing through it would store the same address, but
//     nothing orders their stores).
//   * All calls on a device share the one array.  Two calls that can overlap on the GPU (different
//     streams without an ordering between them) race on it; order them.
//   * The array keeps what the last call left.  The entry point clears the part that must start
//     at zero (the arrival counters) on the caller's stream before each launch.
//   * It calls no cudaMalloc, cudaFree or other allocating routine, and needs no torch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

#define X0NE_NOALLOC_SCRATCH_BYTES (4 << 20)

// Same arguments and result as x0ne_attention_decode_bf16 without the scratch pointer and size:
// q and out are bfloat16 [n_rows][q_heads * head_dim]; one query row per sequence; `splits` blocks
// per (sequence, kv head).  Returns 0, or an error code with the text in x0ne_last_error().
X0NE_API int x0ne_attention_decode_bf16_noalloc(const void* q, void* out, PagedCache cache, const int32_t* row_slot,
                                                const int32_t* row_pos, int n_rows, int q_heads, float scale,
                                                int window, int splits, cudaStream_t stream);

// The largest scratch the entry point can serve, in bytes (X0NE_NOALLOC_SCRATCH_BYTES).
X0NE_API int64_t x0ne_noalloc_scratch_capacity();
