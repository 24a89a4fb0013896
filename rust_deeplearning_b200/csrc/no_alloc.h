// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference (sweengineeringlabs/rust-deeplearning is
// CPU code whose attention allocates freely, rustml/nn/main/src/core/attention.rs:353-450); it
// exists for users of this library only.
//
// Some hosts cannot call cudaMalloc when a step runs: a serving process that has handed every
// free byte of device memory to the cache (an allocation would simply fail), a loop with a
// latency budget that forbids calls which may synchronise the device, a plugin inside another
// runtime that owns the allocator.  For them rdl_attention_decode_static runs the same kernel as
// rdl_attention_decode, but takes its scratch (run counters and partial results) from a fixed
// array inside the library instead of from the caller: it calls no cudaMalloc, no cudaFree and no
// allocating library routine, and needs no torch allocator.
//
//   * The array holds RDL_STATIC_SCRATCH_BYTES (8 MiB) on every device that loads the library,
//     for the life of the process.  A call that needs more - the need is
//     rdl_attention_decode_scratch_bytes(tokens, heads, kv heads, head_dim, max_splits) - is
//     refused with an error and launches nothing.
//   * The fields scratch, scratch_bytes and counter_bytes of the argument are ignored; inputs,
//     outputs, cache and page lists are the caller's, as for rdl_attention_decode.
//   * The first call on a device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside any stream capture.
//   * All calls share the one array and it keeps what the last call left.  The part that must
//     start at zero (the run counters) is cleared on the stream at every call.  Two calls that
//     overlap on the device - different streams, no ordering between them - race on it: order
//     them.
#pragma once

#include "api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define RDL_STATIC_SCRATCH_BYTES (8ll << 20)

int rdl_attention_decode_static(const AttentionArgs* a, void* stream);

#ifdef __cplusplus
}
#endif
