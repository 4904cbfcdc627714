// mrun_attn_decode_static: the split-key decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference (hupe1980/mrun): it exists for programs
// that embed this library where device memory cannot be requested at call time.  Examples are a
// host application that carved up the whole device for its own arena at start-up, so a later
// cudaMalloc would fail or break its accounting; a latency-critical loop that cannot afford the
// device-wide synchronisation an allocation may imply; and an inference-server or plugin
// callback whose contract forbids allocating while it enqueues work.  Such callers cannot give
// the ordinary entry point (mrun_attn_decode) the scratch buffers it asks for.
//
// What it does: exactly what mrun_attn_decode does, with the same kernel and the same arguments
// for inputs and outputs, but the scratch for the splits' partial results and their meeting
// counters lives in a fixed array inside the library instead of in caller-provided buffers.
//
// Limits: blocks <= MRUN_STATIC_MAX_BLOCKS (512), tokens <= MRUN_STATIC_MAX_TOKENS (4096) and
// tokens * kv_heads <= MRUN_STATIC_MAX_PAIRS (4096); larger calls are refused with a message.
// The array takes 512 * 32 * (head size + 2) * 4 + 12289 * 4 bytes of device memory (about 8.2 MiB
// at head size 128) on every GPU that loads the library, from load until the process exits.
// It also holds the step's plan (tiles per token), which this entry point computes itself.
//
// Rules for callers:
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once
//    per device, with that device current).  Make that first call before starting any stream
//    capture on the device.
//  * It calls no cudaMalloc, cudaFree or other allocating routine, on any call.
//  * All calls share the one array and it keeps whatever the last call left.  The entry point
//    clears the part that must start at zero (the counters) on the caller's stream before it
//    launches.  Two calls that overlap on the GPU (different streams, or different threads on the
//    same device) race on the array and give wrong results: serialise them.
//
// Returns 0, or non-zero after storing a message for mrun_last_error().
#pragma once

#include <cuda_runtime.h>

#define MRUN_STATIC_MAX_BLOCKS 512
#define MRUN_STATIC_MAX_TOKENS 4096
#define MRUN_STATIC_MAX_PAIRS 4096

#ifdef __cplusplus
extern "C" {
#endif

int mrun_attn_decode_static(const void* q, long q_stride, void* out, const void* k_cache, const void* v_cache,
                            const int* block_tables, int max_blocks, const int* token_slot, const int* positions,
                            int tokens, int blocks, int min_tiles, int heads, int kv_heads, int head_dim,
                            int page_size, float scale, int window, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
