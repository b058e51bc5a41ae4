// vk_attention_decode_static: split-key decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine; it exists for hosts of this library.
//
// Some programs that embed these kernels cannot give them scratch memory at call time: a serving loop
// that took all of its device memory at start-up and has sworn off cudaMalloc afterwards (an allocation
// may synchronise the device and stall every stream), a plug-in inside another runtime whose memory pool
// owns the device, or a component with a fixed memory budget that is audited once.  vk_attention_decode
// needs scratch for the partial results of the key splits; this variant keeps that scratch inside the
// library, in a file-scope device array of VK_DECODE_STATIC_SCRATCH_BYTES (8 MiB) that every GPU which
// loads the library holds until the process exits.  The caller passes inputs and outputs only.
//
// It calls no cudaMalloc, cudaFree or any allocating routine.  The first call on a device looks up the
// array's device address (cudaGetSymbolAddress, once per device, with that device current); make that
// first call outside any stream capture.  A launch whose partial results would not fit the array is
// refused with VK_TOO_LARGE before anything runs (vk_error_string says so): the need is
// vk_attention_decode_scratch_bytes(n_tokens, nh, nkv, hd, max_context).
//
// All calls share the one array, and it keeps whatever the last call left.  The part that has to start
// at zero (the arrival counters of the splits) is cleared on the caller's stream before each launch.
// Two calls that overlap on the GPU (different streams, or a replay racing a launch) would trample each
// other's partial results: keep calls on one device ordered.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#define VK_DECODE_STATIC_SCRATCH_BYTES ((size_t)8 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as vk_attention_decode without the scratch: q, out [all tokens, nh*hd]; cache: one layer
// [pages][2][nkv][page_size][hd]; block_tables [segments, max_blocks]; token_seg, positions [all tokens];
// tok_list [n_tokens] or null; max_context bounds every position + 1; dtype 0 = float32, 1 = bfloat16.
// Returns 0, a negative refusal (see vk_error_string) or a cudaError_t.
int vk_attention_decode_static(const void* q, const void* cache, const int32_t* block_tables, const int32_t* token_seg,
                               const int32_t* positions, const int32_t* tok_list, void* out, int n_tokens, int nh, int nkv,
                               int hd, int page_size, int max_blocks, int max_context, float scale, int window, int dtype,
                               cudaStream_t stream);

#ifdef __cplusplus
}
#endif
