// llm_paged_attention_decode_noalloc: the split-key decode attention for callers that must not
// allocate device memory.  This entry point has no counterpart in the reference; it exists for
// hosts that embed the kernel library without the engine's Python side.
//
// Who cannot allocate.  A process that has already handed every byte of device memory to a pool
// of its own gets "out of memory" from cudaMalloc, however small the request.  A control loop with
// a deadline cannot pay for cudaMalloc and cudaFree either: both may synchronise the whole device,
// so an allocation in one thread stalls the kernels of every other.  Such callers still own their
// inputs and outputs; what they cannot supply ad hoc is the scratch in which the key splits leave
// their partial results.  Here that scratch is part of the library image.
//
// The scratch.  A file-scope `static __device__ __align__(256)` array of
// LLM_DECODE_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the library is loaded
// holds these 16 MiB from load to process exit, whether or not this entry point is ever called.
// A call needs n_rows * nq * num_splits * (d + 2) floats when num_splits > 1 and none otherwise;
// a call that needs more than the array holds is refused with LLM_REFUSED_SCRATCH and launches
// nothing.  llm_paged_attention_decode_noalloc_needed() returns the number for given sizes, and
// llm_noalloc_strerror() turns any return code of this entry point into a sentence.
//
// First call on a device.  Host code cannot use the array's name as a pointer (on the host the
// name is only a handle for the runtime), so the first call on each device asks the runtime for
// the device address with cudaGetSymbolAddress, with that device current, checks the result and
// keeps it for later calls.  Make that first call during start-up, outside any stream capture.
//
// Sharing.  There is one array per device and every call uses it from its first float.  Each
// split writes its own slots before the merge reads them, so nothing has to be cleared between
// calls; but two calls whose kernels overlap on the GPU (different streams, or the same arguments
// from two threads) write the same slots and race.  Order such calls on one stream or with events.
//
// No cudaMalloc, cudaFree or allocating library routine is called, here or below.
// Arguments are those of llm_paged_attention_decode without `scratch`.
#pragma once

#include <stdint.h>

#define LLM_DECODE_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define LLM_REFUSED_SCRATCH (-4)     // the call needs more scratch than the library's static array holds
#define LLM_SYMBOL_ADDRESS_FAILED (-5)   // cudaGetSymbolAddress did not give the array's device address

#ifdef __cplusplus
extern "C" {
#endif

int llm_paged_attention_decode_noalloc(
    const void* q, void* out, const void* cache, const int32_t* rows, int n_rows, const int32_t* positions,
    const int32_t* token_entry, const int32_t* entry_slot, const int32_t* block_table, int table_stride, int nq,
    int nkv, int d, int page_size, int window, float scale, int num_pages, int num_splits, int32_t* status,
    uintptr_t stream);

long long llm_paged_attention_decode_noalloc_needed(int n_rows, int nq, int d, int num_splits);

const char* llm_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
