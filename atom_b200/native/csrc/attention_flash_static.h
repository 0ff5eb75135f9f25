// Paged attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine; it exists for embedders of
// this library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- a plug-in inside a host
// application that owns the device's memory pool and hands out none of it, a real-time loop
// that may not take the allocator's lock or its implicit device synchronisation, or a
// caller that cannot link a tensor framework whose allocator the regular path relies on for
// the split-K scratch.  Such a caller still owns and passes every input and output array;
// only the scratch for the partial results of the key splits comes from this library.
//
// The scratch is a file-scope array in device memory, ATOM_FLASH_STATIC_SCRATCH_FLOATS
// 32-bit floats (8 MiB), compiled into the library.  Every GPU whose context loads this
// library holds those 8 MiB until the process exits.
//
// Rules of use:
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and sets the kernels' shared-memory attribute, with that device
//     current.  Make that first call outside any stream capture.
//   * A call whose splits need more floats than the array holds,
//         T * nh * num_splits * (head size + 2)  >  ATOM_FLASH_STATIC_SCRATCH_FLOATS,
//     is refused with ATOM_ERR_SCRATCH before anything is launched; num_splits <= 1 needs none.
//   * All calls share the one array and it keeps what the last call left.  Nothing in it has
//     to start at zero: every partial result that the merge step reads is written first by
//     the same call.  Two calls that overlap on the GPU (different streams, no dependency)
//     race on it and give wrong results; serialise them.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define ATOM_FLASH_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define ATOM_ERR_SCRATCH 4   // the call needs more scratch than the static array holds
#define ATOM_ERR_SETUP 5     // the per-device set-up (symbol address) failed

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and meaning as atom_flash_attention, without the scratch pointer.
int atom_flash_attention_static(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                const void* v_pages, const int* block_table, int max_pages,
                                int page_size, const int* cu_q, const int* ctx_len,
                                const int* seq_of_token, int T, int num_seqs, int nh, int nkv, int hd,
                                float scale, int window, int prefill_tiles, int has_short,
                                int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
