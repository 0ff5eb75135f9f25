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

// Causal attention of T query tokens (of num_seqs requests, a request's tokens in a row) over the keys
// and values of their own requests in a paged cache, bf16 in and out, sums in 32-bit.  Only the
// cp.async / mma.sync kernels run on this path (no TMA, no tensor memory), for any page size.
//
//   out            [T, nh * hd] bf16.  A row that no launched tile covers is NOT written: see prefill_tiles.
//   q, q_stride    queries: token t's head h at q + t * q_stride + h * hd (bf16 elements; q_stride a
//                  multiple of 8).  The queries may be the first columns of a wider [q | k | v] array.
//   k_pages, v_pages   [pages, nkv, page_size, hd] bf16 each.
//   block_table    [num_seqs, max_pages] int32: the page of request s that holds its tokens
//                  [i * page_size, (i + 1) * page_size).
//   cu_q           [num_seqs + 1] int32: request s owns the query tokens cu_q[s] .. cu_q[s + 1] - 1.
//   ctx_len        [num_seqs] int32: tokens of request s in the cache, its query tokens of this call
//                  included (they are its last ones; their keys must be in the pages already).
//   seq_of_token   [T] int32: the request of every query token (-1: a padding row, skipped).
//   nh, nkv, hd    query heads, key/value heads (nh a multiple of nkv), head size.  hd must be the one
//                  this library was compiled for (atom_flash_head_dim()).
//   scale          multiplies the scores before the softmax (> 0; usually hd^-0.5).
//   window         > 0: a token sees only the last `window` keys up to itself; 0: all of them.
//   A request's "packed rows" are its query tokens times nh / nkv (the query heads that share a kv head are
//   rows of one tile).  The caller says which kernels are needed:
//   prefill_tiles  the sum, over the requests with MORE than 16 packed rows, of ceil(packed rows / 64)
//                  (requests of 128 rows and more too: the tensor-memory kernel is off on this path);
//                  0 if there is none.  A count that is too small leaves rows of `out` unwritten; one that
//                  is too large costs CTAs that leave at once.
//   has_short      1 if some request has at most 16 packed rows (decoded tokens), else 0.
//   num_splits     >= 1: the key ranges of the short requests are cut into this many pieces that run as
//                  CTAs of their own and are merged afterwards; with 1 nothing is merged and no scratch
//                  is used.  At most 65535, and within the scratch limit above.
//   stream         the CUDA stream of every launch.
// Returns 0, or ATOM_ERR_ARG (1) for sizes the kernels do not take, ATOM_ERR_SCRATCH, ATOM_ERR_SETUP, or
// the launch error code of common.cuh.
int atom_flash_attention_static(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                const void* v_pages, const int* block_table, int max_pages,
                                int page_size, const int* cu_q, const int* ctx_len,
                                const int* seq_of_token, int T, int num_seqs, int nh, int nkv, int hd,
                                float scale, int window, int prefill_tiles, int has_short,
                                int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
