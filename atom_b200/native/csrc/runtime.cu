// Host-side helpers of the core library that launch no kernel: options, and the copy that brings the
// live part of a step's block tables to the device.
#include "common.cuh"

// Sets one of the ATOM_OPT_* options (common.cuh) in the core library.
ATOM_EXPORT int atom_set_option(int key, int value) { return atom::set_option(key, value); }

// Copies ``rows`` rows of ``row_bytes`` bytes from pinned host memory (rows ``src_pitch`` bytes apart) to
// device memory (rows ``dst_pitch`` bytes apart) on ``stream``.  A captured step reads block tables whose
// rows are as long as the longest request the engine takes; each step brings only the rows of the live
// requests, as far as their longest context reaches.
ATOM_EXPORT int atom_copy_rows_h2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                                   int64_t row_bytes, int64_t rows, cudaStream_t stream) {
  if (rows <= 0 || row_bytes <= 0) return ATOM_OK;
  if (dst == nullptr || src == nullptr || dst_pitch < row_bytes || src_pitch < row_bytes) return ATOM_ERR_ARG;
  const cudaError_t e = cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)row_bytes,
                                          (size_t)rows, cudaMemcpyHostToDevice, stream);
  return e == cudaSuccess ? ATOM_OK : ATOM_ERR_LAUNCH;
}
