// Embedding gather: residual[t, :] = table[ids[t], :], widened to 32-bit.
// The residual stream is kept in 32-bit in both precisions, so the gather writes floats.
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int t = blockIdx.x;
  int id = ids[t];
  // Ids are validated on the host; the clamp only keeps a bad id from reading outside the table.
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const T* row = table + (int64_t)id * H;
  float* o = out + (int64_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]);
}

}  // namespace atom

ATOM_EXPORT int atom_embedding(float* out, const void* table, int table_dtype, const int* ids, int T,
                               int H, int V, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || V <= 0) return ATOM_ERR_ARG;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == ATOM_F32) {
    atom::launch_pdl(atom::embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H, V);
  } else if (table_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
