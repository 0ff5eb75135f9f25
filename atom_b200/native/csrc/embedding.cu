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

// bf16 table, H a multiple of 8: 16 bytes per load, all of a thread's loads asked for before the first is used
// (a row is one cold read from HBM: the kernel's time is round trips, not bytes).
__global__ void embedding_bf16_vec_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ table,
                                          const int* __restrict__ ids, int H, int V) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const uint4* row = reinterpret_cast<const uint4*>(table + (int64_t)id * H);
  float4* o = reinterpret_cast<float4*>(out + (int64_t)t * H);
  const int n = H >> 3;
  for (int i0 = threadIdx.x; i0 < n; i0 += 4 * blockDim.x) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      v[u] = i < n ? __ldg(row + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < n) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
        o[2 * i] = make_float4(a.x, a.y, b.x, b.y);
        o[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
      }
    }
  }
}

}  // namespace atom

ATOM_EXPORT int atom_embedding(float* out, const void* table, int table_dtype, const int* ids, int T,
                               int H, int V, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (H <= 0 || V <= 0) return ATOM_ERR_ARG;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == ATOM_F32) {
    atom::launch_pdl(atom::embedding_kernel<float>, dim3(T), dim3(threads), 0, stream, out, (const float*)table, ids, H, V);
  } else if (table_dtype == ATOM_BF16 && H % 8 == 0 && ((uintptr_t)table % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int vt = H >= 4096 ? 128 : (H >= 1024 ? 64 : 32);      // a thread takes up to four 16-byte pieces at a time
    atom::launch_pdl(atom::embedding_bf16_vec_kernel, dim3(T), dim3(vt), 0, stream, out, (const __nv_bfloat16*)table, ids,
                     H, V);
  } else if (table_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::embedding_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
