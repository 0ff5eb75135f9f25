// SiLU-gated product of the feed-forward: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// computed in 32-bit (silu(x) = x / (1 + exp(-x))).
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n, int I) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int64_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

}  // namespace atom

ATOM_EXPORT int atom_silu_mul(void* out, const void* gu, int dtype, int T, int I,
                              cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (I <= 0) return ATOM_ERR_ARG;
  const int64_t n = (int64_t)T * I;
  const int threads = 256;
  int64_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32) {
    atom::silu_mul_kernel<float>
        <<<(int)blocks, threads, 0, stream>>>((float*)out, (const float*)gu, n, I);
  } else if (dtype == ATOM_BF16) {
    atom::silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, n, I);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
