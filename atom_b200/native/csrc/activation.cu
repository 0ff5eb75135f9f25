// SiLU-gated product of the feed-forward: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// computed in 32-bit (silu(x) = x / (1 + exp(-x))).
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n, int I) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int64_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// silu(x) = x / (1 + e^-x) = x * (0.5 + 0.5 * tanh(x / 2)): one special-function operation instead of two
// (the result is rounded to bfloat16, eight times coarser than tanh.approx's error).
__device__ __forceinline__ float silu_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return x * fmaf(0.5f, t, 0.5f);
}

// bf16, I a multiple of 8: 16 bytes of gate and of up per thread.
__global__ void silu_mul_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                         int64_t nvec, int I8) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
    const int64_t t = idx / I8;
    const int i = (int)(idx - t * I8);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + i) * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + i) * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gh[e]), u = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(silu_fast(g.x) * u.x, silu_fast(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = o4;
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
  if (dtype == ATOM_BF16 && I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const int64_t nvec = n / 8;
    int64_t vb = (nvec + threads - 1) / threads;
    if (vb > 148 * 32) vb = 148 * 32;
    atom::launch_pdl(atom::silu_mul_bf16_vec_kernel, dim3((int)vb), dim3(threads), 0, stream, (__nv_bfloat16*)out,
                                                                    (const __nv_bfloat16*)gu, nvec, I / 8);
    return atom::check_launch();
  }
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_F32) {
    atom::launch_pdl(atom::silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (float*)out, (const float*)gu, n, I);
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, n, I);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
