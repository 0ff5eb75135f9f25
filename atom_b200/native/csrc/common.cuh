// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes of the C interface.
#define ATOM_F32 0
#define ATOM_BF16 1

// Return codes of the C interface.
#define ATOM_OK 0
#define ATOM_ERR_ARG 1     // a size or flag the kernel does not take
#define ATOM_ERR_LAUNCH 2  // the CUDA runtime refused the launch
#define ATOM_ERR_LIB 3     // a library call failed

#define ATOM_EXPORT extern "C" __attribute__((visibility("default")))

namespace atom {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Loads element i of a vector whose storage is float or bf16, chosen at run time
// (norm weights and biases may stay in 32-bit beside bf16 activations).
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  return dtype == ATOM_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` holds at least 32 floats; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ATOM_OK : ATOM_ERR_LAUNCH;
}

}  // namespace atom
