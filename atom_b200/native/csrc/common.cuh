// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// ------------------------------------------------------------------ programmatic dependent launch
// Launched with launch_pdl, a kernel may be scheduled as soon as every CTA of the kernel before
// it has passed pdl_trigger() (or exited), that is, while that kernel, and the ones before it,
// still run.  pdl_wait() returns when the kernel before it has completed and its writes are
// visible.  The rules that make a chain of such kernels right:
//   * pdl_trigger() stands at the top of every kernel, so launch latency and prologues overlap
//     whatever is still running;
//   * before pdl_wait() a kernel reads only what no kernel of the same step writes: weights,
//     tables, the step's index arrays (filled by copies before the step's first kernel), cache
//     pages of earlier steps' tokens; it writes nothing to global memory;
//   * every path through a kernel passes pdl_wait() before it ends (in at least one thread of
//     every CTA that could otherwise be the last to finish: simplest, before every early
//     return), so that a completed grid means that everything before it has completed too.
// Option ATOM_OPT_PDL = 0 gives plain launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// ------------------------------------------------------------------ options for measurements and tests
// Choices that the launch code otherwise makes by itself, overridable per process so that both sides
// of a choice can be measured and tested in one run.  Every library built from these sources has its
// own copy, set through its exported set-option function (the Python binding sets all of them).  The
// environment is never read.
#define ATOM_OPT_PDL 0            // 1 (default): programmatic dependent launch; 0: plain launches
#define ATOM_OPT_DECODE_TMA 1     // 1 (default): decode attention through TMA where it applies; 0: cp.async kernel
#define ATOM_OPT_DECODE_KTW 2     // 0 (default): warp tile of the TMA decode kernel by occupancy; 16 or 32: forced
#define ATOM_OPT_COUNT 3
struct Options {
  int v[ATOM_OPT_COUNT] = {1, 1, 0};
};
inline Options& options() {
  static Options o;
  return o;
}
inline int set_option(int key, int value) {
  if (key < 0 || key >= ATOM_OPT_COUNT) return ATOM_ERR_ARG;
  options().v[key] = value;
  return ATOM_OK;
}

inline bool pdl_enabled() { return options().v[ATOM_OPT_PDL] != 0; }

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in check_launch()
}

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? ATOM_OK : ATOM_ERR_LAUNCH;
}

}  // namespace atom
