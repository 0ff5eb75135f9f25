// bf16 matrix products through cuBLAS, where the reference engine calls its GEMM library
// (atom/model_ops/linear.py:960):  C[M, N] = A[M, K] * W[N, K]^T, 32-bit accumulation,
// C in bf16 or in 32-bit (the logits).  Plus the bias add that follows when a layer has one.
#include <cublas_v2.h>

#include "common.cuh"

namespace atom {

static cublasHandle_t g_handle[16] = {};

static cublasHandle_t handle_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  if (g_handle[dev] == nullptr) {
    if (cublasCreate(&g_handle[dev]) != CUBLAS_STATUS_SUCCESS) return nullptr;
  }
  return g_handle[dev];
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ C, const void* __restrict__ bias, int bias_dtype,
                                int64_t n, int N) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    C[i] = from_float<T>(to_float(C[i]) + load_as_float(bias, bias_dtype, i % N));
}

}  // namespace atom

// `workspace` is caller-owned device memory that cuBLAS may use (so that a call inside a
// stream capture allocates nothing).
ATOM_EXPORT int atom_gemm_bf16(void* C, int c_dtype, const void* A, const void* W, int M, int N,
                               int K, int64_t lda, void* workspace, size_t workspace_bytes,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return ATOM_OK;
  if (K <= 0 || lda < K) return ATOM_ERR_ARG;
  cublasHandle_t h = atom::handle_for_current_device();
  if (h == nullptr) return ATOM_ERR_LIB;
  if (cublasSetStream(h, stream) != CUBLAS_STATUS_SUCCESS) return ATOM_ERR_LIB;
  if (workspace != nullptr &&
      cublasSetWorkspace(h, workspace, workspace_bytes) != CUBLAS_STATUS_SUCCESS)
    return ATOM_ERR_LIB;
  const float alpha = 1.f, beta = 0.f;
  cudaDataType ct;
  if (c_dtype == ATOM_F32) ct = CUDA_R_32F;
  else if (c_dtype == ATOM_BF16) ct = CUDA_R_16BF;
  else return ATOM_ERR_ARG;
  // Row-major C[M,N] = A * W^T is column-major C^T[N,M] = W(op T)[N,K] * A^T[K,M].
  cublasStatus_t st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, W, CUDA_R_16BF, K,
                                   A, CUDA_R_16BF, (int)lda, &beta, C, ct, N, CUBLAS_COMPUTE_32F,
                                   CUBLAS_GEMM_DEFAULT);
  return st == CUBLAS_STATUS_SUCCESS ? ATOM_OK : ATOM_ERR_LIB;
}

ATOM_EXPORT int atom_add_bias(void* C, int c_dtype, const void* bias, int bias_dtype, int M, int N,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return ATOM_OK;
  const int64_t n = (int64_t)M * N;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (c_dtype == ATOM_F32)
    atom::launch_pdl(atom::add_bias_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)C, bias, bias_dtype, n, N);
  else if (c_dtype == ATOM_BF16)
    atom::launch_pdl(atom::add_bias_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (__nv_bfloat16*)C, bias, bias_dtype, n, N);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
