// True 32-bit matrix product on the FMA units (no tensor cores, no reduced-precision mode):
//   C[M, N] = A[M, K] * W[N, K]^T (+ bias[N])
// Each output element is one sequential sum over k in increasing order, whatever M is,
// so a row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace atom {

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ W,
                const float* __restrict__ bias, int M, int N, int K, int64_t lda, int64_t ldc) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k per operand: 1024 elements, 4 per thread.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * 256;
      const int r = idx / BK, kk = idx % BK;
      const int k = k0 + kk;
      const int m = m0 + r, n = n0 + r;
      As[kk][r] = (m < M && k < K) ? A[(int64_t)m * lda + k] : 0.f;
      Ws[kk][r] = (n < N && k < K) ? W[(int64_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(int64_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
  }
}

}  // namespace atom

ATOM_EXPORT int atom_gemm_f32(float* C, const float* A, const float* W, const float* bias, int M,
                              int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return ATOM_OK;
  if (K <= 0 || lda < K || ldc < N) return ATOM_ERR_ARG;
  dim3 grid((N + atom::BN - 1) / atom::BN, (M + atom::BM - 1) / atom::BM);
  if (grid.y > 65535) return ATOM_ERR_ARG;
  atom::launch_pdl(atom::gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, C, A, W, bias, M, N, K, lda, ldc);
  return atom::check_launch();
}
