// C interface of the weight-streaming product that shares out rows of W (gemm_rows.cu).
#pragma once
#include <stdint.h>

// One product  C[M, N] = X[M, K] * W[N, K]^T,  X and W bf16, M <= 16, with one of the epilogues
//   plain:     (+ bias), stored as bf16 or 32-bit into out (leading dimension ldc);
//   gated:     W is [2N, K] = [gate ; up], out = silu(X gate^T) * (X up^T);
//   residual:  residual[M, N] (32-bit, in place) += product; xout[M, N] = bf16(residual * norm_w);
//              ssq_out[c * 16 + m] = sum of residual[m, j]^2 over the columns j of CTA c, for every
//              c < atom_gemm_rows_grid()  (out is unused).
// ssq_in != null: output row m is first multiplied by rsqrt(sum_c ssq_in[c * 16 + m] / norm_size + norm_eps),
// c < ssq_parts: with X = xout of a residual product this is the product of RMSNorm(residual) with W,
//     RMSNorm(r) W^T = rstd(r) * ((r . w) W^T),
// without a pass of its own for the norm.
typedef struct AtomRowsOp {
  const void* X;
  int64_t lda;
  const void* W;
  void* out;
  int out_dtype;
  int64_t ldc;
  const void* bias;
  int bias_dtype;
  int N, K, gated;
  const float* ssq_in;
  int ssq_parts, norm_size;
  float norm_eps;
  float* residual;
  const void* norm_w;
  int norm_w_dtype;
  void* xout;
  float* ssq_out;
} AtomRowsOp;
