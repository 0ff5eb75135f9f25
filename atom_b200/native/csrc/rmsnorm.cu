// Fused residual add + RMSNorm.
//   r = residual[row] (+ delta[row]);  residual[row] = r  (unless rows are picked);
//   out[i] = r * rsqrt(mean(r^2) + eps) * w
// The residual stream and all arithmetic are 32-bit; `delta` (the previous block's
// output) and `out` (the next matrix product's input) have the activation type.
// With `rows` given, only those rows are normalised and written densely: this is
// the gather of the rows whose logits are wanted, fused into the final norm.
#include "common.cuh"

namespace atom {

template <typename TA>
__global__ void add_rmsnorm_kernel(TA* __restrict__ out, float* __restrict__ residual,
                                   const TA* __restrict__ delta, const void* __restrict__ w,
                                   int w_dtype, float eps, const int* __restrict__ rows, int H) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  float* res = residual + src * H;
  const TA* d = delta ? delta + src * H : nullptr;
  TA* o = out + (int64_t)r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = res[i];
    if (d) {
      v += to_float(d[i]);
      // Picked rows are not carried further: their sum is formed again in the second pass
      // instead of being written back.
      if (!rows) res[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = res[i];
    if (d && rows) v += to_float(d[i]);
    o[i] = from_float<TA>(v * rstd * load_as_float(w, w_dtype, i));
  }
}

// Plain RMSNorm over the last dimension of a dense [rows, H] array of the activation type.
template <typename TA>
__global__ void rmsnorm_kernel(TA* __restrict__ out, const TA* __restrict__ x,
                               const void* __restrict__ w, int w_dtype, float eps, int H) {
  __shared__ float scratch[32];
  const TA* xi = x + (int64_t)blockIdx.x * H;
  TA* o = out + (int64_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_float(xi[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    o[i] = from_float<TA>(to_float(xi[i]) * rstd * load_as_float(w, w_dtype, i));
}

static inline int norm_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

}  // namespace atom

ATOM_EXPORT int atom_add_rmsnorm(void* out, int act_dtype, float* residual, const void* delta,
                                 const void* w, int w_dtype, float eps, const int* rows, int n_rows,
                                 int H, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  if (act_dtype == ATOM_F32) {
    atom::add_rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>(
        (float*)out, residual, (const float*)delta, w, w_dtype, eps, rows, H);
  } else if (act_dtype == ATOM_BF16) {
    atom::add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

ATOM_EXPORT int atom_rmsnorm(void* out, const void* x, int act_dtype, const void* w, int w_dtype,
                             float eps, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  if (act_dtype == ATOM_F32) {
    atom::rmsnorm_kernel<float>
        <<<n_rows, threads, 0, stream>>>((float*)out, (const float*)x, w, w_dtype, eps, H);
  } else if (act_dtype == ATOM_BF16) {
    atom::rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)x, w, w_dtype, eps, H);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
