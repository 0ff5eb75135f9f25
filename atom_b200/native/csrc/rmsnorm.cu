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
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
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
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
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

// bf16 activations, H a multiple of 8, at most 8 * NV * blockDim: every thread keeps its
// 8 * NV elements in registers, so the row is read once and written once, 16 bytes at a time.
template <int NV>
__global__ void add_rmsnorm_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ residual,
                                            const __nv_bfloat16* __restrict__ delta,
                                            const void* __restrict__ w, int w_dtype, float eps,
                                            const int* __restrict__ rows, int H) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int64_t src = rows ? rows[r] : r;
  // The norm weights do not depend on the kernel in front of this one: they are on their way before the wait.
  float wv[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      if (w_dtype == ATOM_F32) {
        const float4 a = *reinterpret_cast<const float4*>((const float*)w + i);
        const float4 b = *reinterpret_cast<const float4*>((const float*)w + i + 4);
        wv[k][0] = a.x; wv[k][1] = a.y; wv[k][2] = a.z; wv[k][3] = a.w;
        wv[k][4] = b.x; wv[k][5] = b.y; wv[k][6] = b.z; wv[k][7] = b.w;
      } else {
        const uint4 q = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)w + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          wv[k][2 * e] = f.x;
          wv[k][2 * e + 1] = f.y;
        }
      }
    }
  }
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  float* res = residual + src * H;
  const __nv_bfloat16* d = delta ? delta + src * H : nullptr;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      const float4 a = *reinterpret_cast<const float4*>(res + i);
      const float4 b = *reinterpret_cast<const float4*>(res + i + 4);
      v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w;
      v[k][4] = b.x; v[k][5] = b.y; v[k][6] = b.z; v[k][7] = b.w;
      if (d) {
        const uint4 q = *reinterpret_cast<const uint4*>(d + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[k][2 * e] += f.x;
          v[k][2 * e + 1] += f.y;
        }
        if (!rows) {
          *reinterpret_cast<float4*>(res + i) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
          *reinterpret_cast<float4*>(res + i + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (int64_t)r * H;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = (threadIdx.x + k * blockDim.x) * 8;
    if (i < H) {
      uint4 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        h[e] = __floats2bfloat162_rn(v[k][2 * e] * rstd * wv[k][2 * e], v[k][2 * e + 1] * rstd * wv[k][2 * e + 1]);
      *reinterpret_cast<uint4*>(o + i) = q;
    }
  }
}

}  // namespace atom

ATOM_EXPORT int atom_add_rmsnorm(void* out, int act_dtype, float* residual, const void* delta,
                                 const void* w, int w_dtype, float eps, const int* rows, int n_rows,
                                 int H, cudaStream_t stream) {
  if (n_rows <= 0) return ATOM_OK;
  if (H <= 0 || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = atom::norm_threads(H);
  const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                       ((uintptr_t)delta % 16 == 0) && ((uintptr_t)w % 16 == 0);
  if (act_dtype == ATOM_BF16 && H % 8 == 0 && H <= 8 * 2 * 1024 && aligned) {
    // one pass over the row, 16-byte accesses: 128 to 1024 threads, one or two vectors each
    const int vecs = H / 8;
    int nv = 1, th = ((vecs + 31) / 32) * 32;
    if (th > 1024) {
      nv = 2;
      th = (((vecs + 1) / 2 + 31) / 32) * 32;
    }
    if (th < 64) th = 64;
    if (nv == 1)
      atom::launch_pdl(atom::add_rmsnorm_bf16_vec_kernel<1>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H);
    else
      atom::launch_pdl(atom::add_rmsnorm_bf16_vec_kernel<2>, dim3(n_rows), dim3(th), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H);
    return atom::check_launch();
  }
  if (act_dtype == ATOM_F32) {
    atom::launch_pdl(atom::add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (float*)out, residual, (const float*)delta, w, w_dtype, eps, rows, H);
  } else if (act_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (__nv_bfloat16*)out, residual, (const __nv_bfloat16*)delta, w, w_dtype, eps, rows, H);
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
    atom::launch_pdl(atom::rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (float*)out, (const float*)x, w, w_dtype, eps, H);
  } else if (act_dtype == ATOM_BF16) {
    atom::launch_pdl(atom::rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, w, w_dtype, eps, H);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
