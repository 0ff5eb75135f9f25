// Paged causal attention for any head size, 32-bit arithmetic, any mixture of prompt
// portions and single decoded tokens.  One block takes one (query token, query head):
//   o = sum_j softmax_j(scale * q . k_j) v_j   over keys j in [max(0, p - window + 1), p]
// of the token's own request, p being the token's position; keys and values are read
// from the pages named by the request's block-table row.  Keys are processed in chunks
// with a running maximum and sum, so the context length is unbounded.
// This kernel is the true 32-bit path and also serves bf16 head sizes that the tensor-core
// kernels do not take.
#include "common.cuh"

namespace atom {

constexpr int kAttnThreads = 128;
constexpr int kAttnChunk = 256;

template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
paged_attention_generic_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride,
                               const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                               const int* __restrict__ block_table, int max_pages, int page_size,
                               const int* __restrict__ positions,
                               const int* __restrict__ seq_of_token, int nh, int nkv, int hd,
                               float scale, int window) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int64_t* row_off = (int64_t*)smem_raw;           // [kAttnChunk] element offset of a key's row
  float* prob = (float*)(row_off + kAttnChunk);    // [kAttnChunk]
  float* qs = prob + kAttnChunk;                   // [hd]
  __shared__ float scratch[32];

  const int t = blockIdx.x, h = blockIdx.y;
  const int g = h / (nh / nkv);
  const int p = positions[t];
  if (seq_of_token[t] < 0) return;  // a padding row of a fixed-size batch
  const int* bt = block_table + (int64_t)seq_of_token[t] * max_pages;
  const T* qrow = q + (int64_t)t * q_stride + (int64_t)h * hd;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) qs[i] = to_float(qrow[i]);

  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;

  // Each thread owns output elements d = tid, tid + 128, ... (hd <= 512).
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float m = -INFINITY, l = 0.f;
  __syncthreads();

  for (int c0 = lo; c0 <= p; c0 += kAttnChunk) {
    const int n = min(kAttnChunk, p + 1 - c0);
    float cmax = -INFINITY;
    for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
      const int j = c0 + jj;
      const int page = bt[j / page_size];
      const int64_t off = (((int64_t)page * nkv + g) * page_size + (j % page_size)) * hd;
      row_off[jj] = off;
      const T* kr = k_pages + off;
      float s = 0.f;
      for (int i = 0; i < hd; ++i) s += qs[i] * to_float(kr[i]);
      s *= scale;
      prob[jj] = s;
      cmax = fmaxf(cmax, s);
    }
    cmax = block_max(cmax, scratch);
    const float m_new = fmaxf(m, cmax);
    const float corr = expf(m - m_new);  // 0 on the first chunk (m = -inf)
    float lsum = 0.f;
    for (int jj = threadIdx.x; jj < n; jj += blockDim.x) {
      const float e = expf(prob[jj] - m_new);
      prob[jj] = e;
      lsum += e;
    }
    lsum = block_sum(lsum, scratch);  // also orders the prob[] writes before the reads below
    l = l * corr + lsum;
    m = m_new;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int d = threadIdx.x + a * kAttnThreads;
      if (d < hd) {
        float s = acc[a] * corr;
        for (int jj = 0; jj < n; ++jj) s += prob[jj] * to_float(v_pages[row_off[jj] + d]);
        acc[a] = s;
      }
    }
    __syncthreads();  // prob[] and row_off[] are rewritten by the next chunk
  }
  T* orow = out + ((int64_t)t * nh + h) * hd;
  const float inv = 1.f / l;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int d = threadIdx.x + a * kAttnThreads;
    if (d < hd) orow[d] = from_float<T>(acc[a] * inv);
  }
}

}  // namespace atom

// out: [T, nh * hd]; q: row t at q + t * q_stride (elements), heads packed [nh, hd].
// window <= 0 means all keys.
ATOM_EXPORT int atom_paged_attention_generic(void* out, const void* q, int64_t q_stride, int dtype,
                                             const void* k_pages, const void* v_pages,
                                             const int* block_table, int max_pages, int page_size,
                                             const int* positions, const int* seq_of_token, int T,
                                             int nh, int nkv, int hd, float scale, int window,
                                             cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || hd > 4 * atom::kAttnThreads ||
      page_size <= 0 || nh > 65535)
    return ATOM_ERR_ARG;
  const size_t smem = sizeof(float) * (hd + atom::kAttnChunk) + sizeof(int64_t) * atom::kAttnChunk;
  dim3 grid(T, nh);
  if (dtype == ATOM_F32) {
    atom::launch_pdl(atom::paged_attention_generic_kernel<float>, dim3(grid), dim3(atom::kAttnThreads), smem, stream, (float*)out, (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages,
        block_table, max_pages, page_size, positions, seq_of_token, nh, nkv, hd, scale, window);
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::paged_attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(atom::kAttnThreads), smem, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)q, q_stride,
            (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, max_pages,
            page_size, positions, seq_of_token, nh, nkv, hd, scale, window);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
