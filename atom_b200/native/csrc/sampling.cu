// Token sampling from 32-bit logits, one block per row.
//   temperature == 0:  argmax, lowest index on ties.
//   temperature  > 0:  the exponential race  argmax_v softmax(logits / T)_v / E_v,
//                      E_v ~ Exp(1)  (equal in law to drawing from the softmax), run among the
//                      entries that top-k / top-p keep.
// The noise is a pure function of (row seed, row index, v): the same request draws the same
// token whatever else is in the batch.  E_v = -log(u), u = (top 24 bits + 0.5) / 2^24 of a
// 32-bit mix of the three.
// top-k keeps the k most probable entries, top-p those whose strictly more probable
// entries have a total mass <= p; both are found by bisection on the bit pattern of the
// probabilities (positive floats order like their bits), which needs the row's probabilities
// in a caller-owned scratch array.
#include "common.cuh"

namespace atom {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7FEB352Du;
  x ^= x >> 15;
  x *= 0x846CA68Bu;
  x ^= x >> 16;
  return x;
}

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ Best block_best(Best b, Best* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = b;
  __syncthreads();
  Best r = lane < nw ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, other);
  }
  return r;
}

__global__ void __launch_bounds__(1024)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
              const float* __restrict__ temperature, const uint32_t* __restrict__ seeds,
              const uint32_t* __restrict__ indices, const int* __restrict__ top_k,
              const float* __restrict__ top_p, float* __restrict__ probs, int V) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  __shared__ float fscratch[32];
  __shared__ Best bscratch[32];
  const int r = blockIdx.x;
  const float* row = logits + (int64_t)r * V;
  const float T = temperature[r];

  if (T <= 0.f) {
    Best b{-INFINITY, 0x7fffffff};
    for (int v = threadIdx.x; v < V; v += blockDim.x) b = better(b, Best{row[v], v});
    b = block_best(b, bscratch);
    if (threadIdx.x == 0) out[r] = b.i;
    return;
  }

  const float invT = 1.f / T;
  float m = -INFINITY;
  for (int v = threadIdx.x; v < V; v += blockDim.x) m = fmaxf(m, row[v]);
  m = block_max(m, fscratch);

  const int k = top_k ? top_k[r] : -1;
  const float p_keep = top_p ? top_p[r] : 1.f;
  const bool filter = (k > 0 && k < V) || p_keep < 1.f;
  uint32_t thr_bits = 0;  // keep entries whose probability bits are >= thr_bits
  if (filter) {
    float* pr = probs + (int64_t)r * V;
    float z = 0.f;
    for (int v = threadIdx.x; v < V; v += blockDim.x) z += expf((row[v] - m) * invT);
    z = block_sum(z, fscratch);
    const float invz = 1.f / z;
    for (int v = threadIdx.x; v < V; v += blockDim.x) pr[v] = expf((row[v] - m) * invT) * invz;
    __syncthreads();
    if (k > 0 && k < V) {
      // largest t with count(p >= t) >= k
      uint32_t lo = 0, hi = 0x3F800001u;
      while (hi - lo > 1) {
        const uint32_t mid = lo + (hi - lo) / 2;
        float c = 0.f;
        for (int v = threadIdx.x; v < V; v += blockDim.x) c += (__float_as_uint(pr[v]) >= mid) ? 1.f : 0.f;
        c = block_sum(c, fscratch);
        if (c >= (float)k) lo = mid; else hi = mid;
      }
      thr_bits = lo;
    }
    if (p_keep < 1.f) {
      // smallest t with mass(p > t) <= p_keep
      uint32_t lo = 0, hi = 0x3F800000u;
      while (lo < hi) {
        const uint32_t mid = lo + (hi - lo) / 2;
        float s = 0.f;
        for (int v = threadIdx.x; v < V; v += blockDim.x) {
          const float p = pr[v];
          s += (__float_as_uint(p) > mid) ? p : 0.f;
        }
        s = block_sum(s, fscratch);
        if (s <= p_keep) hi = mid; else lo = mid + 1;
      }
      thr_bits = max(thr_bits, hi);
    }
  }

  const uint32_t key = mix32(seeds[r] ^ mix32(indices[r] + 0x9E3779B9u));
  const float* pr = probs + (int64_t)r * V;
  Best b{-INFINITY, 0x7fffffff};
  Best top{-INFINITY, 0x7fffffff};  // most probable entry: always kept
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    const float x = (row[v] - m) * invT;
    top = better(top, Best{x, v});
    if (filter && __float_as_uint(pr[v]) < thr_bits) continue;
    const uint32_t bits = mix32(((uint32_t)(v + 1) * 0x9E3779B1u) ^ key);
    const float u = ((float)(bits >> 8) + 0.5f) * (1.f / 16777216.f);
    const float e = -logf(u);
    b = better(b, Best{x - logf(e), v});
  }
  b = block_best(b, bscratch);
  top = block_best(top, bscratch);
  if (threadIdx.x == 0) out[r] = (b.i == 0x7fffffff) ? top.i : b.i;
}

// Rows without top-k / top-p: the choice is one argmax over the vocabulary,
//   temperature 0:  of the logits;   temperature T:  of logits / T - log(E_v)
// (the race above without the row maximum, which does not change the winner).  The vocabulary is
// cut into `chunks` pieces that as many blocks scan at once; a second kernel picks the best piece.
__global__ void __launch_bounds__(256)
sample_chunk_kernel(Best* __restrict__ part, const float* __restrict__ logits,
                    const float* __restrict__ temperature, const uint32_t* __restrict__ seeds,
                    const uint32_t* __restrict__ indices, int V, int chunk) {
  atom::pdl_wait();
  atom::pdl_trigger();
  __shared__ Best bscratch[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (int64_t)r * V;
  const float T = temperature[r];
  const int v0 = c * chunk, v1 = min(V, v0 + chunk);
  Best b{-INFINITY, 0x7fffffff};
  if (T <= 0.f) {
    for (int v = v0 + threadIdx.x; v < v1; v += 4 * 256) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = (v + k * 256 < v1) ? row[v + k * 256] : -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) b = better(b, Best{x[k], v + k * 256});
    }
  } else {
    const float invT = 1.f / T;
    const uint32_t key = mix32(seeds[r] ^ mix32(indices[r] + 0x9E3779B9u));
    for (int v = v0 + threadIdx.x; v < v1; v += 4 * 256) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = (v + k * 256 < v1) ? row[v + k * 256] : -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int vv = v + k * 256;
        const uint32_t bits = mix32(((uint32_t)(vv + 1) * 0x9E3779B1u) ^ key);
        const float u = ((float)(bits >> 8) + 0.5f) * (1.f / 16777216.f);
        const float e = -logf(u);
        if (vv < v1) b = better(b, Best{x[k] * invT - logf(e), vv});
      }
    }
  }
  b = block_best(b, bscratch);
  if (threadIdx.x == 0) part[(int64_t)r * gridDim.x + c] = b;
}

__global__ void sample_pick_kernel(int* __restrict__ out, const Best* __restrict__ part, int chunks) {
  atom::pdl_wait();
  atom::pdl_trigger();
  const int r = blockIdx.x;
  Best b{-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < chunks; c += 32) b = better(b, part[(int64_t)r * chunks + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
    b = better(b, other);
  }
  if (threadIdx.x == 0) out[r] = b.i == 0x7fffffff ? 0 : b.i;
}

}  // namespace atom

// Rows that use neither top-k nor top-p.  part: scratch of R * chunks * 8 bytes.
ATOM_EXPORT int atom_sample_simple(int* out, const float* logits, const float* temperature,
                                   const uint32_t* seeds, const uint32_t* indices, void* part, int chunks,
                                   int R, int V, cudaStream_t stream) {
  if (R <= 0) return ATOM_OK;
  if (V <= 0 || chunks <= 0 || chunks > 1024 || part == nullptr || R > 65535) return ATOM_ERR_ARG;
  const int chunk = (V + chunks - 1) / chunks;
  atom::launch_pdl(atom::sample_chunk_kernel, dim3(chunks, R), dim3(256), 0, stream, (atom::Best*)part, logits,
                   temperature, seeds, indices, V, chunk);
  atom::launch_pdl(atom::sample_pick_kernel, dim3(R), dim3(32), 0, stream, out, (const atom::Best*)part, chunks);
  return atom::check_launch();
}

// probs: scratch [R, V] floats, needed only when a row filters (may be null otherwise).
ATOM_EXPORT int atom_sample(int* out, const float* logits, const float* temperature,
                            const uint32_t* seeds, const uint32_t* indices, const int* top_k,
                            const float* top_p, float* probs, int R, int V, cudaStream_t stream) {
  if (R <= 0) return ATOM_OK;
  if (V <= 0) return ATOM_ERR_ARG;
  if ((top_k != nullptr || top_p != nullptr) && probs == nullptr) return ATOM_ERR_ARG;
  const int threads = V >= 8192 ? 1024 : (V >= 1024 ? 256 : 128);
  atom::launch_pdl(atom::sample_kernel, dim3(R), dim3(threads), 0, stream, out, logits, temperature, seeds, indices, top_k,
                                                 top_p, probs, V);
  return atom::check_launch();
}


// ------------------------------------------------------------------ log-probability of chosen tokens
namespace atom {
// out[r] = logits[r, ids[r]] - log sum_v exp(logits[r, v]), in 32-bit: the log-probability of
// the sampled token under the model's distribution (as torch.log_softmax(...).gather(...) in
// atom/model_engine/model_runner.py:3233-3240).  One block per row.
__global__ void __launch_bounds__(512)
token_logprob_kernel(float* __restrict__ out, const float* __restrict__ logits, const int* __restrict__ ids, int V) {
  atom::pdl_trigger();
  atom::pdl_wait();
  __shared__ float scratch[32];
  const float* row = logits + (int64_t)blockIdx.x * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, scratch);
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) sum += __expf(row[i] - mx);
  sum = block_sum(sum, scratch);
  if (threadIdx.x == 0) {
    const int id = ids[blockIdx.x];
    out[blockIdx.x] = (id >= 0 && id < V) ? row[id] - mx - __logf(sum) : -INFINITY;
  }
}
}  // namespace atom

ATOM_EXPORT int atom_token_logprob(float* out, const float* logits, const int* ids, int R, int V, cudaStream_t stream) {
  if (R <= 0) return ATOM_OK;
  if (V <= 0) return ATOM_ERR_ARG;
  atom::launch_pdl(atom::token_logprob_kernel, dim3(R), dim3(512), 0, stream, out, logits, ids, V);
  return atom::check_launch();
}
