// Fused per-head q/k RMSNorm + rotary position encoding + paged KV-cache write.
//
// One warp takes one (token, head) of the packed projection output
//   qkv[t] = [ q heads (nh) | k heads (nkv) | v heads (nkv) ], each of width hd.
// q and k heads are normalised over hd (if norm weights are given), rotated over their
// first `rotary_dim` elements in the half-split ("neox") pairing (j, j + rotary_dim/2)
// and written back in place (q) and to the key pages (k); v heads are copied to the
// value pages.  All arithmetic is 32-bit; angles come from a 32-bit table
//   cos_sin[pos] = [cos(pos * f_j) for j < rotary_dim/2 | sin(pos * f_j) ...].
// Page layout: pages[page][kv head][slot in page][hd]; the page of a position comes from
// the request's block-table row: page = block_table[seq][pos / page_size].
#include "common.cuh"

namespace atom {

template <typename T>
__global__ void qknorm_rope_kvwrite_kernel(
    T* __restrict__ qkv, int nh, int nkv, int hd, const void* __restrict__ q_w,
    const void* __restrict__ k_w, int w_dtype, float eps, const float* __restrict__ cos_sin,
    int rotary_dim, int max_pos, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages,
    int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int64_t num_pages,
    int* __restrict__ status) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  const int n_heads_total = nh + 2 * nkv;
  if (head >= n_heads_total) return;
  const bool is_q = head < nh;
  const bool is_k = !is_q && head < nh + nkv;
  const bool write_cache = k_pages != nullptr;
  if (!is_q && !write_cache) return;

  const int seq = seq_of_token[t];
  if (seq < 0) return;  // a padding row of a fixed-size batch: belongs to no request

  T* x = qkv + ((int64_t)t * n_heads_total + head) * hd;
  const int pos = positions[t];

  // Destination in the cache for k and v heads.
  T* dst = nullptr;
  if (!is_q) {
    const int page = block_table[(int64_t)seq * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      // A position without a page is a host-side accounting fault: record it, write nothing.
      if (lane == 0) atomicExch(status, 1);
      return;
    }
    const int kvh = is_k ? head - nh : head - nh - nkv;
    T* base = is_k ? k_pages : v_pages;
    dst = base + (((int64_t)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
  }

  if (!is_q && !is_k) {  // value head: plain copy
    for (int i = lane; i < hd; i += 32) dst[i] = x[i];
    return;
  }

  const void* w = is_q ? q_w : k_w;
  float rstd = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float v = to_float(x[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)hd + eps);
  }
  const int half = rotary_dim >> 1;
  const int p = pos < max_pos ? pos : max_pos - 1;  // host checks pos < max_pos
  const float* cs = cos_sin + (int64_t)p * rotary_dim;
  T* o = is_q ? x : dst;
  for (int j = lane; j < half; j += 32) {
    float x1 = to_float(x[j]) * rstd;
    float x2 = to_float(x[j + half]) * rstd;
    if (w != nullptr) {
      x1 *= load_as_float(w, w_dtype, j);
      x2 *= load_as_float(w, w_dtype, j + half);
    }
    const float c = cs[j], s = cs[half + j];
    o[j] = from_float<T>(x1 * c - x2 * s);
    o[j + half] = from_float<T>(x2 * c + x1 * s);
  }
  for (int i = rotary_dim + lane; i < hd; i += 32) {  // elements beyond the rotary part
    float v = to_float(x[i]) * rstd;
    if (w != nullptr) v *= load_as_float(w, w_dtype, i);
    o[i] = from_float<T>(v);
  }
}

// bf16, hd even, rotary_dim a multiple of 4, at most 32 * MAXP pairs per lane region: a lane
// holds its elements as pairs in registers (read once, 4 bytes at a time, written once).  A
// block is one token; its warps walk over the heads (q, then k, then v) with a stride of
// gridDim.y * warps, so with many tokens one warp serves many heads of a token and reads the
// token's angles and the norm weights once, and with few tokens every head has a warp of its own.
template <int MAXP>
__global__ void qknorm_rope_kvwrite_bf16_kernel(
    __nv_bfloat16* __restrict__ qkv, int nh, int nkv, int hd, const void* __restrict__ q_w,
    const void* __restrict__ k_w, int w_dtype, float eps, const float* __restrict__ cos_sin,
    int rotary_dim, int max_pos, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages,
    int page_size, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
    int64_t num_pages, int* __restrict__ status) {
  // Where the token lies, its angles and the weights are read before the wait for the kernels in
  // front of this one: no kernel of the step writes them.
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int n_heads_total = nh + 2 * nkv;
  const bool write_cache = k_pages != nullptr;
  const int head_end = write_cache ? n_heads_total : nh;
  const int head0 = blockIdx.y * warps + (threadIdx.x >> 5);
  if (head0 >= head_end) {
    atom::pdl_wait();
    return;
  }
  const int seq = seq_of_token[t];
  if (seq < 0) {  // a padding row of a fixed-size batch
    atom::pdl_wait();
    return;
  }
  const int pos = positions[t];

  // where this token's keys and values go
  int64_t kv_row = -1;   // row of the page matrices [pages * nkv * page][hd] for kv head 0
  if (write_cache) {
    const int page = block_table[(int64_t)seq * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (lane == 0 && head0 == 0) atomicExch(status, 1);
      if (head0 >= nh) {                // q heads of the token are still rotated
        atom::pdl_wait();
        return;
      }
    } else {
      kv_row = (int64_t)page * nkv * page_size + (pos % page_size);
    }
  }

  const int half = rotary_dim >> 1, hp = half >> 1;      // hp: pairs in one half of the rotary part
  const int tail_pairs = (hd - rotary_dim) >> 1;
  // the token's angles, and the norm weights of this lane's elements (of the kind of head at hand)
  float2 cc[MAXP], sn[MAXP];
  float2 wa[MAXP], wb[MAXP], wc[MAXP];
  const int p = pos < max_pos ? pos : max_pos - 1;  // host checks pos < max_pos
  const float2* cs2 = reinterpret_cast<const float2*>(cos_sin + (int64_t)p * rotary_dim);
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    const int i = lane + 32 * k;
    cc[k] = sn[k] = make_float2(1.f, 0.f);
    if (i < hp) {
      cc[k] = cs2[i];
      sn[k] = cs2[hp + i];
    }
  }
  auto load_weights = [&](const void* w) {
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      const int i = lane + 32 * k;
      wa[k] = wb[k] = wc[k] = make_float2(1.f, 1.f);
      if (w != nullptr && i < hp) {
        wa[k] = make_float2(load_as_float(w, w_dtype, 2 * i), load_as_float(w, w_dtype, 2 * i + 1));
        wb[k] = make_float2(load_as_float(w, w_dtype, 2 * i + half), load_as_float(w, w_dtype, 2 * i + half + 1));
      }
      if (w != nullptr && i < tail_pairs)
        wc[k] = make_float2(load_as_float(w, w_dtype, rotary_dim + 2 * i),
                            load_as_float(w, w_dtype, rotary_dim + 2 * i + 1));
    }
  };
  bool have_q = false, have_k = false;
  if (head0 < nh) {
    load_weights(q_w);
    have_q = true;
  } else if (head0 < nh + nkv) {
    load_weights(k_w);
    have_k = true;
  }
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int stride = gridDim.y * warps;
  for (int head = head0; head < head_end; head += stride) {
    const bool is_q = head < nh;
    const bool is_k = !is_q && head < nh + nkv;
    __nv_bfloat16* x = qkv + ((int64_t)t * n_heads_total + head) * hd;
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(x);
    __nv_bfloat16* dst = nullptr;
    if (!is_q) {
      if (kv_row < 0) break;   // no page for this token (reported above)
      const int kvh = is_k ? head - nh : head - nh - nkv;
      dst = (is_k ? k_pages : v_pages) + (kv_row + (int64_t)kvh * page_size) * hd;
    }
    if (!is_q && !is_k) {  // value head: plain copy
      __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst);
      for (int i = lane; i < hd / 2; i += 32) d2[i] = x2[i];
      continue;
    }
    if (is_q && !have_q) {
      load_weights(q_w);
      have_q = true;
    } else if (is_k && !have_k) {
      load_weights(k_w);
      have_k = true;
    }
    const void* w = is_q ? q_w : k_w;
    float2 a[MAXP], b[MAXP], c[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      const int i = lane + 32 * k;
      a[k] = b[k] = c[k] = make_float2(0.f, 0.f);
      if (i < hp) {
        a[k] = __bfloat1622float2(x2[i]);
        b[k] = __bfloat1622float2(x2[i + hp]);
        ss += a[k].x * a[k].x + a[k].y * a[k].y + b[k].x * b[k].x + b[k].y * b[k].y;
      }
      if (i < tail_pairs) {
        c[k] = __bfloat1622float2(x2[(rotary_dim >> 1) + i]);
        ss += c[k].x * c[k].x + c[k].y * c[k].y;
      }
    }
    float rstd = 1.f;
    if (w != nullptr) {
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)hd + eps);
    }
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(is_q ? x : dst);
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      const int i = lane + 32 * k;
      if (i < hp) {
        const float2 x1 = make_float2(a[k].x * rstd * wa[k].x, a[k].y * rstd * wa[k].y);
        const float2 xb = make_float2(b[k].x * rstd * wb[k].x, b[k].y * rstd * wb[k].y);
        o2[i] = __floats2bfloat162_rn(x1.x * cc[k].x - xb.x * sn[k].x, x1.y * cc[k].y - xb.y * sn[k].y);
        o2[i + hp] = __floats2bfloat162_rn(xb.x * cc[k].x + x1.x * sn[k].x, xb.y * cc[k].y + x1.y * sn[k].y);
      }
      if (i < tail_pairs)
        o2[(rotary_dim >> 1) + i] = __floats2bfloat162_rn(c[k].x * rstd * wc[k].x, c[k].y * rstd * wc[k].y);
    }
  }
}

// bf16, full rotation (rotary_dim == hd), hd = 16 * LPH: LPH lanes share a head, each holding
// 8 consecutive elements of the first half and the 8 they are rotated with in the second half
// (two 16-byte accesses); a warp takes 32 / LPH heads at a time.  A block is one token (128 threads); the
// token's angles and the norm weights are put into shared memory once and read from there for every head.
template <int LPH>
__global__ void __launch_bounds__(128, 8) qknorm_rope_kvwrite_bf16_vec_kernel(
    __nv_bfloat16* __restrict__ qkv, int nh, int nkv, const void* __restrict__ q_w,
    const void* __restrict__ k_w, int w_dtype, float eps, const float* __restrict__ cos_sin, int max_pos,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
    int max_pages, int page_size, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
    int64_t num_pages, int* __restrict__ status) {
  // (what no kernel of the step writes is read before the wait for the kernels in front of this one)
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  constexpr int HD = 16 * LPH, HPW = 32 / LPH;   // heads a warp takes at a time
  const int lane = threadIdx.x & 31, sub = lane / LPH, l = lane % LPH;
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int n_heads_total = nh + 2 * nkv;
  const bool write_cache = k_pages != nullptr;
  const int head_end = write_cache ? n_heads_total : nh;
  const int seq = seq_of_token[t];
  if (seq < 0) {  // a padding row of a fixed-size batch
    atom::pdl_wait();
    return;
  }
  const int pos = positions[t];
  int64_t kv_row = -1;   // row of the page matrices [pages * nkv * page][hd] for kv head 0
  if (write_cache) {
    const int page = block_table[(int64_t)seq * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && blockIdx.y == 0) atomicExch(status, 1);
    } else {
      kv_row = (int64_t)page * nkv * page_size + (pos % page_size);
    }
  }
  // The token's angles and the norm weights wait in shared memory: held in registers over the heads
  // they cost 48 registers a thread, and with 120 registers an SM holds 16 warps of this kernel
  // where 64 registers let it hold 32 (2,048 tokens: 16.1 -> 13.1 us).
  __shared__ __align__(16) float s_cs[HD];        // cos of the HD/2 pairs' angles, then sin
  __shared__ __align__(16) float s_w[2][HD];      // q norm weights, k norm weights (ones without a norm)
  {
    const int p = pos < max_pos ? pos : max_pos - 1;  // host checks pos < max_pos
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
      s_cs[i] = cos_sin[(int64_t)p * HD + i];
      s_w[0][i] = q_w != nullptr ? load_as_float(q_w, w_dtype, i) : 1.f;
      s_w[1][i] = k_w != nullptr ? load_as_float(k_w, w_dtype, i) : 1.f;
    }
  }
  __syncthreads();
  // (read again for every head: "volatile" keeps the compiler from lifting the loads out of the loop)
  auto lds4 = [](const float* ptr, float* out) {
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(ptr)));
  };
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  const int stride = gridDim.y * warps * HPW;
  // every lane of a warp runs the same number of rounds (the shuffles below need all lanes)
  const int warp_head0 = (blockIdx.y * warps + (threadIdx.x >> 5)) * HPW;
  // Three rounds at a time: their loads are all asked for before the first is used, so that enough
  // bytes are in flight per SM.
  constexpr int UNROLL = 3;
  for (int hbase = warp_head0; hbase < head_end; hbase += UNROLL * stride) {
    uint4 lo[UNROLL], hi[UNROLL];
    __nv_bfloat16* dst[UNROLL];
    int kind[UNROLL];   // 0 q, 1 k, 2 v, -1 nothing to do
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int head = hbase + u * stride + sub;
      kind[u] = head >= head_end ? -1 : (head < nh ? 0 : (head < nh + nkv ? 1 : 2));
      if (kind[u] > 0 && kv_row < 0) kind[u] = -1;        // no page for this token (reported above)
      lo[u] = hi[u] = make_uint4(0, 0, 0, 0);
      dst[u] = nullptr;
      if (kind[u] < 0) continue;
      __nv_bfloat16* x = qkv + ((int64_t)t * n_heads_total + head) * HD;
      lo[u] = *reinterpret_cast<const uint4*>(x + 8 * l);
      hi[u] = *reinterpret_cast<const uint4*>(x + HD / 2 + 8 * l);
      dst[u] = x;
      if (kind[u] > 0) {
        const int kvh = kind[u] == 1 ? head - nh : head - nh - nkv;
        dst[u] = (kind[u] == 1 ? k_pages : v_pages) + (kv_row + (int64_t)kvh * page_size) * HD;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float a[8], b[8];
      {
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo[u]);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(l2[j]), fb = __bfloat1622float2(h2[j]);
          a[2 * j] = fa.x, a[2 * j + 1] = fa.y, b[2 * j] = fb.x, b[2 * j + 1] = fb.y;
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a[j] * a[j] + b[j] * b[j];
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // (every lane, whatever its head)
      if (kind[u] < 0) continue;
      if (kind[u] < 2) {
        const bool is_q = kind[u] == 0;
        const void* w = is_q ? q_w : k_w;
        const float rstd = w != nullptr ? rsqrtf(ss / (float)HD + eps) : 1.f;
        __nv_bfloat162* ol2 = reinterpret_cast<__nv_bfloat162*>(&lo[u]);
        __nv_bfloat162* oh2 = reinterpret_cast<__nv_bfloat162*>(&hi[u]);
#pragma unroll
        for (int j = 0; j < 2; ++j) {   // four column pairs at a time
          float c4[4], s4[4], w1[4], w2[4];
          lds4(s_cs + 8 * l + 4 * j, c4);
          lds4(s_cs + HD / 2 + 8 * l + 4 * j, s4);
          lds4(s_w[is_q ? 0 : 1] + 8 * l + 4 * j, w1);
          lds4(s_w[is_q ? 0 : 1] + HD / 2 + 8 * l + 4 * j, w2);
          float y1[4], y2[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = 4 * j + e;
            const float x1 = a[i] * rstd * w1[e];
            const float x2 = b[i] * rstd * w2[e];
            y1[e] = x1 * c4[e] - x2 * s4[e];
            y2[e] = x2 * c4[e] + x1 * s4[e];
          }
          ol2[2 * j] = __floats2bfloat162_rn(y1[0], y1[1]);
          ol2[2 * j + 1] = __floats2bfloat162_rn(y1[2], y1[3]);
          oh2[2 * j] = __floats2bfloat162_rn(y2[0], y2[1]);
          oh2[2 * j + 1] = __floats2bfloat162_rn(y2[2], y2[3]);
        }
      }
      *reinterpret_cast<uint4*>(dst[u] + 8 * l) = lo[u];
      *reinterpret_cast<uint4*>(dst[u] + HD / 2 + 8 * l) = hi[u];
    }
  }
}

// Per-head RMSNorm of the query and key heads in place, nothing else: for a mixer whose position
// encoding is not a table of angles and runs between the norm and the cache write.
template <typename T>
__global__ void qk_headnorm_kernel(T* __restrict__ qkv, int nh, int nkv, int hd, const void* __restrict__ q_w,
                                   const void* __restrict__ k_w, int w_dtype, float eps,
                                   const int* __restrict__ seq_of_token) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= nh + nkv || seq_of_token[t] < 0) return;
  const void* w = head < nh ? q_w : k_w;
  T* x = qkv + ((int64_t)t * (nh + 2 * nkv) + head) * hd;
  float ss = 0.f;
  for (int i = lane; i < hd; i += 32) {
    const float v = to_float(x[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)hd + eps);
  for (int i = lane; i < hd; i += 32) x[i] = from_float<T>(to_float(x[i]) * rstd * load_as_float(w, w_dtype, i));
}

}  // namespace atom

// qkv: [T, (nh + 2 nkv) * hd] of `dtype`, q part rewritten in place.
// k_pages / v_pages may be null: then only q is processed (a layer that reads another
// layer's cache).  q_w / k_w may be null: no per-head norm.  `status` is a device int that
// is set to 1 if a token's position has no page.
ATOM_EXPORT int atom_qknorm_rope_kvwrite(void* qkv, int dtype, int T, int nh, int nkv, int hd,
                                         const void* q_w, const void* k_w, int w_dtype, float eps,
                                         const float* cos_sin, int rotary_dim, int max_pos,
                                         const int* positions, const int* seq_of_token,
                                         const int* block_table, int max_pages, int page_size,
                                         void* k_pages, void* v_pages, int64_t num_pages,
                                         int* status, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1) ||
      page_size <= 0 || (rotary_dim > 0 && (cos_sin == nullptr || max_pos <= 0)) ||
      ((k_pages == nullptr) != (v_pages == nullptr)))
    return ATOM_ERR_ARG;
  const int warps = 4;
  dim3 grid(T, (nh + 2 * nkv + warps - 1) / warps);
  if (dtype == ATOM_F32) {
    atom::launch_pdl(atom::qknorm_rope_kvwrite_kernel<float>, dim3(grid), dim3(warps * 32), 0, stream, (float*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, cos_sin, rotary_dim, max_pos, positions,
        seq_of_token, block_table, max_pages, page_size, (float*)k_pages, (float*)v_pages,
        num_pages, status);
  } else if (dtype == ATOM_BF16 && hd % 2 == 0 && hd <= 512 && rotary_dim % 4 == 0 && (hd - rotary_dim) <= 256 &&
             (uintptr_t)qkv % 4 == 0 && (uintptr_t)k_pages % 4 == 0 && (uintptr_t)v_pages % 4 == 0 &&
             (uintptr_t)cos_sin % 8 == 0) {
    // (with few tokens the kernel below, a warp per head, is done sooner: measured 2.8 against 3.8 us at 8 tokens)
    const bool vec_ok = T >= 128 && rotary_dim == hd && (hd == 64 || hd == 128 || hd == 256) && (uintptr_t)qkv % 16 == 0 &&
                        (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 && (uintptr_t)cos_sin % 16 == 0 &&
                        (uintptr_t)q_w % 16 == 0 && (uintptr_t)k_w % 16 == 0;
    if (vec_ok) {
      // a warp takes 32 / (hd / 16) heads at a time; few tokens: one round per warp; many: about 2048 blocks
      const int hpw = 32 / (hd / 16);
      int gy = (nh + 2 * nkv + warps * hpw - 1) / (warps * hpw);
      while (gy > 1 && (int64_t)T * gy > 2048) gy = (gy + 1) / 2;
      dim3 g3(T, gy);
#define ATOM_ROPE_VEC(LPH)                                                                                          \
  atom::launch_pdl(atom::qknorm_rope_kvwrite_bf16_vec_kernel<LPH>, dim3(g3), dim3(warps * 32), 0, stream,           \
                   (__nv_bfloat16*)qkv, nh, nkv, q_w, k_w, w_dtype, eps, cos_sin, max_pos, positions, seq_of_token, \
                   block_table, max_pages, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages,  \
                   status)
      if (hd == 64) ATOM_ROPE_VEC(4);
      else if (hd == 128) ATOM_ROPE_VEC(8);
      else ATOM_ROPE_VEC(16);
#undef ATOM_ROPE_VEC
      return atom::check_launch();
    }
    // Few tokens: a warp per head.  Many tokens: fewer, longer-lived warps per token (about two thousand blocks),
    // each serving several heads with the token's angles and the weights in registers.
    const int per_head = (nh + 2 * nkv + warps - 1) / warps;
    int gy = per_head;
    while (gy > 1 && (int64_t)T * gy > 2048) gy = (gy + 1) / 2;
    dim3 g2(T, gy);
    // pairs a lane must hold: of one half of the rotary part, and of the part that is not rotated
    const int need = (rotary_dim / 4 > (hd - rotary_dim) / 2) ? rotary_dim / 4 : (hd - rotary_dim) / 2;
#define ATOM_ROPE_LAUNCH(MAXP)                                                                                     \
  atom::launch_pdl(atom::qknorm_rope_kvwrite_bf16_kernel<MAXP>, dim3(g2), dim3(warps * 32), 0, stream,             \
                   (__nv_bfloat16*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, cos_sin, rotary_dim, max_pos,         \
                   positions, seq_of_token, block_table, max_pages, page_size, (__nv_bfloat16*)k_pages,            \
                   (__nv_bfloat16*)v_pages, num_pages, status)
    if (need <= 32) ATOM_ROPE_LAUNCH(1);
    else if (need <= 64) ATOM_ROPE_LAUNCH(2);
    else ATOM_ROPE_LAUNCH(4);
#undef ATOM_ROPE_LAUNCH
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::qknorm_rope_kvwrite_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, (__nv_bfloat16*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, cos_sin, rotary_dim, max_pos,
        positions, seq_of_token, block_table, max_pages, page_size, (__nv_bfloat16*)k_pages,
        (__nv_bfloat16*)v_pages, num_pages, status);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}

// Per-head RMSNorm of the q and k heads of qkv [T, (nh + 2 nkv) * hd] in place (v untouched, no rotation,
// no cache write).
ATOM_EXPORT int atom_qk_headnorm(void* qkv, int dtype, int T, int nh, int nkv, int hd, const void* q_w,
                                 const void* k_w, int w_dtype, float eps, const int* seq_of_token,
                                 cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || q_w == nullptr || k_w == nullptr) return ATOM_ERR_ARG;
  const int warps = 4;
  dim3 grid(T, (nh + nkv + warps - 1) / warps);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::qk_headnorm_kernel<float>, grid, dim3(warps * 32), 0, stream, (float*)qkv, nh, nkv, hd,
                     q_w, k_w, w_dtype, eps, seq_of_token);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::qk_headnorm_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream,
                     (__nv_bfloat16*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, seq_of_token);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
