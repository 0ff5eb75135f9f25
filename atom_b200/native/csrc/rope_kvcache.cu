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
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  atom::pdl_trigger();   // the next kernel may be scheduled (it waits in the same way)
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

// bf16, hd even and at most 512, rotary_dim a multiple of 4: a lane holds its elements as
// pairs in registers (read once, 4 bytes at a time, written once).
__global__ void qknorm_rope_kvwrite_bf16_kernel(
    __nv_bfloat16* __restrict__ qkv, int nh, int nkv, int hd, const void* __restrict__ q_w,
    const void* __restrict__ k_w, int w_dtype, float eps, const float* __restrict__ cos_sin,
    int rotary_dim, int max_pos, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages,
    int page_size, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
    int64_t num_pages, int* __restrict__ status) {
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  atom::pdl_trigger();   // the next kernel may be scheduled (it waits in the same way)
  constexpr int MAXP = 4;   // pairs per lane and region: hd <= 512
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
  if (seq < 0) return;  // a padding row of a fixed-size batch

  __nv_bfloat16* x = qkv + ((int64_t)t * n_heads_total + head) * hd;
  const int pos = positions[t];
  __nv_bfloat16* dst = nullptr;
  if (!is_q) {
    const int page = block_table[(int64_t)seq * max_pages + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicExch(status, 1);
      return;
    }
    const int kvh = is_k ? head - nh : head - nh - nkv;
    __nv_bfloat16* base = is_k ? k_pages : v_pages;
    dst = base + (((int64_t)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
  }
  const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(x);
  if (!is_q && !is_k) {  // value head: plain copy
    __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst);
    for (int i = lane; i < hd / 2; i += 32) d2[i] = x2[i];
    return;
  }
  const int half = rotary_dim >> 1, hp = half >> 1;      // hp: pairs in one half of the rotary part
  const int tail_pairs = (hd - rotary_dim) >> 1;
  float2 a[MAXP], b[MAXP], c[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    const int i = lane + 32 * k;
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
  const void* w = is_q ? q_w : k_w;
  float rstd = 1.f;
  if (w != nullptr) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / (float)hd + eps);
  }
  const int p = pos < max_pos ? pos : max_pos - 1;  // host checks pos < max_pos
  const float2* cs2 = reinterpret_cast<const float2*>(cos_sin + (int64_t)p * rotary_dim);
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(is_q ? x : dst);
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    const int i = lane + 32 * k;
    if (i < hp) {
      float2 x1 = make_float2(a[k].x * rstd, a[k].y * rstd), xb = make_float2(b[k].x * rstd, b[k].y * rstd);
      if (w != nullptr) {
        x1.x *= load_as_float(w, w_dtype, 2 * i);
        x1.y *= load_as_float(w, w_dtype, 2 * i + 1);
        xb.x *= load_as_float(w, w_dtype, 2 * i + half);
        xb.y *= load_as_float(w, w_dtype, 2 * i + half + 1);
      }
      const float2 cc = cs2[i], sn = cs2[hp + i];
      o2[i] = __floats2bfloat162_rn(x1.x * cc.x - xb.x * sn.x, x1.y * cc.y - xb.y * sn.y);
      o2[i + hp] = __floats2bfloat162_rn(xb.x * cc.x + x1.x * sn.x, xb.y * cc.y + x1.y * sn.y);
    }
    if (i < tail_pairs) {
      float2 v = make_float2(c[k].x * rstd, c[k].y * rstd);
      if (w != nullptr) {
        v.x *= load_as_float(w, w_dtype, rotary_dim + 2 * i);
        v.y *= load_as_float(w, w_dtype, rotary_dim + 2 * i + 1);
      }
      o2[(rotary_dim >> 1) + i] = __floats2bfloat162_rn(v.x, v.y);
    }
  }
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
  } else if (dtype == ATOM_BF16 && hd % 2 == 0 && hd <= 512 && rotary_dim % 4 == 0 &&
             (uintptr_t)qkv % 4 == 0 && (uintptr_t)k_pages % 4 == 0 && (uintptr_t)v_pages % 4 == 0 &&
             (uintptr_t)cos_sin % 8 == 0) {
    atom::launch_pdl(atom::qknorm_rope_kvwrite_bf16_kernel, dim3(grid), dim3(warps * 32), 0, stream, (__nv_bfloat16*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, cos_sin, rotary_dim, max_pos, positions,
        seq_of_token, block_table, max_pages, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages,
        num_pages, status);
  } else if (dtype == ATOM_BF16) {
    atom::launch_pdl(atom::qknorm_rope_kvwrite_kernel<__nv_bfloat16>, dim3(grid), dim3(warps * 32), 0, stream, (__nv_bfloat16*)qkv, nh, nkv, hd, q_w, k_w, w_dtype, eps, cos_sin, rotary_dim, max_pos,
        positions, seq_of_token, block_table, max_pages, page_size, (__nv_bfloat16*)k_pages,
        (__nv_bfloat16*)v_pages, num_pages, status);
  } else {
    return ATOM_ERR_ARG;
  }
  return atom::check_launch();
}
