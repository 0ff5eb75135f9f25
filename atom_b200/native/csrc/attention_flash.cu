// Paged causal attention on the tensor cores (bf16 operands, 32-bit softmax and accumulation),
// for one head size fixed at compile time (-DATOM_HD=<multiple of 16, at most 256>).
//
// A step's batch holds, per request s, q_len(s) new tokens at positions
// [ctx_len(s) - q_len(s), ctx_len(s)); their keys and values are already in the pages.  Query
// rows of the G = nh / nkv heads that share one kv head are packed into one tile
// (row = token * G + head in group), so a tile reads each key once for all G heads.
//
//   portions (more than 16 packed rows): one CTA = 64 rows of one (request, kv head); its 4
//       warps take 16 rows each and walk over the keys in tiles of 64.
//   short (at most 16 packed rows: decoded tokens, portions of a few tokens): one CTA = one
//       (request, kv head, split of the keys); its 4 warps take 16 keys each of every tile of
//       64 and are merged at the end.  With more than one split the CTA writes unnormalised
//       partial sums with their maximum and denominator to scratch, and a second kernel
//       merges the splits.
//
// Keys of a tile come into shared memory with cp.async (rows beyond the request's length, or
// on pages a window has given back, are zero-filled), in a ring of stages; S = Q K^T and
// O += P V run on mma.sync.m16n8k16 with P rounded to bf16.
//
// Where the head size is a multiple of 64 and a page holds a power of two >= 8 of tokens, short
// requests run on another kernel (flash_decode_tma_kernel): pages come as TMA boxes (a warp's
// own cp.async stream carries ~2.5 bytes a clock, far less than the memory system gives a CTA),
// and the products are transposed, S^T = K Q^T and O^T = V^T P^T, so that the 16-wide side of
// the instruction runs over keys and the 8-wide side over the few query rows.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "tma.cuh"

#ifndef ATOM_HD
#error "compile with -DATOM_HD=<head size>"
#endif

namespace atom {
namespace flash {

constexpr int HD = ATOM_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16, at most 256");
constexpr int LDS = HD + 8;   // shared-memory row stride in elements: rows shift by one 16-byte bank group
constexpr int BN = 64;        // keys per tile
constexpr int BM = 64;        // packed query rows per CTA (portions)
constexpr int NT = 128;       // threads per CTA
constexpr int CH = HD / 8;    // 16-byte chunks per row
constexpr bool Q_IN_REGS = HD <= 128;

struct Params {
  __nv_bfloat16* out;          // [T, nh * HD]
  const __nv_bfloat16* q;      // token t, head h at q + t * q_stride + h * HD
  int64_t q_stride;
  const __nv_bfloat16* k_pages;  // [pages, nkv, page_size, HD]
  const __nv_bfloat16* v_pages;
  const int* block_table;      // [S, max_pages]
  int max_pages, page_size, page_shift;   // page_shift >= 0 when page_size is a power of two
  const int* cu_q;             // [S + 1]
  const int* ctx_len;          // [S] tokens of the request in the cache after this step
  int num_seqs, nh, nkv, group;
  float scale_log2;            // scale * log2(e)
  int window;                  // <= 0: all keys
  int num_splits;
  float* part_o;               // [T, nh, num_splits, HD]
  float* part_ml;              // [T, nh, num_splits, 2]
  int* error;                  // device flag raised when a bounded wait ran out
  int long_rows;               // requests with at least this many packed rows go to the tcgen05 kernel
  // A decode step (one new token per request) may leave the per-head norm, the rotation and the cache write
  // of its new tokens to the TMA decode kernel: q then points at the raw projection [q | k | v] of a token.
  const float* rot_table;      // [max_pos, rotary_dim] cos of every pair's angle, then sin; null: q and the cache are ready
  const int* rot_rows;         // [T] table row of every token
  int rotary_dim, rot_max_pos;
  const void* q_norm_w;        // [HD] or null
  const void* k_norm_w;
  int norm_w_dtype;
  float norm_eps;
  __nv_bfloat16* k_write;      // the pages again, to be written (null: this call writes no cache)
  __nv_bfloat16* v_write;
  int64_t num_pages;
  int* status;                 // set when a new token has no page
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// What one CTA works on.
struct Work {
  int seq, kvh;
  int q_begin;        // first token row of the request in the batch
  int q_start;        // position of the request's first new token
  int rows_total;     // q_len * group
  int row0;           // first packed row of this CTA
  int ctx;            // ctx_len
  const int* bt;
};

// Copies keys and values [tile * BN, tile * BN + BN) of the request into one stage.
// Consecutive threads take consecutive 16-byte chunks of a row (whole 128-byte lines per
// request); a thread's rows are row0, row0 + NT / CH, ...  Offsets are formed in units of 16
// bytes in 32-bit arithmetic (a layer's pages stay below 64 GB).
__device__ __forceinline__ void load_kv_tile(const Params& p, const Work& w, int tile, int key_end,
                                             __nv_bfloat16* sK, __nv_bfloat16* sV) {
  constexpr int ROWS_PER_PASS = NT / CH > 0 ? NT / CH : 1;   // rows covered by one pass of the CTA
  const uint32_t head_stride = (uint32_t)p.page_size * CH;           // 16-byte units
  const uint32_t page_stride = head_stride * (uint32_t)p.nkv;
  const uint4* kp = reinterpret_cast<const uint4*>(p.k_pages);
  const uint4* vp = reinterpret_cast<const uint4*>(p.v_pages);
  if (NT % CH == 0) {
    const int ch = threadIdx.x % CH, row0 = threadIdx.x / CH;
    const uint32_t fixed = (uint32_t)w.kvh * head_stride + ch;
    const int soff = ch * 8;
#pragma unroll
    for (int i = 0; i < BN / ROWS_PER_PASS; ++i) {
      const int row = row0 + i * ROWS_PER_PASS;
      const int j = tile * BN + row;
      bool valid = j < key_end;
      uint32_t off = 0;
      if (valid) {
        const int lp = p.page_shift >= 0 ? (j >> p.page_shift) : (j / p.page_size);
        const int in_page = j - lp * p.page_size;
        const int page = w.bt[lp];
        valid = page >= 0;
        if (valid) off = (uint32_t)page * page_stride + (uint32_t)in_page * CH + fixed;
      }
      cp_async16(sK + row * LDS + soff, kp + off, valid);
      cp_async16(sV + row * LDS + soff, vp + off, valid);
    }
  } else {
    for (int c = threadIdx.x; c < BN * CH; c += NT) {
      const int row = c / CH, ch = c % CH;
      const int j = tile * BN + row;
      bool valid = j < key_end;
      uint32_t off = 0;
      if (valid) {
        const int lp = p.page_shift >= 0 ? (j >> p.page_shift) : (j / p.page_size);
        const int in_page = j - lp * p.page_size;
        const int page = w.bt[lp];
        valid = page >= 0;
        if (valid) off = (uint32_t)page * page_stride + (uint32_t)w.kvh * head_stride + (uint32_t)in_page * CH + ch;
      }
      cp_async16(sK + row * LDS + ch * 8, kp + off, valid);
      cp_async16(sV + row * LDS + ch * 8, vp + off, valid);
    }
  }
}

// Copies ROWS packed query rows starting at w.row0 into shared memory (zero beyond the last).
template <int ROWS>
__device__ __forceinline__ void load_q_tile(const Params& p, const Work& w, __nv_bfloat16* sQ) {
  for (int c = threadIdx.x; c < ROWS * CH; c += NT) {
    const int row = c / CH, ch = c % CH;
    const int R = w.row0 + row;
    const bool valid = R < w.rows_total;
    int64_t off = 0;
    if (valid) {
      const int tok = R / p.group, hig = R - tok * p.group;
      off = (int64_t)(w.q_begin + tok) * p.q_stride + (int64_t)(w.kvh * p.group + hig) * HD + ch * 8;
    }
    cp_async16(sQ + row * LDS + ch * 8, p.q + off, valid);
  }
}

// Per-warp running state of 16 query rows: this thread holds rows g and g + 8.
struct Acc {
  float o[HD / 8][4];
  float m[2], l[2];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// One tile step of a warp: 16 query rows (fragments in qf or read from sQ) against KT * 8
// keys starting at row `kw` of the stage.  pos0 / pos1: positions of the thread's two rows
// (-1: row does not exist).  key0: index of the stage's first key.
template <int KT>
__device__ __forceinline__ void warp_tile(Acc& acc, uint32_t (*qf)[4], const __nv_bfloat16* sQw,
                                          const __nv_bfloat16* sK, const __nv_bfloat16* sV, int kw,
                                          int key0, int pos0, int pos1, int window, float c, bool mask) {
  const int lane = threadIdx.x & 31;
  float s[KT][4];
#pragma unroll
  for (int i = 0; i < KT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;

  // S = Q K^T
  {
    const int mat = lane >> 3, r8 = lane & 7;
    const __nv_bfloat16* kbase = sK + (kw + (mat >> 1) * 8 + r8) * LDS + (mat & 1) * 8;
    const __nv_bfloat16* qbase = sQw + ((mat & 1) * 8 + r8) * LDS + (mat >> 1) * 8;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4];
      if (Q_IN_REGS) {
        a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3];
      } else {
        ldmatrix_x4(a, qbase + ks * 16);
      }
#pragma unroll
      for (int n2 = 0; n2 < KT / 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4(b, kbase + n2 * 16 * LDS + ks * 16);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }
  }

  // mask
  if (mask) {
    const int t4 = lane & 3;
#pragma unroll
    for (int n = 0; n < KT; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = key0 + kw + n * 8 + 2 * t4 + (e & 1);
        const int pos = (e < 2) ? pos0 : pos1;
        bool ok = j <= pos;
        if (window > 0) ok = ok && (j > pos - window);
        if (!ok) s[n][e] = -INFINITY;
      }
    }
  }

  // online softmax
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float mx = -INFINITY;
#pragma unroll
    for (int n = 0; n < KT; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * r], s[n][2 * r + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(acc.m[r], mx);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float corr = exp2f((acc.m[r] - m_use) * c);
    acc.m[r] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int n = 0; n < KT; ++n) {
      const float p0 = exp2f((s[n][2 * r] - m_use) * c);
      const float p1 = exp2f((s[n][2 * r + 1] - m_use) * c);
      s[n][2 * r] = p0;
      s[n][2 * r + 1] = p1;
      sum += p0 + p1;
    }
    acc.l[r] = acc.l[r] * corr + sum;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      acc.o[d][2 * r] *= corr;
      acc.o[d][2 * r + 1] *= corr;
    }
  }

  // O += P V
  {
    const int mat = lane >> 3, r8 = lane & 7;
    const __nv_bfloat16* vbase = sV + (kw + (mat & 1) * 8 + r8) * LDS + (mat >> 1) * 8;
#pragma unroll
    for (int kk = 0; kk < KT / 2; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < HD / 16; ++d2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vbase + kk * 16 * LDS + d2 * 16);
        mma_bf16(acc.o[2 * d2], a, b[0], b[1]);
        mma_bf16(acc.o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
  }
}

__device__ __forceinline__ void load_q_frags(uint32_t (*qf)[4], const __nv_bfloat16* sQw) {
  const int lane = threadIdx.x & 31;
  const int mat = lane >> 3, r8 = lane & 7;
  const __nv_bfloat16* qbase = sQw + ((mat & 1) * 8 + r8) * LDS + (mat >> 1) * 8;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], qbase + ks * 16);
}

// ------------------------------------------------------------------ portions

constexpr int PREFILL_STAGES = 2;
constexpr size_t prefill_smem_bytes() {
  return sizeof(__nv_bfloat16) * (size_t)(BM * LDS + PREFILL_STAGES * 2 * BN * LDS);
}

__global__ void __launch_bounds__(NT) flash_prefill_kernel(const Params p) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sKV = sQ + BM * LDS;

  // Which (request, row tile) is this CTA?  Requests with at most 16 packed rows belong to
  // the other kernel.  Within a request the last (longest) tiles come first.
  Work w;
  {
    int tile = blockIdx.y, s = 0, nt = 0;   // (blocks are handed out with x fastest: all kv heads of the longest tile first)
    for (; s < p.num_seqs; ++s) {
      const int rows = (p.cu_q[s + 1] - p.cu_q[s]) * p.group;
      nt = (rows > 16 && rows < p.long_rows) ? (rows + BM - 1) / BM : 0;
      if (tile < nt) break;
      tile -= nt;
    }
    if (s == p.num_seqs) return;
    w.seq = s;
    w.kvh = blockIdx.x;
    w.q_begin = p.cu_q[s];
    const int q_len = p.cu_q[s + 1] - w.q_begin;
    w.ctx = p.ctx_len[s];
    w.q_start = w.ctx - q_len;
    w.rows_total = q_len * p.group;
    w.row0 = (nt - 1 - tile) * BM;
    w.bt = p.block_table + (int64_t)s * p.max_pages;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2;

  const int row_last = min(w.row0 + BM, w.rows_total) - 1;
  const int pos_first = w.q_start + w.row0 / p.group;
  const int pos_last = w.q_start + row_last / p.group;
  const int key_end = pos_last + 1;
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, pos_first - p.window + 1);
  const int tile_begin = key_lo / BN, tile_end = (key_end + BN - 1) / BN;

  load_q_tile<BM>(p, w, sQ);
  load_kv_tile(p, w, tile_begin, key_end, sKV, sKV + BN * LDS);
  cp_async_commit();

  const int R0 = w.row0 + warp * 16 + g, R1 = R0 + 8;
  const int pos0 = R0 < w.rows_total ? w.q_start + R0 / p.group : -1;
  const int pos1 = R1 < w.rows_total ? w.q_start + R1 / p.group : -1;
  // Positions of this warp's first and last row decide which tiles need the mask.
  const int wr_first = w.row0 + warp * 16, wr_last = min(wr_first + 15, w.rows_total - 1);
  const int wpos_first = w.q_start + wr_first / p.group;
  const int wpos_last = w.q_start + max(wr_last, wr_first) / p.group;
  const bool warp_has_rows = wr_first < w.rows_total;

  Acc acc;
  acc.init();
  uint32_t qf[Q_IN_REGS ? HD / 16 : 1][4];
  const __nv_bfloat16* sQw = sQ + warp * 16 * LDS;

  for (int t = tile_begin; t < tile_end; ++t) {
    const int st = (t - tile_begin) & 1;
    __nv_bfloat16* sK = sKV + st * 2 * BN * LDS;
    __nv_bfloat16* sV = sK + BN * LDS;
    cp_async_wait<0>();
    __syncthreads();
    if (t + 1 < tile_end) {
      __nv_bfloat16* nK = sKV + (st ^ 1) * 2 * BN * LDS;
      load_kv_tile(p, w, t + 1, key_end, nK, nK + BN * LDS);
    }
    cp_async_commit();
    if (t == tile_begin && Q_IN_REGS) load_q_frags(qf, sQw);
    const int key0 = t * BN;
    // Skip tiles that lie wholly after this warp's last position (another warp needs them).
    if (!warp_has_rows || key0 > wpos_last) continue;
    bool mask = (key0 + BN - 1 > wpos_first) || !(wr_first + 15 < w.rows_total);
    if (p.window > 0) mask = mask || (key0 <= wpos_last - p.window);
    warp_tile<BN / 8>(acc, qf, sQw, sK, sV, 0, key0, pos0, pos1, p.window, p.scale_log2, mask);
  }
  cp_async_wait<0>();

  // normalise and write
  const int t4 = lane & 3;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = acc.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int R = r == 0 ? R0 : R1;
    if (R >= w.rows_total) continue;
    const float inv = 1.f / l;
    const int tok = R / p.group, hig = R - tok * p.group;
    __nv_bfloat16* orow = p.out + ((int64_t)(w.q_begin + tok) * p.nh + (w.kvh * p.group + hig)) * HD;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      *reinterpret_cast<__nv_bfloat162*>(orow + d * 8 + 2 * t4) =
          __floats2bfloat162_rn(acc.o[d][2 * r] * inv, acc.o[d][2 * r + 1] * inv);
    }
  }
}

// ------------------------------------------------------------------ short requests (decode)

// Combines the four warps' partial results (each saw other keys) that lie in shared memory,
// mo[warp][16 rows][MLD], mm / ml [warp][16], and writes the result or this split's partial sums.
constexpr int MLD = HD + 8;   // padded row: conflict-free fragment stores
__device__ __forceinline__ void decode_combine(const Params& p, const Work& w, int split, const float* mo,
                                               const float* mm, const float* ml) {
  for (int idx = threadIdx.x; idx < w.rows_total * HD; idx += NT) {
    const int row = idx / HD, d = idx - row * HD;
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) M = fmaxf(M, mm[k * 16 + row]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float f = exp2f((mm[k * 16 + row] - Mu) * p.scale_log2);
      L += ml[k * 16 + row] * f;
      O += mo[(k * 16 + row) * MLD + d] * f;
    }
    const int tok = row / p.group, hig = row - tok * p.group;
    const int64_t th = (int64_t)(w.q_begin + tok) * p.nh + (w.kvh * p.group + hig);
    if (p.num_splits == 1) {
      p.out[th * HD + d] = __float2bfloat16_rn(O / L);
    } else {
      p.part_o[(th * p.num_splits + split) * HD + d] = O;
      if (d == 0) {
        p.part_ml[(th * p.num_splits + split) * 2] = M;
        p.part_ml[(th * p.num_splits + split) * 2 + 1] = L;
      }
    }
  }
}


constexpr int DECODE_STAGES = 3;
constexpr size_t decode_smem_bytes() {
  const size_t ring = sizeof(__nv_bfloat16) * (size_t)(16 * LDS + DECODE_STAGES * 2 * BN * LDS);
  const size_t merge = sizeof(float) * (size_t)(4 * 16 * (HD + 8 + 2));
  return ring > merge ? ring : merge;
}

__global__ void __launch_bounds__(NT, 2) flash_decode_kernel(const Params p) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  atom::pdl_wait();      // inputs written by the kernel before this one are visible from here on
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sKV = sQ + 16 * LDS;

  Work w;
  w.seq = blockIdx.x;
  w.kvh = blockIdx.y;
  const int split = blockIdx.z;
  w.q_begin = p.cu_q[w.seq];
  const int q_len = p.cu_q[w.seq + 1] - w.q_begin;
  w.rows_total = q_len * p.group;
  if (w.rows_total <= 0 || w.rows_total > 16) return;
  w.ctx = p.ctx_len[w.seq];
  w.q_start = w.ctx - q_len;
  w.row0 = 0;
  w.bt = p.block_table + (int64_t)w.seq * p.max_pages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int key_end = w.ctx;
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, w.q_start - p.window + 1);
  const int first_tile = key_lo / BN, n_tiles = (key_end + BN - 1) / BN - first_tile;
  const int per_split = (n_tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(tile_begin + per_split, first_tile + n_tiles);

  const int pos0 = g < w.rows_total ? w.q_start + g / p.group : -1;
  const int pos1 = g + 8 < w.rows_total ? w.q_start + (g + 8) / p.group : -1;

  Acc acc;
  acc.init();
  if (tile_begin < tile_end) {
    load_q_tile<16>(p, w, sQ);
#pragma unroll
    for (int i = 0; i < DECODE_STAGES - 1; ++i) {
      if (tile_begin + i < tile_end) {
        __nv_bfloat16* sK = sKV + i * 2 * BN * LDS;
        load_kv_tile(p, w, tile_begin + i, key_end, sK, sK + BN * LDS);
      }
      cp_async_commit();
    }
    uint32_t qf[Q_IN_REGS ? HD / 16 : 1][4];
    for (int t = tile_begin; t < tile_end; ++t) {
      const int st = (t - tile_begin) % DECODE_STAGES;
      __nv_bfloat16* sK = sKV + st * 2 * BN * LDS;
      __nv_bfloat16* sV = sK + BN * LDS;
      cp_async_wait<DECODE_STAGES - 2>();
      __syncthreads();
      const int nx = t + DECODE_STAGES - 1;
      if (nx < tile_end) {
        __nv_bfloat16* nK = sKV + ((nx - tile_begin) % DECODE_STAGES) * 2 * BN * LDS;
        load_kv_tile(p, w, nx, key_end, nK, nK + BN * LDS);
      }
      cp_async_commit();
      if (t == tile_begin && Q_IN_REGS) load_q_frags(qf, sQ);
      // The mask is needed where a key of the warp's 16 may lie after the first new token, or
      // before the window of the last one.
      const int kfirst = t * BN + warp * 16;
      bool mask = kfirst + 15 > w.q_start;
      if (p.window > 0) mask = mask || (kfirst <= w.ctx - 1 - p.window);
      warp_tile<2>(acc, qf, sQ, sK, sV, warp * 16, t * BN, pos0, pos1, p.window, p.scale_log2, mask);
    }
    cp_async_wait<0>();
  }
  __syncthreads();   // the ring is free: it becomes the merge buffer

  // Merge the four warps (each saw other keys).
  float* mo = reinterpret_cast<float*>(smem_raw);       // [4][16][MLD]
  float* mm = mo + 4 * 16 * MLD;                         // [4][16]
  float* ml = mm + 4 * 16;                               // [4][16]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = acc.l[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = g + 8 * r;
    if (t4 == 0) {
      mm[warp * 16 + row] = acc.m[r];
      ml[warp * 16 + row] = l;
    }
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      float2 v = make_float2(acc.o[d][2 * r], acc.o[d][2 * r + 1]);
      *reinterpret_cast<float2*>(mo + (warp * 16 + row) * MLD + d * 8 + 2 * t4) = v;
    }
  }
  __syncthreads();
  decode_combine(p, w, split, mo, mm, ml);
}

#if ATOM_HD % 64 == 0
// ------------------------------------------------------------------ short requests, TMA and transposed products
//
// Every warp works alone: it takes tiles w, w + 4, ... (KTW keys each) of the CTA's keys through a
// ring of its own (RING stages, one mbarrier each), and refills a stage itself as soon as it has
// left it, so there is no CTA-wide barrier in the loop and a warp only ever waits for a phase
// that it started itself.  (With a ring shared by the warps a warp could run two phases ahead of
// a stage whose earlier tile belongs to another warp, which a parity wait cannot tell apart.)
// A stage holds its keys as boxes of min(page, KTW) keys (one page, or a piece of a larger one),
// each box laid out [64-column half][key][64 columns] with the 128-byte swizzle.  Lane
// l < 2 * boxes issues box l / 2 of K (l even) or V (l odd), with the page looked up one tile
// ahead.  Every box is always issued, so a stage always receives the same number of bytes: a box
// past the request's end, or on a page that a window gave back, is read from the request's last
// page instead and masked like any key outside the causal range (the cache holds finite numbers
// everywhere, so 0 * V is 0).
//
// Launched with programmatic stream serialization, the kernel asks for the pages that hold only
// earlier steps' keys before it waits for the kernels in front of it: within a step the cache
// receives only that step's new keys and values.
//
// A warp's tile: S^T[KTW keys, 8 NQ rows] = K Q^T (A = K from ldmatrix, B = Q^T held in
// registers; two accumulators over the head size to shorten the dependent chain), softmax down
// the key axis (a thread holds keys g, g + 8 of each 16 for columns 2 t4, 2 t4 + 1; the maximum
// goes over the lanes of equal t4, the denominator stays a per-thread partial sum until the
// end), P^T to bf16 and through movmatrix into B fragments, and O^T[HD, 8 NQ] += V^T P^T
// (A = V^T from ldmatrix.trans).
//
// KTW, the keys of a warp's tile, is 16 or 32: with 16 two CTAs share an SM, which overlaps one
// CTA's start and end with the other's loads (better for grids of several waves); with 32 the
// per-tile costs are spread over more keys (better where every CTA has an SM to itself).
constexpr int RING = 3;                    // stages of a warp's ring
__host__ __device__ constexpr int tma_stage_bytes(int ktw) { return 2 * ktw * HD * 2; }
constexpr size_t decode_tma_smem_bytes(int ktw) {
  const size_t ring = 1024 + (size_t)4 * RING * tma_stage_bytes(ktw) + sizeof(__nv_bfloat16) * 16 * LDS +
                      sizeof(uint64_t) * 4 * RING;
  const size_t merge = sizeof(float) * (size_t)(4 * 16 * (MLD + 2));
  return ring > merge ? ring : merge;
}
constexpr bool decode_tma_fits(int ktw) { return decode_tma_smem_bytes(ktw) <= 227 * 1024; }
// CTAs that share an SM
constexpr int decode_tma_ctas(int ktw) { return decode_tma_smem_bytes(ktw) + 1024 <= (227 * 1024) / 2 ? 2 : 1; }
static_assert(decode_tma_fits(16), "the rings must fit an SM");

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

// Running state of a warp over NQ * 8 query rows, transposed: o[dm][nq] is the C fragment of
// O^T rows dm * 16 + {g, g + 8}, columns nq * 8 + {2 t4, 2 t4 + 1}.
template <int NQ>
struct AccT {
  float o[HD / 16][NQ][4];
  float m[NQ][2], l[NQ][2];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < HD / 16; ++i)
#pragma unroll
      for (int n = 0; n < NQ; ++n) o[i][n][0] = o[i][n][1] = o[i][n][2] = o[i][n][3] = 0.f;
#pragma unroll
    for (int n = 0; n < NQ; ++n) {
      m[n][0] = m[n][1] = -INFINITY;
      l[n][0] = l[n][1] = 0.f;
    }
  }
};

// One KTW-key tile of a warp.  sK / sV: the stage's K and V; qf: B fragments of Q^T (or read from
// sQ when they do not fit in registers); pos[nq][j]: position of query row nq * 8 + 2 t4 + j (-1: none).
template <int NQ, int KTW>
__device__ __forceinline__ void warp_tile_t(AccT<NQ>& acc, const uint32_t (*qf)[NQ][2], const __nv_bfloat16* sQ,
                                            const unsigned char* sK, const unsigned char* sV, int key0,
                                            const int (*pos)[2], int window, float c, bool mask, int box_shift) {
  constexpr int MT = KTW / 16;
  const int lane = threadIdx.x & 31;
  const int mat = lane >> 3, r8 = lane & 7, g = lane >> 2;
  const int half_stride = 128 << box_shift;
  // byte offset of key row kr (first half, chunk 0) in a stage
  auto sw_row = [&](int kr) {
    return (((kr >> box_shift) * HD) << (box_shift + 1)) + (kr & ((1 << box_shift) - 1)) * 128;
  };
  float s[MT][NQ][4];

  // S^T = K Q^T, even and odd 16-column steps in accumulators of their own
  {
    float s2[MT][NQ][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < NQ; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[mt][n][e] = s2[mt][n][e] = 0.f;
    int krow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) krow[mt] = sw_row(mt * 16 + (mat & 1) * 8 + r8);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t b[NQ][2];
      if (Q_IN_REGS) {
#pragma unroll
        for (int n = 0; n < NQ; ++n) b[n][0] = qf[ks][n][0], b[n][1] = qf[ks][n][1];
      } else {
#pragma unroll
        for (int n = 0; n < NQ; ++n) {
          const __nv_bfloat16* qrow = sQ + (n * 8 + g) * LDS + ks * 16 + 2 * (lane & 3);
          b[n][0] = *reinterpret_cast<const uint32_t*>(qrow);
          b[n][1] = *reinterpret_cast<const uint32_t*>(qrow + 8);
        }
      }
      const int koff = (ks >> 2) * half_stride + ((((ks * 2) & 7) + (mat >> 1)) ^ r8) * 16;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a[4];
        ldmatrix_x4(a, sK + krow[mt] + koff);
#pragma unroll
        for (int n = 0; n < NQ; ++n) {
          if (ks & 1)
            mma_bf16(s2[mt][n], a, b[n][0], b[n][1]);
          else
            mma_bf16(s[mt][n], a, b[n][0], b[n][1]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < NQ; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[mt][n][e] += s2[mt][n][e];
  }

  if (mask) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < NQ; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + mt * 16 + g + (e >> 1) * 8;
          const int ps = pos[n][e & 1];
          bool ok = j <= ps;
          if (window > 0) ok = ok && (j > ps - window);
          if (!ok) s[mt][n][e] = -INFINITY;
        }
  }

  // online softmax down the keys
  bool changed = false;
  float corr[NQ][2];
#pragma unroll
  for (int n = 0; n < NQ; ++n)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float mx = -INFINITY;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) mx = fmaxf(mx, fmaxf(s[mt][n][j], s[mt][n][j + 2]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(acc.m[n][j], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      changed = changed || (m_new > acc.m[n][j]);
      corr[n][j] = exp2f((acc.m[n][j] - m_use) * c);
      acc.m[n][j] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const float p0 = exp2f((s[mt][n][j] - m_use) * c);
        const float p1 = exp2f((s[mt][n][j + 2] - m_use) * c);
        s[mt][n][j] = p0;
        s[mt][n][j + 2] = p1;
        sum += p0 + p1;
      }
      acc.l[n][j] = acc.l[n][j] * corr[n][j] + sum;
    }
  if (__any_sync(0xffffffffu, changed)) {
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm)
#pragma unroll
      for (int n = 0; n < NQ; ++n) {
        acc.o[dm][n][0] *= corr[n][0];
        acc.o[dm][n][1] *= corr[n][1];
        acc.o[dm][n][2] *= corr[n][0];
        acc.o[dm][n][3] *= corr[n][1];
      }
  }

  // O^T += V^T P^T
  {
    uint32_t pb[MT][NQ][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int n = 0; n < NQ; ++n) {
        pb[mt][n][0] = movmatrix_trans(pack_bf16(s[mt][n][0], s[mt][n][1]));
        pb[mt][n][1] = movmatrix_trans(pack_bf16(s[mt][n][2], s[mt][n][3]));
      }
    int vrow[MT];
#pragma unroll
    for (int kk = 0; kk < MT; ++kk) vrow[kk] = sw_row(kk * 16 + (mat >> 1) * 8 + r8);
#pragma unroll
    for (int dm = 0; dm < HD / 16; ++dm) {
      const int voff = (dm >> 2) * half_stride + ((((dm * 2) & 7) + (mat & 1)) ^ r8) * 16;
#pragma unroll
      for (int kk = 0; kk < MT; ++kk) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, sV + vrow[kk] + voff);
#pragma unroll
        for (int n = 0; n < NQ; ++n) mma_bf16(acc.o[dm][n], a, pb[kk][n][0], pb[kk][n][1]);
      }
    }
  }
}

// One head row of a new token, normalised over the head (if a weight is given) and rotated over its first
// rotary_dim elements in the half-split pairing (j, j + rotary_dim / 2), by one warp: lane l holds the
// EPL = HD / 32 consecutive elements from l * EPL, so an element's partner lies in the same slot of the lane
// rotary_dim / 2 / EPL further on (rotary_dim a multiple of 2 EPL).  32-bit throughout, rounded once.
// What does not depend on the kernels before this one (the token's angles, the norm weights) is read first.
constexpr int EPL = HD / 32 > 0 ? HD / 32 : 1;
struct Rotation {
  float c[EPL], s[EPL];      // cos and sin of this lane's elements' pairs (1, 0 beyond the rotary part)
  int src;                   // the lane that holds the partners
  bool first, second;        // this lane's elements are the first / the second of their pairs
  __device__ __forceinline__ void init(const float* table_row, int rotary_dim) {
    const int lane = threadIdx.x & 31;
    const int half = rotary_dim >> 1, D = half / EPL;
    first = lane < D;
    second = !first && lane < 2 * D;
    src = first ? lane + D : (second ? lane - D : lane);
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      c[e] = 1.f;
      s[e] = 0.f;
      if (first || second) {
        const int j = (first ? lane : lane - D) * EPL + e;
        c[e] = table_row[j];
        s[e] = table_row[half + j];
      }
    }
  }
};
__device__ __forceinline__ void load_norm_weight(const void* nw, int w_dtype, float (&w)[EPL]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int e = 0; e < EPL; ++e) w[e] = nw != nullptr ? atom::load_as_float(nw, w_dtype, lane * EPL + e) : 1.f;
}
__device__ __forceinline__ void load_row(const __nv_bfloat16* x, __nv_bfloat16 (&raw)[EPL]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int e = 0; e < EPL; ++e) raw[e] = x[lane * EPL + e];
}
__device__ __forceinline__ void rotated_row(const __nv_bfloat16 (&raw)[EPL], bool normed, const float (&w)[EPL], float eps,
                                            const Rotation& r, float (&out)[EPL]) {
  float v[EPL];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    v[e] = __bfloat162float(raw[e]);
    ss += v[e] * v[e];
  }
  if (normed) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = v[e] * rstd * w[e];
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const float other = __shfl_sync(0xffffffffu, v[e], r.src);
    out[e] = r.first ? v[e] * r.c[e] - other * r.s[e] : (r.second ? v[e] * r.c[e] + other * r.s[e] : v[e]);
  }
}

// The work of one warp of a short-request CTA over KTW-key tiles [tile_begin, tile_end) of the
// request.  ring / full: this warp's stages and their barriers.
template <int NQ, int KTW>
__device__ __forceinline__ void decode_tma_body(const Params& p, const Work& w, unsigned char* ring, uint64_t* full,
                                                const CUtensorMap* kmap, const CUtensorMap* vmap, int* aborted,
                                                __nv_bfloat16* sQ, int tile_begin, int tile_end,
                                                int key_end, int split, unsigned char* smem_raw) {
  constexpr int TMA_STAGE_BYTES = tma_stage_bytes(KTW);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  int box_shift = p.page_shift, kt_shift = 0;
  while ((1 << kt_shift) < KTW) ++kt_shift;
  box_shift = min(box_shift, kt_shift);
  const int boxes = KTW >> box_shift;
  const bool issuer = lane < 2 * boxes;
  const int my_box = lane >> 1;
  const CUtensorMap* my_map = (lane & 1) ? vmap : kmap;
  const uint32_t my_dst = ((lane & 1) ? KTW * HD * 2 : 0) + ((my_box * HD) << (box_shift + 1));
  const int safe_page = (issuer && key_end > 0) ? max(w.bt[(key_end - 1) >> p.page_shift], 0) : 0;
  // Row of this lane's box of tile t in the page matrix [pages * nkv * page][HD].
  auto box_row = [&](int t) -> int {
    if (!issuer || t >= tile_end) return 0;
    const int j0 = t * KTW + (my_box << box_shift);
    int page = safe_page, in_page = 0;
    if (j0 < key_end) {
      const int pg = w.bt[j0 >> p.page_shift];
      if (pg >= 0) {
        page = pg;
        in_page = j0 & (p.page_size - 1);
      }
    }
    return (page * p.nkv + w.kvh) * p.page_size + in_page;
  };
  auto issue = [&](int st, int row) {
    if (lane == 0) atom::tma::mbar_expect_tx(&full[st], TMA_STAGE_BYTES);
    __syncwarp();
    if (issuer) atom::tma::load_chunks(ring + st * TMA_STAGE_BYTES + my_dst, my_map, row, 0, &full[st]);
  };

  // The warp's first RING tiles.  Those that hold only keys from before this step are asked for at
  // once: the kernel before this one (which may still be running) writes the step's new keys and
  // nothing else of the cache, and the step's arrays were filled before it began.  The others, and Q,
  // follow once that kernel has completed.
  // Where this kernel rotates the step's new tokens itself: the token's angles and the norm weights, and
  // which warp will meet the new token's tile, before the wait for the kernels in front of it.
  const bool rotating = p.rot_table != nullptr;
  Rotation rot;
  float qw[EPL], kw[EPL];
  bool will_patch = false;
  __nv_bfloat16 new_k[EPL], new_v[EPL];    // the new token's key (normalised, rotated) and value, held by the warp that will meet their tile
  if (rotating) {
    const int row_of = min(p.rot_rows[w.q_begin], p.rot_max_pos - 1);
    rot.init(p.rot_table + (int64_t)row_of * p.rotary_dim, p.rotary_dim);
    load_norm_weight(p.q_norm_w, p.norm_w_dtype, qw);
    const int t_new = (w.ctx - 1) / KTW;
    will_patch = p.k_write != nullptr && w.ctx >= 1 && t_new >= tile_begin && t_new < tile_end &&
                 ((t_new - tile_begin) & 3) == warp;
    if (will_patch) load_norm_weight(p.k_norm_w, p.norm_w_dtype, kw);
  }
  int row_next;
  {
    int rows[RING + 1];
#pragma unroll
    for (int i = 0; i <= RING; ++i) rows[i] = box_row(tile_begin + warp + 4 * i);
    bool early[RING];
#pragma unroll
    for (int i = 0; i < RING; ++i) {
      const int t = tile_begin + warp + 4 * i;
      // (where this kernel writes the new token's key and value itself, no kernel of the step writes the cache)
      early[i] = t < tile_end && ((t + 1) * KTW <= w.q_start || p.k_write != nullptr);
      if (early[i]) issue(i, rows[i]);
    }
    atom::pdl_wait();      // inputs written by the kernels before this one are visible from here on
#pragma unroll
    for (int i = 0; i < RING; ++i)
      if (!early[i] && tile_begin + warp + 4 * i < tile_end) issue(i, rows[i]);
    row_next = rows[RING];
  }
  if (tile_begin < tile_end) {
    if (rotating) {
      // the raw projection's query rows of this kv head, normalised and rotated on their way into sQ; what
      // the warp needs from the projection (its query rows, the new key and value) is asked for at once
      const __nv_bfloat16* raw = p.q + (int64_t)w.q_begin * p.q_stride;
      __nv_bfloat16 xq[4][EPL];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (warp + 4 * i < w.rows_total) load_row(raw + (int64_t)(w.kvh * p.group + warp + 4 * i) * HD, xq[i]);
      if (will_patch) {
        load_row(raw + (int64_t)(p.nh + w.kvh) * HD, new_k);
        load_row(raw + (int64_t)(p.nh + p.nkv + w.kvh) * HD, new_v);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int R = warp + 4 * i;
        float qv[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) qv[e] = 0.f;
        if (R < w.rows_total) rotated_row(xq[i], p.q_norm_w != nullptr, qw, p.norm_eps, rot, qv);
#pragma unroll
        for (int e = 0; e < EPL; ++e) sQ[R * LDS + lane * EPL + e] = __float2bfloat16_rn(qv[e]);
      }
      if (will_patch) {
        float kv[EPL];
        rotated_row(new_k, p.k_norm_w != nullptr, kw, p.norm_eps, rot, kv);
#pragma unroll
        for (int e = 0; e < EPL; ++e) new_k[e] = __float2bfloat16_rn(kv[e]);
      }
    } else {
      load_q_tile<16>(p, w, sQ);
      cp_async_commit();
      cp_async_wait<0>();
    }
  }
  __syncthreads();

  int pos[NQ][2];
#pragma unroll
  for (int n = 0; n < NQ; ++n)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int R = n * 8 + 2 * t4 + j;
      pos[n][j] = R < w.rows_total ? w.q_start + R / p.group : -1;
    }
  uint32_t qf[Q_IN_REGS ? HD / 16 : 1][NQ][2];
  if (Q_IN_REGS) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
#pragma unroll
      for (int n = 0; n < NQ; ++n) {
        const __nv_bfloat16* qrow = sQ + (n * 8 + g) * LDS + ks * 16 + 2 * t4;
        qf[ks][n][0] = *reinterpret_cast<const uint32_t*>(qrow);
        qf[ks][n][1] = *reinterpret_cast<const uint32_t*>(qrow + 8);
      }
  }

  AccT<NQ> acc;
  acc.init();
  int st = 0;
  uint32_t phase = 0;
  for (int t = tile_begin + warp; t < tile_end; t += 4) {
    const int refill = t + 4 * RING;
    const int row_after = box_row(refill + 4);   // in flight during the tile's arithmetic
    atom::tma::mbar_wait(&full[st], phase, aborted, p.error);
    unsigned char* sK = ring + st * TMA_STAGE_BYTES;
    const int key0 = t * KTW;
    if (will_patch && w.ctx - 1 >= key0 && w.ctx - 1 < key0 + KTW) {
      // The tile of the request's new token: its key and value replace what the page held at that place
      // in this stage, and go to the page.
      const int newpos = w.ctx - 1, kr = newpos - key0;
      const int page = w.bt[newpos >> p.page_shift];
      const bool has_page = page >= 0 && page < p.num_pages;
      if (!has_page && lane == 0) atomicExch(p.status, 1);     // a position without a page: recorded, not written
      const int64_t at = (((int64_t)(has_page ? page : 0) * p.nkv + w.kvh) * p.page_size + (newpos & (p.page_size - 1))) * HD;
      const int half_stride = 128 << box_shift;
      const int rbase = (((kr >> box_shift) * HD) << (box_shift + 1)) + (kr & ((1 << box_shift) - 1)) * 128;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const int d = lane * EPL + e;
        const int off = rbase + (d >> 6) * half_stride + ((((d & 63) >> 3) ^ (kr & 7)) << 4) + (d & 7) * 2;
        *reinterpret_cast<__nv_bfloat16*>(sK + off) = new_k[e];
        *reinterpret_cast<__nv_bfloat16*>(sK + KTW * HD * 2 + off) = new_v[e];
        if (has_page) {
          p.k_write[at + d] = new_k[e];
          p.v_write[at + d] = new_v[e];
        }
      }
      __syncwarp();
    }
    bool mask = key0 + KTW - 1 > w.q_start;
    if (p.window > 0) mask = mask || (key0 <= w.ctx - 1 - p.window);
    warp_tile_t<NQ, KTW>(acc, qf, sQ, sK, sK + KTW * HD * 2, key0, pos, p.window, p.scale_log2, mask, box_shift);
    if (refill < tile_end) {
      __syncwarp();
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // this warp's reads before the refill's writes
      issue(st, row_next);
    }
    row_next = row_after;
    if (++st == RING) {
      st = 0;
      phase ^= 1;
    }
  }
  __syncthreads();   // every warp has consumed all it asked for: the rings become the merge buffer

  float* mo = reinterpret_cast<float*>(smem_raw);       // [4][16][MLD]
  float* mm = mo + 4 * 16 * MLD;                         // [4][16]
  float* ml = mm + 4 * 16;                               // [4][16]
#pragma unroll
  for (int n = 0; n < NQ; ++n)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float l = acc.l[n][j];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      const int row = n * 8 + 2 * t4 + j;
      if (g == 0) {
        mm[warp * 16 + row] = acc.m[n][j];
        ml[warp * 16 + row] = l;
      }
#pragma unroll
      for (int dm = 0; dm < HD / 16; ++dm) {
        mo[(warp * 16 + row) * MLD + dm * 16 + g] = acc.o[dm][n][j];
        mo[(warp * 16 + row) * MLD + dm * 16 + g + 8] = acc.o[dm][n][j + 2];
      }
    }
  __syncthreads();
  decode_combine(p, w, split, mo, mm, ml);
}

template <int KTW>
__global__ void __launch_bounds__(NT, decode_tma_ctas(KTW)) flash_decode_tma_kernel(const Params p,
                                                                 const __grid_constant__ CUtensorMap kmap,
                                                                 const __grid_constant__ CUtensorMap vmap) {
  constexpr int TMA_STAGE_BYTES = tma_stage_bytes(KTW);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int aborted;
  unsigned char* rings = smem_raw + ((1024 - (atom::tma::smem_u32(smem_raw) & 1023)) & 1023);
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(rings + 4 * RING * TMA_STAGE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(sQ + 16 * LDS);
  if (threadIdx.x == 0) {
    aborted = 0;
#pragma unroll
    for (int i = 0; i < 4 * RING; ++i) atom::tma::mbar_init(&full[i], 1);
    atom::tma::mbar_fence_init();
    atom::tma::prefetch_map(&kmap);
    atom::tma::prefetch_map(&vmap);
  }
  __syncthreads();
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  // (no wait for the kernels before this one yet: see decode_tma_body.  No kernel of the step writes the arrays read here.)

  Work w;
  w.seq = blockIdx.x;
  w.kvh = blockIdx.y;
  const int split = blockIdx.z;
  w.q_begin = p.cu_q[w.seq];
  const int q_len = p.cu_q[w.seq + 1] - w.q_begin;
  w.rows_total = q_len * p.group;
  if (w.rows_total <= 0 || w.rows_total > 16) {
    atom::pdl_wait();   // a grid is complete only after what came before it
    return;
  }
  w.ctx = p.ctx_len[w.seq];
  w.q_start = w.ctx - q_len;
  w.row0 = 0;
  w.bt = p.block_table + (int64_t)w.seq * p.max_pages;

  // The splits are cut in units of BN keys, as in the kernel above; tiles are counted in KTW keys.
  const int key_end = w.ctx;
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, w.q_start - p.window + 1);
  const int first_tile = key_lo / BN, n_tiles = (key_end + BN - 1) / BN - first_tile;
  const int per_split = (n_tiles + p.num_splits - 1) / p.num_splits;
  const int big_begin = first_tile + split * per_split;
  const int big_end = max(big_begin, min(big_begin + per_split, first_tile + n_tiles));
  const int tile_begin = big_begin * (BN / KTW);
  const int tile_end = min(big_end * (BN / KTW), (key_end + KTW - 1) / KTW);

  const int warp = threadIdx.x >> 5;
  unsigned char* ring = rings + warp * RING * TMA_STAGE_BYTES;
  if (w.rows_total <= 8)
    decode_tma_body<1, KTW>(p, w, ring, full + warp * RING, &kmap, &vmap, &aborted, sQ, tile_begin, tile_end, key_end,
                       split, smem_raw);
  else
    decode_tma_body<2, KTW>(p, w, ring, full + warp * RING, &kmap, &vmap, &aborted, sQ, tile_begin, tile_end, key_end,
                       split, smem_raw);
}
#endif

// Merges the splits of every (token, head) of the short requests: one warp each.  Lanes
// first take one split each to find the common maximum and the weights, then one output
// element each (all loads of a pass are independent).  At most 64 splits.
__global__ void flash_merge_kernel(const Params p, const int* __restrict__ seq_of_token, int T) {
  atom::pdl_trigger();   // the next kernel may be scheduled at once: before its own wait it reads nothing a kernel of this step writes
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int s = -1, rows = 0;
  if (warp < T * p.nh) {
    s = seq_of_token[warp / p.nh];   // (no kernel of the step writes the step's arrays)
    if (s >= 0) rows = (p.cu_q[s + 1] - p.cu_q[s]) * p.group;
  }
  atom::pdl_wait();      // inputs written by the kernels before this one are visible from here on
  if (s < 0 || rows > 16) return;   // beyond the batch, a padding row of a fixed-size batch, or not a short request
  const float* ml = p.part_ml + (int64_t)warp * p.num_splits * 2;
  const float* po = p.part_o + (int64_t)warp * p.num_splits * HD;
  constexpr int VEC = HD / 32 > 0 ? HD / 32 : 1;   // (head sizes of 128, 256: a lane holds VEC consecutive elements)
  constexpr bool WIDE = HD % 128 == 0;
  constexpr int BATCH = 8;              // splits whose partial sums are asked for together
  constexpr int NV = VEC / 4 > 0 ? VEC / 4 : 1;      // 16-byte pieces of a lane's elements
  float4 first[WIDE ? BATCH * NV : 1];
  if constexpr (WIDE) {
    // the first splits' partial sums are asked for before the weights are known: one round trip, not two
#pragma unroll
    for (int k = 0; k < BATCH; ++k)
#pragma unroll
      for (int v = 0; v < VEC / 4; ++v)
        first[k * (VEC / 4) + v] = k < p.num_splits
                                       ? __ldcg(reinterpret_cast<const float4*>(po + (int64_t)k * HD + lane * VEC) + v)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int k0 = lane, k1 = lane + 32;
  const float m0 = k0 < p.num_splits ? ml[2 * k0] : -INFINITY;
  const float m1 = k1 < p.num_splits ? ml[2 * k1] : -INFINITY;
  const float l0 = k0 < p.num_splits ? ml[2 * k0 + 1] : 0.f;
  const float l1 = k1 < p.num_splits ? ml[2 * k1 + 1] : 0.f;
  float M = fmaxf(m0, m1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  const float Mu = (M == -INFINITY) ? 0.f : M;
  float w0 = exp2f((m0 - Mu) * p.scale_log2), w1 = exp2f((m1 - Mu) * p.scale_log2);
  float L = l0 * w0 + l1 * w1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
  const float inv = 1.f / L;
  w0 *= inv;
  w1 *= inv;
  if constexpr (WIDE) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int kb = 0; kb < p.num_splits; kb += BATCH) {
      float4 part[BATCH * NV];
#pragma unroll
      for (int k = 0; k < BATCH; ++k)
#pragma unroll
        for (int v = 0; v < VEC / 4; ++v) {
          if (kb == 0)
            part[k * (VEC / 4) + v] = first[k * (VEC / 4) + v];
          else
            part[k * (VEC / 4) + v] = kb + k < p.num_splits
                                          ? __ldcg(reinterpret_cast<const float4*>(po + (int64_t)(kb + k) * HD + lane * VEC) + v)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int k = 0; k < BATCH; ++k) {
        const int kk = kb + k;
        const float wk = __shfl_sync(0xffffffffu, kk < 32 ? w0 : w1, kk & 31);     // (0 beyond the last split)
#pragma unroll
        for (int v = 0; v < VEC / 4; ++v) {
          const float4 x = part[k * (VEC / 4) + v];
          acc[4 * v] += x.x * wk;
          acc[4 * v + 1] += x.y * wk;
          acc[4 * v + 2] += x.z * wk;
          acc[4 * v + 3] += x.w * wk;
        }
      }
    }
    __nv_bfloat16* o = p.out + (int64_t)warp * HD + lane * VEC;
#pragma unroll
    for (int e = 0; e < VEC; e += 2) *reinterpret_cast<__nv_bfloat162*>(o + e) = __floats2bfloat162_rn(acc[e], acc[e + 1]);
    return;
  }
  float acc[(HD + 31) / 32];
#pragma unroll
  for (int i = 0; i < (HD + 31) / 32; ++i) acc[i] = 0.f;
  for (int k = 0; k < p.num_splits; ++k) {
    const float wk = __shfl_sync(0xffffffffu, k < 32 ? w0 : w1, k & 31);
#pragma unroll
    for (int i = 0; i < (HD + 31) / 32; ++i) {
      const int d = lane + i * 32;
      if (d < HD) acc[i] += po[k * HD + d] * wk;
    }
  }
#pragma unroll
  for (int i = 0; i < (HD + 31) / 32; ++i) {
    const int d = lane + i * 32;
    if (d < HD) p.out[(int64_t)warp * HD + d] = __float2bfloat16_rn(acc[i]);
  }
}

}  // namespace flash
}  // namespace atom

#if ATOM_HD == 128
#include "attention_flash_tc.cuh"
#include "attention_flash_tc2.cuh"
#endif

namespace atom {
namespace flash {
// Raised by a kernel of this library whose bounded wait ran out.
static __device__ int g_error_flag;
static int* g_error_addr[64] = {};      // per device: the caller's flag if it gave one, else this library's own
static int* error_flag_address() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (g_error_addr[dev] == nullptr && cudaGetSymbolAddress((void**)&g_error_addr[dev], g_error_flag) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return g_error_addr[dev];
}
}  // namespace flash
}  // namespace atom

// From now on the kernels launched on the current device raise ``flag`` (a device int that outlives
// them) instead of the library's own word; nullptr goes back to the library's own.
ATOM_EXPORT int atom_flash_set_error_flag(int* flag) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ATOM_ERR_LAUNCH;
  atom::flash::g_error_addr[dev] = flag;
  return ATOM_OK;
}

// Reads and clears the error flag of this library on the current device (synchronises): 0 if all is well.
ATOM_EXPORT int atom_flash_take_error() {
  int* a = atom::flash::error_flag_address();
  int v = 0;
  if (a == nullptr || cudaMemcpy(&v, a, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    (void)cudaMemcpy(a, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

// Sets one of the ATOM_OPT_* options (common.cuh) in this library.
ATOM_EXPORT int atom_flash_set_option(int key, int value) { return atom::set_option(key, value); }

// 1 if this library has the tcgen05 kernel for long portions (head size 128).
ATOM_EXPORT int atom_flash_has_tc() {
#if ATOM_HD == 128
  return 1;
#else
  return 0;
#endif
}

#define ATOM_CAT_(a, b) a##b
#define ATOM_CAT(a, b) ATOM_CAT_(a, b)

// Head size this library was compiled for.
ATOM_EXPORT int atom_flash_head_dim() { return atom::flash::HD; }

namespace atom {
namespace flash {
// A kernel's shared-memory attribute belongs to a device: one flag per (device, kind of kernel).
static bool& attr_done(int kind) {
  static bool done[64][4] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  return done[dev][kind];
}
}  // namespace flash
}  // namespace atom

// Bytes of scratch that `num_splits` splits need for T tokens.
ATOM_EXPORT int64_t atom_flash_scratch_bytes(int T, int nh, int num_splits) {
  return num_splits <= 1 ? 0 : (int64_t)T * nh * num_splits * (atom::flash::HD + 2) * (int64_t)sizeof(float);
}

// What a decode step hands over when the kernel is to normalise, rotate and store its new tokens itself
// (atom_flash_attention_rotating): see Params.
struct AtomFlashRotation {
  const float* table;
  const int* rows;
  int rotary_dim, max_pos;
  const void* q_norm_w;
  const void* k_norm_w;
  int norm_w_dtype;
  float norm_eps;
  int write_cache;
  int* status;
};

namespace atom {
namespace flash {
static bool decode_tma_usable(int page_size, int64_t num_pages, int nkv) {
#if ATOM_HD % 64 == 0
  const bool pow2 = page_size >= 8 && (page_size & (page_size - 1)) == 0;
  return pow2 && atom::options().v[ATOM_OPT_DECODE_TMA] != 0 && num_pages > 0 &&
         (uint64_t)num_pages * nkv * page_size < 0x7fffffffull && atom::tma::encode_fn() != nullptr;
#else
  return false;
#endif
}
}  // namespace flash
}  // namespace atom

// 1 if a decode step of these sizes can leave norm, rotation and cache write to the decode kernel.
ATOM_EXPORT int atom_flash_rotating_supports(int page_size, int64_t num_pages, int nh, int nkv, int rotary_dim) {
#if ATOM_HD % 64 == 0
  return nkv > 0 && nh % nkv == 0 && nh / nkv <= 16 && rotary_dim > 0 && rotary_dim <= atom::flash::HD &&
         rotary_dim % (2 * atom::flash::EPL) == 0 && atom::flash::decode_tma_usable(page_size, num_pages, nkv);
#else
  return 0;
#endif
}

static int flash_run(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                     const void* v_pages, int64_t num_pages, const int* block_table, int max_pages,
                                     int page_size, const int* cu_q, const int* ctx_len,
                                     const int* seq_of_token, int T, int num_seqs, int nh, int nkv,
                                     int hd, float scale, int window, int long_tiles, int long_rows,
                                     int prefill_tiles, int has_short, int num_splits, void* scratch,
                                     cudaStream_t stream, const AtomFlashRotation* rot) {
  using namespace atom::flash;
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (hd != HD || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || num_splits < 1 ||
      nkv > 65535 || num_splits > 65535 || long_tiles > 65535 || prefill_tiles > 65535 || (q_stride % 8) != 0 || (num_splits > 1 && scratch == nullptr) ||
      !(scale > 0.f))
    return ATOM_ERR_ARG;
  Params p;
  p.out = (__nv_bfloat16*)out;
  p.q = (const __nv_bfloat16*)q;
  p.q_stride = q_stride;
  p.k_pages = (const __nv_bfloat16*)k_pages;
  p.v_pages = (const __nv_bfloat16*)v_pages;
  p.block_table = block_table;
  p.max_pages = max_pages;
  p.page_size = page_size;
  p.page_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    int s = 0;
    while ((1 << s) < page_size) ++s;
    p.page_shift = s;
  }
  p.cu_q = cu_q;
  p.ctx_len = ctx_len;
  p.num_seqs = num_seqs;
  p.nh = nh;
  p.nkv = nkv;
  p.group = nh / nkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.num_splits = num_splits;
  p.error = atom::flash::error_flag_address();
  p.long_rows = long_tiles > 0 ? long_rows : 0x7fffffff;
  if (long_tiles > 0 && (!atom_flash_has_tc() || window > 0 || long_rows < 17 || p.error == nullptr)) return ATOM_ERR_ARG;
  p.part_o = (float*)scratch;
  p.part_ml = p.part_o ? p.part_o + (int64_t)T * nh * num_splits * HD : nullptr;
  p.rot_table = nullptr;
  p.rot_rows = nullptr;
  p.rotary_dim = p.rot_max_pos = 0;
  p.q_norm_w = p.k_norm_w = nullptr;
  p.norm_w_dtype = ATOM_F32;
  p.norm_eps = 0.f;
  p.k_write = p.v_write = nullptr;
  p.num_pages = num_pages;
  p.status = nullptr;
  if (rot != nullptr) {
    // one new token per request, all of them short, on the TMA decode kernel
    if (!atom_flash_rotating_supports(page_size, num_pages, nh, nkv, rot->rotary_dim) || T != num_seqs ||
        long_tiles > 0 || prefill_tiles > 0 || !has_short || rot->table == nullptr || rot->rows == nullptr ||
        rot->max_pos <= 0 || rot->status == nullptr || p.error == nullptr ||
        (rot->norm_w_dtype != ATOM_F32 && rot->norm_w_dtype != ATOM_BF16))
      return ATOM_ERR_ARG;
    p.rot_table = rot->table;
    p.rot_rows = rot->rows;
    p.rotary_dim = rot->rotary_dim;
    p.rot_max_pos = rot->max_pos;
    p.q_norm_w = rot->q_norm_w;
    p.k_norm_w = rot->k_norm_w;
    p.norm_w_dtype = rot->norm_w_dtype;
    p.norm_eps = rot->norm_eps;
    if (rot->write_cache) {
      p.k_write = (__nv_bfloat16*)const_cast<void*>(k_pages);
      p.v_write = (__nv_bfloat16*)const_cast<void*>(v_pages);
    }
    p.status = rot->status;
  }

  bool& attr_set = attr_done(0);
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)prefill_smem_bytes()) != cudaSuccess ||
        cudaFuncSetAttribute(flash_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)decode_smem_bytes()) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
#if ATOM_HD == 128
  if (long_tiles > 0) {
    // TMA loading needs pages of 8, 16, ..., 128 (or more, a power of two) tokens and a group size that
    // divides 128; otherwise the cp.async loaders take any sizes.
    const int ps = page_size, G = p.group;
    const bool ps_ok = (ps & (ps - 1)) == 0 && ps >= 8;
    bool use_tma = ps_ok && G <= 128 && 128 % G == 0 && num_pages > 0 && (uint64_t)num_pages * nkv * ps < 0x7fffffffull && atom::tma::encode_fn() != nullptr && (q_stride % 8) == 0;
    tc::Maps maps;
    memset(&maps, 0, sizeof(maps));
    if (use_tma) {
      const uint64_t rows = (uint64_t)num_pages * nkv * ps;     // the page matrices [pages * nkv * page][128]
      const uint32_t box_rows = ps < tc::TN ? ps : tc::TN;
      uint64_t d2[2] = {128, rows}, s2[1] = {256};
      uint32_t b2[2] = {64, box_rows};
      uint64_t d3[3] = {128, (uint64_t)(nh + 2 * nkv), (uint64_t)T}, s3[2] = {256, (uint64_t)q_stride * 2};
      uint32_t b3[3] = {64, (uint32_t)G, (uint32_t)(128 / G)};
      use_tma = atom::tma::make_map_raw(&maps.k, k_pages, 2, d2, s2, b2) &&
                atom::tma::make_map_raw(&maps.v, v_pages, 2, d2, s2, b2) &&
                atom::tma::make_map_raw(&maps.q, q, 3, d3, s3, b3);
    }
    if (use_tma) {
      // The two-tile kernel trades registers between its warpgroups (setmaxnreg), which waits without a bound
      // if the CTA's pool is smaller than the kernel assumes: it runs only if it was compiled to the register
      // count its numbers are made for.
      static int tc2_regs = -1;
      if (tc2_regs < 0) {
        cudaFuncAttributes fa;
        tc2_regs = cudaFuncGetAttributes(&fa, tc2::flash_prefill_tc2_kernel) == cudaSuccess ? fa.numRegs : 0;
      }
      if (tc2_regs != tc2::LAUNCH_REGS) use_tma = false;
    }
    if (use_tma) {
      bool& tc2_attr = attr_done(1);
      if (!tc2_attr) {
        if (cudaFuncSetAttribute(tc2::flash_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)tc2::smem_bytes2()) != cudaSuccess)
          return ATOM_ERR_LAUNCH;
        tc2_attr = true;
      }
      // (long_tiles counts 128-row tiles: an upper bound of the 256-row tiles; the CTAs beyond them leave at once)
      atom::launch_pdl(tc2::flash_prefill_tc2_kernel, dim3(nkv, long_tiles), dim3(tc2::NTHREADS2), tc2::smem_bytes2(),
                       stream, p, long_rows, maps);
    } else {
      bool& tc_attr = attr_done(2);
      if (!tc_attr) {
        if (cudaFuncSetAttribute(tc::flash_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)tc::smem_bytes()) != cudaSuccess)
          return ATOM_ERR_LAUNCH;
        tc_attr = true;
      }
      atom::launch_pdl(tc::flash_prefill_tc_kernel, dim3(nkv, long_tiles), dim3(tc::NTHREADS), tc::smem_bytes(), stream, p,
                       long_rows);
    }
  }
#endif
  if (prefill_tiles > 0) {
    dim3 grid(nkv, prefill_tiles);
    atom::launch_pdl(flash_prefill_kernel, dim3(grid), dim3(NT), prefill_smem_bytes(), stream, p);
  }
  if (has_short) {
    dim3 grid(num_seqs, nkv, num_splits);
    bool tma_done = false;
#if ATOM_HD % 64 == 0
    // One TMA box per page needs pages of a power of two >= 8 tokens and the size of the page matrices.
    const bool tma_off = atom::options().v[ATOM_OPT_DECODE_TMA] == 0;
    const uint64_t page_rows = (uint64_t)num_pages * nkv * page_size;
    if (!tma_off && p.page_shift >= 3 && num_pages > 0 && page_rows < 0x7fffffffull && p.error != nullptr) {
      // 32-key warp tiles where every CTA has an SM to itself (and they fit), else 16-key tiles and two CTAs an SM.
      static int sms = 0;
      if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
          return ATOM_ERR_LAUNCH;
      }
      const int forced = atom::options().v[ATOM_OPT_DECODE_KTW];
      const bool wide = decode_tma_fits(32) && (forced == 32 || (forced != 16 && (int64_t)num_seqs * nkv * num_splits <= sms));
      const int ktw = wide ? 32 : 16;
      const uint32_t box_rows = page_size < ktw ? page_size : ktw;
      CUtensorMap kmap, vmap;
      if (atom::tma::cached_map(&kmap, k_pages, page_rows, HD, HD, box_rows, HD / 64) &&
          atom::tma::cached_map(&vmap, v_pages, page_rows, HD, HD, box_rows, HD / 64)) {
        bool& tma_attr = attr_done(3);
        if (!tma_attr) {
          if (cudaFuncSetAttribute(flash_decode_tma_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)decode_tma_smem_bytes(16)) != cudaSuccess)
            return ATOM_ERR_LAUNCH;
          if (decode_tma_fits(32) &&
              cudaFuncSetAttribute(flash_decode_tma_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)decode_tma_smem_bytes(32)) != cudaSuccess)
            return ATOM_ERR_LAUNCH;
          tma_attr = true;
        }
        if (wide)
          atom::launch_pdl(flash_decode_tma_kernel<32>, dim3(grid), dim3(NT), decode_tma_smem_bytes(32), stream, p, kmap,
                           vmap);
        else
          atom::launch_pdl(flash_decode_tma_kernel<16>, dim3(grid), dim3(NT), decode_tma_smem_bytes(16), stream, p, kmap,
                           vmap);
        tma_done = true;
      }
    }
#endif
    if (!tma_done && rot != nullptr) return ATOM_ERR_LIB;      // (the tensor maps were refused)
    if (!tma_done) atom::launch_pdl(flash_decode_kernel, dim3(grid), dim3(NT), decode_smem_bytes(), stream, p);
    if (num_splits > 1) {
      const int warps = T * nh;
      atom::launch_pdl(flash_merge_kernel, dim3((warps + 3) / 4), dim3(128), 0, stream, p, seq_of_token, T);
    }
  }
  return atom::check_launch();
}

// num_pages: pages of k_pages / v_pages (used to bound the TMA maps; 0: unknown, no TMA loading).
// long_tiles > 0: requests with at least long_rows packed rows run on the tcgen05 kernel
// (long_tiles = sum over them of ceil(rows / 128); needs atom_flash_has_tc() and window <= 0).
// prefill_tiles: sum over the other requests with more than 16 packed rows of ceil(rows / 64); 0: none.
// has_short: some request has at most 16 packed rows.  scratch: atom_flash_scratch_bytes bytes
// when num_splits > 1.
ATOM_EXPORT int atom_flash_attention(void* out, const void* q, int64_t q_stride, const void* k_pages,
                                     const void* v_pages, int64_t num_pages, const int* block_table, int max_pages,
                                     int page_size, const int* cu_q, const int* ctx_len,
                                     const int* seq_of_token, int T, int num_seqs, int nh, int nkv,
                                     int hd, float scale, int window, int long_tiles, int long_rows,
                                     int prefill_tiles, int has_short, int num_splits, void* scratch,
                                     cudaStream_t stream) {
  return flash_run(out, q, q_stride, k_pages, v_pages, num_pages, block_table, max_pages, page_size, cu_q, ctx_len,
                   seq_of_token, T, num_seqs, nh, nkv, hd, scale, window, long_tiles, long_rows, prefill_tiles,
                   has_short, num_splits, scratch, stream, nullptr);
}

// A decode step (T == num_seqs: one new token per request; requests of a fixed-size batch without one
// have ctx_len 0) whose tokens' queries and keys are still raw: q points at the projection's rows
// [q heads | k heads | v heads] of width hd each.  The decode kernel normalises every query and key head
// (weights of hd elements, or null), rotates it by the table row rows[t], writes the key and the value to
// the token's page (write_cache; a token without a page sets *status) and attends over the pages and the
// new token.  Needs atom_flash_rotating_supports.
ATOM_EXPORT int atom_flash_attention_rotating(void* out, const void* qkv, int64_t q_stride, void* k_pages,
                                              void* v_pages, int64_t num_pages, const int* block_table,
                                              int max_pages, int page_size, const int* cu_q, const int* ctx_len,
                                              const int* seq_of_token, int T, int num_seqs, int nh, int nkv, int hd,
                                              float scale, int window, int num_splits, void* scratch,
                                              const float* table, const int* rows, int rotary_dim, int max_pos,
                                              const void* q_norm_w, const void* k_norm_w, int norm_w_dtype,
                                              float norm_eps, int write_cache, int* status, cudaStream_t stream) {
  AtomFlashRotation rot = {table, rows, rotary_dim, max_pos, q_norm_w, k_norm_w, norm_w_dtype, norm_eps, write_cache,
                           status};
  return flash_run(out, qkv, q_stride, k_pages, v_pages, num_pages, block_table, max_pages, page_size, cu_q, ctx_len,
                   seq_of_token, T, num_seqs, nh, nkv, hd, scale, window, 0, 0, 0, 1, num_splits, scratch, stream,
                   &rot);
}

// ------------------------------------------------------------------ allocation-free entry point
// See attention_flash_static.h for who this is for and the rules of use.
#include "attention_flash_static.h"

namespace atom {
namespace flash {

// Scratch for the partial results of the key splits.  In host code this name is only a
// stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_static_scratch[ATOM_FLASH_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {};

// Once per device, with that device current: the array's address on that device.
static float* static_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_static_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_static_scratch_addr[dev] = ptr;
  }
  return g_static_scratch_addr[dev];
}

}  // namespace flash
}  // namespace atom

ATOM_EXPORT int atom_flash_attention_static(void* out, const void* q, int64_t q_stride,
                                            const void* k_pages, const void* v_pages,
                                            const int* block_table, int max_pages, int page_size,
                                            const int* cu_q, const int* ctx_len,
                                            const int* seq_of_token, int T, int num_seqs, int nh,
                                            int nkv, int hd, float scale, int window,
                                            int prefill_tiles, int has_short, int num_splits,
                                            cudaStream_t stream) {
  using namespace atom::flash;
  if (T <= 0 || num_seqs <= 0) return ATOM_OK;
  if (nh <= 0 || num_splits < 1) return ATOM_ERR_ARG;
  float* scratch = nullptr;
  if (num_splits > 1) {
    const int64_t need = (int64_t)T * nh * num_splits * (HD + 2);
    if (need > (int64_t)ATOM_FLASH_STATIC_SCRATCH_FLOATS) return ATOM_ERR_SCRATCH;
    scratch = static_scratch_for_current_device();
    if (scratch == nullptr) return ATOM_ERR_SETUP;
  }
  return atom_flash_attention(out, q, q_stride, k_pages, v_pages, 0, block_table, max_pages, page_size,
                              cu_q, ctx_len, seq_of_token, T, num_seqs, nh, nkv, hd, scale, window,
                              0, 0, prefill_tiles, has_short, num_splits, scratch, stream);
}
