// Paged causal attention for long portions on the 5th-generation tensor cores (tcgen05), head
// size 128, bf16, for any page size and group size (where pages and query rows come as TMA boxes
// the kernel of attention_flash_tc2.cuh runs instead; it uses the primitives defined here).
// Included by attention_flash.cu (namespace atom::flash, its Params / Work).
//
// One CTA takes 128 packed query rows (row = token * G + head in group) of one (request, kv
// head) and walks over that request's keys in tiles of 128:
//     S = Q K^T        tcgen05.mma, Q and K from shared memory (K-major, 128-byte swizzle),
//                      S (128 x 128, 32-bit) in tensor memory, two buffers
//     P = softmax      four warps, one row per thread: tcgen05.ld of the row, running
//                      maximum and sum in 32-bit, P rounded to bf16 into shared memory
//     O += P V         tcgen05.mma, P from shared memory, V as it lies in the pages
//                      (MN-major), O (128 x 128, 32-bit) in tensor memory
// Warp roles: 0-3 softmax and epilogue (warp w owns TMEM lanes 32 w .. 32 w + 31), 4-11 load
// Q, K, V with cp.async into the swizzled layout (pages of any size), 12 allocates tensor
// memory and issues every MMA from one thread.  The MMA thread runs one S ahead: while the
// softmax warps work on tile j the tensor cores compute S of tile j + 1 and then O of tile j.
// O is rescaled in tensor memory only when some row's maximum has grown.
// All waits are bounded (see tma.cuh); tensor memory is freed on every path.
#pragma once
#include "tma.cuh"

namespace atom {
namespace flash {
namespace tc {

using atom::tma::mbar_arrive;
using atom::tma::mbar_fence_init;
using atom::tma::mbar_init;
using atom::tma::mbar_wait;
using atom::tma::smem_u32;

constexpr int TM = 128;          // packed query rows per CTA
constexpr int TN = 128;          // keys per tile
constexpr int LOADERS = 256;                  // loader threads: eight warps copy with cp.async (~2.5 B/clk per warp)
constexpr int NTHREADS = 128 + LOADERS + 32;  // 4 softmax warps, the loaders, 1 MMA warp
constexpr int MMA_WARP = (128 + LOADERS) / 32;
constexpr int BLOCK = 128 * 128; // bytes of one [128 rows][64 elements] swizzled block
constexpr int K_STAGES = 3, V_STAGES = 2;   // K is wanted one tile ahead of V and is free again sooner
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t S_COL0 = 0, S_COL1 = 128, O_COL = 256;

// shared memory: Q (2 blocks), K stages (2 blocks each), V stages (2 blocks each), P (2 blocks)
constexpr int SMEM_Q = 0, SMEM_K = 2 * BLOCK, SMEM_V = SMEM_K + K_STAGES * 2 * BLOCK,
              SMEM_P = SMEM_V + V_STAGES * 2 * BLOCK, SMEM_DATA = SMEM_P + 2 * BLOCK;
constexpr size_t smem_bytes() { return 1024 + SMEM_DATA + 256; }

// ---- tcgen05 primitives

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; 128 x N x 16 per call, bf16 in, 32-bit out.
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// The same with A taken from tensor memory: lane = row, 16 bf16 of a row in 8 consecutive 32-bit columns.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// The same for 16 columns.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, blocks of [rows][64 elements]:
//   bits 0-13 start address / 16, 16-29 leading byte offset / 16, 32-45 stride byte offset / 16,
//   46-47 version (1), 61-63 layout (2 = 128-byte swizzle).
// K-major operand: 8-row groups are `sbo` bytes apart (1024); the leading offset is unused.
// MN-major operand: 64-element groups along MN are `lbo` bytes apart, 8-row groups along K `sbo`.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: 32-bit accumulate (bit 4), bf16 A and B (bits 7, 10), B MN-major (bit 16),
// N / 8 at bit 17, M / 16 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// The largest of three in one instruction.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two 32-bit lanes in one instruction: (x0, x1) = (x0, x1) * c + d, and (s0, s1) += (x0, x1).
__device__ __forceinline__ void fma2(float& x0, float& x1, float c, float d) {
  asm("{\n.reg .b64 a, b, cc, r;\nmov.b64 a, {%0, %1};\nmov.b64 b, {%2, %2};\nmov.b64 cc, {%3, %3};\n"
      "fma.rn.f32x2 r, a, b, cc;\nmov.b64 {%0, %1}, r;\n}\n"
      : "+f"(x0), "+f"(x1) : "f"(c), "f"(d));
}
__device__ __forceinline__ void add2(float& s0, float& s1, float x0, float x1) {
  asm("{\n.reg .b64 a, b, r;\nmov.b64 a, {%0, %1};\nmov.b64 b, {%2, %3};\nadd.rn.f32x2 r, a, b;\nmov.b64 {%0, %1}, r;\n}\n"
      : "+f"(s0), "+f"(s1) : "f"(x0), "f"(x1));
}
// 2^x, one instruction of the special-function unit (2^-inf = 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp16(uint32_t smem, const void* g, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(g), "r"(n) : "memory");
}

// Address of chunk `ch` (16 bytes, 0..15 over the 128 elements of a row) of row `row` in a pair
// of swizzled blocks that starts at `base` (1024-byte aligned).
__device__ __forceinline__ uint32_t sw_addr(uint32_t base, int row, int ch) {
  return base + (ch >> 3) * BLOCK + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
}

// Development aid: with -DATOM_TC_TRACE the first CTA records clock64() at its hand-over points
// into the scratch array (slot * 64 + tile), to see which role the others wait for.
#ifdef ATOM_TC_TRACE
#define TC_TRACE(slot, idx) do { if (blockIdx.x == 0 && blockIdx.y == 0 && p.part_o) reinterpret_cast<long long*>(p.part_o)[(slot) * 64 + (idx)] = clock64(); } while (0)
#else
#define TC_TRACE(slot, idx) do { } while (0)
#endif

struct Bars {
  uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES], s_full[2], p_full, o_full;
  uint32_t tmem_base;
  int aborted;
};

// Tensor maps of the TMA path: the K and V pages as matrices [pages * nkv * page_size, 128] with boxes of
// 64 x min(page_size, 128), and the packed projection output as [tokens][heads][128] with boxes of
// 64 x group x (128 / group), which lands as the CTA's 128 packed rows.
struct Maps {
  CUtensorMap k, v, q;
};

__global__ void __launch_bounds__(NTHREADS, 1)
flash_prefill_tc_kernel(const Params p, int min_rows) {
  static_assert(HD == 128, "the tcgen05 attention kernel is written for head size 128");
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  Bars* bars = reinterpret_cast<Bars*>(smem_raw + (sbase - smem_u32(smem_raw)) + SMEM_DATA);

  // Which (request, 128-row tile) is this CTA?  Requests with fewer than min_rows packed rows
  // belong to the other kernels.  Within a request the last (longest) tiles come first.
  Work w;
  {
    int tile = blockIdx.y, s = 0, nt = 0;   // (blocks are handed out with x fastest: all kv heads of the longest tile first)
    for (; s < p.num_seqs; ++s) {
      const int rows = (p.cu_q[s + 1] - p.cu_q[s]) * p.group;
      nt = rows >= min_rows ? (rows + TM - 1) / TM : 0;
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
    w.row0 = (nt - 1 - tile) * TM;
    w.bt = p.block_table + (int64_t)s * p.max_pages;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_last = min(w.row0 + TM, w.rows_total) - 1;
  const int key_end = w.q_start + row_last / p.group + 1;       // keys [0, key_end) are visible to some row
  const int n_tiles = (key_end + TN - 1) / TN;

  if (threadIdx.x == 0) {
    for (int i = 0; i < K_STAGES; ++i) {
      mbar_init(&bars->k_full[i], LOADERS);
      mbar_init(&bars->k_empty[i], 1);
    }
    for (int i = 0; i < V_STAGES; ++i) {
      mbar_init(&bars->v_full[i], LOADERS);
      mbar_init(&bars->v_empty[i], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_full, 128);
    mbar_init(&bars->o_full, 1);
    bars->aborted = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&bars->tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* aborted = &bars->aborted;

  if (warp >= 4 && warp < MMA_WARP) {
   {
    // ------------------------------------------------------------------ loaders
    constexpr int RSTEP = LOADERS / 16, RPT = 128 / RSTEP;   // a thread's rows are r0, r0 + RSTEP, ...: RPT of them
    const int t = threadIdx.x - 128;               // 0 .. LOADERS - 1
    const int ch = t & 15, r0 = t >> 4;            // chunk of a row (RSTEP is a multiple of 8: row & 7 == r0 & 7)
    const uint32_t head_stride = (uint32_t)p.page_size * 16;    // 16-byte units
    const uint32_t page_stride = head_stride * (uint32_t)p.nkv;
    const uint4* kp = reinterpret_cast<const uint4*>(p.k_pages);
    const uint4* vp = reinterpret_cast<const uint4*>(p.v_pages);
    // Q: rows of this CTA (zero beyond the request's last row)
#pragma unroll 4
    for (int i = 0; i < RPT; ++i) {
      const int row = r0 + RSTEP * i, R = w.row0 + row;
      const bool valid = R < w.rows_total;
      int64_t off = 0;
      if (valid) {
        const int tok = R / p.group, hig = R - tok * p.group;
        off = (int64_t)(w.q_begin + tok) * p.q_stride + (int64_t)(w.kvh * p.group + hig) * HD + ch * 8;
      }
      cp16(sw_addr(sbase + SMEM_Q, row, ch), p.q + off, valid);
    }
    // The loader keeps copies of later tiles in flight while earlier ones are computed on (an L2
    // hit takes over a thousand cycles): every tile half (K or V) is one cp.async group, issued
    // as soon as its stage is free.  The page ids a
    // thread needs for a tile are read one tile ahead, so no copy waits for a table lookup.
    // Order of issue: K0 (with Q), V0, K1, V1, K2, V2, K3, ...   (group g: g = 0 is K0, odd g is
    // V((g - 1) / 2), even g is K(g / 2)).
    const uint32_t fixed = (uint32_t)w.kvh * head_stride + ch;
    const uint32_t srow_off = (ch >> 3) * BLOCK + (((ch & 7) ^ (r0 & 7)) << 4);   // row & 7 == r0 & 7
    auto fetch_pages = [&](int j, int* pg) {          // page of each of this thread's rows of tile j (-1: none)
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int key = j * TN + r0 + RSTEP * i;
        pg[i] = -1;
        if (j < n_tiles && key < key_end) {
          const int lp = p.page_shift >= 0 ? (key >> p.page_shift) : (key / p.page_size);
          pg[i] = __ldg(w.bt + lp);
        }
      }
    };
    auto issue = [&](const uint4* pages, uint32_t dst, int j, const int* pg) {
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int row = r0 + RSTEP * i;
        const int key = j * TN + row;
        const int lp = p.page_shift >= 0 ? (key >> p.page_shift) : (key / p.page_size);
        const bool valid = pg[i] >= 0;
        const uint32_t off = valid ? (uint32_t)pg[i] * page_stride + (uint32_t)(key - lp * p.page_size) * 16 + fixed : 0u;
        cp16(dst + srow_off + row * 128, pages + off, valid);
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    // A group is published by the hardware: the thread's arrival on the stage's barrier is
    // triggered when all copies it has issued so far have landed (no thread waits for them).
    auto arrive_when_landed = [&](uint64_t* bar) {
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
    };
    int pg_k[RPT], pg_v[RPT];
    fetch_pages(0, pg_k);
#pragma unroll
    for (int i = 0; i < RPT; ++i) pg_v[i] = pg_k[i];
    const int n_groups = 2 * n_tiles;     // K0, V0, K1, V1, ...: K(j) is group 2 j, V(j) group 2 j + 1
#pragma unroll 1
    for (int g = 0; g < n_groups; ++g) {
      const bool is_k = (g & 1) == 0;
      const int j = g >> 1;
      if (is_k) {
        if (j >= K_STAGES) mbar_wait(&bars->k_empty[j % K_STAGES], ((j / K_STAGES) & 1) ^ 1, aborted, p.error);
        if (t == 0) TC_TRACE(11, j);
        issue(kp, sbase + SMEM_K + (j % K_STAGES) * 2 * BLOCK, j, pg_k);
        arrive_when_landed(&bars->k_full[j % K_STAGES]);
        if (t == 0) TC_TRACE(12, j);
        fetch_pages(j + 1, pg_k);         // for K(j + 1), two groups from now
      } else {
        if (j >= V_STAGES) mbar_wait(&bars->v_empty[j % V_STAGES], ((j / V_STAGES) & 1) ^ 1, aborted, p.error);
        if (t == 0) TC_TRACE(8, j);
        issue(vp, sbase + SMEM_V + (j % V_STAGES) * 2 * BLOCK, j, pg_v);
        arrive_when_landed(&bars->v_full[j % V_STAGES]);
        if (t == 0) TC_TRACE(10, j);
        fetch_pages(j + 1, pg_v);
      }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");   // nothing of this thread is in flight when it leaves
   }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = instr_desc(TM, TN, false), idesc_o = instr_desc(TM, HD, true);
      auto issue_s = [&](int j) {
        const int st = j % K_STAGES;
        mbar_wait(&bars->k_full[st], (j / K_STAGES) & 1, aborted, p.error);
        tc_fence_after();
        TC_TRACE(6, j);
        const uint32_t d = tmem + ((j & 1) ? S_COL1 : S_COL0);
        const uint32_t qa = sbase + SMEM_Q, ka = sbase + SMEM_K + st * 2 * BLOCK;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t o = (ks >> 2) * BLOCK + (ks & 3) * 32;
          umma(d, smem_desc(qa + o, 16, 1024), smem_desc(ka + o, 16, 1024), idesc_s, ks > 0);
        }
        umma_commit(&bars->s_full[j & 1]);
        umma_commit(&bars->k_empty[st]);
      };
      if (n_tiles > 0) issue_s(0);
      for (int j = 0; j < n_tiles; ++j) {
        if (j + 1 < n_tiles) issue_s(j + 1);
        const int st = j % V_STAGES;
        mbar_wait(&bars->v_full[st], (j / V_STAGES) & 1, aborted, p.error);
        mbar_wait(&bars->p_full, j & 1, aborted, p.error);
        tc_fence_after();
        TC_TRACE(7, j);
        const uint32_t pa = sbase + SMEM_P, va = sbase + SMEM_V + st * 2 * BLOCK;
#pragma unroll
        for (int ks = 0; ks < TN / 16; ++ks) {
          // P: K-major along the keys; V: MN-major, 16 keys are 2048 bytes further, the second
          // 64 of the head size one block further.
          umma(tmem + O_COL, smem_desc(pa + (ks >> 2) * BLOCK + (ks & 3) * 32, 16, 1024),
               smem_desc(va + ks * 2048, BLOCK, 1024), idesc_o, (j > 0 || ks > 0));
        }
        umma_commit(&bars->v_empty[st]);
        umma_commit(&bars->o_full);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax and epilogue
    const int r = threadIdx.x;                       // row of the tile = TMEM lane
    const int R = w.row0 + r;
    const int pos = R < w.rows_total ? w.q_start + R / p.group : -1;
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    const float c = p.scale_log2;
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < n_tiles; ++j) {
      if (threadIdx.x == 0) TC_TRACE(0, j);
      mbar_wait(&bars->s_full[j & 1], (j >> 1) & 1, aborted, p.error);
      tc_fence_after();
      if (threadIdx.x == 0) TC_TRACE(1, j);
     {
      // Two passes over the row in tensor memory, 32 columns at a time (few live registers, the
      // next chunk's load in flight while this one is worked on): first the maximum, then P.
      const uint32_t scol = tmem + lane_base + ((j & 1) ? S_COL1 : S_COL0);
      const int key0 = j * TN;
      const bool diag = key0 + TN - 1 > pos;   // the diagonal crosses this tile for this row (or the row does not exist)
      float buf[2][32];
      float mx4[4] = {m, -INFINITY, -INFINITY, -INFINITY};
      tmem_ld32(scol, buf[0]);
#pragma unroll 2
      for (int q = 0; q < TN / 32; ++q) {
        float* cur = buf[q & 1];
        tmem_wait_ld();
        if (q + 1 < TN / 32) tmem_ld32(scol + (q + 1) * 32, buf[(q + 1) & 1]);
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + q * 32 + i > pos) cur[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx4[0] = fmaxf(mx4[0], cur[i]);
          mx4[1] = fmaxf(mx4[1], cur[i + 1]);
          mx4[2] = fmaxf(mx4[2], cur[i + 2]);
          mx4[3] = fmaxf(mx4[3], cur[i + 3]);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = ex2((m - m_use) * c);
      const float mc = m_use * c;
      if (threadIdx.x == 0) TC_TRACE(2, j);
      tmem_ld32(scol, buf[0]);                 // first chunk of the second pass, in flight during the wait below
      // O of the tile before and the P buffer are free when that tile's second MMA is done.
      if (threadIdx.x == 0) TC_TRACE(3, j);
      if (j > 0) {
        mbar_wait(&bars->o_full, (j - 1) & 1, aborted, p.error);
        tc_fence_after();
        if (threadIdx.x == 0) TC_TRACE(4, j);
        if (__any_sync(0xffffffffu, mx > m)) {      // some row of this warp has a new maximum: rescale O
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < HD / 32; ++q) {
            float* o = buf[1];
            tmem_ld32(tmem + lane_base + O_COL + q * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(tmem + lane_base + O_COL + q * 32, o);
          }
          tmem_wait_st();
        }
      }
      m = mx;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int q = 0; q < TN / 32; ++q) {
        float* cur = buf[q & 1];
        tmem_wait_ld();
        if (q + 1 < TN / 32) tmem_ld32(scol + (q + 1) * 32, buf[(q + 1) & 1]);
        if (diag) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + q * 32 + i > pos) cur[i] = -INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            cur[i + e] = ex2(fmaf(cur[i + e], c, -mc));
            sum4[e] += cur[i + e];
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(cur[8 * k + 2 * e], cur[8 * k + 2 * e + 1]);
            pk[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          const uint32_t a = sw_addr(sbase + SMEM_P, r, q * 4 + k);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(a), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]),
                       "r"(pk[3])
                       : "memory");
        }
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
     }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_full);
      if (threadIdx.x == 0) TC_TRACE(5, j);
    }
    // epilogue: O / l -> bf16 -> global
    if (n_tiles > 0) {
      mbar_wait(&bars->o_full, (n_tiles - 1) & 1, aborted, p.error);
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = nullptr;
      if (R < w.rows_total) {
        const int tok = R / p.group, hig = R - tok * p.group;
        orow = p.out + ((int64_t)(w.q_begin + tok) * p.nh + (w.kvh * p.group + hig)) * HD;
      }
#pragma unroll
      for (int q = 0; q < HD / 32; ++q) {
        float o[32];
        tmem_ld32(tmem + lane_base + O_COL + q * 32, o);
        tmem_wait_ld();
        if (orow != nullptr && !*aborted) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(o[8 * k + 2 * e] * inv, o[8 * k + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(orow + q * 32 + k * 8) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tc
}  // namespace flash
}  // namespace atom
