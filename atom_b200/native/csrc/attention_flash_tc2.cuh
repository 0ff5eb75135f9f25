// Paged causal attention for long portions on tcgen05, two query tiles per CTA: head size 128,
// bf16, pages of a power of two of 8 to 128 tokens, a group size that divides 128 (the sizes
// whose pages and packed query rows come as TMA boxes).  Included by attention_flash.cu after
// attention_flash_tc.cuh, whose primitives it uses.
//
// One CTA takes 256 packed query rows (row = token * G + head in group) of one (request, kv
// head) as two tiles A and B of 128 rows, and walks over the request's keys in tiles of 128:
//     S_X = Q_X K^T     tcgen05.mma, operands from shared memory, S_X (128 x 128, 32-bit) in
//                       tensor memory, one buffer per query tile
//     P_X = softmax     two warpgroups per query tile, two threads per row (each takes 64 of the
//                       128 keys: tcgen05.ld of its half row, the two halves' maxima exchanged
//                       through shared memory, running maximum and sums in 32-bit); P_X goes
//                       back into the first 64 columns of S_X as bf16 pairs
//     O_X += P_X V      tcgen05.mma with A from tensor memory, V as it lies in the pages
// The single MMA-issuing thread alternates between the tiles, S_A(0) S_B(0) | PV_A(0) S_A(1)
// | PV_B(0) S_B(1) | PV_A(1) ..., so while one warpgroup computes exponentials the tensor
// cores work for the other tile, and every K and V tile that comes into shared memory is used
// for twice the rows.  Tensor memory: S_A, S_B, O_A, O_B = 512 columns.  Shared memory: Q 64 KB,
// two stages of K and of V, 32 KB each.
// Warps 0-7 softmax and epilogue of tile A (0-3 the keys 0..63 of a key tile, 4-7 the keys 64..127),
// warps 8-15 of tile B (warp w owns TMEM lanes 32 (w mod 4) ...; a thread holds its half row of S in
// registers; the fifth warpgroup cedes registers to these four with setmaxnreg), warp 16 issues the TMA
// boxes, warp 17 allocates tensor memory and issues every MMA from one thread, warps 18 and 19 only fill
// the fifth warpgroup.  A tile's exponentials (one special-function operation per score, the unit
// does 16 a clock) thus run on all four schedulers at once, which halves the time a tile's chain
// softmax -> PV -> next S spends in its softmax.
// All waits are bounded; tensor memory is freed on every path.
#pragma once
#include "attention_flash_tc.cuh"

namespace atom {
namespace flash {
namespace tc2 {

using namespace atom::flash::tc;

constexpr int ROWS2 = 2 * TM;                 // packed query rows per CTA
constexpr int NTHREADS2 = 640;                // four softmax warpgroups and a fifth with the loader warp and the MMA warp
// Registers per thread after the warpgroups have traded them.  setmaxnreg.inc waits, without a bound, until the
// CTA's own pool (threads x registers per thread at launch) has that many to give, so the sum must fit the pool:
// 512 x 104 + 128 x 64 = 640 x 96; the launch code checks the compiled kernel's register count against it.
constexpr int SOFTMAX_REGS = 104, OTHER_REGS = 64, LAUNCH_REGS = 96;
static_assert(16 * 32 * SOFTMAX_REGS + 4 * 32 * OTHER_REGS <= 640 * LAUNCH_REGS, "the warpgroups' registers exceed the CTA's pool");
constexpr int SOFTMAX_WARPS = 16, LOAD_WARP = 16, MMA_WARP2 = 17;
constexpr int HALF = TN / 2;                  // keys of a thread per key tile
constexpr int KV_STAGES = 2;
constexpr uint32_t SA_COL = 0, SB_COL = 128, OA_COL = 256, OB_COL = 384;
// shared memory: Q_A, Q_B (2 blocks each), K stages (2 blocks each), V stages (2 blocks each)
constexpr int S2_Q = 0, S2_K = 4 * BLOCK, S2_V = S2_K + KV_STAGES * 2 * BLOCK, S2_DATA = S2_V + KV_STAGES * 2 * BLOCK;
constexpr size_t smem_bytes2() { return 1024 + S2_DATA + 256 + 2 * 2 * 2 * TM * 4; }

struct Bars2 {
  uint64_t q_full, k_full[KV_STAGES], k_empty[KV_STAGES], v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], p_full[2], o_full[2];   // [0] tile A, [1] tile B
  uint32_t tmem_base;
  int aborted;
  float xch[2][2][2][TM];                     // [step parity][query tile][half][row]: the halves' row maxima (at the end: sums)
};

__global__ void __launch_bounds__(NTHREADS2, 1)
flash_prefill_tc2_kernel(const Params p, int min_rows, const __grid_constant__ Maps maps) {
  static_assert(HD == 128, "the tcgen05 attention kernel is written for head size 128");
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  Bars2* bars = reinterpret_cast<Bars2*>(smem_raw + (sbase - smem_u32(smem_raw)) + S2_DATA);

  // Which (request, 256-row tile) is this CTA?  Requests with fewer than min_rows packed rows
  // belong to the other kernels.  Within a request the last (longest) tiles come first.  The
  // grid is sized for 128-row tiles, an upper bound: CTAs beyond the last tile leave at once.
  Work w;
  {
    int tile = blockIdx.y, s = 0, nt = 0;   // (blocks are handed out with x fastest: all kv heads of the longest tile first)
    for (; s < p.num_seqs; ++s) {
      const int rows = (p.cu_q[s + 1] - p.cu_q[s]) * p.group;
      nt = rows >= min_rows ? (rows + ROWS2 - 1) / ROWS2 : 0;
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
    w.row0 = (nt - 1 - tile) * ROWS2;
    w.bt = p.block_table + (int64_t)s * p.max_pages;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key tiles of each query tile (0: the tile has no row)
  int n_of[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int first = w.row0 + x * TM;
    if (first >= w.rows_total) {
      n_of[x] = 0;
    } else {
      const int last = min(first + TM, w.rows_total) - 1;
      n_of[x] = (w.q_start + last / p.group + 1 + TN - 1) / TN;
    }
  }
  const int n_tiles = max(n_of[0], n_of[1]);     // (tile B sees at least the keys tile A sees)
  const int key_end = w.q_start + (min(w.row0 + ROWS2, w.rows_total) - 1) / p.group + 1;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&bars->s_full[x], 1);
      mbar_init(&bars->p_full[x], 256);
      mbar_init(&bars->o_full[x], 1);
    }
    bars->aborted = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP2) tmem_alloc(&bars->tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* aborted = &bars->aborted;
  // The softmax threads hold a whole row of S (128 values) in registers: the third warpgroup gives
  // up registers it does not need and the softmax warpgroups take them.
  if (warp >= SOFTMAX_WARPS) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(OTHER_REGS));
   if (warp == LOAD_WARP) {
    // ------------------------------------------------------------------ loader: TMA boxes
    // A tile of 128 keys is 128 / page_size pages (or part of one page when pages are larger);
    // every page gives two boxes, one per 64-element half of the head.  Lane l issues box l.
    const int ps = p.page_size;
    const int box_rows = ps < TN ? ps : TN;
    const int ppt = TN / box_rows;                   // pages (boxes per half) of a tile
    const int n_ops = 2 * ppt;
    const int my_pg = lane >> 1, my_half = lane & 1;
    const bool active = lane < n_ops;
    // Row of the page matrix where this lane's box of tile j starts.  Pages beyond the last key
    // are replaced by the request's first page: finite values that the causal mask removes.
    auto box_row = [&](int j) -> int {
      const int key = j * TN + my_pg * box_rows;
      int lp = p.page_shift >= 0 ? (key >> p.page_shift) : (key / ps);
      int in_page = key - lp * ps;
      if (key >= key_end) { lp = 0; in_page = 0; }
      const int page = active ? __ldg(w.bt + lp) : 0;
      return (page * p.nkv + w.kvh) * ps + in_page;
    };
    if (lane < 4) {   // Q: each 128-row tile is 128 / group tokens of the group's heads, two 64-column boxes
      if (lane == 0) atom::tma::mbar_expect_tx(&bars->q_full, 4 * BLOCK);
      __syncwarp(0xfu);
      const int x = lane >> 1, half = lane & 1;
      // a tile without rows still gets a box (of rows that exist or of the fill value): the byte count stays fixed
      const int tok0 = w.q_begin + min(w.row0 + x * TM, max(w.rows_total - 1, 0)) / p.group;
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::
              "r"(sbase + S2_Q + (x * 2 + half) * BLOCK),
          "l"(&maps.q), "r"(half * 64), "r"(w.kvh * p.group), "r"(tok0), "r"(smem_u32(&bars->q_full))
          : "memory");
    }
    int row_k = box_row(0), row_v = row_k;
    const int n_groups = 2 * n_tiles;     // K0, V0, K1, V1, ...
#pragma unroll 1
    for (int g = 0; g < n_groups; ++g) {
      const bool is_k = (g & 1) == 0;
      const int j = g >> 1, st = j % KV_STAGES;
      uint64_t* full = is_k ? &bars->k_full[st] : &bars->v_full[st];
      if (j >= KV_STAGES)
        mbar_wait(is_k ? &bars->k_empty[st] : &bars->v_empty[st], ((j / KV_STAGES) & 1) ^ 1, aborted, p.error);
      if (lane == 0) atom::tma::mbar_expect_tx(full, 2 * BLOCK);
      __syncwarp();
      if (active) {
        const uint32_t dst = sbase + (is_k ? S2_K : S2_V) + st * 2 * BLOCK + my_half * BLOCK + my_pg * box_rows * 128;
        atom::tma::load_box(reinterpret_cast<void*>(0), is_k ? &maps.k : &maps.v, my_half * 64, is_k ? row_k : row_v, full, dst);
      }
      if (is_k) row_k = box_row(j + 1); else row_v = box_row(j + 1);   // looked up a tile ahead
    }
  } else if (warp == MMA_WARP2) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = instr_desc(TM, TN, false), idesc_o = instr_desc(TM, HD, true);
      const uint32_t s_col[2] = {SA_COL, SB_COL}, o_col[2] = {OA_COL, OB_COL};
      int k_ready = -1;     // the last K tile whose arrival has been waited for
      auto issue_s = [&](int x, int j) {
        const int st = j % KV_STAGES;
        if (k_ready < j) {
          mbar_wait(&bars->k_full[st], (j / KV_STAGES) & 1, aborted, p.error);
          tc_fence_after();
          k_ready = j;
        }
        const uint32_t qa = sbase + S2_Q + x * 2 * BLOCK, ka = sbase + S2_K + st * 2 * BLOCK;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t o = (ks >> 2) * BLOCK + (ks & 3) * 32;
          umma(tmem + s_col[x], smem_desc(qa + o, 16, 1024), smem_desc(ka + o, 16, 1024), idesc_s, ks > 0);
        }
        umma_commit(&bars->s_full[x]);
      };
      // K(j) is free when the last S of tile j has been issued and completed: tile B's if it has that tile,
      // else tile A's.
      auto last_user = [&](int j) { return j < n_of[1] ? 1 : 0; };
      auto issue_pv = [&](int x, int j) {
        const int st = j % KV_STAGES;
        mbar_wait(&bars->p_full[x], j & 1, aborted, p.error);
        tc_fence_after();
        const uint32_t va = sbase + S2_V + st * 2 * BLOCK;
#pragma unroll
        for (int ks = 0; ks < TN / 16; ++ks)
          umma_ts(tmem + o_col[x], tmem + s_col[x] + ks * 8, smem_desc(va + ks * 2048, BLOCK, 1024), idesc_o,
                  (j > 0 || ks > 0));
        umma_commit(&bars->o_full[x]);
      };
      mbar_wait(&bars->q_full, 0, aborted, p.error);
      for (int x = 0; x < 2; ++x)
        if (n_of[x] > 0) {
          issue_s(x, 0);
          if (last_user(0) == x) umma_commit(&bars->k_empty[0]);
        }
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % KV_STAGES;
        bool v_waited = false;
        for (int x = 0; x < 2; ++x) {
          if (j >= n_of[x]) continue;
          if (!v_waited) {
            mbar_wait(&bars->v_full[st], (j / KV_STAGES) & 1, aborted, p.error);
            v_waited = true;
          }
          issue_pv(x, j);
          if (last_user(j) == x) umma_commit(&bars->v_empty[st]);
          if (j + 1 < n_of[x]) {
            issue_s(x, j + 1);
            if (last_user(j + 1) == x) umma_commit(&bars->k_empty[(j + 1) % KV_STAGES]);
          }
        }
      }
    }
   }
  } else {
    // ------------------------------------------------------------------ softmax and epilogue of tile x, keys / columns of half c
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(SOFTMAX_REGS));
    const int x = warp >> 3, c2 = (warp >> 2) & 1;
    const int r = (warp & 3) * 32 + lane;            // row of the tile = TMEM lane
    const int R = w.row0 + x * TM + r;
    const int pos = R < w.rows_total ? w.q_start + R / p.group : -1;
    const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
    const uint32_t scol = tmem + lane_base + (x ? SB_COL : SA_COL);
    const uint32_t ocol = tmem + lane_base + (x ? OB_COL : OA_COL) + c2 * (HD / 2);
    const int pair_bar = 1 + x * 4 + (warp & 3);     // named barrier of the two warps that share these 32 rows
    const float c = p.scale_log2;
    const int n_mine = n_of[x];
    float m = -INFINITY, l = 0.f;                    // l: the sum over this thread's keys only
    for (int j = 0; j < n_mine; ++j) {
      if (r == 0 && c2 == 0) TC_TRACE(x * 4 + 0, j);
      mbar_wait(&bars->s_full[x], j & 1, aborted, p.error);
      tc_fence_after();
      if (r == 0 && c2 == 0) TC_TRACE(x * 4 + 1, j);
      const int key0 = j * TN + c2 * HALF;
      const bool diag = key0 + HALF - 1 > pos;   // the diagonal crosses this half tile for this row (or the row does not exist)
      // the half row in registers: one round trip to tensor memory per tile
      float s[HALF];
#pragma unroll
      for (int q = 0; q < HALF / 32; ++q) tmem_ld32(scol + c2 * HALF + q * 32, s + q * 32);
      tmem_wait_ld();
      if (diag) {
#pragma unroll
        for (int i = 0; i < HALF; ++i)
          if (key0 + i > pos) s[i] = -INFINITY;
      }
      float mx8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) mx8[e] = -INFINITY;
#pragma unroll
      for (int i = 0; i < HALF; i += 16) {
#pragma unroll
        for (int e = 0; e < 8; ++e) mx8[e] = max3(mx8[e], s[i + e], s[i + 8 + e]);
      }
      float mt = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]));
      // The row's maximum over both halves.  After this barrier both threads of the row have read their
      // scores, so the first 64 columns of S may take P.
      bars->xch[j & 1][x][c2][r] = mt;
      asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
      mt = fmaxf(mt, bars->xch[j & 1][x][c2 ^ 1][r]);
      // The exponent's offset m follows the row maximum lazily: it moves (and O and l are rescaled)
      // only when the maximum has outgrown it by more than 2^8, so P stays below 256 and most tiles
      // need no pass over O.  The quotient O / l does not depend on the offset.  Both threads of a row
      // see the same maxima and decide alike.
      const bool grow = (mt - m) * c > 8.f || (m == -INFINITY && mt != -INFINITY);
      const bool rescale = __any_sync(0xffffffffu, grow);
      const float mx = rescale ? fmaxf(m, mt) : m;
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = ex2((m - m_use) * c);     // 1 where the offset stays (2^-inf = 0 where it was -inf: O and l are 0 there)
      const float mc = m_use * c;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < HALF; i += 4) {      // (the softmax warps are bound by the instructions they issue: two lanes per FMA and per add)
        fma2(s[i], s[i + 1], c, -mc);
        fma2(s[i + 2], s[i + 3], c, -mc);
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i + e] = ex2(s[i + e]);
        add2(sum4[0], sum4[1], s[i], s[i + 1]);
        add2(sum4[2], sum4[3], s[i + 2], s[i + 3]);
      }
      if (r == 0 && c2 == 0) TC_TRACE(x * 4 + 2, j);
      m = mx;
      // P as bf16 pairs into the first 64 columns of the same buffer: this thread's 64 keys are 32 columns
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(s[q * 32 + 2 * e], s[q * 32 + 2 * e + 1]);
          pk[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        tmem_st16(scol + c2 * 32 + q * 16, pk);
      }
      // O of the tile before: its MMA was issued before this tile's S, so it is complete by now; the
      // wait only makes that visible to this thread.  (After P has left the registers, before the word
      // that lets the next product add to O.)
      if (j > 0) {
        mbar_wait(&bars->o_full[x], (j - 1) & 1, aborted, p.error);
        tc_fence_after();
        if (rescale) {      // some row of this warp moves its offset: rescale this thread's half of O
#pragma unroll
          for (int q = 0; q < HD / 64; ++q) {
            float o[32];
            tmem_ld32(ocol + q * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(ocol + q * 32, o);
          }
        }
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars->p_full[x]);
      if (r == 0 && c2 == 0) TC_TRACE(x * 4 + 3, j);
    }
    // epilogue: O / l -> bf16 -> global, this thread's 64 columns of the row
    if (n_mine > 0) {
      bars->xch[n_mine & 1][x][c2][r] = l;
      asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
      l += bars->xch[n_mine & 1][x][c2 ^ 1][r];
      mbar_wait(&bars->o_full[x], (n_mine - 1) & 1, aborted, p.error);
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = nullptr;
      if (R < w.rows_total) {
        const int tok = R / p.group, hig = R - tok * p.group;
        orow = p.out + ((int64_t)(w.q_begin + tok) * p.nh + (w.kvh * p.group + hig)) * HD + c2 * (HD / 2);
      }
#pragma unroll
      for (int q = 0; q < HD / 64; ++q) {
        float o[32];
        tmem_ld32(ocol + q * 32, o);
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
  if (warp == MMA_WARP2) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace tc2
}  // namespace flash
}  // namespace atom
