// Matrix product for many rows on the 5th-generation tensor cores, two CTAs to a tile (tcgen05 with
// cta_group::2), bf16 in, 32-bit sums in tensor memory, bf16 out:
//     plain:   C[M, N] = X[M, K] W[N, K]^T
//     gated:   W = [gate ; up] of N rows each, C[M, N] = silu(X gate^T) * (X up^T)
// It is the prefill feed-forward's first product with the activation in its epilogue: the sums never
// leave the chip, and the activation kernel with its pass over [M, 2N] goes away.
//
// A pair of CTAs (a cluster of two) owns a tile of 256 rows x 512 columns of sums, held as two halves of
// 256 columns that share the X blocks.  CTA r of the pair loads rows 128 r .. 128 r + 127 of the tile's X
// rows and, for each half, 128 rows of W; one thread of the pair's first CTA issues MMAs of 256 x 256 x 16
// that read both CTAs' shared memory, and every CTA finds its 128 rows x 512 columns in its own tensor
// memory.  Against a tile of 256 x 256 per pair this needs a quarter fewer bytes per MMA: with the
// smaller tile the TMA unit (about 64 bytes a clock into an SM) was as busy as the tensor cores.
// A half stands alone: in a gated product its columns 0..127 hold the gate sums and 128..255 the up sums
// of the same 128 outputs (the pair's first CTA loads the gate rows, the second the up rows), so a tile
// can be handed out as two work items, which is done for the last, ragged wave of tiles.
//
// Roles in a CTA of 384 threads: warps 0, 10 and 11 each load one block of a stage (X, W of half 0, W of
// half 1) with TMA, the bytes of both CTAs counted at the first CTA's barrier; warp 1 allocates tensor
// memory and (first CTA) issues the MMAs; warps 2-9 read the sums (a warp may read the quarter of the
// tensor memory's lanes that its index selects), apply the epilogue and write blocks of 128 rows x 64
// columns to shared memory, from where TMA stores take them (rows and columns beyond the matrix are cut
// off by the store, rows and columns beyond X and W are read as zeros).  The tensor memory is full with
// one tile, so the MMAs of a tile wait until the epilogue of the one before has read the sums (a gated
// tile's outputs fit in registers as bf16, so its stores come after that); the loads do not wait.
// All waits are bounded (tma.cuh); tensor memory is freed on every path.
#include "tma.cuh"
#include <cuda_bf16.h>

namespace atom {
namespace pairs {

using namespace atom::tma;

constexpr int STAGES = 4;
constexpr int BLK = 128 * 64 * 2;               // one [128][64] bf16 block, 128-byte swizzle
constexpr int STAGE_BYTES = 3 * BLK;            // the X block and the W blocks of the two halves
constexpr int OUT_OFF = STAGES * STAGE_BYTES;   // two blocks of output on their way to global memory
constexpr int BARS_OFF = OUT_OFF + 2 * BLK;
constexpr int NTHREADS = 384;
constexpr int EPI_THREADS = 256;
constexpr int MMA_WARP = 1, EPI_WARP0 = 2, W_WARP0 = 10;

struct Bars {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int aborted;
};
constexpr size_t SMEM = 1024 + BARS_OFF + 256;

struct Params {
  int M, N, K;        // N: columns of C (gated: W has 2 N rows)
  int mt, nt;         // tiles of 256 rows, tiles of 512 columns of sums
  int full_items;     // work items [0, full_items) are whole tiles, the others halves of the tiles that follow
  int items;
  int* error;
};

// ---- the cluster
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
// The address, in the cluster's window, of the same place in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t d;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(d) : "r"(addr), "r"(rank));
  return d;
}
__device__ __forceinline__ void arrive_at(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded like tma::mbar_wait, for a barrier at which the other CTA arrives.
__device__ __forceinline__ void wait_cluster(uint64_t* bar, uint32_t parity, volatile int* aborted, int* error) {
  const int limit = *aborted ? 64 : (1 << 24);
  for (int i = 0; i < limit; ++i)
    if (try_wait_cluster(bar, parity)) return;
  *aborted = 1;
  atomicExch(error, 2);
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// ---- TMA
// A box into this CTA's shared memory; its bytes are counted at `bar_cluster`, a barrier of the pair's
// first CTA given by its address in the cluster's window.
__device__ __forceinline__ void load_box_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
// A block of shared memory to the box at (column x, row y) of the mapped matrix; x and y are never negative.
__device__ __forceinline__ void store_box(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n" ::"l"(map), "r"(x),
               "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// All but the newest group of this thread's stores have read their source.
__device__ __forceinline__ void stores_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory"); }
__device__ __forceinline__ void stores_done() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(EPI_THREADS) : "memory"); }

// ---- tcgen05 for a pair of CTAs
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// D[tmem of both CTAs] (+)= A * B: 256 x 256 x 16; each CTA gives 128 rows of A and 128 rows of B from the
// same place in its shared memory and receives its 128 rows of D.
__device__ __forceinline__ void umma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// One arrival at the barrier at this address in both CTAs when every MMA issued so far has completed.
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::
                   "r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
// 32 consecutive 32-bit columns of this thread's lane of the tensor memory.
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
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// Shared-memory matrix descriptor of a K-major [rows][64] block in the 128-byte swizzle: start address / 16,
// leading offset (unused) / 16 at bit 16, 1024 bytes between 8-row groups / 16 at bit 32, version 1 at bit 46,
// layout 2 (128-byte swizzle) at bit 61.  16 elements further along K: + 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: 32-bit sums (bit 4), bf16 A and B (bits 7, 10), both K-major, N / 8 at bit 17, M / 16 at bit 24.
__device__ __forceinline__ uint32_t instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// x * sigmoid(x) as x (0.5 + 0.5 tanh(x / 2)): one special-function operation.
__device__ __forceinline__ float silu(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(t) : "f"(0.5f * x));
  return x * (0.5f + 0.5f * t);
}

struct Item {
  int tile;
  bool h0, h1;   // which halves of the tile
};
__device__ __forceinline__ Item item_of(const Params& p, int i) {
  Item w;
  if (i < p.full_items) {
    w.tile = i; w.h0 = w.h1 = true;
  } else {
    const int j = i - p.full_items;
    w.tile = p.full_items + (j >> 1); w.h0 = (j & 1) == 0; w.h1 = !w.h0;
  }
  return w;
}

template <bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
gemm_pairs_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW,
                  const __grid_constant__ CUtensorMap mapC, const Params p) {
  atom::pdl_trigger();
  extern __shared__ unsigned char smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  Bars* bars = reinterpret_cast<Bars*>(smem_raw + (sbase - smem_u32(smem_raw)) + BARS_OFF);
  volatile int* aborted = &bars->aborted;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int KT = (p.K + 63) / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&bars->acc_full[h], 1);
      mbar_init(&bars->acc_empty[h], 2 * (EPI_THREADS / 32));     // the epilogue warps of both CTAs
    }
    bars->aborted = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc_pair(&bars->tmem_base, 512);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything arrives at them
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0 || warp >= W_WARP0) {
    // ------------------------------------------------------------------ loaders: one block of every stage each
    if (lane == 0) {
      const int which = warp == 0 ? 0 : warp - W_WARP0 + 1;       // 0: X, 1: W of half 0, 2: W of half 1
      const CUtensorMap* map = which == 0 ? &mapX : &mapW;
      prefetch_map(map);
      if (which == 0) atom::pdl_wait();      // X is written by the kernel before this one; W is not
      int it = 0;
      for (int i = pair; i < p.items; i += n_pairs) {
        const Item w = item_of(p, i);
        const int m0 = (w.tile % p.mt) * 256, nti = w.tile / p.mt;
        const bool mine = which == 0 || (which == 1 ? w.h0 : w.h1);
        const uint32_t bytes = 2 * BLK * (1 + (int)w.h0 + (int)w.h1);
        int row;
        if (which == 0) row = m0 + 128 * (int)rank;
        else if (GATED) row = (int)rank * p.N + nti * 256 + (which - 1) * 128;
        else row = nti * 512 + (which - 1) * 256 + 128 * (int)rank;
        for (int kt = 0; kt < KT; ++kt, ++it) {
          if (!mine) continue;
          const int s = it % STAGES;
          if (it >= STAGES) mbar_wait(&bars->empty[s], ((it / STAGES) - 1) & 1, aborted, p.error);
          if (which == 0 && rank == 0) mbar_expect_tx(&bars->full[s], bytes);
          load_box_pair(sbase + s * STAGE_BYTES + which * BLK, map, kt * 64, row, map_to_rank(smem_u32(&bars->full[s]), 0));
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer (the pair's first CTA)
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = instr_desc(256, 256);
      int it = 0;
      int used0 = 0, used1 = 0;       // how often a half of the tensor memory has been filled
      for (int i = pair; i < p.items; i += n_pairs) {
        const Item w = item_of(p, i);
        if (w.h0 && used0 > 0) wait_cluster(&bars->acc_empty[0], (used0 - 1) & 1, aborted, p.error);
        if (w.h1 && used1 > 0) wait_cluster(&bars->acc_empty[1], (used1 - 1) & 1, aborted, p.error);
        tc_fence_after();
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = it % STAGES;
          mbar_wait(&bars->full[s], (it / STAGES) & 1, aborted, p.error);
          tc_fence_after();
          const uint32_t a = sbase + s * STAGE_BYTES;
          const uint64_t dx = smem_desc(a), d0 = smem_desc(a + BLK), d1 = smem_desc(a + 2 * BLK);
          const uint32_t acc = kt != 0;
          if (w.h0) {
            umma_pair(tmem, dx, d0, idesc, acc);
            umma_pair(tmem, dx + 2, d0 + 2, idesc, 1);
            umma_pair(tmem, dx + 4, d0 + 4, idesc, 1);
            umma_pair(tmem, dx + 6, d0 + 6, idesc, 1);
          }
          if (w.h1) {
            umma_pair(tmem + 256, dx, d1, idesc, acc);
            umma_pair(tmem + 256, dx + 2, d1 + 2, idesc, 1);
            umma_pair(tmem + 256, dx + 4, d1 + 4, idesc, 1);
            umma_pair(tmem + 256, dx + 6, d1 + 6, idesc, 1);
          }
          commit_pair(&bars->empty[s]);
        }
        if (w.h0) { commit_pair(&bars->acc_full[0]); ++used0; }
        if (w.h1) { commit_pair(&bars->acc_full[1]); ++used1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 8 warps, blocks of 64 output columns
    const int q = warp & 3;                       // the quarter of the tensor memory's lanes this warp may read
    const int ch = (warp - EPI_WARP0) >> 2;       // which 32 of a block's 64 columns this warp writes
    const int r = 32 * q + lane;                  // row of the CTA's 128
    const bool issuer = threadIdx.x == EPI_WARP0 * 32;
    const uint32_t empty0[2] = {map_to_rank(smem_u32(&bars->acc_empty[0]), 0), map_to_rank(smem_u32(&bars->acc_empty[1]), 0)};
    const uint32_t tbase = tmem + ((uint32_t)(32 * q) << 16);
    int used[2] = {0, 0};
    int blocks = 0;                               // output blocks written so far (they alternate between two buffers)
    // 32 values of this thread's row (16 registers of bf16 pairs) into the block buffer, and the block on its way.
    auto put_block = [&](const uint32_t* v, int x, int y) {
      if (issuer && blocks >= 2) stores_read_but_one();   // the store that read this buffer two blocks ago is through with it
      epi_sync();
      const uint32_t buf = sbase + OUT_OFF + (blocks & 1) * BLK;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t dst = buf + r * 128 + (((ch * 4 + c) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "r"(v[4 * c]), "r"(v[4 * c + 1]), "r"(v[4 * c + 2]),
                     "r"(v[4 * c + 3])
                     : "memory");
      }
      fence_async_smem();
      epi_sync();
      if (issuer) {
        if (y < p.M && x < p.N) store_box(&mapC, x, y, buf);
        store_commit();      // (an empty group where nothing of the block lies inside C, so that the count of groups holds)
      }
      ++blocks;
    };
    auto pack = [](const float* v, uint32_t* o) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        o[j] = *reinterpret_cast<uint32_t*>(&h2);
      }
    };
    for (int i = pair; i < p.items; i += n_pairs) {
      const Item w = item_of(p, i);
      const int m0 = (w.tile % p.mt) * 256, nti = w.tile / p.mt;
      const int y = m0 + 128 * (int)rank;
      if (GATED) {
        // First everything out of the tensor memory (a tile's 256 outputs of this thread's row and column half
        // fit in 64 registers as bf16), so that the next tile's MMAs wait for the reads only; then the stores.
        uint32_t o[2][2][16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!(h == 0 ? w.h0 : w.h1)) continue;
          mbar_wait(&bars->acc_full[h], used[h] & 1, aborted, p.error);
          ++used[h];
          tc_fence_after();
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float g[32], u[32];
            tmem_ld32(tbase + h * 256 + b * 64 + ch * 32, g);
            tmem_ld32(tbase + h * 256 + 128 + b * 64 + ch * 32, u);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = silu(g[j]) * u[j];
            pack(g, o[h][b]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) arrive_at(empty0[h]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!(h == 0 ? w.h0 : w.h1)) continue;
#pragma unroll
          for (int b = 0; b < 2; ++b) put_block(o[h][b], nti * 256 + h * 128 + b * 64, y);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (!(h == 0 ? w.h0 : w.h1)) continue;
          mbar_wait(&bars->acc_full[h], used[h] & 1, aborted, p.error);
          ++used[h];
          tc_fence_after();
          for (int b = 0; b < 4; ++b) {
            float v[32];
            uint32_t o[16];
            tmem_ld32(tbase + h * 256 + b * 64 + ch * 32, v);
            tmem_wait_ld();
            if (b == 3) {       // the sums of this half are in registers: the next tile may overwrite them
              tc_fence_before();
              __syncwarp();
              if (lane == 0) arrive_at(empty0[h]);
            }
            pack(v, o);
            put_block(o, nti * 512 + h * 256 + b * 64, y);
          }
        }
      }
    }
    if (issuer) stores_done();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the other CTA's shared memory and tensor memory are in use until both are here
  if (warp == MMA_WARP) tmem_dealloc_pair(tmem, 512);
}

// Pairs of CTAs that the device holds at once.
static int resident_pairs() {
  static int pairs = 0;
  if (pairs == 0) {
    if (cudaFuncSetAttribute(gemm_pairs_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_pairs_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(NTHREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pairs_kernel<true>, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      return 0;
    }
    pairs = n;
  }
  return pairs;
}

}  // namespace pairs
}  // namespace atom

// Pairs of CTAs of a launch (0: the kernel cannot run on this device).
ATOM_EXPORT int atom_gemm_pairs_resident(void) { return atom::pairs::resident_pairs(); }

// 1 if the kernel takes a product of these sizes (N: columns of C).
ATOM_EXPORT int atom_gemm_pairs_supports(int M, int N, int K, int64_t lda, int64_t ldc) {
  return M >= 1 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && lda >= K && ldc % 8 == 0 && ldc >= N &&
         atom::tma::encode_fn() != nullptr;
}

// The work items of a product on `pairs` pairs: whole tiles, and the last, ragged wave in halves where that
// shortens it.  Returns the number of items; *full_items of them are whole tiles.
static int plan_items(int tiles, int pairs, int* full_items) {
  const int rem = tiles % pairs;
  if (tiles > pairs && rem > 0 && 2 * rem <= pairs) {
    *full_items = tiles - rem;
    return tiles + rem;
  }
  *full_items = tiles;
  return tiles;
}

ATOM_EXPORT int atom_gemm_pairs(const void* X, int64_t lda, const void* W, void* out, int64_t ldc, int M, int N, int K,
                                int gated, int* error, cudaStream_t stream) {
  using namespace atom::pairs;
  if (X == nullptr || W == nullptr || out == nullptr || error == nullptr || !atom_gemm_pairs_supports(M, N, K, lda, ldc) ||
      ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0 || ((uintptr_t)out % 16) != 0)
    return ATOM_ERR_ARG;
  int pairs = resident_pairs();
  if (pairs < 1) return ATOM_ERR_LIB;
  CUtensorMap mx, mw, mc;
  if (!atom::tma::cached_map(&mx, X, M, K, lda, 128) || !atom::tma::cached_map(&mw, W, gated ? 2 * (int64_t)N : N, K, K, 128) ||
      !atom::tma::cached_map(&mc, out, M, N, ldc, 128))
    return ATOM_ERR_LIB;
  Params p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.mt = (M + 255) / 256;
  p.nt = gated ? (N + 255) / 256 : (N + 511) / 512;
  p.error = error;
  const int tiles = p.mt * p.nt;
  if (pairs > tiles) pairs = tiles;
  p.items = plan_items(tiles, pairs, &p.full_items);
  if (gated) atom::launch_pdl(gemm_pairs_kernel<true>, dim3(2 * pairs), dim3(NTHREADS), SMEM, stream, mx, mw, mc, p);
  else atom::launch_pdl(gemm_pairs_kernel<false>, dim3(2 * pairs), dim3(NTHREADS), SMEM, stream, mx, mw, mc, p);
  return atom::check_launch();
}
