// Weight-streaming matrix product for few rows (decode):  C[M, N] = X[M, K] * W[N, K]^T, M <= 16.
//
// The time of this product is the time to read W once from HBM, so the kernel is built
// around keeping many bytes in flight per SM.  A persistent CTA takes slabs of W rows over
// all of K.  One producer warp streams a slab (and the matching columns of X) into a ring of
// shared-memory stages with tensor-map TMA loads that complete on an mbarrier; a stage holds
// 256 k elements as four blocks of rows x 64 elements in the 128-byte swizzle, and one load
// operation brings all four (the matrix is mapped as [k chunk][row][64]), because the copy
// engine's rate is counted in operations as much as in bytes.
// Four consumer warps take one box each and feed mma.sync.m16n8k16 with W rows as the 16-row
// operand and the tokens as the 8-column operand, so padding the few tokens to 8 wastes
// tensor flops, not bytes.  At the end of a slab the four warps put their partial sums into
// one of two buffers in shared memory and go on with the next slab at once; a sixth warp adds
// them in a fixed order (the result does not depend on timing) and writes them as bf16 or
// 32-bit, with an optional bias, or, in gated mode, as silu(gate) * up for
// W = [gate rows ; up rows]: the feed-forward's activation never travels through memory.
// The consumers never stand still for an epilogue, so stages are released and loads are asked
// for without a pause: one SM's stream from HBM runs at no more than ~22 bytes a clock, about
// its share of the memory bandwidth, and every pause of it is lost for good.
//
// Work is the sequence of all (slab, 256-k stage) pairs, slab-major, cut into one contiguous
// range per CTA of equal length (+-1 stage), so every CTA streams the same number of bytes
// whatever the number of slabs.  A range may begin and end inside a slab.  Such a slab has
// several contributors: each writes its partial sums to its own slot of a scratch buffer and
// counts itself in; the one that arrives last adds the slots in the order of the ranges (so
// the sum does not depend on who was last), applies the epilogue and clears the counter.
// Nobody waits for anybody.  Without scratch the ranges are rounded to whole slabs.
//
// Takes K that is a multiple of 64 and leading dimensions that are multiples of 8 elements;
// the caller uses the library product for other sizes.  Every mbarrier wait is bounded: when one runs
// out the kernel raises the device error flag and finishes without hanging.
#include <stdlib.h>

#include "gemm_smallm.cuh"

namespace atom {
namespace smallm {

struct Params {
  void* out;
  int out_dtype;
  int64_t ldc;
  const void* bias;
  int bias_dtype;
  int M, N, K;
  int gated;
  int* error;
  int num_slabs;
  long long total;      // stages of all slabs
  float* slots;         // [CTAs][2][8 MT][ROWS] partial sums of ranges that begin or end inside a slab
  int* counters;        // [num_slabs] contributors that have arrived; zero between launches
  int whole_slabs;      // 1: ranges are rounded to whole slabs (no scratch)
};

// First stage of CTA c's range.
__device__ __forceinline__ long long range_begin(const Params& p, int c, int num_kt) {
  if (p.whole_slabs) return ((long long)p.num_slabs * c / gridDim.x) * num_kt;
  return p.total * c / gridDim.x;
}

template <int MT, int RT, int NS>
__global__ void __launch_bounds__(NTHREADS)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   const Params p) {
  atom::pdl_trigger();   // the next kernel may be scheduled; this one waits below, after its first loads of W
  using C = Cfg<MT, RT, NS>;
  constexpr int ROWS = C::ROWS, MP = C::MP, RLD = C::RLD;
  extern __shared__ unsigned char smem_raw[];
  // boxes of the 128-byte swizzle start on 1024-byte boundaries
  unsigned char* ring = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  float* red = reinterpret_cast<float*>(ring + C::RING);   // two buffers [NCONS][MP][RLD]
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + C::RING + C::RED);
  uint64_t* empty = full + NS;
  uint64_t* red_full = empty + NS;     // [2] the consumers have put a segment's sums into the buffer
  uint64_t* red_empty = red_full + 2;  // [2] the epilogue warp has taken them out
  __shared__ int aborted;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    aborted = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NCONS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&red_full[b], NCONS);
      mbar_init(&red_empty[b], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();

  // Rows of W in a slab.  Gated: the first half are gate rows, the second the matching up rows.
  const int out_per_slab = p.gated ? ROWS / 2 : ROWS;
  const int num_kt = (p.K + BK - 1) / BK;
  const long long g_begin = range_begin(p, blockIdx.x, num_kt), g_end = range_begin(p, blockIdx.x + 1, num_kt);

  if (warp == NCONS) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_map(&wmap);
      prefetch_map(&xmap);
    }
    // W is written by no kernel, X by the one before this: the first ring of W loads goes out
    // at once, then the producer waits for the kernels before it, then X follows.
    // One operation per operand and stage: W rows (gate rows when gated), X, and the up rows
    // when gated.  A gated stage is [gate: 4 blocks of ROWS/2 rows][up: the same][X].
    {
      Walk w(g_begin, g_end, num_kt);
      for (int it = 0; it < NS && w.valid(); ++it, w.advance()) {
        const int n0 = w.slab * out_per_slab;
        unsigned char* stage = ring + (size_t)it * C::STAGE;
        if (lane == 0) {
          mbar_expect_tx(&full[it], (uint32_t)C::STAGE);
          load_chunks(stage, &wmap, n0, w.kt * NCONS, &full[it]);
        } else if (lane == 2 && p.gated) {
          load_chunks(stage + NCONS * C::W_BOX / 2, &wmap, p.N + n0, w.kt * NCONS, &full[it]);
        }
      }
    }
    atom::pdl_wait();
    int s = 0, u = 0, it = 0;   // stage s of the ring, in its u-th use
    for (Walk w(g_begin, g_end, num_kt); w.valid(); w.advance(), ++it) {
      const int n0 = w.slab * out_per_slab;
      unsigned char* stage = ring + (size_t)s * C::STAGE;
      const int kc = w.kt * NCONS;
      if (it < NS) {   // W of the first ring is on its way already
        if (lane == 1) load_chunks(stage + NCONS * C::W_BOX, &xmap, 0, kc, &full[s]);
      } else {
        mbar_wait(&empty[s], (u & 1) ^ 1, &aborted, p.error);
        if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)C::STAGE);
        __syncwarp();
        if (lane == 0) {
          load_chunks(stage, &wmap, n0, kc, &full[s]);
        } else if (lane == 1) {
          load_chunks(stage + NCONS * C::W_BOX, &xmap, 0, kc, &full[s]);
        } else if (lane == 2 && p.gated) {
          load_chunks(stage + NCONS * C::W_BOX / 2, &wmap, p.N + n0, kc, &full[s]);
        }
      }
      if (++s == NS) {
        s = 0;
        ++u;
      }
    }
    return;
  }

  const int head_slab = (int)(g_begin / num_kt);
  auto write_out = [&](int m, int col, float v, float uval) {
    if (p.gated) {
      v = v / (1.f + __expf(-v)) * uval;
    } else if (p.bias != nullptr) {
      v += load_as_float(p.bias, p.bias_dtype, col);
    }
    if (p.out_dtype == ATOM_F32)
      reinterpret_cast<float*>(p.out)[(int64_t)m * p.ldc + col] = v;
    else
      reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.ldc + col] = __float2bfloat16_rn(v);
  };
  // Outputs first, first + stride, ... of a slab that this CTA holds whole: the four warps' sums, added in order.
  auto write_whole = [&](const float* rb, int n0, int first, int stride) {
    const int n_out = out_per_slab * p.M;
    for (int idx = first; idx < n_out; idx += stride) {
      const int m = idx / out_per_slab, r = idx - m * out_per_slab;
      if (n0 + r >= p.N) continue;
      float v = 0.f, uval = 0.f;
#pragma unroll
      for (int wv = 0; wv < NCONS; ++wv) v += rb[((size_t)wv * MP + m) * RLD + r];
      if (p.gated) {
#pragma unroll
        for (int wv = 0; wv < NCONS; ++wv) uval += rb[((size_t)wv * MP + m) * RLD + ROWS / 2 + r];
      }
      write_out(m, n0 + r, v, uval);
    }
  };
  if (warp == NCONS + 1) {
    // ---------------------------------------------------------------- epilogue warp
    __shared__ int part_slot[MAX_GRID];   // for the contributors of a shared slab: index of the slot each wrote
    Walk walk(g_begin, g_end, num_kt);
    for (int seg = 0; walk.valid(); ++seg) {
      int slab, kt_first, kt_last;
      next_segment(walk, slab, kt_first, kt_last);
      const int n0 = slab * out_per_slab;
      const int b = seg & 1;
      const float* rb = red + (size_t)b * (C::RED1 / sizeof(float));
      mbar_wait(&red_full[b], (seg >> 1) & 1, &aborted, p.error);

      // Does this range hold the whole slab?  If not: which CTAs share it, and which of them is this one.
      const bool whole = kt_first == 0 && kt_last == num_kt;
      int c_first = blockIdx.x, nparts = 1;
      bool finish = true;
      if (!whole) {
        const long long s_begin = (long long)slab * num_kt, s_end = s_begin + num_kt, G = gridDim.x;
        c_first = (int)(((s_begin + 1) * G + p.total - 1) / p.total) - 1;   // the last CTA whose range begins at or before the slab's first stage
        const int c_last = (int)((s_end * G + p.total - 1) / p.total) - 1;  // ... at or before its last stage
        nparts = c_last - c_first + 1;
        // this CTA's slot: 0 if the slab is the first of its range, else 1
        float* slot = p.slots + ((size_t)blockIdx.x * 2 + (slab == head_slab ? 0 : 1)) * (MP * ROWS);
        for (int idx = lane; idx < MP * ROWS; idx += 32) {
          const int m = idx / ROWS, r = idx - m * ROWS;
          float v = 0.f;
#pragma unroll
          for (int wv = 0; wv < NCONS; ++wv) v += rb[((size_t)wv * MP + m) * RLD + r];
          slot[idx] = v;
        }
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          const int old = atomicAdd(p.counters + slab, 1);
          last = old == nparts - 1;
          if (last) p.counters[slab] = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        finish = last != 0;
        if (finish) {
          __threadfence();
          for (int j = lane; j < nparts; j += 32) {
            const int c = c_first + j;
            const bool head = (range_begin(p, c, num_kt) / num_kt) == slab;   // the slab is the first of c's range
            part_slot[j] = c * 2 + (head ? 0 : 1);
          }
          __syncwarp();
        }
      }
      if (finish) {
        const int n_out = out_per_slab * p.M;
        if (whole) {
          // the last segment of the walk has nothing after it to hide behind: the consumer warps share its outputs
          const bool shared = !walk.valid();
          write_whole(rb, n0, shared ? NCONS * 32 + lane : lane, shared ? (NCONS + 1) * 32 : 32);
        } else {
          // The contributors' sums come from L2: eight outputs of a lane at a time, all their loads in
          // flight together, added in the order of the ranges.
          constexpr int E = 8;
          for (int base = 0; base < n_out; base += 32 * E) {
            float v[E], uval[E];
            int off[E];
#pragma unroll
            for (int e = 0; e < E; ++e) {
              const int idx = base + e * 32 + lane;
              const int m = idx / out_per_slab, r = idx - m * out_per_slab;
              off[e] = (idx < n_out && n0 + r < p.N) ? m * ROWS + r : -1;
              v[e] = uval[e] = 0.f;
            }
            for (int j = 0; j < nparts; ++j) {
              const float* slot = p.slots + (size_t)part_slot[j] * (MP * ROWS);
              float t[E], tu[E];
#pragma unroll
              for (int e = 0; e < E; ++e) {
                t[e] = off[e] >= 0 ? __ldcg(slot + off[e]) : 0.f;
                tu[e] = (off[e] >= 0 && p.gated) ? __ldcg(slot + off[e] + ROWS / 2) : 0.f;
              }
#pragma unroll
              for (int e = 0; e < E; ++e) {
                v[e] += t[e];
                uval[e] += tu[e];
              }
            }
#pragma unroll
            for (int e = 0; e < E; ++e) {
              if (off[e] < 0) continue;
              const int idx = base + e * 32 + lane;
              const int m = idx / out_per_slab, r = idx - m * out_per_slab;
              write_out(m, n0 + r, v[e], uval[e]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[b]);   // the buffer may take the segment after the next
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  // (their first full barrier completes only after the producer's wait, so everything that is
  // written to global memory, by the epilogue warp, comes after the kernels before this one)
  const int mat = lane >> 3, r8 = lane & 7;
  int s = 0, u = 0;   // stage s of the ring, in its u-th use
  Walk walk(g_begin, g_end, num_kt);
  for (int seg = 0; walk.valid(); ++seg) {
    const int kt_first = walk.kt, slab = walk.slab;
    float acc[RT][MT][4];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    int kt_last = kt_first;   // exclusive
    for (; walk.valid() && walk.slab == slab && walk.kt == kt_last; walk.advance()) {
      const int kt = kt_last++;
      mbar_wait(&full[s], u & 1, &aborted, p.error);
      const unsigned char* stage = ring + (size_t)s * C::STAGE;
      // this warp's block of W rows; gated: its block of gate rows, the up rows half a W region on
      const int prows = p.gated ? ROWS / 2 : ROWS;
      const unsigned char* wbox = stage + warp * prows * 128;
      const unsigned char* xbox = stage + NCONS * C::W_BOX + warp * C::X_BOX;
      const int kbase = kt * BK + warp * BOX_COLS;
#pragma unroll
      for (int ks = 0; ks < BOX_COLS / 16; ++ks) {
        if (kbase + ks * 16 < p.K) {
          uint32_t b[MT][2];
          if (MT == 1) {
            uint32_t t2[2];
            ldsm_x2(t2, swizzled(xbox, r8, ks * 2 + ((lane >> 3) & 1)));
            b[0][0] = t2[0];
            b[0][1] = t2[1];
          } else {
#pragma unroll
            for (int j = 0; j < MT / 2; ++j) {
              uint32_t t4[4];
              ldsm_x4(t4, swizzled(xbox, j * 16 + (mat >> 1) * 8 + r8, ks * 2 + (mat & 1)));
              b[2 * j][0] = t4[0];
              b[2 * j][1] = t4[1];
              b[2 * j + 1][0] = t4[2];
              b[2 * j + 1][1] = t4[3];
            }
          }
#pragma unroll
          for (int i = 0; i < RT; ++i) {
            uint32_t a[4];
            const bool up = p.gated && i >= RT / 2;
            const unsigned char* wb = up ? wbox + NCONS * C::W_BOX / 2 : wbox;
            const int row = (up ? i - RT / 2 : i) * 16 + (mat & 1) * 8 + r8;
            ldsm_x4(a, swizzled(wb, row, ks * 2 + (mat >> 1)));
#pragma unroll
            for (int j = 0; j < MT; ++j) mma16816(acc[i][j], a, b[j][0], b[j][1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == NS) {
        s = 0;
        ++u;
      }
    }
    // The warp's partial sums go to the segment's buffer as soon as the epilogue warp has emptied it.
    {
      const int b = seg & 1;
      float* rb = red + (size_t)b * (C::RED1 / sizeof(float));
      mbar_wait(&red_empty[b], ((seg >> 1) & 1) ^ 1, &aborted, p.error);
      const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          float* base = rb + ((size_t)warp * MP + j * 8 + 2 * t4) * RLD + i * 16 + g4;
          base[0] = acc[i][j][0];
          base[RLD] = acc[i][j][1];
          base[8] = acc[i][j][2];
          base[RLD + 8] = acc[i][j][3];
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[b]);
      if (!walk.valid() && kt_first == 0 && kt_last == num_kt) {
        // the walk's last segment, a whole slab: every warp writes a share of its outputs
        mbar_wait(&red_full[b], (seg >> 1) & 1, &aborted, p.error);
        write_whole(rb, slab * out_per_slab, warp * 32 + lane, (NCONS + 1) * 32);
      }
    }
  }
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// Stage depth for a tile shape: as many stages as fit beside the reduction buffer, at most 8.
template <int MT, int RT>
struct Shape {
  static constexpr size_t STAGE = (size_t)NCONS * (RT * 16 + MT * 8) * 128;
  static constexpr size_t RED = 2 * (sizeof(float) * (size_t)NCONS * MT * 8 * (RT * 16 + 1) + 16);   // two buffers
  static constexpr int FIT = (int)((220 * 1024 - RED - 1024 - 256) / STAGE);
  static constexpr int NS = FIT > 8 ? 8 : FIT;
  static_assert(NS >= 2, "at least two stages");
  static constexpr size_t W_IN_FLIGHT = (size_t)NS * NCONS * RT * 16 * 128;
};

template <int MT, int RT>
static int launch(Params p, const void* X, int64_t lda, const void* W, void* scratch, int64_t scratch_bytes,
                  cudaStream_t stream) {
  using S = Shape<MT, RT>;
  using C = Cfg<MT, RT, S::NS>;
  static_assert(C::SMEM <= 227 * 1024, "shared memory of a CTA");
  auto kern = gemm_smallm_kernel<MT, RT, S::NS>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
  CUtensorMap wmap, xmap;
  const int w_rows = p.gated ? 2 * p.N : p.N;
  if (!cached_map(&wmap, W, w_rows, p.K, p.K, p.gated ? C::ROWS / 2 : C::ROWS, NCONS) ||
      !cached_map(&xmap, X, p.M, p.K, lda, C::MP, NCONS))
    return ATOM_ERR_LIB;
  const int out_per_slab = p.gated ? C::ROWS / 2 : C::ROWS;
  const int num_kt = (p.K + BK - 1) / BK;
  p.num_slabs = (p.N + out_per_slab - 1) / out_per_slab;
  p.total = (long long)p.num_slabs * num_kt;
  // Scratch: [grid][2] slots of MP x ROWS floats, then one counter per slab.
  int grid = sm_count() < MAX_GRID ? sm_count() : MAX_GRID;
  // (the counters lie behind the largest slot area any shape needs, so no shape's slots ever cover them)
  const int64_t slot_bytes = (int64_t)MAX_GRID * 2 * 16 * 64 * (int64_t)sizeof(float);
  const int64_t need = slot_bytes + (int64_t)p.num_slabs * (int64_t)sizeof(int);
  p.whole_slabs = (scratch == nullptr || scratch_bytes < need || ((uintptr_t)scratch % 16) != 0) ? 1 : 0;
  if (p.whole_slabs) {
    if (grid > p.num_slabs) grid = p.num_slabs;
    p.slots = nullptr;
    p.counters = nullptr;
  } else {
    if ((long long)grid > p.total) grid = (int)p.total;
    p.slots = reinterpret_cast<float*>(scratch);
    p.counters = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(scratch) + slot_bytes);
  }
  atom::launch_pdl(kern, dim3(grid), dim3(NTHREADS), C::SMEM, stream, wmap, xmap, p);
  return check_launch();
}

// Rows of W per slab.  With ranges cut anywhere the balance does not depend on it: the tallest
// slab that leaves every CTA a few stages reads X least often (X travels once per slab and stage).
// With whole slabs: the height whose slab count fills the CTAs' rounds best.
static double slab_cost(int n_out, int out_per_slab, int rows, double in_flight_bytes, int G) {
  const int slabs = (n_out + out_per_slab - 1) / out_per_slab;
  const int full = slabs / G, rem = slabs % G;
  double t = full;
  if (rem > 0) {
    double f = rem * in_flight_bytes / 10.0e6;
    if (f > 1.0) f = 1.0;
    double part = ((double)rem / G) / f;
    if (part > 1.0) part = 1.0;
    if (full == 0 && f < 1.0) part = ((double)rem / G) / f;   // a lone partial round is latency bound
    t += part;
  }
  return t * rows + 0.15 * rows * (full + (rem > 0));           // plus a fill/drain share per round
}

template <int MT>
static int launch_mt(const Params& p, const void* X, int64_t lda, const void* W, void* scratch, int64_t scratch_bytes,
                     cudaStream_t stream) {
  const int G = sm_count();
  int rt = 2;
  const int forced = atom::options().v[ATOM_OPT_GEMM_ROW_TILE];
  // Ranges cut inside slabs pay where a CTA streams much (the settling of a shared slab costs a few
  // microseconds of its consumers' time): measured better from about half a megabyte of W per CTA.
  const int mode = atom::options().v[ATOM_OPT_GEMM_CUT];
  const double w_bytes_per_cta = 2.0 * (p.gated ? 2.0 : 1.0) * p.N * (double)p.K / G;
  const bool cut = mode < 0 ? w_bytes_per_cta >= 512.0 * 1024 : mode != 0;
  if (!cut) scratch = nullptr;
  if (scratch != nullptr) {
    // stages per CTA with slabs of 64 rows: at least 4, else lower slabs
    const long long num_kt = (p.K + BK - 1) / BK;
    rt = 4;
    while (rt > (p.gated ? 2 : 1) && ((long long)((p.N + (p.gated ? rt * 8 : rt * 16) - 1) / (p.gated ? rt * 8 : rt * 16)) * num_kt) < 4LL * G)
      rt = p.gated ? rt - 2 : rt - 1;
  } else {
    double best = 1e300;
    const int n_out = p.N;
#define ATOM_TRY(RT)                                                                              \
  {                                                                                               \
    const int rows = RT * 16, out = p.gated ? rows / 2 : rows;                                    \
    const double c = slab_cost(n_out, out, rows, (double)Shape<MT, RT>::W_IN_FLIGHT, G);          \
    if (c < best) { best = c; rt = RT; }                                                          \
  }
    if (!p.gated) ATOM_TRY(1)
    ATOM_TRY(2)
    if (!p.gated) ATOM_TRY(3)
    ATOM_TRY(4)
#undef ATOM_TRY
  }
  if (forced >= 1 && forced <= 4 && !(p.gated && (forced & 1))) rt = forced;
  switch (rt) {
    case 1: return launch<MT, 1>(p, X, lda, W, scratch, scratch_bytes, stream);
    case 2: return launch<MT, 2>(p, X, lda, W, scratch, scratch_bytes, stream);
    case 3: return launch<MT, 3>(p, X, lda, W, scratch, scratch_bytes, stream);
    default: return launch<MT, 4>(p, X, lda, W, scratch, scratch_bytes, stream);
  }
}

}  // namespace smallm
}  // namespace atom

// 1 if the kernel takes these sizes (the caller uses the library product otherwise).
ATOM_EXPORT int atom_gemm_smallm_supports(int M, int N, int K, int64_t lda) {
  return M >= 1 && M <= 16 && N >= 1 && K >= 64 && K % 64 == 0 && lda % 8 == 0 && lda >= K &&
         atom::tma::encode_fn() != nullptr;
}

// C[M, N] = X[M, K] * W[N, K]^T (+ bias), or with gated != 0: W is [2N, K] = [gate ; up] and
// C[M, N] = silu(X gate^T) * (X up^T).  X, W bf16; C bf16 or float32.  `error` is a device int
// that is set to 2 if a wait inside the kernel ran out.  `scratch` (16-byte aligned, zero before
// its first use and left zero where it matters; may be null): room for the partial sums of slabs
// that several CTAs share, atom_gemm_smallm_scratch_bytes(N) bytes; one launch at a time may use it.
ATOM_EXPORT int64_t atom_gemm_smallm_scratch_bytes(int N) {
  using namespace atom::smallm;
  return (int64_t)MAX_GRID * 2 * 16 * 64 * (int64_t)sizeof(float) + ((int64_t)(N + 7) / 8) * (int64_t)sizeof(int);
}

ATOM_EXPORT int atom_gemm_smallm(void* C, int c_dtype, int64_t ldc, const void* X, int64_t lda, const void* W,
                                 const void* bias, int bias_dtype, int M, int N, int K, int gated, int* error,
                                 void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
  using namespace atom::smallm;
  if (M <= 0 || N <= 0) return ATOM_OK;
  if (!atom_gemm_smallm_supports(M, N, K, lda) || ldc < N || (gated && bias != nullptr) || error == nullptr ||
      (c_dtype != ATOM_F32 && c_dtype != ATOM_BF16) || ((uintptr_t)X % 16) != 0 || ((uintptr_t)W % 16) != 0)
    return ATOM_ERR_ARG;
  Params p;
  p.out = C;
  p.out_dtype = c_dtype;
  p.ldc = ldc;
  p.bias = bias;
  p.bias_dtype = bias_dtype;
  p.M = M;
  p.N = N;
  p.K = K;
  p.gated = gated ? 1 : 0;
  p.error = error;
  p.num_slabs = 0;
  p.total = 0;
  p.slots = nullptr;
  p.counters = nullptr;
  p.whole_slabs = 1;
  if (M <= 8) return launch_mt<1>(p, X, lda, W, scratch, scratch_bytes, stream);
  return launch_mt<2>(p, X, lda, W, scratch, scratch_bytes, stream);
}
