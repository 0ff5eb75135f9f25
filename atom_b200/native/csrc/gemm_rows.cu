// Weight-streaming product of a decode step (at most 16 rows of X):
//
//     C[M, N] = epilogue( X[M, K] * W[N, K]^T )
//
// The time of such a product is the time to read W once.  Rows of W, not tiles of work, are shared
// out: CTA c owns the output columns [N c / G, N (c+1) / G) and walks all of K for them, so every
// CTA streams the same number of bytes to within one row of W, no output has two contributors and
// nothing is settled between CTAs (the kernel's end is a CTA's last stage, not a reduction over
// CTAs).  The rows of a CTA are taken in sub-slabs of h <= 64 rows (h is whatever ceil(N / G) needs,
// e.g. 28 for 4096 rows on 148 SMs): a pipeline stage is one TMA box of [KC chunks of 64 k][h rows]
// (two for [gate ; up]) plus the X columns of those chunks.  The chunks lie h * 128 bytes apart,
// which is no multiple of 1024, so the 128-byte swizzle is undone with the row's absolute position
// in the stage, not its position in the chunk.  The last 16-row MMA tile of a sub-slab reads rows
// that are not the CTA's (the neighbour's, or whatever lies behind the box); their sums are never
// written.
//
// Warps: one streams W into the ring and never waits for the kernels before this one (W is written by
// nobody), so the first ring of weights arrives while they finish; one brings the X columns of a stage
// once the kernels before have completed; one turns the sums of squares into the rows' factors beside
// the stream (inside the X producer it held the stages' X back by 1-2 us); sixteen consume (one
// mma.sync warp per scheduler keeps the tensor cores busy for a fraction of the time only, and with a
// handful of stages per CTA the consumers' time per stage is on the critical path): 8 along k (half
// chunks of two 16-k steps each, so that all work on a stage of four chunks too) times 2 over the 16-row
// tiles, each warp with one or two 8-token tiles (up to 8 or 16 rows of X; with 16 the ring has 4 stages).  At a sub-slab's end the warps' sums meet in shared
// memory and each of the 512 consumer threads settles one output (a single epilogue warp took 2-5 us
// for it).
//
// The norm between two products needs no pass of its own:
//     RMSNorm(r) W^T = rstd(r) * ((r . w) W^T)
//   * a product in residual mode adds its result to the 32-bit residual stream r[M, N], writes
//     x' = bf16(r * w) (w: the following norm's weight) as the next product's X, and every CTA writes
//     the sums of r^2 over its own columns, per row, to ssq_out[CTA][16];
//   * a product with ssq_in multiplies output row m by rsqrt(sum_c ssq_in[c][m] / size + eps) before
//     bias or activation; the parts are added in their order, so the factor does not depend on timing.
// Every wait is bounded; one that runs out raises the device error flag and the kernel finishes.
#include "gemm_rows.h"

#include "common.cuh"
#include "tma.cuh"

namespace atom {
namespace rows {

using namespace atom::tma;

__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int KG = 8, TG = 2, NCW = KG * TG;      // consumer warps: k groups times tile groups
constexpr int CTHREADS = (NCW + 3) * 32;          // consumers, W producer, X producer, the rows' factors
constexpr int KC_MAX = 8;                         // chunks of 64 k in a stage, at most
constexpr int RLD = 65;                           // stride of the buffer of sums [k group][token][row]

// MT: 8-token column tiles of the MMA (M <= 8 MT).
template <int MT>
struct Cfg {
  static constexpr int MP = 8 * MT;
  static constexpr int NS = MT == 1 ? 5 : 4;                     // stages of the ring
  static constexpr int W_MAX = (MT == 1 ? 32 : 30) * 1024;       // bytes of W in a stage, at most
  static constexpr int X_MAX = KC_MAX * MP * 128;                // bytes of X in a stage, at most
  static constexpr int STAGE = W_MAX + X_MAX;
  static constexpr size_t RED = ((sizeof(float) * (size_t)KG * MP * RLD + 15) / 16) * 16;
  // ring (1024-aligned), 2 KB that a last tile may read into, the sums, the barriers
  static constexpr size_t SMEM = 1024 + (size_t)NS * STAGE + 2048 + RED + (2 * NS + 2) * sizeof(uint64_t) + 16;
  static_assert(SMEM + 1024 <= 227 * 1024, "shared memory of a CTA");
};

struct Params {
  int M;
  int* error;
  void* out;
  int out_dtype;
  int64_t ldc;
  const void* bias;
  int bias_dtype;
  int N, K, gated;
  int h, KC, S, num_kt;   // rows of a sub-slab, chunks of a stage, sub-slabs of a CTA, stages of a sub-slab
  const float* ssq_in;
  int ssq_parts;
  float inv_norm_size, norm_eps;
  float* residual;
  const void* norm_w;
  int norm_w_dtype;
  __nv_bfloat16* xout;
  float* ssq_out;
};

__device__ __forceinline__ int row_begin(const Params& p, int c) { return (int)((long long)p.N * c / gridDim.x); }

// Barrier among the consumer warps only (the producers never join it).
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(NCW * 32) : "memory"); }

// rstd of every token's row from the partial sums [parts][16] that the CTAs of the product before wrote,
// added in a fixed order; run by one whole warp, which then arrives at `bar`.
__device__ __forceinline__ void row_factors(const Params& p, float* out, uint64_t* bar, int lane) {
  float ss[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) ss[m] = 0.f;
  const float4* in4 = reinterpret_cast<const float4*>(p.ssq_in);
  for (int j0 = lane; j0 < p.ssq_parts; j0 += 64) {
    float4 t[2][4];
#pragma unroll
    for (int uu = 0; uu < 2; ++uu)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        t[uu][q] = (j0 + 32 * uu < p.ssq_parts) ? __ldcg(in4 + (size_t)(j0 + 32 * uu) * 4 + q)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int uu = 0; uu < 2; ++uu)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ss[4 * q] += t[uu][q].x;
        ss[4 * q + 1] += t[uu][q].y;
        ss[4 * q + 2] += t[uu][q].z;
        ss[4 * q + 3] += t[uu][q].w;
      }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    const float tot = warp_sum(ss[m]);
    if (lane == m) out[m] = m < p.M ? rsqrtf(tot * p.inv_norm_size + p.norm_eps) : 0.f;
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

template <int MT>
__global__ void __launch_bounds__(CTHREADS, 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const __grid_constant__ Params p) {
  using C = Cfg<MT>;
  constexpr int NS = C::NS, MP = C::MP, STAGE = C::STAGE, W_MAX = C::W_MAX;
  atom::pdl_trigger();
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  float* red = reinterpret_cast<float*>(ring + (size_t)NS * STAGE + 2048);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + C::RED);
  uint64_t* empty = full + NS;
  uint64_t* scale_bar = empty + NS;       // the rows' factors are there
  __shared__ int aborted;
  __shared__ float row_scale[16];
  __shared__ float sq_part[MT][NCW];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R0 = row_begin(p, blockIdx.x), R1 = row_begin(p, blockIdx.x + 1);
  if (R0 >= R1) {
    // (fewer rows than CTAs) this CTA owns none; its part of the sums of squares is zero
    atom::pdl_wait();
    if (p.residual != nullptr && threadIdx.x < 16) p.ssq_out[(size_t)blockIdx.x * 16 + threadIdx.x] = 0.f;
    return;
  }
  if (threadIdx.x == 0) {
    aborted = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 2);        // the W producer's and the X producer's arrival, each with its bytes
      mbar_init(&empty[s], NCW);
    }
    mbar_init(scale_bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const int h = p.h, KC = p.KC;

  if (warp == NCW) {
    // ---------------------------------------------------------------- W producer: never waits for a kernel
    if (lane == 0) prefetch_map(&map_w);
    const uint32_t w_bytes = (uint32_t)((p.gated ? 2 : 1) * h * KC * 128);
    int s = 0, u = 0;
    long long it = 0;
    for (int sl = 0; sl < p.S; ++sl) {
      const int r0 = R0 + sl * h;
      if (r0 >= R1) break;
      for (int kt = 0; kt < p.num_kt; ++kt, ++it) {
        if (it >= NS) mbar_wait(&empty[s], (u & 1) ^ 1, &aborted, p.error);
        unsigned char* stage = ring + (size_t)s * STAGE;
        if (lane == 0) mbar_expect_tx(&full[s], w_bytes);
        __syncwarp();
        if (lane == 0) {
          load_chunks(stage, &map_w, r0, kt * KC, &full[s]);
        } else if (lane == 1 && p.gated) {
          load_chunks(stage + h * KC * 128, &map_w, p.N + r0, kt * KC, &full[s]);
        }
        if (++s == NS) {
          s = 0;
          ++u;
        }
      }
    }
    return;
  }

  if (warp == NCW + 1) {
    // ---------------------------------------------------------------- X producer: after the kernels before
    if (lane == 0) prefetch_map(&map_x);
    atom::pdl_wait();
    const uint32_t x_bytes = (uint32_t)(KC * MP * 128);
    int s = 0, u = 0;
    long long it = 0;
    for (int sl = 0; sl < p.S; ++sl) {
      if (R0 + sl * h >= R1) break;
      for (int kt = 0; kt < p.num_kt; ++kt, ++it) {
        if (it >= NS) mbar_wait(&empty[s], (u & 1) ^ 1, &aborted, p.error);
        unsigned char* stage = ring + (size_t)s * STAGE;
        if (lane == 0) {
          mbar_expect_tx(&full[s], x_bytes);
          load_chunks(stage + W_MAX, &map_x, 0, kt * KC, &full[s]);
        }
        if (++s == NS) {
          s = 0;
          ++u;
        }
      }
    }
    return;
  }

  if (warp == NCW + 2) {
    // ---------------------------------------------------------------- the rows' factors, beside the stream
    if (p.ssq_in != nullptr) {
      atom::pdl_wait();
      row_factors(p, row_scale, scale_bar, lane);
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  // warp = tile group * 8 + k group: it takes the chunks kg, kg + 8, ... of a stage and the 16-row tiles
  // tg, tg + 2 (gated: tiles 0, 1 are gate rows, 2, 3 the up rows, so a warp holds a gate tile and its up
  // tile).  At a sub-slab's end thread t settles the token t / 64 (+ 8 for the second token tile) and the
  // row t % 64 of the sub-slab.
  atom::pdl_wait();      // (the residual stream that the epilogue reads is written by the kernels before)
  const int mat = lane >> 3, r8 = lane & 7;
  const int kg = warp & (KG - 1), tg = warp >> 3;
  const int em = threadIdx.x >> 6, er = threadIdx.x & 63;
  const bool gated = p.gated != 0, res_mode = p.residual != nullptr;
  const int tiles = (h + 15) >> 4;                 // 16-row tiles of a sub-slab (gated: of its gate rows, at most 2)
  const uint32_t up_off = (uint32_t)(h * KC * 128);
  const uint32_t lrow = (uint32_t)((mat & 1) * 8 + r8), lcol = (uint32_t)(mat >> 1);
  float scale[MT], sq[MT];
#pragma unroll
  for (int nt = 0; nt < MT; ++nt) scale[nt] = 1.f, sq[nt] = 0.f;
  bool have_scale = p.ssq_in == nullptr;
  int s = 0, u = 0;
  for (int sl = 0; sl < p.S; ++sl) {
    const int r0 = R0 + sl * h;
    if (r0 >= R1) break;
    const int v = min(h, R1 - r0);                 // rows of this sub-slab that are the CTA's
    // two accumulators per tile (even and odd k steps): the chains of dependent MMAs stay short
    float acc[MT][2][2][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int q = 0; q < 2; ++q) acc[nt][j][q][0] = acc[nt][j][q][1] = acc[nt][j][q][2] = acc[nt][j][q][3] = 0.f;
    for (int kt = 0; kt < p.num_kt; ++kt) {
      mbar_wait(&full[s], u & 1, &aborted, p.error);
      const uint32_t wbase = smem_u32(ring + (size_t)s * STAGE);
      const unsigned char* xreg = ring + (size_t)s * STAGE + W_MAX;
      // a k group takes half chunks (two 16-k steps): kg, kg + 8, ... of the stage's 2 KC, so that all eight
      // groups work on a stage of four chunks too (the stages of [gate ; up])
      for (int un = kg; un < 2 * KC; un += KG) {
        const int ck = un >> 1, ks0 = (un & 1) * 2;
        const unsigned char* xbox = xreg + ck * (MP * 128);
        const uint32_t crow = (uint32_t)(ck * h) + lrow;
        uint32_t xb[MT][2][2];
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
#pragma unroll
          for (int k2 = 0; k2 < 2; ++k2)
            ldsm_x2(xb[nt][k2], swizzled(xbox, nt * 8 + r8, (ks0 + k2) * 2 + ((lane >> 3) & 1)));
        uint32_t a[2][2][4];
        bool valid[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int t = tg + 2 * j;                  // plain: tile t; gated: j = 0 gate tile tg, j = 1 up tile tg
          const bool up = gated && j == 1;
          const int tt = gated ? tg : t;
          valid[j] = tt < tiles;
          if (valid[j]) {
            const uint32_t off = (crow + (uint32_t)(tt * 16)) * 128u + (up ? up_off : 0u);
            const uint32_t rowaddr = wbase + off, sw = (off >> 7) & 7u;
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2)
              asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                           : "=r"(a[j][k2][0]), "=r"(a[j][k2][1]), "=r"(a[j][k2][2]), "=r"(a[j][k2][3])
                           : "r"(rowaddr + ((((uint32_t)((ks0 + k2) * 2) + lcol) ^ sw) << 4)));
          }
        }
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (valid[j]) {
#pragma unroll
              for (int nt = 0; nt < MT; ++nt) mma16816(acc[nt][j][k2], a[j][k2], xb[nt][k2][0], xb[nt][k2][1]);
            }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      if (++s == NS) {
        s = 0;
        ++u;
      }
    }
    // ---- the sub-slab's end.  What this thread's outputs need from memory is asked for first.
    const bool my_row = er < v && (!gated || er < 32);
    const int col = r0 + er;
    float old[MT], nw = 0.f, bias = 0.f;
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) old[nt] = 0.f;
    if (my_row) {
      if (res_mode) {
        nw = load_as_float(p.norm_w, p.norm_w_dtype, col);
#pragma unroll
        for (int nt = 0; nt < MT; ++nt)
          if (em + 8 * nt < p.M) old[nt] = __ldcg(p.residual + (int64_t)(em + 8 * nt) * p.N + col);
      } else if (p.bias != nullptr) {
        bias = load_as_float(p.bias, p.bias_dtype, col);
      }
    }
    consumers_sync();       // everybody has read the sums of the sub-slab before
    {
      // plain: tile t at rows 16 t; gated: gate tile tg at rows 16 tg, its up tile 32 rows behind
      const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll
      for (int nt = 0; nt < MT; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int t = tg + 2 * j;
          float* base = red + ((size_t)kg * MP + nt * 8 + 2 * t4) * RLD + t * 16 + g4;
          base[0] = acc[nt][j][0][0] + acc[nt][j][1][0];
          base[RLD] = acc[nt][j][0][1] + acc[nt][j][1][1];
          base[8] = acc[nt][j][0][2] + acc[nt][j][1][2];
          base[RLD + 8] = acc[nt][j][0][3] + acc[nt][j][1][3];
        }
    }
    consumers_sync();       // the sums are complete
    if (!have_scale) {
      have_scale = true;
      mbar_wait(scale_bar, 0, &aborted, p.error);
#pragma unroll
      for (int nt = 0; nt < MT; ++nt) scale[nt] = row_scale[em + 8 * nt];
    }
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
      const int m = em + 8 * nt;
      // the k groups' sums are added in a fixed order
      float sum = 0.f, up = 0.f;
#pragma unroll
      for (int wv = 0; wv < KG; ++wv) sum += red[((size_t)wv * MP + m) * RLD + er];
      if (gated) {
#pragma unroll
        for (int wv = 0; wv < KG; ++wv) up += red[((size_t)wv * MP + m) * RLD + 32 + (er & 31)];
      }
      sum *= scale[nt];
      if (my_row && m < p.M) {
        if (res_mode) {
          const int64_t at = (int64_t)m * p.N + col;
          const float rr = old[nt] + sum;
          p.residual[at] = rr;
          p.xout[at] = __float2bfloat16_rn(rr * nw);
          sq[nt] += rr * rr;
        } else {
          if (gated)
            sum = sum / (1.f + __expf(-sum)) * (up * scale[nt]);
          else
            sum += bias;
          if (p.out_dtype == ATOM_F32)
            reinterpret_cast<float*>(p.out)[(int64_t)m * p.ldc + col] = sum;
          else
            reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.ldc + col] = __float2bfloat16_rn(sum);
        }
      }
    }
  }
  // ---- the end: this CTA's part of every row's sum of squares
  if (res_mode) {
    // a warp holds one token's rows 0..31 or 32..63 of every sub-slab
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
      const float tot = warp_sum(sq[nt]);
      if (lane == 0) sq_part[nt][warp] = tot;
    }
    consumers_sync();
    if (threadIdx.x < 16) {
      const int m = threadIdx.x, nt = m >> 3, e = m & 7;
      p.ssq_out[(size_t)blockIdx.x * 16 + m] = nt < MT ? sq_part[nt][2 * e] + sq_part[nt][2 * e + 1] : 0.f;
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

template <int MT>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int grid, cudaStream_t stream) {
  auto kern = gemm_rows_kernel<MT>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<MT>::SMEM) != cudaSuccess)
      return ATOM_ERR_LAUNCH;
    attr_set = true;
  }
  atom::launch_pdl(kern, dim3(grid), dim3(CTHREADS), Cfg<MT>::SMEM, stream, mw, mx, p);
  return atom::check_launch();
}

}  // namespace rows
}  // namespace atom

// 1 if the kernel takes a product of these sizes.
ATOM_EXPORT int atom_gemm_rows_supports(int M, int N, int K, int64_t lda) {
  return M >= 1 && M <= 16 && N >= 1 && K >= 64 && K % 64 == 0 && lda % 8 == 0 && lda >= K &&
         atom::tma::encode_fn() != nullptr;
}

// CTAs of a launch: the parts of ssq_out that a residual product writes, and of ssq_in that its reader sums.
ATOM_EXPORT int atom_gemm_rows_grid(void) {
  const int g = atom::rows::sm_count();
  return g > 256 ? 256 : g;
}

ATOM_EXPORT int atom_gemm_rows(const AtomRowsOp* op, int M, int* error, cudaStream_t stream) {
  using namespace atom::rows;
  if (op == nullptr || error == nullptr) return ATOM_ERR_ARG;
  const AtomRowsOp& a = *op;
  const bool res = a.residual != nullptr;
  if (!atom_gemm_rows_supports(M, a.N, a.K, a.lda) || (a.gated && a.bias != nullptr) ||
      ((uintptr_t)a.X % 16) != 0 || ((uintptr_t)a.W % 16) != 0)
    return ATOM_ERR_ARG;
  if (!res && (a.out == nullptr || a.ldc < a.N || (a.out_dtype != ATOM_F32 && a.out_dtype != ATOM_BF16)))
    return ATOM_ERR_ARG;
  if (res && (a.gated || a.bias != nullptr || a.norm_w == nullptr || a.xout == nullptr || a.ssq_out == nullptr ||
              (a.norm_w_dtype != ATOM_F32 && a.norm_w_dtype != ATOM_BF16)))
    return ATOM_ERR_ARG;
  if (a.ssq_in != nullptr && (a.ssq_parts <= 0 || a.norm_size <= 0 || ((uintptr_t)a.ssq_in % 16) != 0))
    return ATOM_ERR_ARG;
  const int grid = atom_gemm_rows_grid();
  const int MT = M <= 8 ? 1 : 2;
  Params p;
  p.M = M;
  p.error = error;
  // rows of a CTA, in sub-slabs of h rows; chunks of a stage
  const int rmax = (a.N + grid - 1) / grid;
  const int hmax = a.gated ? 32 : 64;
  p.S = (rmax + hmax - 1) / hmax;
  p.h = (rmax + p.S - 1) / p.S;
  const int rows = a.gated ? 2 * p.h : p.h;
  int kc = (MT == 1 ? atom::rows::Cfg<1>::W_MAX : atom::rows::Cfg<2>::W_MAX) / (rows * 128);
  if (kc > KC_MAX) kc = KC_MAX;
  if (kc > a.K / 64) kc = a.K / 64;
  if (kc < 1) kc = 1;
  p.KC = kc;
  p.num_kt = (a.K / 64 + kc - 1) / kc;
  CUtensorMap mw, mx;
  const int w_rows = a.gated ? 2 * a.N : a.N;
  if (!atom::tma::cached_map(&mw, a.W, w_rows, a.K, a.K, p.h, kc) ||
      !atom::tma::cached_map(&mx, a.X, M, a.K, a.lda, 8 * MT, kc))
    return ATOM_ERR_LIB;
  p.out = a.out;
  p.out_dtype = a.out_dtype;
  p.ldc = a.ldc;
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.N = a.N;
  p.K = a.K;
  p.gated = a.gated ? 1 : 0;
  p.ssq_in = a.ssq_in;
  p.ssq_parts = a.ssq_parts;
  p.inv_norm_size = a.norm_size > 0 ? 1.f / (float)a.norm_size : 0.f;
  p.norm_eps = a.norm_eps;
  p.residual = a.residual;
  p.norm_w = a.norm_w;
  p.norm_w_dtype = a.norm_w_dtype;
  p.xout = reinterpret_cast<__nv_bfloat16*>(a.xout);
  p.ssq_out = a.ssq_out;
  return MT == 1 ? launch<1>(mw, mx, p, grid, stream) : launch<2>(mw, mx, p, grid, stream);
}
