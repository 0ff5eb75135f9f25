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
// tensor flops, not bytes.  At the end of a slab the four warps' partial sums are added in
// shared memory in a fixed order (the result does not depend on timing) and written as bf16
// or 32-bit, with an optional bias, or, in gated mode, as silu(gate) * up for
// W = [gate rows ; up rows]: the feed-forward's activation never travels through memory.
// Meanwhile the producer is already streaming the next slab.
//
// Takes K that is a multiple of 64 and leading dimensions that are multiples of 8 elements;
// the caller uses the library product for other sizes.  Every mbarrier wait is bounded: when one runs
// out the kernel raises the device error flag and finishes without hanging.
#include "common.cuh"
#include "tma.cuh"

namespace atom {
namespace smallm {

using namespace atom::tma;

constexpr int NCONS = 4;                 // consumer warps, one 64-element box of a stage each
constexpr int NTHREADS = (NCONS + 1) * 32;
constexpr int BK = NCONS * BOX_COLS;     // k elements per stage

struct Params {
  void* out;
  int out_dtype;
  int64_t ldc;
  const void* bias;
  int bias_dtype;
  int M, N, K;
  int gated;
  int* error;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
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

// MT: 8-token column tiles (tokens padded to 8 * MT).  RT: 16-row tiles of W per slab.  NS: stages.
template <int MT, int RT, int NS>
struct Cfg {
  static constexpr int ROWS = RT * 16, MP = MT * 8;
  static constexpr int W_BOX = ROWS * 128, X_BOX = MP * 128;             // bytes of one 64-element box
  static constexpr int STAGE = NCONS * (W_BOX + X_BOX);
  static constexpr size_t RING = (size_t)NS * STAGE;
  static constexpr int RLD = ROWS + 1;   // padded stride of the reduction buffer [warp][token][row]
  static constexpr size_t RED = sizeof(float) * (size_t)NCONS * MP * RLD;
  static constexpr size_t SMEM = 1024 + RING + ((RED + 15) / 16) * 16 + 2 * NS * sizeof(uint64_t) + 16;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(NCONS * 32) : "memory"); }

template <int MT, int RT, int NS>
__global__ void __launch_bounds__(NTHREADS)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   const Params p, int num_slabs) {
  atom::pdl_trigger();   // the next kernel may be scheduled; this one waits below, after its first loads of W
  using C = Cfg<MT, RT, NS>;
  constexpr int ROWS = C::ROWS, MP = C::MP, RLD = C::RLD;
  extern __shared__ unsigned char smem_raw[];
  // boxes of the 128-byte swizzle start on 1024-byte boundaries
  unsigned char* ring = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  float* red = reinterpret_cast<float*>(ring + C::RING);   // [NCONS][MP][RLD]
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + C::RING + ((C::RED + 15) / 16) * 16);
  uint64_t* empty = full + NS;
  __shared__ int aborted;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    aborted = 0;
    for (int s = 0; s < NS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NCONS);
    }
    mbar_fence_init();
  }
  __syncthreads();

  // Rows of W in a slab.  Gated: the first half are gate rows, the second the matching up rows.
  const int out_per_slab = p.gated ? ROWS / 2 : ROWS;
  const int num_kt = (p.K + BK - 1) / BK;

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
      int it = 0;
      for (int slab = blockIdx.x; slab < num_slabs && it < NS; slab += gridDim.x) {
        const int n0 = slab * out_per_slab;
        for (int kt = 0; kt < num_kt && it < NS; ++kt, ++it) {
          unsigned char* stage = ring + (size_t)it * C::STAGE;
          if (lane == 0) {
            mbar_expect_tx(&full[it], (uint32_t)C::STAGE);
            load_chunks(stage, &wmap, n0, kt * NCONS, &full[it]);
          } else if (lane == 2 && p.gated) {
            load_chunks(stage + NCONS * C::W_BOX / 2, &wmap, p.N + n0, kt * NCONS, &full[it]);
          }
        }
      }
    }
    atom::pdl_wait();
    int it = 0;   // stages issued so far, over all slabs
    for (int slab = blockIdx.x; slab < num_slabs; slab += gridDim.x) {
      const int n0 = slab * out_per_slab;
      for (int kt = 0; kt < num_kt; ++kt, ++it) {
        const int s = it % NS, u = it / NS;
        unsigned char* stage = ring + (size_t)s * C::STAGE;
        const int kc = kt * NCONS;
        if (it < NS) {   // W of the first ring is on its way already
          if (lane == 1) load_chunks(stage + NCONS * C::W_BOX, &xmap, 0, kc, &full[s]);
          continue;
        }
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
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  // (their first full barrier completes only after the producer's wait, so the outputs below
  // are written after the kernels before this one have completed)
  const int mat = lane >> 3, r8 = lane & 7;
  const int tid = threadIdx.x;   // 0 .. NCONS * 32 - 1
  int it = 0;
  for (int slab = blockIdx.x; slab < num_slabs; slab += gridDim.x) {
    const int n0 = slab * out_per_slab;
    float acc[RT][MT][4];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
      for (int j = 0; j < MT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    for (int kt = 0; kt < num_kt; ++kt, ++it) {
      const int s = it % NS, u = it / NS;
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
    }
    // Add the four warps' partial sums in a fixed order and write the slab's outputs.
    {
      const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
      for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          float* base = red + ((size_t)warp * MP + j * 8 + 2 * t4) * RLD + i * 16 + g;
          base[0] = acc[i][j][0];
          base[RLD] = acc[i][j][1];
          base[8] = acc[i][j][2];
          base[RLD + 8] = acc[i][j][3];
        }
    }
    consumer_sync();
    for (int idx = tid; idx < out_per_slab * p.M; idx += NCONS * 32) {
      const int m = idx / out_per_slab, r = idx - m * out_per_slab;
      const int col = n0 + r;
      if (col >= p.N) continue;
      float v = 0.f;
#pragma unroll
      for (int wv = 0; wv < NCONS; ++wv) v += red[((size_t)wv * MP + m) * RLD + r];
      if (p.gated) {
        float uval = 0.f;
#pragma unroll
        for (int wv = 0; wv < NCONS; ++wv) uval += red[((size_t)wv * MP + m) * RLD + ROWS / 2 + r];
        v = v / (1.f + __expf(-v)) * uval;
      } else if (p.bias != nullptr) {
        v += load_as_float(p.bias, p.bias_dtype, col);
      }
      if (p.out_dtype == ATOM_F32)
        reinterpret_cast<float*>(p.out)[(int64_t)m * p.ldc + col] = v;
      else
        reinterpret_cast<__nv_bfloat16*>(p.out)[(int64_t)m * p.ldc + col] = __float2bfloat16_rn(v);
    }
    consumer_sync();   // the reduction buffer is free for the next slab
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
  static constexpr size_t RED = sizeof(float) * (size_t)NCONS * MT * 8 * (RT * 16 + 1) + 16;
  static constexpr int FIT = (int)((220 * 1024 - RED - 1024 - 256) / STAGE);
  static constexpr int NS = FIT > 8 ? 8 : FIT;
  static_assert(NS >= 2, "at least two stages");
  static constexpr size_t W_IN_FLIGHT = (size_t)NS * NCONS * RT * 16 * 128;
};

template <int MT, int RT>
static int launch(const Params& p, const void* X, int64_t lda, const void* W, cudaStream_t stream) {
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
  const int num_slabs = (p.N + out_per_slab - 1) / out_per_slab;
  const int grid = num_slabs < sm_count() ? num_slabs : sm_count();
  atom::launch_pdl(kern, dim3(grid), dim3(NTHREADS), C::SMEM, stream, wmap, xmap, p, num_slabs);
  return check_launch();
}

// Estimated time (arbitrary unit) of streaming N rows in slabs of `rows` over G persistent
// CTAs: whole rounds run at full bandwidth; a last partial round of r CTAs is limited by the
// bytes those CTAs keep in flight (about 10 MB saturate the memory system).
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
static int launch_mt(const Params& p, const void* X, int64_t lda, const void* W, cudaStream_t stream) {
  const int G = sm_count();
  double best = 1e300;
  int rt = 2;
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
  switch (rt) {
    case 1: return launch<MT, 1>(p, X, lda, W, stream);
    case 2: return launch<MT, 2>(p, X, lda, W, stream);
    case 3: return launch<MT, 3>(p, X, lda, W, stream);
    default: return launch<MT, 4>(p, X, lda, W, stream);
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
// that is set to 2 if a wait inside the kernel ran out.
ATOM_EXPORT int atom_gemm_smallm(void* C, int c_dtype, int64_t ldc, const void* X, int64_t lda, const void* W,
                                 const void* bias, int bias_dtype, int M, int N, int K, int gated, int* error,
                                 cudaStream_t stream) {
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
  if (M <= 8) return launch_mt<1>(p, X, lda, W, stream);
  return launch_mt<2>(p, X, lda, W, stream);
}
