// Device pieces shared by the weight-streaming products (gemm_smallm.cu: slabs of W and ranges of k
// shared out among the CTAs; gemm_rows.cu: rows of W shared out): the stage layout of the ring, the
// walk of a CTA through its range of (slab, k stage) pairs, and the mma.sync wrappers.
#pragma once
#include "common.cuh"
#include "tma.cuh"

namespace atom {
namespace smallm {

using namespace atom::tma;

constexpr int NCONS = 4;                 // consumer warps, one 64-element box of a stage each
constexpr int NTHREADS = (NCONS + 2) * 32;   // + the producer warp and the epilogue warp
constexpr int BK = NCONS * BOX_COLS;     // k elements per stage
constexpr int MAX_GRID = 256;            // most CTAs of a launch whose ranges may share slabs

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

// The order in which a CTA walks the stages [b, e) of its range: first the piece of the slab
// that its range ends in, then the piece of the slab that it begins in, then the whole slabs
// between them.  The shared slabs are thus settled early, while the stream of the whole slabs
// is already on its way, and the kernel's end is a plain slab's.
struct Walk {
  long long pb[3], pe[3];
  int n, pi, num_kt;
  long long g;
  int slab, kt;
  __device__ __forceinline__ void seek() {
    if (pi < n) {
      g = pb[pi];
      slab = (int)(g / num_kt);
      kt = (int)(g - (long long)slab * num_kt);
    }
  }
  __device__ __forceinline__ Walk(long long b, long long e, int nkt) : n(0), pi(0), num_kt(nkt), g(0), slab(0), kt(0) {
    const long long head_end = (b / nkt + 1) * nkt;        // end of the slab that b lies in
    const long long tail_begin = (e / nkt) * nkt;          // begin of the slab that e lies in
    const bool head_cut = b % nkt != 0, tail_cut = e % nkt != 0;
    if (b >= e) {
    } else if (head_end >= e || (!head_cut && tail_begin <= b)) {
      // at most one slab is touched, or the range is one run: whole slabs, then a cut tail
      if (tail_cut && tail_begin > b) {
        pb[n] = tail_begin, pe[n] = e, ++n;
        pb[n] = b, pe[n] = tail_begin, ++n;
      } else {
        pb[n] = b, pe[n] = e, ++n;
      }
    } else {
      long long wb = b, we = e;
      if (tail_cut) pb[n] = tail_begin, pe[n] = e, ++n, we = tail_begin;
      if (head_cut) pb[n] = b, pe[n] = head_end, ++n, wb = head_end;
      if (wb < we) pb[n] = wb, pe[n] = we, ++n;
    }
    seek();
  }
  __device__ __forceinline__ bool valid() const { return pi < n; }
  __device__ __forceinline__ void advance() {
    ++g;
    if (++kt == num_kt) {
      kt = 0;
      ++slab;
    }
    if (g == pe[pi]) {
      ++pi;
      seek();
    }
  }
};

// MT: 8-token column tiles (tokens padded to 8 * MT).  RT: 16-row tiles of W per slab.  NS: stages.
template <int MT, int RT, int NS>
struct Cfg {
  static constexpr int ROWS = RT * 16, MP = MT * 8;
  static constexpr int W_BOX = ROWS * 128, X_BOX = MP * 128;             // bytes of one 64-element box
  static constexpr int STAGE = NCONS * (W_BOX + X_BOX);
  static constexpr size_t RING = (size_t)NS * STAGE;
  static constexpr int RLD = ROWS + 1;   // padded stride of the reduction buffer [warp][token][row]
  static constexpr size_t RED1 = ((sizeof(float) * (size_t)NCONS * MP * RLD + 15) / 16) * 16;   // one buffer
  static constexpr size_t RED = 2 * RED1;
  static constexpr size_t SMEM = 1024 + RING + RED + (2 * NS + 4) * sizeof(uint64_t) + 16;
};

// The next piece of a CTA's walk that lies in one slab: stages [kt_first, kt_last) of `slab`.
__device__ __forceinline__ void next_segment(Walk& w, int& slab, int& kt_first, int& kt_last) {
  slab = w.slab;
  kt_first = kt_last = w.kt;
  while (w.valid() && w.slab == slab && w.kt == kt_last) {
    ++kt_last;
    w.advance();
  }
}

}  // namespace smallm
}  // namespace atom
