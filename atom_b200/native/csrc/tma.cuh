// Tensor-map TMA helpers shared by the matrix-product kernels: host-side creation of a 2-D
// tensor map (through the driver entry point, so the library does not link against the
// driver), and the device-side load, mbarrier and swizzle primitives.
//
// A map describes a row-major bf16 matrix [rows, cols] with a row pitch in elements; a load
// brings a box of `box_rows` x 64 elements (64 bf16 = 128 bytes, the widest box the 128-byte
// swizzle takes) into shared memory, rows 128 bytes apart, with the 16-byte chunks of every row
// XOR-ed with (row mod 8) so that ldmatrix and the tensor cores read them without bank
// conflicts.  Parts of a box outside the matrix are filled with zeros, and the byte count
// signalled to the mbarrier is always that of the whole box.
// The innermost coordinate of every load must be a multiple of 8 elements (16 bytes).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace atom {
namespace tma {

constexpr int BOX_COLS = 64;   // elements per box row (128 bytes of bf16)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Map of a bf16 matrix [rows, cols], `pitch` elements between rows, boxes of box_rows x 64.
// Needs: base 16-byte aligned, pitch a multiple of 8, box_rows <= 256.  False if refused.
inline bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                     uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || ((uintptr_t)base % 16) != 0 || pitch % 8 != 0 || box_rows == 0 || box_rows > 256 ||
      rows == 0 || cols == 0)
    return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch * 2};
  cuuint32_t box[2] = {(cuuint32_t)BOX_COLS, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same matrix seen as [k chunk][row][64]: dimension 0 the 64 elements of a chunk, dimension
// 1 the rows, dimension 2 the chunks of 64 along a row.  One load then brings `box_chunks`
// chunks of `box_rows` rows, laid out in shared memory chunk after chunk, each chunk a
// [box_rows][64] block in the 128-byte swizzle: a whole pipeline stage in one operation.
// Needs cols to be a multiple of 64 (a chunk never runs into the next row).
inline bool make_map_chunked(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                             uint32_t box_rows, uint32_t box_chunks) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || ((uintptr_t)base % 16) != 0 || pitch % 8 != 0 || box_rows == 0 || box_rows > 256 ||
      box_chunks == 0 || box_chunks > 256 || rows == 0 || cols == 0 || cols % BOX_COLS != 0)
    return false;
  cuuint64_t dims[3] = {(cuuint64_t)BOX_COLS, rows, cols / BOX_COLS};
  cuuint64_t strides[2] = {pitch * 2, (cuuint64_t)BOX_COLS * 2};
  cuuint32_t box[3] = {(cuuint32_t)BOX_COLS, box_rows, box_chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A bf16 map of rank 2 or 3 given outright: sizes (innermost first), byte strides of the outer
// dimensions, box sizes; 128-byte swizzle (box[0] must be 64).
inline bool make_map_raw(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                         const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || rank < 2 || rank > 3 || ((uintptr_t)base % 16) != 0 || box[0] != (uint32_t)BOX_COLS) return false;
  cuuint64_t d[3], st[2];
  cuuint32_t b[3], es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    if (dims[i] == 0 || box[i] == 0 || box[i] > 256) return false;
    d[i] = dims[i];
    b[i] = box[i];
  }
  for (int i = 0; i < rank - 1; ++i) {
    if (strides[i] % 16 != 0) return false;
    st[i] = strides[i];
  }
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, st, b, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Maps are cached by what they describe: encoding costs a few microseconds on the host.
struct MapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, box_chunks;   // box_chunks 0: the 2-D map
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows &&
           box_chunks == o.box_chunks;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.pitch;
    h = h * 1000003u ^ k.box_rows;
    h = h * 1000003u ^ k.box_chunks;
    return h;
  }
};

inline bool cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                       uint32_t box_rows, uint32_t box_chunks = 0) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, cols, pitch, box_rows, box_chunks};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    const bool ok = box_chunks == 0 ? make_map(&m, base, rows, cols, pitch, box_rows)
                                    : make_map_chunked(&m, base, rows, cols, pitch, box_rows, box_chunks);
    if (!ok) return false;
    if (cache.size() > 65536) cache.clear();
    it = cache.emplace(key, m).first;
  }
  *out = it->second;
  return true;
}

// ------------------------------------------------------------------ device side

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about a second, raises the flags and returns, so that a fault
// in the pipeline ends the kernel instead of hanging it.  After the first wait that ran out
// (shared flag set) later waits give up at once.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* aborted, int* error) {
  const int limit = *aborted ? 64 : (1 << 24);
  for (int i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return;
  *aborted = 1;
  atomicExch(error, 2);
}

// Loads the box whose first element is (row y, column x) of the mapped matrix.
__device__ __forceinline__ void load_box(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// The same with the destination given as a 32-bit shared-memory address (`smem_dst` is ignored).
__device__ __forceinline__ void load_box(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                         uint32_t smem_addr) {
  (void)smem_dst;
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(smem_addr),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Chunked map: loads chunks [chunk, chunk + box_chunks) of rows [row, row + box_rows).
__device__ __forceinline__ void load_chunks(void* smem_dst, const CUtensorMap* map, int row, int chunk,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], "
      "[%5];\n" ::"r"(smem_u32(smem_dst)),
      "l"(map), "r"(0), "r"(row), "r"(chunk), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}

// Address of the 16-byte chunk `chunk` (0..7) of row `row` inside a box that starts at a
// 1024-byte aligned shared-memory address.
__device__ __forceinline__ const unsigned char* swizzled(const unsigned char* box, int row, int chunk) {
  return box + row * 128 + ((chunk ^ (row & 7)) << 4);
}

}  // namespace tma
}  // namespace atom
