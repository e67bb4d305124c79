// TMA and mbarrier helpers shared by the kernels that are fed by the tensor memory accelerator.
// Every wait is bounded in time: mbar_wait gives up after `limit_ns` nanoseconds and says so.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace sllm {

constexpr uint64_t TMA_WAIT_NS = 1000000000ull;          // a wait gives up after a second
constexpr uint64_t TMA_DRAIN_NS = 1000000ull;            // waiting for copies in flight after a failure: a millisecond

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// false if the phase did not complete within `limit_ns` (the clock is read every 256 polls)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = TMA_WAIT_NS) {
  const uint32_t addr = smem_u32(bar);
  uint64_t start = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (__builtin_expect(ok, 1)) return true;
    if ((i & 255u) == 255u) {
      const uint64_t now = global_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) return false;
    }
  }
}
// the same for a wait that is usually short and stands in a hot loop: one test first, the bounded loop after it
__device__ __forceinline__ bool mbar_wait_hot(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  if (__builtin_expect(ok, 1)) return true;
  return mbar_wait(bar, parity);
}
// one test of the phase that never suspends the thread
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// ---- host side: tensor maps through the driver entry point (no link against libcuda) ------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// rows x K bfloat16, row-major; boxes of box_rows x 64 elements, 128-byte swizzle, zeros outside
inline bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows,
                     CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promotion,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A result matrix rows x cols (bfloat16 or float32, row-major) for TMA stores: boxes of 32 rows x 128 bytes,
// 128-byte swizzle; what a box holds beyond the matrix's edges is not written.  cols * elem_bytes must be a
// multiple of 16.
inline bool make_map_store(CUtensorMap* map, void* base, int rows, int cols, int elem_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), 32};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides,
            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// one box from this CTA's shared memory to the matrix at (x, y); completion is tracked by bulk groups
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `N` groups have been read out of shared memory (their buffers may be written again)
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// all but the newest `N` groups are complete (their writes are done)
template <int N> __device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }

// rows x (halves * 64) bfloat16, row-major, seen as [rows][halves][64]: one box takes box_rows whole
// rows (all halves), stored as consecutive 128-byte units (row-major, half fastest), 128-byte swizzle
inline bool make_map_rows(CUtensorMap* map, const void* base, long long rows, int halves, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64, (cuuint64_t)halves, (cuuint64_t)rows};
  cuuint64_t strides[2] = {128, (cuuint64_t)halves * 128};
  cuuint32_t box[3] = {64, (cuuint32_t)halves, (cuuint32_t)box_rows};
  cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The paged cache [pages][kv heads][page_size][hd] bfloat16 seen as a 5-d tensor whose last dimension
// walks the pages: one box then takes `run_pages` pages with CONSECUTIVE IDS of one kv head (they are
// not adjacent in memory; the page dimension has its own stride).  rows_major: the box lands as
// [page][row][half][64] (the decode kernel's tile layout); else as [half][page][row][64] (the K-major
// operand layout of the tcgen05 kernel).  128-byte swizzle either way.
inline bool make_map_page_run(CUtensorMap* map, const void* base, long long num_pages, int nkv, int ps, int hd, int run_pages,
                              bool rows_major) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t halves = (cuuint64_t)hd / 64, row_b = (cuuint64_t)hd * 2, head_b = row_b * ps, page_b = head_b * nkv;
  cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  if (rows_major) {
    cuuint64_t dims[5] = {64, halves, (cuuint64_t)ps, (cuuint64_t)nkv, (cuuint64_t)num_pages};
    cuuint64_t strides[4] = {128, row_b, head_b, page_b};
    cuuint32_t box[5] = {64, (cuuint32_t)halves, (cuuint32_t)ps, 1, (cuuint32_t)run_pages};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  cuuint64_t dims[5] = {64, (cuuint64_t)ps, (cuuint64_t)num_pages, halves, (cuuint64_t)nkv};
  cuuint64_t strides[4] = {row_b, page_b, 128, head_b};
  cuuint32_t box[5] = {64, (cuuint32_t)ps, (cuuint32_t)run_pages, (cuuint32_t)halves, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__device__ __forceinline__ void tma_load_5d(void* smem, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

}  // namespace sllm
