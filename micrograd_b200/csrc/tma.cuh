// Thin wrappers over the sm_100a bulk-tensor copy (TMA), mbarrier and FP64
// tensor-core (mma.sync ... f64) instructions, plus host-side tensor-map
// construction.  No cluster multicast is used anywhere.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

namespace mg {

// ---------------------------------------------------------------------------
// Host: tensor maps.  cuTensorMapEncodeTiled is fetched through the runtime so
// that the library has no link-time dependency on libcuda.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                         &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return (EncodeTiledFn) nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// Row-major fp64 matrix [rows][cols] viewed as a 2-D tensor (x = column,
// y = row), copied in boxes of box_cols x box_rows with the 128-byte swizzle
// (16-byte chunk index XOR row index mod 8).  Out-of-range elements read as 0.
// Requirements: base 16-byte aligned, cols even, box_cols * 8 <= 128.
inline bool make_tensor_map_f64(CUtensorMap *map, const double *base, size_t rows, size_t cols,
                                unsigned box_cols, unsigned box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(double)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, const_cast<double *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The same matrix when cols is a multiple of 16, viewed as a 3-D tensor
// (x = column within a 16-column group, y = row, z = column group) so that one
// copy brings `box_groups` adjacent 16-column groups x `box_rows` rows: the
// shared-memory image is `box_groups` consecutive [box_rows][16] swizzled
// sub-tiles, identical to what box_groups separate 2-D copies produce.
inline bool make_tensor_map_f64_grouped(CUtensorMap *map, const double *base, size_t rows,
                                        size_t cols, unsigned box_rows, unsigned box_groups) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || (cols % 16) != 0) return false;
  cuuint64_t dims[3] = {16, (cuuint64_t)rows, (cuuint64_t)(cols / 16)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * sizeof(double), 16 * sizeof(double)};
  cuuint32_t box[3] = {16, box_rows, box_groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3, const_cast<double *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS && getenv("MG_DEBUG"))
    fprintf(stderr, "grouped tensor map rejected: CUresult %d (rows %zu cols %zu box %u x %u)\n",
            (int)r, rows, cols, box_rows, box_groups);
  return r == CUDA_SUCCESS;
}

// ---------------------------------------------------------------------------
// Device: mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `limit_cycles` SM clock cycles (about two
// seconds) or as soon as another thread of the CTA has raised *abort_flag.
// Returns false on give-up; the caller then raises the kernel fault word and
// leaves its loops, so a lost copy can never hang the GPU.
constexpr long long kWaitLimitCycles = 4000000000ll;

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

// ---------------------------------------------------------------------------
// Device: TMA 2-D tile load, global -> shared, completion on an mbarrier.
// x is the innermost (column) coordinate and must be a multiple of 2 doubles
// (16 bytes); every call site passes multiples of 16.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_dst),
      "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// 3-D form for the grouped view above: x is always 0, y the first row, z the
// first 16-column group.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap *map, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];" ::"r"(smem_dst),
      "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------
// Device: FP64 tensor-core MMA (D = A.B + D), the four shapes sm_100a accepts.
// Fragment ownership for lane = 4*g + t (g = 0..7, t = 0..3):
//   A (m x k, row):  rows g (and g+8 for m16), k slots t, t+4, t+8, t+12
//   B (k x 8, col):  k slots t, t+4, ..., column g
//   C/D (m x 8):     rows g (c0,c1) and g+8 (c2,c3), columns 2t and 2t+1
// ---------------------------------------------------------------------------
__device__ __forceinline__ void dmma_m8n8k4(double &c0, double &c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1)
               : "d"(a), "d"(b));
}

__device__ __forceinline__ void dmma_m16n8k4(double (&c)[4], double a0, double a1, double b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
      "{%0,%1,%2,%3};"
      : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
      : "d"(a0), "d"(a1), "d"(b0));
}

__device__ __forceinline__ void dmma_m16n8k8(double (&c)[4], double a0, double a1, double a2,
                                             double a3, double b0, double b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
      : "d"(a0), "d"(a1), "d"(a2), "d"(a3), "d"(b0), "d"(b1));
}

__device__ __forceinline__ void dmma_m16n8k16(double (&c)[4], double a0, double a1, double a2,
                                              double a3, double a4, double a5, double a6, double a7,
                                              double b0, double b1, double b2, double b3) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, "
      "{%4,%5,%6,%7,%8,%9,%10,%11}, {%12,%13,%14,%15}, {%0,%1,%2,%3};"
      : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
      : "d"(a0), "d"(a1), "d"(a2), "d"(a3), "d"(a4), "d"(a5), "d"(a6), "d"(a7), "d"(b0), "d"(b1),
        "d"(b2), "d"(b3));
}

}  // namespace mg
