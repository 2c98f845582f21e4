// Shared host-side plumbing of the device backend: the per-process context
// (device, streams, scratch), error reporting and launch-geometry helpers.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>

#include "mg_cuda.h"

namespace mg {

// Number of partial sums the two-level reductions use.  Fixed (not derived from
// the device) so that a sum has the same association order on every run.
constexpr int kReducePartials = 1184;  // 148 SMs x 8
constexpr int kReduceThreads = 256;

struct Context {
  bool ready = false;
  int device = -1;
  int sm_count = 0;
  cudaStream_t stream = nullptr;       // compute stream (ordered)
  cudaStream_t comm_stream = nullptr;  // NCCL all-reduces
  cudaStream_t copy_stream = nullptr;  // host -> device prefetch of the next batch
  cudaEvent_t copy_fork_event = nullptr;  // compute -> copy ordering (buffer is allocated)
  cudaEvent_t fork_event = nullptr;    // compute -> comm ordering
  cudaEvent_t join_event = nullptr;    // comm -> compute ordering
  // Scratch for reductions: partial sums and the "blocks done" ticket.
  double *reduce_partials = nullptr;   // kReducePartials doubles (x2 for row/col use)
  unsigned int *reduce_ticket = nullptr;
  // Column-sum scratch (add_row backward, bias gradients): [kColSplit][N].
  double *colsum_scratch = nullptr;
  size_t colsum_scratch_elems = 0;
  // Split-K scratch for the transposed-A GEMM.
  double *splitk_scratch = nullptr;
  size_t splitk_scratch_elems = 0;
  // Kernel fault word: kernels write a non-zero code here instead of trapping.
  int *kernel_status = nullptr;        // device
  int *status_host = nullptr;          // pinned mirror of kernel_status (mg_kernel_status_mirror)
  // L2 flush buffer.
  void *flush_buf = nullptr;
  size_t flush_bytes = 0;
  unsigned long long launches = 0;
  // True between mg_graph_begin() and mg_graph_end(): everything enqueued on the
  // compute stream is being recorded into a CUDA graph instead of executed.
  bool capturing = false;
};

Context &ctx();
int ensure_init();

// Records a formatted message for mg_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

// Grows a scratch buffer (stream-ordered free + alloc) to at least `elems`.
int ensure_scratch(double **buf, size_t *have, size_t elems);

// Frees the segment tables the GEMM dispatcher caches on the device.
void gemm_release_tables();
// Clears the arrival counters of split-contraction tiles (after a kernel fault).
void gemm_reset_tickets();

inline void count_launch() { ctx().launches++; }

#define MG_CUDA_TRY(expr)                                                                          \
  do {                                                                                             \
    cudaError_t mg_e_ = (expr);                                                                    \
    if (mg_e_ != cudaSuccess) return ::mg::cuda_fail(mg_e_, #expr);                                \
  } while (0)

#define MG_ENSURE_INIT()                                                                           \
  do {                                                                                             \
    int mg_rc_ = ::mg::ensure_init();                                                              \
    if (mg_rc_ != MG_OK) return mg_rc_;                                                            \
  } while (0)

// Entry points that wait for the device, touch other streams or read host memory
// later cannot be part of a recorded step.
#define MG_NOT_WHILE_RECORDING(name)                                                               \
  do {                                                                                             \
    if (::mg::ctx().capturing)                                                                     \
      return ::mg::fail(MG_ERR_INVALID, name ": not allowed while a step is being recorded "       \
                                             "(between mg_graph_begin and mg_graph_end)");         \
  } while (0)

#define MG_LAUNCH_CHECK(name)                                                                      \
  do {                                                                                             \
    ::mg::count_launch();                                                                          \
    cudaError_t mg_e_ = cudaGetLastError();                                                        \
    if (mg_e_ != cudaSuccess) return ::mg::cuda_fail(mg_e_, name);                                 \
  } while (0)

// 32-byte vector of four doubles: sm_100 has 256-bit global loads and stores
// (ld/st.global.v4.f64).  The streaming forms keep once-touched data out of L1.
struct __align__(32) double4v {
  double x, y, z, w;
};
#ifdef __CUDACC__
__device__ __forceinline__ double4v ld_stream_v4(const double4v *p) {
  double4v v;
  asm volatile("ld.global.cs.v4.f64 {%0,%1,%2,%3}, [%4];"
               : "=d"(v.x), "=d"(v.y), "=d"(v.z), "=d"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_v4(double4v *p, double4v v) {
  asm volatile("st.global.cs.v4.f64 [%0], {%1,%2,%3,%4};" ::"l"(p), "d"(v.x), "d"(v.y), "d"(v.z),
               "d"(v.w)
               : "memory");
}
#endif

// Grid for a grid-stride kernel over `work_items` with `threads` per CTA:
// enough CTAs to cover the work, capped at `ctas_per_sm` resident CTAs per SM
// so the grid is a whole number of waves on the 148-SM part.
inline unsigned grid_for(size_t work_items, int threads, int ctas_per_sm) {
  size_t need = (work_items + (size_t)threads - 1) / (size_t)threads;
  size_t cap = (size_t)ctx().sm_count * (size_t)ctas_per_sm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

}  // namespace mg
