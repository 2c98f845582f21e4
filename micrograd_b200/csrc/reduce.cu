// Reductions: full sum, last-axis sum, column sum (bias gradients), softmax
// cross-entropy and row argmax.
//
// Every reduction has a fixed association order: per-thread strided partial
// sums, a warp-shuffle butterfly, a shared-memory tree across the warps of a
// CTA, and a second level over a fixed number of per-CTA partials that the last
// CTA to finish folds in index order.  The order depends only on the problem
// size, never on scheduling, so a result is reproducible from run to run.
#include "common.cuh"

#include <mutex>

namespace mg {

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

__device__ __forceinline__ double warp_max(double v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// Sum of `v` over the CTA (blockDim.x a multiple of 32, at most 1024); the
// result is valid in thread 0.
__device__ __forceinline__ double block_sum(double v, double *smem32) {
  const int lane_id = threadIdx.x & 31, warp_id = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane_id == 0) smem32[warp_id] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  double t = (threadIdx.x < nwarps) ? smem32[threadIdx.x] : 0.0;
  if (warp_id == 0) t = warp_sum(t);
  __syncthreads();
  return t;
}

// Second level: CTA `blockIdx.x` publishes its partial; the last CTA to arrive
// (ticket counter) sums all partials in index order, scales, and stores or
// accumulates the result.  The ticket is reset for the next launch.
__device__ __forceinline__ void finish_partials(double partial, double *partials,
                                                unsigned int *ticket, double *out, double scale,
                                                double *smem32) {
  __shared__ bool is_last;
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = partial;
    __threadfence();
    unsigned int t = atomicAdd(ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  double acc = 0.0;
  for (unsigned i = threadIdx.x; i < gridDim.x; i += blockDim.x) acc += __ldcg(partials + i);
  acc = block_sum(acc, smem32);
  if (threadIdx.x == 0) {
    out[0] = acc * scale;
    *ticket = 0u;
  }
}

// ---------------------------------------------------------------------------
// Full sum (src/ops/Reduction.cpp:17-21).  8 B of traffic per element.
// 256-thread CTAs, at least four resident per SM, at most kSumCtas of them (three
// per SM on a 148-SM part, but a fixed number: the association order must depend on
// n alone), four independent 32-byte loads in flight per thread.  Chosen from a
// sweep on B200 over CTA sizes 128-1024, 2-8 loads in flight and 148-1184 CTAs:
// 25.1 us at 2^24 elements and 296 us at 2^28 (7.25 TB/s).  A CTA of 1024 threads
// that needs 64 registers is alone on its SM, and its end-of-CTA fold then idles
// the SM: 28 us at 2^24.
// ---------------------------------------------------------------------------
constexpr int kSumThreads = 256;
constexpr int kSumMinCtasPerSm = 4;
constexpr int kSumCtas = 444;
static_assert(kSumCtas <= kReducePartials, "partials buffer too small");

template <int VEC>
__global__ void __launch_bounds__(kSumThreads, kSumMinCtasPerSm)
sum_all_kernel(const double *__restrict__ x, size_t n, double *partials, unsigned int *ticket,
               double *out) {
  __shared__ double smem32[32];
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
  if (VEC == 4) {
    const double4v *xv = reinterpret_cast<const double4v *>(x);
    const size_t nvec = n >> 2;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      double4v v0 = ld_stream_v4(xv + i), v1 = ld_stream_v4(xv + i + stride),
               v2 = ld_stream_v4(xv + i + 2 * stride), v3 = ld_stream_v4(xv + i + 3 * stride);
      a0 += (v0.x + v0.y) + (v0.z + v0.w);
      a1 += (v1.x + v1.y) + (v1.z + v1.w);
      a2 += (v2.x + v2.y) + (v2.z + v2.w);
      a3 += (v3.x + v3.y) + (v3.z + v3.w);
    }
    for (; i < nvec; i += stride) {
      double4v v = ld_stream_v4(xv + i);
      a0 += (v.x + v.y) + (v.z + v.w);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 3)) a1 += x[(nvec << 2) + threadIdx.x];
  } else if (VEC == 2) {
    const double2 *xv = reinterpret_cast<const double2 *>(x);
    const size_t nvec = n >> 1;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      double2 v0 = __ldcs(xv + i), v1 = __ldcs(xv + i + stride), v2 = __ldcs(xv + i + 2 * stride),
              v3 = __ldcs(xv + i + 3 * stride);
      a0 += v0.x + v0.y;
      a1 += v1.x + v1.y;
      a2 += v2.x + v2.y;
      a3 += v3.x + v3.y;
    }
    for (; i < nvec; i += stride) {
      double2 v = __ldcs(xv + i);
      a0 += v.x + v.y;
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) a1 += x[n - 1];
  } else {
    for (; i < n; i += stride) a0 += __ldcs(x + i);
  }
  double t = block_sum((a0 + a1) + (a2 + a3), smem32);
  finish_partials(t, partials, ticket, out, 1.0, smem32);
}

// ---------------------------------------------------------------------------
// Last-axis sum [M,N] -> [M]: one warp per row, four warps per CTA (small CTAs
// spread a few thousand rows evenly over the SMs), lanes stride the row in
// 32-byte words with four loads in flight, butterfly at the end.
// ---------------------------------------------------------------------------
constexpr int kLastAxisThreads = 128;

template <int VEC>
__global__ void __launch_bounds__(kLastAxisThreads)
sum_lastaxis_kernel(const double *__restrict__ x, double *__restrict__ out, size_t M, size_t N) {
  const int lane_id = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  for (; row < M; row += warps) {
    const double *r = x + row * N;
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    if (VEC == 4) {
      const double4v *rv = reinterpret_cast<const double4v *>(r);
      const size_t nvec = N >> 2;
      size_t j = lane_id;
      for (; j + 96 < nvec; j += 128) {
        double4v v0 = ld_stream_v4(rv + j), v1 = ld_stream_v4(rv + j + 32),
                 v2 = ld_stream_v4(rv + j + 64), v3 = ld_stream_v4(rv + j + 96);
        a0 += (v0.x + v0.y) + (v0.z + v0.w);
        a1 += (v1.x + v1.y) + (v1.z + v1.w);
        a2 += (v2.x + v2.y) + (v2.z + v2.w);
        a3 += (v3.x + v3.y) + (v3.z + v3.w);
      }
      for (; j < nvec; j += 32) {
        double4v v = ld_stream_v4(rv + j);
        a0 += (v.x + v.y) + (v.z + v.w);
      }
    } else if (VEC == 2) {
      const double2 *rv = reinterpret_cast<const double2 *>(r);
      const size_t nvec = N >> 1;
      size_t j = lane_id;
      for (; j + 32 < nvec; j += 64) {
        double2 v0 = __ldcs(rv + j), v1 = __ldcs(rv + j + 32);
        a0 += v0.x + v0.y;
        a1 += v1.x + v1.y;
      }
      for (; j < nvec; j += 32) {
        double2 v = __ldcs(rv + j);
        a0 += v.x + v.y;
      }
    } else {
      for (size_t j = lane_id; j < N; j += 32) a0 += __ldcs(r + j);
    }
    double t = warp_sum((a0 + a1) + (a2 + a3));
    if (lane_id == 0) out[row] = t;
  }
}

// ---------------------------------------------------------------------------
// Column sum over rows (bias gradient; add_row backward), optionally fused with
// the pass-through gx += g so that g is read once: 24 B per element with gx,
// 8 B without.
//   stage 1: grid (column tiles, S row chunks); thread (tx, ty) walks rows
//            ty, ty+TY, ... of its chunk for column word tx; shared-memory fold
//            over ty in index order -> partials[s][col]
//   stage 2: one thread per column folds the S partials in index order.
// ---------------------------------------------------------------------------
template <int VEC, int TX>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const double *__restrict__ g, double *__restrict__ gx, bool gx_accumulate,
                      double *__restrict__ partials, size_t M, size_t N, size_t rows_per_chunk,
                      double *__restrict__ direct_out, bool direct_accumulate) {
  constexpr int TY = 256 / TX;
  __shared__ double sm[TY][TX * VEC + 1];
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  const size_t ncol = N / VEC;
  const size_t cv = (size_t)blockIdx.x * TX + tx;
  const size_t r0 = (size_t)blockIdx.y * rows_per_chunk;
  size_t r1 = r0 + rows_per_chunk;
  if (r1 > M) r1 = M;
  double acc[VEC];
#pragma unroll
  for (int l = 0; l < VEC; l++) acc[l] = 0.0;
  if (cv < ncol) {
    if (VEC == 2) {
      // Four rows per trip, all loads issued before the first store, so a thread
      // keeps 4-8 independent 16-byte requests in flight.
      const double2 *gv = reinterpret_cast<const double2 *>(g);
      double2 *xv = reinterpret_cast<double2 *>(gx);
      size_t r = r0 + ty;
      for (; r + 3 * TY < r1; r += 4 * TY) {
        double2 v[4], o[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = __ldcs(gv + (r + u * TY) * ncol + cv);
        if (gx && gx_accumulate) {
#pragma unroll
          for (int u = 0; u < 4; u++) o[u] = __ldcs(xv + (r + u * TY) * ncol + cv);
        } else {
#pragma unroll
          for (int u = 0; u < 4; u++) o[u] = make_double2(0.0, 0.0);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          acc[0] += v[u].x;
          acc[VEC - 1] += v[u].y;
          if (gx) {
            o[u].x += v[u].x;
            o[u].y += v[u].y;
            __stcs(xv + (r + u * TY) * ncol + cv, o[u]);
          }
        }
      }
      for (; r < r1; r += TY) {
        const size_t at = r * ncol + cv;
        double2 v = __ldcs(gv + at);
        acc[0] += v.x;
        acc[VEC - 1] += v.y;
        if (gx) {
          double2 o = gx_accumulate ? __ldcs(xv + at) : make_double2(0.0, 0.0);
          o.x += v.x;
          o.y += v.y;
          __stcs(xv + at, o);
        }
      }
    } else {
      for (size_t r = r0 + ty; r < r1; r += TY) {
        const size_t at = r * ncol + cv;
        double v = __ldcs(g + at);
        acc[0] += v;
        if (gx) {
          double o = gx_accumulate ? __ldcs(gx + at) : 0.0;
          __stcs(gx + at, o + v);
        }
      }
    }
  }
#pragma unroll
  for (int l = 0; l < VEC; l++) sm[ty][tx * VEC + l] = acc[l];
  __syncthreads();
  if (ty == 0 && cv < ncol) {
#pragma unroll
    for (int l = 0; l < VEC; l++) {
      double t = 0.0;
      for (int y = 0; y < TY; y++) t += sm[y][tx * VEC + l];
      if (direct_out) {
        // A single row chunk: this is already the column sum; no second stage.
        double *dst = direct_out + cv * VEC + l;
        *dst = direct_accumulate ? *dst + t : t;
      } else {
        partials[(size_t)blockIdx.y * N + cv * VEC + l] = t;
      }
    }
  }
}

// One warp per column: lane l folds partials l, l+32, ... in index order, then a
// butterfly over the lanes — a fixed order, so the result is reproducible.
__global__ void colsum_finish_kernel(const double *__restrict__ partials, size_t S, size_t N,
                                     double *__restrict__ out, bool accumulate) {
  const int lane_id = threadIdx.x & 31;
  const size_t j = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (j >= N) return;
  double t = 0.0;
  for (size_t s = lane_id; s < S; s += 32) t += partials[s * N + j];
  t = warp_sum(t);
  if (lane_id == 0) out[j] = accumulate ? out[j] + t : t;
}

// ---------------------------------------------------------------------------
// Softmax cross-entropy over rows, one warp per row.
//   m = max_j z_j ; s = sum_j exp(z_j - m) ; loss_i = -(z_y - m - log s)
// Forward folds the per-row losses with the same two-level scheme as the full
// sum and divides by `denom`.  Backward recomputes m and s (the logits row is
// C doubles, far cheaper to re-read than to save the probabilities).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void row_max_sumexp(const double *r, size_t C, int lane_id, double &mx,
                                               double &s) {
  double m = -INFINITY;
  for (size_t j = lane_id; j < C; j += 32) m = fmax(m, r[j]);
  m = warp_max(m);
  double t = 0.0;
  for (size_t j = lane_id; j < C; j += 32) t += exp(r[j] - m);
  s = warp_sum(t);
  mx = m;
}

__global__ void __launch_bounds__(kReduceThreads)
softmax_xent_fwd_kernel(const double *__restrict__ z, const int *__restrict__ labels, size_t M,
                        size_t C, double inv_scale_denom, double *partials, unsigned int *ticket,
                        double *out, int *status) {
  __shared__ double smem32[32];
  const int lane_id = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  double local = 0.0;
  for (size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps) {
    const double *r = z + row * C;
    double mx, s;
    row_max_sumexp(r, C, lane_id, mx, s);
    if (lane_id == 0) {
      int y = labels[row];
      if (y < 0 || (size_t)y >= C) {
        atomicExch(status, 101);  // label out of range: flag it, count no loss
      } else {
        local += -(r[y] - mx - log(s));
      }
    }
  }
  double t = block_sum(local, smem32);
  finish_partials(t, partials, ticket, out, inv_scale_denom, smem32);
}

__global__ void __launch_bounds__(256)
softmax_xent_bwd_kernel(const double *__restrict__ z, const int *__restrict__ labels,
                        const double *__restrict__ gloss, double *__restrict__ gz, size_t M,
                        size_t C, double denom, bool accumulate) {
  const int lane_id = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const double gl = __ldg(gloss);
  for (size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps) {
    const double *r = z + row * C;
    double mx, s;
    row_max_sumexp(r, C, lane_id, mx, s);
    const int y = labels[row];
    for (size_t j = lane_id; j < C; j += 32) {
      const double p = exp(r[j] - mx) / s;
      const double v = gl * (p - ((int)j == y ? 1.0 : 0.0)) / denom;
      double *dst = gz + row * C + j;
      *dst = accumulate ? (*dst + v) : v;
    }
  }
}

// Row argmax: first index of the strict maximum (ties keep the lower index).
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const double *__restrict__ x, int *__restrict__ out, size_t M, size_t N) {
  const int lane_id = threadIdx.x & 31;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t row = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps) {
    const double *r = x + row * N;
    double best = -INFINITY;
    unsigned long long best_j = ~0ull;  // "no candidate yet"
    for (size_t j = lane_id; j < N; j += 32) {
      double v = r[j];
      if (best_j == ~0ull || v > best) {
        best = v;
        best_j = j;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      double ov = __shfl_xor_sync(0xffffffffu, best, off);
      unsigned long long oj = __shfl_xor_sync(0xffffffffu, best_j, off);
      if (oj != ~0ull && (best_j == ~0ull || ov > best || (ov == best && oj < best_j))) {
        best = ov;
        best_j = oj;
      }
    }
    if (lane_id == 0) out[row] = (int)best_j;
  }
}

// Narrow rows (N <= kNarrowCols, the ten logits of a classifier): a warp per row
// leaves most lanes idle and serialises on one dependent load per row.  Here a CTA
// takes kNarrowRows consecutive rows — one contiguous range of the matrix — copies
// it to shared memory with coalesced loads, and every thread then walks one row left
// to right exactly as the reference's loop does (src/main.cpp:29-32: `>` against the
// best so far, so ties keep the lower index and a NaN never replaces anything).
constexpr int kNarrowRows = 128;
constexpr int kNarrowCols = 32;

__global__ void __launch_bounds__(kNarrowRows)
argmax_narrow_rows_kernel(const double *__restrict__ x, int *__restrict__ out, size_t M, int N) {
  extern __shared__ double tile[];  // kNarrowRows x stride doubles, sized by the launch
  const int stride = N | 1;         // odd row pitch: the column walk spreads over the banks
  const size_t tiles = (M + kNarrowRows - 1) / kNarrowRows;
  for (size_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const size_t row0 = t * kNarrowRows;
    const int rows = (int)(M - row0 < (size_t)kNarrowRows ? M - row0 : (size_t)kNarrowRows);
    const double *src = x + row0 * (size_t)N;
    const int count = rows * N;
    for (int i = threadIdx.x; i < count; i += kNarrowRows) {
      const int r = i / N;
      tile[r * stride + (i - r * N)] = src[i];
    }
    __syncthreads();
    if ((int)threadIdx.x < rows) {
      const double *r = tile + threadIdx.x * stride;
      double best = r[0];
      int best_j = 0;
      for (int j = 1; j < N; j++) {
        const double v = r[j];
        if (v > best) {
          best = v;
          best_j = j;
        }
      }
      out[row0 + threadIdx.x] = best_j;
    }
    __syncthreads();
  }
}

static unsigned sum_grid(size_t vectors) {
  // Enough CTAs that each thread has a few vectors, never more than kSumCtas.
  size_t need = (vectors + (size_t)kSumThreads * 4 - 1) / ((size_t)kSumThreads * 4);
  if (need < 1) need = 1;
  if (need > (size_t)kSumCtas) need = kSumCtas;
  return (unsigned)need;
}

}  // namespace mg

using namespace mg;

extern "C" {

int mg_sum_all_fwd(const double *x, double *out1, size_t n) {
  MG_ENSURE_INIT();
  if (!out1) return fail(MG_ERR_INVALID, "mg_sum_all_fwd: null output");
  if (n == 0) return mg_fill(out1, 0.0, 1);
  if (!x) return fail(MG_ERR_INVALID, "mg_sum_all_fwd: null input");
  Context &c = ctx();
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x);
  if ((bits & 31) == 0) {
    sum_all_kernel<4><<<sum_grid((n + 3) / 4), kSumThreads, 0, c.stream>>>(x, n, c.reduce_partials,
                                                                          c.reduce_ticket, out1);
  } else if ((bits & 15) == 0) {
    sum_all_kernel<2><<<sum_grid((n + 1) / 2), kSumThreads, 0, c.stream>>>(x, n, c.reduce_partials,
                                                                          c.reduce_ticket, out1);
  } else {
    sum_all_kernel<1><<<sum_grid(n), kSumThreads, 0, c.stream>>>(x, n, c.reduce_partials,
                                                                c.reduce_ticket, out1);
  }
  MG_LAUNCH_CHECK("sum_all_fwd");
  return MG_OK;
}

int mg_sum_lastaxis_fwd(const double *x, double *out, size_t M, size_t N) {
  MG_ENSURE_INIT();
  if (M == 0) return MG_OK;
  if (!out) return fail(MG_ERR_INVALID, "mg_sum_lastaxis_fwd: null output");
  if (N == 0) return mg_fill(out, 0.0, M);
  if (!x) return fail(MG_ERR_INVALID, "mg_sum_lastaxis_fwd: null input");
  Context &c = ctx();
  // 16 CTAs of four warps are resident per SM; two waves of them at most.
  const unsigned grid = grid_for(M * 32, kLastAxisThreads, 32);
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x);
  if ((N % 4 == 0) && (bits & 31) == 0)
    sum_lastaxis_kernel<4><<<grid, kLastAxisThreads, 0, c.stream>>>(x, out, M, N);
  else if ((N % 2 == 0) && (bits & 15) == 0)
    sum_lastaxis_kernel<2><<<grid, kLastAxisThreads, 0, c.stream>>>(x, out, M, N);
  else
    sum_lastaxis_kernel<1><<<grid, kLastAxisThreads, 0, c.stream>>>(x, out, M, N);
  MG_LAUNCH_CHECK("sum_lastaxis_fwd");
  return MG_OK;
}

int mg_add_row_bwd(const double *g, double *gx, double *grow, size_t M, size_t N, int flags) {
  MG_ENSURE_INIT();
  if (M == 0 || N == 0 || (!gx && !grow)) return MG_OK;
  if (!g) return fail(MG_ERR_INVALID, "mg_add_row_bwd: null upstream gradient");
  if (!grow) {
    // Only the pass-through: a plain accumulate.
    return mg_unary_bwd(MG_SADD, nullptr, nullptr, 0.0, g, gx, M * N, flags & MG_ACC_STORE_A);
  }
  if (M == 1) {
    // A single row is its own column sum: one accumulate per destination instead
    // of the two-stage reduction (batch-1 training steps are all launch cost).
    int rc = mg_unary_bwd(MG_SADD, nullptr, nullptr, 0.0, g, grow, N, (flags & MG_ACC_STORE_B) ? MG_ACC_STORE_A : 0);
    if (rc != MG_OK || !gx) return rc;
    return mg_unary_bwd(MG_SADD, nullptr, nullptr, 0.0, g, gx, N, flags & MG_ACC_STORE_A);
  }
  Context &c = ctx();
  uintptr_t bits = reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gx);
  const bool vec = (N % 2 == 0) && (bits & 15) == 0;
  const size_t ncol = vec ? N / 2 : N;
  const int TX = ncol >= 32 ? 32 : 8;
  const int TY = 256 / TX;
  const size_t gridx = (ncol + TX - 1) / TX;
  // Row chunks: about sixteen CTAs per SM (streaming kernels on this part run
  // fastest with many more CTAs than are resident at once), each CTA at least 4
  // passes of TY rows.
  size_t S = (size_t)(c.sm_count * 16) / gridx;
  size_t max_s = (M + (size_t)TY * 4 - 1) / ((size_t)TY * 4);
  if (S > max_s) S = max_s;
  if (S < 1) S = 1;
  if (S > 65535) S = 65535;
  const size_t rows_per_chunk = (M + S - 1) / S;
  S = (M + rows_per_chunk - 1) / rows_per_chunk;
  int rc = ensure_scratch(&c.colsum_scratch, &c.colsum_scratch_elems, S * N);
  if (rc != MG_OK) return rc;
  dim3 grid((unsigned)gridx, (unsigned)S);
  const bool gx_acc = !(flags & MG_ACC_STORE_A);
  // One row chunk (few rows: the small-batch steps): the first stage writes the
  // result itself, the same value the second stage would produce from one partial.
  double *direct = S == 1 ? grow : nullptr;
  const bool direct_acc = !(flags & MG_ACC_STORE_B);
  if (vec) {
    if (TX == 32)
      colsum_partial_kernel<2, 32><<<grid, 256, 0, c.stream>>>(g, gx, gx_acc, c.colsum_scratch, M, N, rows_per_chunk, direct, direct_acc);
    else
      colsum_partial_kernel<2, 8><<<grid, 256, 0, c.stream>>>(g, gx, gx_acc, c.colsum_scratch, M, N, rows_per_chunk, direct, direct_acc);
  } else {
    if (TX == 32)
      colsum_partial_kernel<1, 32><<<grid, 256, 0, c.stream>>>(g, gx, gx_acc, c.colsum_scratch, M, N, rows_per_chunk, direct, direct_acc);
    else
      colsum_partial_kernel<1, 8><<<grid, 256, 0, c.stream>>>(g, gx, gx_acc, c.colsum_scratch, M, N, rows_per_chunk, direct, direct_acc);
  }
  MG_LAUNCH_CHECK("colsum_partial");
  if (direct) return MG_OK;
  colsum_finish_kernel<<<(unsigned)((N * 32 + 255) / 256), 256, 0, c.stream>>>(
      c.colsum_scratch, S, N, grow, !(flags & MG_ACC_STORE_B));
  MG_LAUNCH_CHECK("colsum_finish");
  return MG_OK;
}

int mg_softmax_xent_fwd(const double *logits, const int *labels, double *loss1, size_t M,
                        size_t C, double denom) {
  MG_ENSURE_INIT();
  if (!loss1) return fail(MG_ERR_INVALID, "mg_softmax_xent_fwd: null output");
  if (M == 0 || C == 0) return mg_fill(loss1, 0.0, 1);
  if (!logits || !labels) return fail(MG_ERR_INVALID, "mg_softmax_xent_fwd: null input");
  if (!(denom > 0.0)) return fail(MG_ERR_INVALID, "mg_softmax_xent_fwd: denom must be positive");
  Context &c = ctx();
  size_t need = (M * 32 + kReduceThreads - 1) / kReduceThreads;
  unsigned grid = (unsigned)(need < (size_t)kReducePartials ? (need ? need : 1) : kReducePartials);
  softmax_xent_fwd_kernel<<<grid, kReduceThreads, 0, c.stream>>>(
      logits, labels, M, C, 1.0 / denom, c.reduce_partials, c.reduce_ticket, loss1, c.kernel_status);
  MG_LAUNCH_CHECK("softmax_xent_fwd");
  return MG_OK;
}

int mg_softmax_xent_bwd(const double *logits, const int *labels, const double *gloss1,
                        double *glogits, size_t M, size_t C, double denom, int flags) {
  MG_ENSURE_INIT();
  if (M == 0 || C == 0 || !glogits) return MG_OK;
  if (!logits || !labels || !gloss1) return fail(MG_ERR_INVALID, "mg_softmax_xent_bwd: null input");
  if (!(denom > 0.0)) return fail(MG_ERR_INVALID, "mg_softmax_xent_bwd: denom must be positive");
  Context &c = ctx();
  unsigned grid = grid_for(M * 32, 256, 8);
  softmax_xent_bwd_kernel<<<grid, 256, 0, c.stream>>>(logits, labels, gloss1, glogits, M, C, denom,
                                                      !(flags & MG_ACC_STORE_A));
  MG_LAUNCH_CHECK("softmax_xent_bwd");
  return MG_OK;
}

int mg_argmax_rows(const double *x, int *out, size_t M, size_t N) {
  MG_ENSURE_INIT();
  if (M == 0) return MG_OK;
  if (!x || !out) return fail(MG_ERR_INVALID, "mg_argmax_rows: null pointer");
  if (N == 0) return fail(MG_ERR_INVALID, "mg_argmax_rows: rows are empty");
  Context &c = ctx();
  if (N <= (size_t)kNarrowCols) {
    const size_t tiles = (M + kNarrowRows - 1) / kNarrowRows;
    // The tile is sized by the actual column count (11 KB for ten columns, 34 KB at
    // most), so shared memory does not cap residency; about four waves of CTAs.
    const size_t tile_bytes = (size_t)kNarrowRows * (N | 1) * sizeof(double);
    const size_t cap = (size_t)c.sm_count * 40;
    argmax_narrow_rows_kernel<<<(unsigned)(tiles < cap ? tiles : cap), kNarrowRows, tile_bytes,
                                c.stream>>>(x, out, M, (int)N);
  } else {
    argmax_rows_kernel<<<grid_for(M * 32, 256, 8), 256, 0, c.stream>>>(x, out, M, N);
  }
  MG_LAUNCH_CHECK("argmax_rows");
  return MG_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Column sum without any allocation.
//
// Some callers must not allocate device memory at the moment they need a bias
// gradient: code running inside a latency-critical loop where a cudaMalloc
// would stall the whole device, a process whose memory has been handed in full
// to another component's pool, or a host framework that forbids allocation
// between two of its own synchronisation points.  For them the partial sums of
// the two-stage column reduction live in a fixed array in the library's own
// device image instead of in pool memory.  Each GPU that loads the library
// carries that array (1 MiB) until the process exits.
//
// Inside host code the array's name is only a handle for the runtime; it is not
// a device address.  The address is looked up once per device with
// cudaGetSymbolAddress, with that device current, and handed to the kernels.
// ---------------------------------------------------------------------------
namespace mg {

constexpr size_t kNoAllocScratchElems = (size_t)1 << 17;  // 131072 doubles = 1 MiB
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) double g_noalloc_colsum_scratch[kNoAllocScratchElems];
static double *g_noalloc_scratch_addr[kNoAllocMaxDevices];  // per device, filled on first use

// Device address of the static scratch on the context's device (looked up once,
// under a lock).  The lookup is keyed on the device the context is bound to, and
// refused when the calling thread has a different device current: a fresh host
// thread starts on device 0, and resolving the symbol there would create a
// context (an allocation) on a GPU this process does not use.
static std::mutex g_noalloc_mutex;

static int noalloc_scratch(double **out) {
  const int device = ctx().device;
  int current = -1;
  MG_CUDA_TRY(cudaGetDevice(&current));
  if (current != device)
    return fail(MG_ERR_INVALID,
                "mg_colsum_noalloc: the calling thread has device %d current but the library is "
                "bound to device %d; call cudaSetDevice(%d) on this thread first",
                current, device, device);
  if (device < 0 || device >= kNoAllocMaxDevices)
    return fail(MG_ERR_INVALID, "mg_colsum_noalloc: device ordinal %d not supported", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_scratch_addr[device]) {
    double *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_colsum_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static column-sum scratch)");
    if (!ptr) return fail(MG_ERR_CUDA, "mg_colsum_noalloc: static scratch has no device address");
    g_noalloc_scratch_addr[device] = ptr;
  }
  *out = g_noalloc_scratch_addr[device];
  return MG_OK;
}

}  // namespace mg

extern "C" int mg_colsum_noalloc(const double *g, double *out_row, size_t M, size_t N,
                                 int accumulate) {
  // No implicit initialisation here: bringing the context up allocates.
  Context &c = ctx();
  if (!c.ready)
    return fail(MG_ERR_INVALID,
                "mg_colsum_noalloc: call mg_init() during set-up; this entry point never allocates");
  if (M == 0 || N == 0) return MG_OK;
  if (!g || !out_row) return fail(MG_ERR_INVALID, "mg_colsum_noalloc: null pointer");
  if (N > kNoAllocScratchElems)
    return fail(MG_ERR_INVALID,
                "mg_colsum_noalloc: %zu columns exceed the static scratch limit of %zu; use "
                "mg_add_row_bwd, which takes its scratch from the pool",
                N, kNoAllocScratchElems);
  double *scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc != MG_OK) return rc;

  const bool vec = (N % 2 == 0) && (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  const size_t ncol = vec ? N / 2 : N;
  const int TX = ncol >= 32 ? 32 : 8;
  const int TY = 256 / TX;
  const size_t gridx = (ncol + TX - 1) / TX;
  // Row chunks as in the pooled path, capped so that S x N partials fit the array.
  size_t S = (size_t)(c.sm_count * 16) / gridx;
  const size_t max_rows = (M + (size_t)TY * 4 - 1) / ((size_t)TY * 4);
  const size_t max_fit = kNoAllocScratchElems / N;
  if (S > max_rows) S = max_rows;
  if (S > max_fit) S = max_fit;
  if (S < 1) S = 1;
  if (S > 65535) S = 65535;
  const size_t rows_per_chunk = (M + S - 1) / S;
  S = (M + rows_per_chunk - 1) / rows_per_chunk;
  // Every partial that stage 2 reads is written by stage 1 of the same call, so
  // nothing left in the array by an earlier call can leak into this result.
  dim3 grid((unsigned)gridx, (unsigned)S);
  if (vec) {
    if (TX == 32)
      colsum_partial_kernel<2, 32><<<grid, 256, 0, c.stream>>>(g, nullptr, false, scratch, M, N, rows_per_chunk, nullptr, false);
    else
      colsum_partial_kernel<2, 8><<<grid, 256, 0, c.stream>>>(g, nullptr, false, scratch, M, N, rows_per_chunk, nullptr, false);
  } else {
    if (TX == 32)
      colsum_partial_kernel<1, 32><<<grid, 256, 0, c.stream>>>(g, nullptr, false, scratch, M, N, rows_per_chunk, nullptr, false);
    else
      colsum_partial_kernel<1, 8><<<grid, 256, 0, c.stream>>>(g, nullptr, false, scratch, M, N, rows_per_chunk, nullptr, false);
  }
  MG_LAUNCH_CHECK("colsum_partial (static scratch)");
  colsum_finish_kernel<<<(unsigned)((N * 32 + 255) / 256), 256, 0, c.stream>>>(scratch, S, N, out_row,
                                                                          accumulate != 0);
  MG_LAUNCH_CHECK("colsum_finish (static scratch)");
  return MG_OK;
}
