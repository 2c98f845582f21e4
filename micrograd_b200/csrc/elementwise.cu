// Elementwise forward/backward kernels, row-broadcast add, SGD update, fill.
//
// All of these are HBM-bound streaming kernels: one generic grid-stride "map"
// kernel moves 32-byte vectors (four doubles, the 256-bit global loads/stores of
// sm_100; 16-byte vectors or scalars when a pointer is less aligned) with 64
// bytes per operand in flight per thread, and a small functor supplies the
// arithmetic.  The grid is a whole number of waves (SM count x resident CTAs),
// each thread striding through the array so that consecutive threads touch
// consecutive vectors.
//
// This file is compiled with -fmad=false: the reference rounds every multiply
// and add separately (it is built without FMA contraction), and add, sub, mul,
// relu, their gradients and the SGD update are bit-identical to it only if the
// device does the same.
#include "common.cuh"

namespace mg {

constexpr int kEwThreads = 256;
constexpr int kEwUnroll = 4;
constexpr int kEwWaves = 16;

template <int VEC> struct VecT;
template <> struct VecT<2> {
  using type = double2;
  static __device__ __forceinline__ double2 zero() { return make_double2(0.0, 0.0); }
};
template <> struct VecT<4> {
  using type = double4v;
  static __device__ __forceinline__ double4v zero() { return double4v{0.0, 0.0, 0.0, 0.0}; }
};
template <> struct VecT<1> {
  using type = double;
  static __device__ __forceinline__ double zero() { return 0.0; }
};

__device__ __forceinline__ double lane(const double &v, int) { return v; }
__device__ __forceinline__ double lane(const double2 &v, int i) { return i == 0 ? v.x : v.y; }
__device__ __forceinline__ void set_lane(double &v, int, double x) { v = x; }
__device__ __forceinline__ void set_lane(double2 &v, int i, double x) {
  if (i == 0) v.x = x; else v.y = x;
}

__device__ __forceinline__ double lane(const double4v &v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}
__device__ __forceinline__ void set_lane(double4v &v, int i, double x) {
  if (i == 0) v.x = x; else if (i == 1) v.y = x; else if (i == 2) v.z = x; else v.w = x;
}
__device__ __forceinline__ double4v ld_stream(const double4v *p) { return ld_stream_v4(p); }
__device__ __forceinline__ void st_stream(double4v *p, double4v v) { st_stream_v4(p, v); }

// Streaming loads/stores: every element is touched once, so keep it out of L1.
template <class V> __device__ __forceinline__ V ld_stream(const V *p) { return __ldcs(p); }
template <class V> __device__ __forceinline__ void st_stream(V *p, V v) { __stcs(p, v); }

// F provides: static constexpr int NI, NO; const double *in[NI]; double *out[NO];
// __device__ void compute(const double (&i)[NI], double (&o)[NO]) const.
// A null in[k] reads as 0.0 without touching memory; a null out[k] is skipped.
template <int VEC, class F>
__global__ void __launch_bounds__(kEwThreads) map_kernel(F f, size_t n) {
  using V = typename VecT<VEC>::type;
  constexpr int NI = F::NI, NO = F::NO;
  constexpr int kUnroll = VEC == 4 ? kEwUnroll / 2 : kEwUnroll;  // same bytes in flight per thread
  const size_t nvec = n / VEC;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;

  auto process = [&](const V(&v)[NI > 0 ? NI : 1], size_t at) {
    V o[NO];
#pragma unroll
    for (int l = 0; l < VEC; l++) {
      double si[NI > 0 ? NI : 1], so[NO];
#pragma unroll
      for (int k = 0; k < NI; k++) si[k] = lane(v[k], l);
      f.compute(si, so);
#pragma unroll
      for (int k = 0; k < NO; k++) set_lane(o[k], l, so[k]);
    }
#pragma unroll
    for (int k = 0; k < NO; k++)
      if (f.out[k]) st_stream(reinterpret_cast<V *>(f.out[k]) + at, o[k]);
  };

  // Main loop: kEwUnroll independent vectors per thread; all loads are issued
  // before the first store so they overlap.
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    V v[kUnroll][NI > 0 ? NI : 1];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
#pragma unroll
      for (int k = 0; k < NI; k++)
        v[u][k] = f.in[k] ? ld_stream(reinterpret_cast<const V *>(f.in[k]) + i + u * stride)
                          : VecT<VEC>::zero();
    }
#pragma unroll
    for (int u = 0; u < kUnroll; u++) process(v[u], i + u * stride);
  }
  for (; i < nvec; i += stride) {
    V v[NI > 0 ? NI : 1];
#pragma unroll
    for (int k = 0; k < NI; k++)
      v[k] = f.in[k] ? ld_stream(reinterpret_cast<const V *>(f.in[k]) + i) : VecT<VEC>::zero();
    process(v, i);
  }
  // Tail elements of the vector paths (n not a multiple of VEC).
  if (VEC > 1 && blockIdx.x == 0 && threadIdx.x < (unsigned)(n % VEC)) {
    const size_t at = nvec * VEC + threadIdx.x;
    double si[NI > 0 ? NI : 1], so[NO];
#pragma unroll
    for (int k = 0; k < NI; k++) si[k] = f.in[k] ? f.in[k][at] : 0.0;
    f.compute(si, so);
#pragma unroll
    for (int k = 0; k < NO; k++)
      if (f.out[k]) f.out[k][at] = so[k];
  }
}

template <class F> static uintptr_t pointer_bits(const F &f) {
  uintptr_t bits = 0;
  for (int k = 0; k < F::NI; k++) bits |= reinterpret_cast<uintptr_t>(f.in[k]);
  for (int k = 0; k < F::NO; k++) bits |= reinterpret_cast<uintptr_t>(f.out[k]);
  return bits;
}

// Grid of a streaming kernel: up to kEwWaves times the CTAs that are resident at
// once (occupancy of this very instantiation x SM count), never more than the
// work needs.  Measured on B200 (1R+1W, 2R+1W and read-modify-write maps, 2^24 to
// 2^28 elements, waves = 1, 2, 3, 4, 6, 8, 16, 64): a grid of exactly one
// resident wave is the slowest choice — relu at 2^24 elements 5.39 TB/s with one
// wave, 5.66 with two, 5.99 with four, 6.12 with sixteen; at 2^26 5.87 / 6.14 /
// 6.42 / 6.61 — because SMs do not stream at equal speed and the hardware
// scheduler can only even that out while it has CTAs left to hand out.  Beyond
// sixteen the one-input maps fall off again (the loop degenerates to one vector
// per thread), so sixteen it is.
template <class Kernel> static int resident_ctas_per_sm(Kernel kernel, int threads) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = 1;
  }
  return n;
}

template <int VEC, class F> static unsigned map_grid(size_t n) {
  static const int resident = resident_ctas_per_sm(map_kernel<VEC, F>, kEwThreads);
  return grid_for((n + VEC - 1) / VEC, kEwThreads, resident * kEwWaves);
}

template <class F> static int launch_map(const F &f, size_t n, const char *name) {
  if (n == 0) return MG_OK;
  Context &c = ctx();
  const uintptr_t bits = pointer_bits(f);
  if ((bits & 31) == 0 && n >= 4096) {
    map_kernel<4, F><<<map_grid<4, F>(n), kEwThreads, 0, c.stream>>>(f, n);
  } else if ((bits & 15) == 0) {
    map_kernel<2, F><<<map_grid<2, F>(n), kEwThreads, 0, c.stream>>>(f, n);
  } else {
    map_kernel<1, F><<<map_grid<1, F>(n), kEwThreads, 0, c.stream>>>(f, n);
  }
  MG_LAUNCH_CHECK(name);
  return MG_OK;
}

// ---------------------------------------------------------------------------
// Functors
// ---------------------------------------------------------------------------
template <int OP> struct BinaryFwd {
  static constexpr int NI = 2, NO = 1;
  const double *in[NI];
  double *out[NO];
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    if (OP == MG_ADD) o[0] = i[0] + i[1];
    else if (OP == MG_SUB) o[0] = i[0] - i[1];
    else if (OP == MG_MUL) o[0] = i[0] * i[1];
    else o[0] = i[0] / i[1];
  }
};

// in: g, a, b, old ga, old gb.  out: ga, gb.  Null "old" pointers read as 0, which
// turns the accumulation into a plain store of the same value.
template <int OP> struct BinaryBwd {
  static constexpr int NI = 5, NO = 2;
  const double *in[NI];
  double *out[NO];
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    const double g = i[0], a = i[1], b = i[2];
    if (OP == MG_ADD) {
      o[0] = i[3] + g;
      o[1] = i[4] + g;
    } else if (OP == MG_SUB) {
      o[0] = i[3] + g;
      o[1] = i[4] - g;
    } else if (OP == MG_MUL) {
      o[0] = i[3] + g * b;
      o[1] = i[4] + g * a;
    } else {
      o[0] = i[3] + g / b;
      o[1] = i[4] - (g * a) / (b * b);
    }
  }
};

// ---------------------------------------------------------------------------
// tanh without branches.  The library tanh takes two different paths around
// |x| = 0.55, so nearly every warp of a mixed-sign, unit-scale input executes
// both and the kernel becomes bound by the FP64 pipe instead of by HBM.  This
// form has one path of about 35 FP64 instructions:
//   e = expm1(-2|x|) = 2^k (expm1(r) + 1) - 1   with -2|x| = k ln2 + r, |r| <= ln2/2
//   tanh|x| = -e / (2 + e)
// expm1(r) is the degree-13 Taylor polynomial (truncation below 5e-17 relative);
// the quotient uses the hardware reciprocal seed refined twice plus a remainder
// step (the divisor lies in [1, 2], so no scaling cases arise).  |x| is clamped
// to 20, beyond which the result is 1 in double precision.  tanh(+-0) = +-0,
// subnormal inputs are returned exactly, NaN propagates.  Against a correctly
// rounded tanh the result differs by at most 3 units in the last place
// (6.7e-16 relative); std::tanh of the reference (src/ops/Activations.cpp:74)
// is itself accurate to about 1.
// ---------------------------------------------------------------------------
__device__ __forceinline__ double tanh_onepath(double x) {
  const double am = fmin(fabs(x), 20.0);
  const double z = -2.0 * am;
  const double kMagic = 6755399441055744.0;  // 1.5 * 2^52: adding it rounds to an integer
  const double km = fma(z, 1.4426950408889634074, kMagic);
  const double kd = km - kMagic;
  double r = fma(kd, -6.93147180369123816490e-01, z);
  r = fma(kd, -1.90821492927058770002e-10, r);
  double q = 1.0 / 6227020800.0;
  q = fma(q, r, 1.0 / 479001600.0);
  q = fma(q, r, 1.0 / 39916800.0);
  q = fma(q, r, 1.0 / 3628800.0);
  q = fma(q, r, 1.0 / 362880.0);
  q = fma(q, r, 1.0 / 40320.0);
  q = fma(q, r, 1.0 / 5040.0);
  q = fma(q, r, 1.0 / 720.0);
  q = fma(q, r, 1.0 / 120.0);
  q = fma(q, r, 1.0 / 24.0);
  q = fma(q, r, 1.0 / 6.0);
  q = fma(q, r, 0.5);
  const double p = fma(r * r, q, r);  // expm1(r)
  const int k = __double2loint(km);   // low word of km holds k in two's complement
  const double s = __hiloint2double((k + 1023) << 20, 0);  // 2^k, k in [-58, 0]
  const double e = fma(s, p, s - 1.0);
  const double d = 2.0 + e, n = -e;
  double y;
  asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(d));
  double err = fma(-d, y, 1.0);
  y = fma(y, err, y);
  err = fma(-d, y, 1.0);
  y = fma(y, err, y);
  double t = n * y;
  t = fma(fma(-d, t, n), y, t);
  t = copysign(t, x);
  return (x != x) ? x + x : t;
}

template <int OP> struct UnaryFwd {
  static constexpr int NI = 1, NO = 1;
  const double *in[NI];
  double *out[NO];
  double s;
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    const double x = i[0];
    if (OP == MG_SADD) o[0] = x + s;
    else if (OP == MG_SSUB) o[0] = x - s;
    else if (OP == MG_SMUL) o[0] = x * s;
    else if (OP == MG_SDIV) o[0] = x / s;
    else if (OP == MG_POW) o[0] = pow(x, s);
    else if (OP == MG_RELU) o[0] = x > 0 ? x : 0.0;
    else if (OP == MG_SIGMOID) o[0] = 1.0 / (1.0 + exp(-x));
    else if (OP == MG_TANH) o[0] = tanh_onepath(x);
    else o[0] = exp(x);
  }
};

// in: g, a (forward input), y (forward output), old ga.  out: ga.
template <int OP> struct UnaryBwd {
  static constexpr int NI = 4, NO = 1;
  const double *in[NI];
  double *out[NO];
  double s;
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    const double g = i[0], a = i[1], y = i[2], old = i[3];
    if (OP == MG_SADD || OP == MG_SSUB) o[0] = old + g;
    else if (OP == MG_SMUL) o[0] = old + g * s;
    else if (OP == MG_SDIV) o[0] = old + g / s;
    else if (OP == MG_POW) o[0] = old + (g * s) * pow(a, s - 1.0);
    else if (OP == MG_RELU) o[0] = old + g * (a > 0 ? 1.0 : 0.0);
    else if (OP == MG_SIGMOID) o[0] = old + (g * y) * (1.0 - y);
    else if (OP == MG_TANH) o[0] = old + g * (1.0 - y * y);
    else o[0] = old + g * y;
  }
};

struct FillFn {
  static constexpr int NI = 0, NO = 1;
  const double *in[1];
  double *out[NO];
  double value;
  __device__ __forceinline__ void compute(const double (&)[1], double (&o)[NO]) const {
    o[0] = value;
  }
};

// in: p, g.  out: p.  p - (lr*g) with the product rounded first (src/nn.cpp:74).
struct SgdFn {
  static constexpr int NI = 2, NO = 1;
  const double *in[NI];
  double *out[NO];
  double lr;
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    o[0] = i[0] - lr * i[1];
  }
};

// ---------------------------------------------------------------------------
// Row-broadcast add: out[r, c] = x[r, c] + row[c].  Each thread owns flat vectors
// (32, 16 or 8 bytes) and advances its column incrementally, so the loop has no
// division; two vectors are in flight per thread.  x and out may be the same
// buffer (the in-place accumulate of sum(axis=0) backward): every thread reads
// its own words before it writes them, and neither pointer is declared restrict.
// ---------------------------------------------------------------------------
constexpr int kRowUnroll = 2;

template <int VEC>
__global__ void __launch_bounds__(kEwThreads)
add_row_kernel(const double *x, const double *__restrict__ row, double *out, size_t M, size_t N) {
  using V = typename VecT<VEC>::type;
  const size_t ncol = N / VEC;  // vectors per row
  const size_t total = M * ncol;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t dcol = stride % ncol;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t c = i % ncol;
  const V *xv = reinterpret_cast<const V *>(x);
  const V *rv = reinterpret_cast<const V *>(row);
  V *ov = reinterpret_cast<V *>(out);
  auto next_col = [&](size_t col) {
    col += dcol;
    return col >= ncol ? col - ncol : col;
  };
  for (; i + (kRowUnroll - 1) * stride < total; i += kRowUnroll * stride) {
    V a[kRowUnroll], b[kRowUnroll];
    size_t col = c;
#pragma unroll
    for (int u = 0; u < kRowUnroll; u++) {
      a[u] = ld_stream(xv + i + u * stride);
      b[u] = rv[col];
      col = next_col(col);
    }
    c = col;
#pragma unroll
    for (int u = 0; u < kRowUnroll; u++) {
      V o;
#pragma unroll
      for (int l = 0; l < VEC; l++) set_lane(o, l, lane(a[u], l) + lane(b[u], l));
      st_stream(ov + i + u * stride, o);
    }
  }
  for (; i < total; i += stride) {
    V a = ld_stream(xv + i);
    V b = rv[c];
    V o;
#pragma unroll
    for (int l = 0; l < VEC; l++) set_lane(o, l, lane(a, l) + lane(b, l));
    st_stream(ov + i, o);
    c = next_col(c);
  }
}


// sum() backward: gx[i] += g[0], the scalar read from device memory
// (src/ops/Reduction.cpp:26-30).  in: old gx.  out: gx.
struct ScalarBroadcastBwd {
  static constexpr int NI = 1, NO = 1;
  const double *in[NI];
  double *out[NO];
  const double *g0;
  __device__ __forceinline__ void compute(const double (&i)[NI], double (&o)[NO]) const {
    o[0] = i[0] + __ldg(g0);
  }
};

// Last-axis-sum backward: gx[r, c] += g[r].  Same walk as the row-broadcast add,
// tracking the row as well.
template <int VEC>
__global__ void __launch_bounds__(kEwThreads)
row_scalar_bwd_kernel(const double *__restrict__ g, double *__restrict__ gx, size_t M, size_t N,
                      bool accumulate) {
  using V = typename VecT<VEC>::type;
  const size_t ncol = N / VEC;
  const size_t total = M * ncol;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t drow = stride / ncol, dcol = stride % ncol;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t r = i / ncol, c = i % ncol;
  V *gv = reinterpret_cast<V *>(gx);
  auto advance = [&](size_t &row, size_t &col) {
    col += dcol;
    row += drow;
    if (col >= ncol) {
      col -= ncol;
      row++;
    }
  };
  for (; i + (kRowUnroll - 1) * stride < total; i += kRowUnroll * stride) {
    V o[kRowUnroll];
    double sc[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; u++) {
      sc[u] = __ldg(g + r);
      o[u] = accumulate ? ld_stream(gv + i + u * stride) : VecT<VEC>::zero();
      advance(r, c);
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; u++) {
#pragma unroll
      for (int l = 0; l < VEC; l++) set_lane(o[u], l, lane(o[u], l) + sc[u]);
      st_stream(gv + i + u * stride, o[u]);
    }
  }
  for (; i < total; i += stride) {
    const double sc = __ldg(g + r);
    V o = accumulate ? ld_stream(gv + i) : VecT<VEC>::zero();
#pragma unroll
    for (int l = 0; l < VEC; l++) set_lane(o, l, lane(o, l) + sc);
    st_stream(gv + i, o);
    advance(r, c);
  }
}

// 2x2 mean pooling of 28x28 images stored as rows of 784 values -> rows of 196
// (src/nn.cpp:17-35): ((a + b) + c) + d, then / 4.0, in the reference's order.
__global__ void avg_pool_28_kernel(const double *__restrict__ x, double *__restrict__ out,
                                   size_t batch) {
  const size_t total = batch * 196;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t b = i / 196, cell = i % 196;
    const size_t py = cell / 14, px = cell % 14;
    const double *img = x + b * 784 + (py * 2) * 28 + px * 2;
    double sum = 0.0;
    sum += img[0];
    sum += img[1];
    sum += img[28];
    sum += img[29];
    out[i] = sum / 4.0;
  }
}

// dst[i] = src[i] / divisor, the byte widened to double first (pixel / 255.0 of
// src/mnist.cpp:21: one IEEE division, so the values equal the host's).
__global__ void u8_scale_kernel(const unsigned char *__restrict__ src, double *__restrict__ dst,
                                size_t n, double divisor) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = (double)src[i] / divisor;
}

__global__ void f64_to_i32_kernel(const double *__restrict__ src, int *__restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = (int)src[i];
}

}  // namespace mg

using namespace mg;

// Dispatch a runtime op code to the functor template.
#define MG_DISPATCH_BINARY(OPVAR, CALL)                                                            \
  switch (OPVAR) {                                                                                 \
    case MG_ADD: { constexpr int OP = MG_ADD; CALL; } break;                                       \
    case MG_SUB: { constexpr int OP = MG_SUB; CALL; } break;                                       \
    case MG_MUL: { constexpr int OP = MG_MUL; CALL; } break;                                       \
    case MG_DIV: { constexpr int OP = MG_DIV; CALL; } break;                                       \
    default: return fail(MG_ERR_INVALID, "unknown binary op %d", OPVAR);                           \
  }

#define MG_DISPATCH_UNARY(OPVAR, CALL)                                                             \
  switch (OPVAR) {                                                                                 \
    case MG_SADD: { constexpr int OP = MG_SADD; CALL; } break;                                     \
    case MG_SSUB: { constexpr int OP = MG_SSUB; CALL; } break;                                     \
    case MG_SMUL: { constexpr int OP = MG_SMUL; CALL; } break;                                     \
    case MG_SDIV: { constexpr int OP = MG_SDIV; CALL; } break;                                     \
    case MG_POW: { constexpr int OP = MG_POW; CALL; } break;                                       \
    case MG_RELU: { constexpr int OP = MG_RELU; CALL; } break;                                     \
    case MG_SIGMOID: { constexpr int OP = MG_SIGMOID; CALL; } break;                               \
    case MG_TANH: { constexpr int OP = MG_TANH; CALL; } break;                                     \
    case MG_EXP: { constexpr int OP = MG_EXP; CALL; } break;                                       \
    default: return fail(MG_ERR_INVALID, "unknown unary op %d", OPVAR);                            \
  }

template <int OP>
static int binary_bwd_one(const double *a, const double *b, const double *g, double *ga, double *gb,
                          size_t n, int flags) {
  BinaryBwd<OP> f;
  const bool needs_ab = (OP == MG_MUL || OP == MG_DIV);
  f.in[0] = g;
  f.in[1] = needs_ab ? a : nullptr;
  f.in[2] = needs_ab ? b : nullptr;
  f.in[3] = (ga && !(flags & MG_ACC_STORE_A)) ? ga : nullptr;
  f.in[4] = (gb && !(flags & MG_ACC_STORE_B)) ? gb : nullptr;
  f.out[0] = ga;
  f.out[1] = gb;
  return launch_map(f, n, "binary_bwd");
}

// Several small parameter tensors in one launch (the per-tensor form costs a
// launch each, which is all a batch-1 training step consists of).  p - (lr*g)
// with the product rounded first, like SgdFn.
struct SgdBatch {
  double *param[8];
  const double *grad[8];
  unsigned long long n[8];
  int count;
};

__global__ void __launch_bounds__(256) sgd_multi_kernel(SgdBatch b, double lr) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int t = 0; t < b.count; t++) {
    double *p = b.param[t];
    const double *g = b.grad[t];
    const size_t n = (size_t)b.n[t];
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) == 0) {
      const size_t pairs = n >> 1;
      for (; i < pairs; i += stride) {
        double2 pv = reinterpret_cast<double2 *>(p)[i];
        const double2 gv = reinterpret_cast<const double2 *>(g)[i];
        pv.x = pv.x - lr * gv.x;
        pv.y = pv.y - lr * gv.y;
        reinterpret_cast<double2 *>(p)[i] = pv;
      }
      if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) p[n - 1] = p[n - 1] - lr * g[n - 1];
    } else {
      for (; i < n; i += stride) p[i] = p[i] - lr * g[i];
    }
  }
}

// Widest vector (in doubles) that the row length and all the pointers allow.
static int row_vector_width(size_t N, uintptr_t pointer_bits) {
  if (N % 4 == 0 && (pointer_bits & 31) == 0) return 4;
  if (N % 2 == 0 && (pointer_bits & 15) == 0) return 2;
  return 1;
}

// `resident` caches the occupancy of one kernel instantiation (0 = not asked yet).
template <class Kernel> static unsigned row_grid(Kernel kernel, size_t items, int *resident) {
  if (*resident == 0) *resident = resident_ctas_per_sm(kernel, kEwThreads);
  return grid_for(items, kEwThreads, *resident * kEwWaves);
}

extern "C" {

int mg_fill(double *dst, double value, size_t n) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!dst) return fail(MG_ERR_INVALID, "mg_fill: null pointer");
  if (value == 0.0) {  // +0.0 is all-zero bits
    MG_CUDA_TRY(cudaMemsetAsync(dst, 0, n * sizeof(double), ctx().stream));
    return MG_OK;
  }
  FillFn f;
  f.in[0] = nullptr;
  f.out[0] = dst;
  f.value = value;
  return launch_map(f, n, "fill");
}

int mg_binary_fwd(int op, const double *a, const double *b, double *out, size_t n) {
  MG_ENSURE_INIT();
  if (n && (!a || !b || !out)) return fail(MG_ERR_INVALID, "mg_binary_fwd: null pointer");
  int rc = MG_OK;
  MG_DISPATCH_BINARY(op, {
    BinaryFwd<OP> f;
    f.in[0] = a; f.in[1] = b; f.out[0] = out;
    rc = launch_map(f, n, "binary_fwd");
  });
  return rc;
}

int mg_binary_bwd(int op, const double *a, const double *b, const double *g, double *ga,
                  double *gb, size_t n, int flags) {
  MG_ENSURE_INIT();
  if (n == 0 || (!ga && !gb)) return MG_OK;
  if (!g) return fail(MG_ERR_INVALID, "mg_binary_bwd: null upstream gradient");
  if ((op == MG_MUL || op == MG_DIV) && (!a || !b))
    return fail(MG_ERR_INVALID, "mg_binary_bwd: mul/div need both forward operands");
  int rc = MG_OK;
  if (ga && ga == gb) {
    // Both operands are one tensor: apply the two updates one after the other,
    // in the reference's order (first operand, then second).
    MG_DISPATCH_BINARY(op, {
      rc = binary_bwd_one<OP>(a, b, g, ga, nullptr, n, flags & MG_ACC_STORE_A);
      if (rc == MG_OK) rc = binary_bwd_one<OP>(a, b, g, nullptr, gb, n, 0);
    });
    return rc;
  }
  MG_DISPATCH_BINARY(op, { rc = binary_bwd_one<OP>(a, b, g, ga, gb, n, flags); });
  return rc;
}

int mg_unary_fwd(int op, const double *a, double s, double *out, size_t n) {
  MG_ENSURE_INIT();
  if (n && (!a || !out)) return fail(MG_ERR_INVALID, "mg_unary_fwd: null pointer");
  int rc = MG_OK;
  MG_DISPATCH_UNARY(op, {
    UnaryFwd<OP> f;
    f.in[0] = a; f.out[0] = out; f.s = s;
    rc = launch_map(f, n, "unary_fwd");
  });
  return rc;
}

int mg_unary_bwd(int op, const double *a, const double *out, double s, const double *g,
                 double *ga, size_t n, int flags) {
  MG_ENSURE_INIT();
  if (n == 0 || !ga) return MG_OK;
  if (!g) return fail(MG_ERR_INVALID, "mg_unary_bwd: null upstream gradient");
  const bool needs_a = (op == MG_POW || op == MG_RELU);
  const bool needs_y = (op == MG_SIGMOID || op == MG_TANH || op == MG_EXP);
  if ((needs_a && !a) || (needs_y && !out))
    return fail(MG_ERR_INVALID, "mg_unary_bwd: op %d needs its forward %s", op,
                needs_a ? "input" : "output");
  int rc = MG_OK;
  MG_DISPATCH_UNARY(op, {
    UnaryBwd<OP> f;
    f.in[0] = g;
    f.in[1] = needs_a ? a : nullptr;
    f.in[2] = needs_y ? out : nullptr;
    f.in[3] = (flags & MG_ACC_STORE_A) ? nullptr : ga;
    f.out[0] = ga;
    f.s = s;
    rc = launch_map(f, n, "unary_bwd");
  });
  return rc;
}

int mg_sgd_step(double *param, const double *grad, double lr, size_t n) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!param || !grad) return fail(MG_ERR_INVALID, "mg_sgd_step: null pointer");
  SgdFn f;
  f.in[0] = param; f.in[1] = grad; f.out[0] = param; f.lr = lr;
  return launch_map(f, n, "sgd_step");
}

int mg_sgd_step_multi(double *const *params, const double *const *grads, const size_t *sizes, int count,
                      double lr) {
  MG_ENSURE_INIT();
  if (count <= 0) return MG_OK;
  if (!params || !grads || !sizes) return fail(MG_ERR_INVALID, "mg_sgd_step_multi: null pointer");
  Context &c = ctx();
  for (int first = 0; first < count; first += 8) {
    SgdBatch b;
    b.count = 0;
    size_t longest = 0;
    for (int t = first; t < count && t < first + 8; t++) {
      if (sizes[t] == 0) continue;
      if (!params[t] || !grads[t]) return fail(MG_ERR_INVALID, "mg_sgd_step_multi: null tensor %d", t);
      b.param[b.count] = params[t];
      b.grad[b.count] = grads[t];
      b.n[b.count] = sizes[t];
      longest = sizes[t] > longest ? sizes[t] : longest;
      b.count++;
    }
    if (b.count == 0) continue;
    sgd_multi_kernel<<<grid_for(longest, 256, 8), 256, 0, c.stream>>>(b, lr);
    MG_LAUNCH_CHECK("sgd_multi");
  }
  return MG_OK;
}

int mg_add_row_fwd(const double *x, const double *row, double *out, size_t M, size_t N) {
  MG_ENSURE_INIT();
  if (M == 0 || N == 0) return MG_OK;
  if (!x || !row || !out) return fail(MG_ERR_INVALID, "mg_add_row_fwd: null pointer");
  Context &c = ctx();
  uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(row) |
                   reinterpret_cast<uintptr_t>(out);
  static int resident[3] = {0, 0, 0};
  switch (row_vector_width(N, bits)) {
    case 4:
      add_row_kernel<4><<<row_grid(add_row_kernel<4>, M * (N / 4), &resident[2]), kEwThreads, 0, c.stream>>>(x, row, out, M, N);
      break;
    case 2:
      add_row_kernel<2><<<row_grid(add_row_kernel<2>, M * (N / 2), &resident[1]), kEwThreads, 0, c.stream>>>(x, row, out, M, N);
      break;
    default:
      add_row_kernel<1><<<row_grid(add_row_kernel<1>, M * N, &resident[0]), kEwThreads, 0, c.stream>>>(x, row, out, M, N);
  }
  MG_LAUNCH_CHECK("add_row_fwd");
  return MG_OK;
}

int mg_sum_all_bwd(const double *g1, double *gx, size_t n, int flags) {
  MG_ENSURE_INIT();
  if (n == 0 || !gx) return MG_OK;
  if (!g1) return fail(MG_ERR_INVALID, "mg_sum_all_bwd: null upstream gradient");
  ScalarBroadcastBwd f;
  f.in[0] = (flags & MG_ACC_STORE_A) ? nullptr : gx;
  f.out[0] = gx;
  f.g0 = g1;
  return launch_map(f, n, "sum_all_bwd");
}

int mg_sum_lastaxis_bwd(const double *g, double *gx, size_t M, size_t N, int flags) {
  MG_ENSURE_INIT();
  if (M == 0 || N == 0 || !gx) return MG_OK;
  if (!g) return fail(MG_ERR_INVALID, "mg_sum_lastaxis_bwd: null upstream gradient");
  Context &c = ctx();
  const bool acc = !(flags & MG_ACC_STORE_A);
  static int resident[3] = {0, 0, 0};
  switch (row_vector_width(N, reinterpret_cast<uintptr_t>(gx))) {
    case 4:
      row_scalar_bwd_kernel<4><<<row_grid(row_scalar_bwd_kernel<4>, M * (N / 4), &resident[2]), kEwThreads, 0, c.stream>>>(g, gx, M, N, acc);
      break;
    case 2:
      row_scalar_bwd_kernel<2><<<row_grid(row_scalar_bwd_kernel<2>, M * (N / 2), &resident[1]), kEwThreads, 0, c.stream>>>(g, gx, M, N, acc);
      break;
    default:
      row_scalar_bwd_kernel<1><<<row_grid(row_scalar_bwd_kernel<1>, M * N, &resident[0]), kEwThreads, 0, c.stream>>>(g, gx, M, N, acc);
  }
  MG_LAUNCH_CHECK("sum_lastaxis_bwd");
  return MG_OK;
}

int mg_avg_pool_28(const double *x, double *out, size_t batch) {
  MG_ENSURE_INIT();
  if (batch == 0) return MG_OK;
  if (!x || !out) return fail(MG_ERR_INVALID, "mg_avg_pool_28: null pointer");
  avg_pool_28_kernel<<<grid_for(batch * 196, 256, 8), 256, 0, ctx().stream>>>(x, out, batch);
  MG_LAUNCH_CHECK("avg_pool_28");
  return MG_OK;
}

int mg_upload_u8_scaled(double *dst, const unsigned char *src_host, size_t n, double divisor) {
  MG_ENSURE_INIT();
  MG_NOT_WHILE_RECORDING("mg_upload_u8_scaled");
  if (n == 0) return MG_OK;
  if (!dst || !src_host) return fail(MG_ERR_INVALID, "mg_upload_u8_scaled: null pointer");
  if (divisor == 0.0) return fail(MG_ERR_INVALID, "mg_upload_u8_scaled: divisor is zero");
  Context &c = ctx();
  unsigned char *staged = nullptr;
  MG_CUDA_TRY(cudaMallocAsync(&staged, n, c.stream));
  MG_CUDA_TRY(cudaMemcpyAsync(staged, src_host, n, cudaMemcpyHostToDevice, c.stream));
  u8_scale_kernel<<<grid_for(n, 256, 8), 256, 0, c.stream>>>(staged, dst, n, divisor);
  MG_LAUNCH_CHECK("u8_scale");
  MG_CUDA_TRY(cudaFreeAsync(staged, c.stream));
  return MG_OK;
}

int mg_f64_to_i32(const double *src, int *dst, size_t n) {
  MG_ENSURE_INIT();
  if (n == 0) return MG_OK;
  if (!src || !dst) return fail(MG_ERR_INVALID, "mg_f64_to_i32: null pointer");
  f64_to_i32_kernel<<<grid_for(n, 256, 4), 256, 0, ctx().stream>>>(src, dst, n);
  MG_LAUNCH_CHECK("f64_to_i32");
  return MG_OK;
}

}  // extern "C"
