/*
 * ref_fast.c — CPU restatement of micrograd's fp64 tensor-op path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA backend is
 * compared against; the product never links, imports or calls it.
 *
 * Every function keeps, for each output element, the exact sequence of
 * floating-point operations of the reference project's loops (file:line cited
 * per function), so that with `-O2 -ffp-contract=off` (no FMA contraction, no
 * reassociation) results are bit-identical to the reference's own code.  The
 * only liberties taken are flat indexing instead of at({i,j}) and OpenMP across
 * independent output elements.  Bit-identity against the reference's compiled
 * sources is asserted by tests/test_oracle.py.
 *
 * Ops that the reference does not have (exp, row-broadcast add, last-axis sum,
 * softmax cross-entropy, argmax) are restated as plain sequential fp64 loops in
 * the same style; the reference pins no values for them ("parity unpinned" for
 * those ops only).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared (see Makefile).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef long long idx_t; /* signed loop index for OpenMP */

int rf_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void rf_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* Tensor-tensor elementwise ops: src/ops/Arithmetic.cpp:9-135                */
/* op: 0 add, 1 sub, 2 mul, 3 div                                             */
/* ------------------------------------------------------------------------- */
void rf_binary_fwd(int op, size_t n, const double *a, const double *b, double *out) {
  idx_t N = (idx_t)n;
  switch (op) {
  case 0: /* Arithmetic.cpp:24-26 */
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) out[i] = a[i] + b[i];
    break;
  case 1: /* Arithmetic.cpp:55-57 */
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) out[i] = a[i] - b[i];
    break;
  case 2: /* Arithmetic.cpp:87-89 */
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) out[i] = a[i] * b[i];
    break;
  case 3: /* Arithmetic.cpp:119-121 */
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) out[i] = a[i] / b[i];
    break;
  default:
    break;
  }
}

/* Backward closures: Arithmetic.cpp:31-36, 62-67, 94-99, 126-132.
 * ga and gb accumulate; they may alias (x op x), in which case the two updates
 * of one element happen in the reference's order (ga first, then gb).  Pointers
 * are volatile-free but not restrict, so aliasing is honoured. */
void rf_binary_bwd(int op, size_t n, const double *a, const double *b, const double *g,
                   double *ga, double *gb) {
  idx_t N = (idx_t)n;
  switch (op) {
  case 0:
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) {
      ga[i] += g[i];
      gb[i] += g[i];
    }
    break;
  case 1:
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) {
      ga[i] += g[i];
      gb[i] -= g[i];
    }
    break;
  case 2:
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) {
      ga[i] += g[i] * b[i];
      gb[i] += g[i] * a[i];
    }
    break;
  case 3:
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < N; i++) {
      ga[i] += g[i] / b[i];
      gb[i] -= g[i] * a[i] / (b[i] * b[i]);
    }
    break;
  default:
    break;
  }
}

/* ------------------------------------------------------------------------- */
/* Tensor-scalar ops and pow: Arithmetic.cpp:137-266                          */
/* op: 0 add, 1 sub, 2 mul, 3 div, 4 pow                                      */
/* ------------------------------------------------------------------------- */
void rf_scalar_fwd(int op, size_t n, const double *a, double s, double *out) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) {
    switch (op) {
    case 0: out[i] = a[i] + s; break;      /* :147-149 */
    case 1: out[i] = a[i] - s; break;      /* :173-175 */
    case 2: out[i] = a[i] * s; break;      /* :199-201 */
    case 3: out[i] = a[i] / s; break;      /* :225-227 */
    case 4: out[i] = pow(a[i], s); break;  /* :251-253 */
    default: break;
    }
  }
}

void rf_scalar_bwd(int op, size_t n, const double *a, double s, const double *g, double *ga) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) {
    switch (op) {
    case 0: ga[i] += g[i]; break;                            /* :154-158 */
    case 1: ga[i] += g[i]; break;                            /* :180-184 */
    case 2: ga[i] += g[i] * s; break;                        /* :206-210 */
    case 3: ga[i] += g[i] / s; break;                        /* :232-236 */
    case 4: ga[i] += g[i] * s * pow(a[i], s - 1); break;     /* :258-263 */
    default: break;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Activations: src/ops/Activations.cpp.  op: 0 relu, 1 sigmoid, 2 tanh,      */
/* 3 exp (not in the reference; std::exp forward, g*out backward).            */
/* ------------------------------------------------------------------------- */
void rf_unary_fwd(int op, size_t n, const double *a, double *out) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) {
    switch (op) {
    case 0: out[i] = a[i] > 0 ? a[i] : 0; break;        /* Activations.cpp:18-20 */
    case 1: out[i] = 1.0 / (1.0 + exp(-a[i])); break;   /* :45-47 */
    case 2: out[i] = tanh(a[i]); break;                 /* :73-75 */
    case 3: out[i] = exp(a[i]); break;
    default: break;
    }
  }
}

void rf_unary_bwd(int op, size_t n, const double *a, const double *out, const double *g,
                  double *ga) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) {
    switch (op) {
    case 0: ga[i] += g[i] * (a[i] > 0 ? 1.0 : 0.0); break;  /* :25-30 */
    case 1: {                                                /* :52-58 */
      double s = out[i];
      ga[i] += g[i] * s * (1.0 - s);
    } break;
    case 2: {                                                /* :80-85 */
      double t = out[i];
      ga[i] += g[i] * (1.0 - t * t);
    } break;
    case 3: ga[i] += g[i] * out[i]; break;
    default: break;
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Full sum: src/ops/Reduction.cpp:17-30.  Strictly left to right from 0.0.   */
/* ------------------------------------------------------------------------- */
double rf_sum(size_t n, const double *a) {
  double total = 0.0;
  for (size_t i = 0; i < n; i++) total += a[i];
  return total;
}

void rf_sum_bwd(size_t n, double g0, double *ga) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) ga[i] += g0;
}

/* Long-double sum, used only to show which side of a sum comparison is off. */
double rf_sum_longdouble(size_t n, const double *a) {
  long double total = 0.0L;
  for (size_t i = 0; i < n; i++) total += (long double)a[i];
  return (double)total;
}

/* ------------------------------------------------------------------------- */
/* matmul: src/ops/Matmul.cpp.  A[m,k] B[k,n] C[m,n], row-major.               */
/* ------------------------------------------------------------------------- */
/* Forward (:30-38): C[i,j] = ((0.0 + A[i,0]*B[0,j]) + A[i,1]*B[1,j]) + ...     */
void rf_matmul_fwd(size_t m, size_t k, size_t n, const double *A, const double *B, double *C) {
  idx_t M = (idx_t)m;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < M; i++) {
    double *c = C + (size_t)i * n;
    for (size_t j = 0; j < n; j++) c[j] = 0.0;
    for (size_t p = 0; p < k; p++) {
      double a = A[(size_t)i * k + p];
      const double *b = B + p * n;
      for (size_t j = 0; j < n; j++) c[j] += a * b[j];
    }
  }
}

/* Backward (:43-58): first gA[i,j] += gC[i,p]*B[j,p] for p ascending over n,
 * accumulating into the existing gradient value; then gB[i,j] += A[p,i]*gC[p,j]
 * for p ascending over m.  gA and gB may alias when A and B are one tensor. */
void rf_matmul_bwd(size_t m, size_t k, size_t n, const double *A, const double *B,
                   const double *gC, double *gA, double *gB) {
  idx_t M = (idx_t)m, K = (idx_t)k;
  if (gA) {
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < M; i++) {
      const double *g = gC + (size_t)i * n;
      for (size_t j = 0; j < k; j++) {
        const double *b = B + j * n;
        double acc = gA[(size_t)i * k + j];
        for (size_t p = 0; p < n; p++) acc += g[p] * b[p];
        gA[(size_t)i * k + j] = acc;
      }
    }
  }
  if (gB) {
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < K; i++) {
      double *gb = gB + (size_t)i * n;
      for (size_t p = 0; p < m; p++) {
        double a = A[p * k + (size_t)i];
        const double *g = gC + p * n;
        for (size_t j = 0; j < n; j++) gb[j] += a * g[j];
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* SGD: src/nn.cpp:71-77.  p -= (lr*g): product rounded, then subtracted.      */
/* ------------------------------------------------------------------------- */
void rf_sgd_step(size_t n, double *p, const double *g, double lr) {
  idx_t N = (idx_t)n;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < N; i++) p[i] -= lr * g[i];
}

/* ------------------------------------------------------------------------- */
/* Ops the reference lacks (plain sequential restatements).                   */
/* ------------------------------------------------------------------------- */
/* Row-broadcast add out[i,j] = x[i,j] + r[j].  Equals the reference-only
 * encoding x + ones[M,1]@r[1,N], whose product term is 0.0 + 1.0*r[j] = r[j]. */
void rf_add_row_fwd(size_t M, size_t N, const double *x, const double *r, double *out) {
  idx_t MM = (idx_t)M;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < MM; i++)
    for (size_t j = 0; j < N; j++) out[(size_t)i * N + j] = x[(size_t)i * N + j] + r[j];
}

/* gx += g; gr[j] += g[i,j] for i ascending (the ones-matmul's gB loop order). */
void rf_add_row_bwd(size_t M, size_t N, const double *g, double *gx, double *gr) {
  idx_t NN = (idx_t)N, T = (idx_t)(M * N);
  if (gx) {
#pragma omp parallel for schedule(static)
    for (idx_t i = 0; i < T; i++) gx[i] += g[i];
  }
  if (gr) {
#pragma omp parallel for schedule(static)
    for (idx_t j = 0; j < NN; j++) {
      double acc = gr[j];
      for (size_t i = 0; i < M; i++) acc += g[i * N + (size_t)j];
      gr[j] = acc;
    }
  }
}

/* Last-axis sum: out[i] = left-to-right sum of row i; bwd gx[i,j] += g[i]. */
void rf_sum_lastaxis_fwd(size_t M, size_t N, const double *x, double *out) {
  idx_t MM = (idx_t)M;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < MM; i++) {
    double t = 0.0;
    for (size_t j = 0; j < N; j++) t += x[(size_t)i * N + j];
    out[i] = t;
  }
}

void rf_sum_lastaxis_bwd(size_t M, size_t N, const double *g, double *gx) {
  idx_t MM = (idx_t)M;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < MM; i++)
    for (size_t j = 0; j < N; j++) gx[(size_t)i * N + j] += g[i];
}

/* Softmax cross-entropy with integer labels, mean over `denom` rows
 * (denom = global batch, so that a row shard yields its share of the mean).
 * Per row: m = max_j z; s = sum_j exp(z_j - m) left to right;
 * loss_i = -(z_y - m - log s).  Returns (sum_i loss_i) / denom. */
double rf_softmax_xent_fwd(size_t M, size_t C, const double *z, const int *labels, double denom) {
  double total = 0.0;
  for (size_t i = 0; i < M; i++) {
    const double *r = z + i * C;
    double mx = r[0];
    for (size_t j = 1; j < C; j++)
      if (r[j] > mx) mx = r[j];
    double s = 0.0;
    for (size_t j = 0; j < C; j++) s += exp(r[j] - mx);
    total += -(r[labels[i]] - mx - log(s));
  }
  return total / denom;
}

/* gz[i,j] += gloss * (exp(z_ij - m)/s - [j == y_i]) / denom. */
void rf_softmax_xent_bwd(size_t M, size_t C, const double *z, const int *labels, double denom,
                         double gloss, double *gz) {
  idx_t MM = (idx_t)M;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < MM; i++) {
    const double *r = z + (size_t)i * C;
    double mx = r[0];
    for (size_t j = 1; j < C; j++)
      if (r[j] > mx) mx = r[j];
    double s = 0.0;
    for (size_t j = 0; j < C; j++) s += exp(r[j] - mx);
    for (size_t j = 0; j < C; j++) {
      double p = exp(r[j] - mx) / s;
      double onehot = ((int)j == labels[i]) ? 1.0 : 0.0;
      gz[(size_t)i * C + j] += gloss * (p - onehot) / denom;
    }
  }
}

/* Row argmax: first index of the strict maximum, as the reference trainer's
 * prediction loop does with `>` (src/main.cpp:29-32). */
void rf_argmax_rows(size_t M, size_t N, const double *x, int *out) {
  idx_t MM = (idx_t)M;
#pragma omp parallel for schedule(static)
  for (idx_t i = 0; i < MM; i++) {
    const double *r = x + (size_t)i * N;
    size_t best = 0;
    for (size_t j = 0; j < N; j++)
      if (r[j] > r[best]) best = j;
    out[i] = (int)best;
  }
}
