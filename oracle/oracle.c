/*
 * oracle.c — CPU restatement of the semantics of gorgonia's CPU engine for the ops that the
 * B200 engine executes. TEST INFRASTRUCTURE ONLY: it is the checker for tests/, for
 * __graft_entry__.smoke() and for bench.py's CPU-baseline legs. Nothing in the product
 * (gorgonia_b200/, libgorgonia_b200.so) links, imports or calls it.
 *
 * What it follows. gorgonia's own repository holds the dispatch and the nn kernels; the
 * arithmetic of the dense ops lives in modules that the repository pins but does not vendor:
 *   gorgonia.org/tensor v0.9.23 (StdEng Add..Pow, Lt..ElNe, MatMul/MatVecMul/Outer, SoftMax,
 *   Repeat, Transpose, Sum/Max, ByIndices), gonum.org/v1/gonum v0.11.0 (blas/gonum Sgemm,
 *   Sgemv, Sger), github.com/chewxy/math32 v1.10.1 (float32 Exp/Log/Pow/...).
 * Those are restated from their published behaviour: IEEE arithmetic per element without
 * FMA contraction; BLAS-3/2 as plain sums of products. Each function cites the gorgonia
 * file:line whose call it stands for.
 *
 * Pinned against: the golden tables of gorgonia's tests (tests/golden/, extracted from
 * op_math_test.go, op_softmax_test.go, nn_test.go, known_issues_test.go,
 * op_by_indices_test.go, example_*_test.go and others; tests/test_oracle_golden.py).
 * PARITY UNPINNED for: last-ulp behaviour of math32's float32 transcendentals, gonum's
 * Sgemm summation order, tensor.SoftMax's internal formulation, and tensor.SoftMaxB /
 * LogSoftMaxB (the softmax derivatives); no bit-level vector exists for them in gorgonia.
 * Here float32 transcendentals are computed in double and rounded once, and sums of products
 * are accumulated in double. The backward ops maxPoolDiff and col2im are integer-indexed
 * additions whose order the repository spells out; their known answers are derived from the
 * configurations of TestMaxPool2D and TestIm2Col (nn_test.go:13-89,140-193).
 *
 * Build: make -C oracle   (gcc -O3 -fopenmp -ffp-contract=off).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* op codes: identical to B200_OP_* of include/gorgonia_b200.h */
enum {
  OP_ADD = 0, OP_SUB, OP_MUL, OP_DIV, OP_POW, OP_MOD, OP_LT, OP_GT, OP_LTE, OP_GTE, OP_EQ, OP_NE,
  OP_ABS = 32, OP_SIGN, OP_CEIL, OP_FLOOR, OP_SIN, OP_COS, OP_EXP, OP_LN, OP_LOG2, OP_NEG, OP_SQUARE,
  OP_SQRT, OP_INV, OP_INVSQRT, OP_CUBE, OP_TANH, OP_SIGMOID, OP_LOG1P, OP_EXPM1, OP_SOFTPLUS
};

int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1 to their children; a timed CPU leg that is
 * meant to use the whole host sets its thread count here instead. Returns the count in effect. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ---- scalar semantics -----------------------------------------------------------------
 * binary: operatorPointwise_binary.go:40-293 (scalar lambdas) and
 *         operatorPointwise_binary_const.go:5-22 (tensor.Add.. / tensor.Lt..); compare ops
 *         as used by the graphs of nn.go:104-112,154-155 (retSame: 1/0 in operand dtype).
 * unary:  operatorPointwise_unary_const.go:10-71, math_nooptim.go:18-51 (tanh f32 through
 *         float64, sigmoid f32 thresholds -88/15 through float64, invsqrt = 1/sqrt),
 *         operatorPointwise_unary.go (sign, square, cube, softplus lambdas). */

static inline float bin_f32(int op, float x, float y) {
  switch (op) {
    case OP_ADD: return x + y;
    case OP_SUB: return x - y;
    case OP_MUL: return x * y;
    case OP_DIV: return x / y;
    case OP_POW: return (float)pow((double)x, (double)y);
    case OP_MOD: return (float)fmod((double)x, (double)y);
    case OP_LT: return x < y ? 1.f : 0.f;
    case OP_GT: return x > y ? 1.f : 0.f;
    case OP_LTE: return x <= y ? 1.f : 0.f;
    case OP_GTE: return x >= y ? 1.f : 0.f;
    case OP_EQ: return x == y ? 1.f : 0.f;
    case OP_NE: return x != y ? 1.f : 0.f;
  }
  return NAN;
}
static inline double bin_f64(int op, double x, double y) {
  switch (op) {
    case OP_ADD: return x + y;
    case OP_SUB: return x - y;
    case OP_MUL: return x * y;
    case OP_DIV: return x / y;
    case OP_POW: return pow(x, y);
    case OP_MOD: return fmod(x, y);
    case OP_LT: return x < y ? 1. : 0.;
    case OP_GT: return x > y ? 1. : 0.;
    case OP_LTE: return x <= y ? 1. : 0.;
    case OP_GTE: return x >= y ? 1. : 0.;
    case OP_EQ: return x == y ? 1. : 0.;
    case OP_NE: return x != y ? 1. : 0.;
  }
  return NAN;
}
static inline double un_f64(int op, double x) {
  switch (op) {
    case OP_ABS: return fabs(x);
    case OP_SIGN: return (double)((x > 0) - (x < 0));
    case OP_CEIL: return ceil(x);
    case OP_FLOOR: return floor(x);
    case OP_SIN: return sin(x);
    case OP_COS: return cos(x);
    case OP_EXP: return exp(x);
    case OP_LN: return log(x);
    case OP_LOG2: return log2(x);
    case OP_NEG: return -x;
    case OP_SQUARE: return x * x;
    case OP_SQRT: return sqrt(x);
    case OP_INV: return 1.0 / x;
    case OP_INVSQRT: return 1.0 / sqrt(x);
    case OP_CUBE: return x * x * x;
    case OP_TANH: return tanh(x);
    case OP_SIGMOID: /* math_nooptim.go:24-33 */
      if (x < -709) return 0;
      if (x > 19) return 1;
      return 1.0 / (1.0 + exp(-x));
    case OP_LOG1P: return log1p(x);
    case OP_EXPM1: return expm1(x);
    case OP_SOFTPLUS: /* operatorPointwise_unary.go softplus lambda; thresholds as the kernels */
      if (x < -708) return 0;
      if (x > 16) return x;
      return log1p(exp(x));
  }
  return NAN;
}
static inline float un_f32(int op, float x) {
  switch (op) {
    case OP_ABS: return fabsf(x);
    case OP_SIGN: return (float)((x > 0) - (x < 0));
    case OP_CEIL: return ceilf(x);
    case OP_FLOOR: return floorf(x);
    case OP_NEG: return -x;
    case OP_SQUARE: return x * x;
    case OP_SQRT: return sqrtf(x);
    case OP_INV: return 1.0f / x;
    case OP_INVSQRT: return 1.0f / sqrtf(x);
    case OP_CUBE: return x * x * x;
    case OP_SIGMOID: /* math_nooptim.go:36-45 */
      if (x < -88) return 0;
      if (x > 15) return 1;
      return (float)(1.0 / (1.0 + exp((double)(-x))));
    case OP_SOFTPLUS:
      if (x < -103) return 0;
      if (x > 14) return x;
      return (float)log1p(exp((double)x));
    default: /* transcendental: evaluate in double, round once */
      return (float)un_f64(op, (double)x);
  }
}

/* dst[i] = a[ai] op b[bi]; stride 0 on an operand makes it a scalar (vs / sv forms of
 * cuda/arith.go:67-130). dst may alias a or b. */
void oracle_binary_f32(int op, float *dst, const float *a, const float *b, int64_t n, int a_scalar, int b_scalar) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = bin_f32(op, a[a_scalar ? 0 : i], b[b_scalar ? 0 : i]);
}
void oracle_binary_f64(int op, double *dst, const double *a, const double *b, int64_t n, int a_scalar,
                       int b_scalar) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = bin_f64(op, a[a_scalar ? 0 : i], b[b_scalar ? 0 : i]);
}
void oracle_unary_f32(int op, float *dst, const float *a, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = un_f32(op, a[i]);
}
void oracle_unary_f64(int op, double *dst, const double *a, int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) dst[i] = un_f64(op, a[i]);
}

/* Broadcast binary: gorgonia materialises the small operand with repeatOp and then runs the
 * plain op (broadcast.go:69-129, op_tensor.go:354-473); element i of the repeated operand is
 * small[(i / div) % mod]. */
void oracle_binary_bcast_f32(int op, float *dst, const float *a, const float *b, int64_t n, int64_t div,
                             int64_t mod, int bcast_is_a) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t k = (i / div) % mod;
    dst[i] = bcast_is_a ? bin_f32(op, a[k], b[i]) : bin_f32(op, a[i], b[k]);
  }
}
void oracle_binary_bcast_f64(int op, double *dst, const double *a, const double *b, int64_t n, int64_t div,
                             int64_t mod, int bcast_is_a) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t k = (i / div) % mod;
    dst[i] = bcast_is_a ? bin_f64(op, a[k], b[i]) : bin_f64(op, a[i], b[k]);
  }
}

/* ---- linear algebra ---------------------------------------------------------------------
 * C[M,N] = op(A) op(B), row-major with leading dimensions, alpha=1 beta=0: the result of
 * linAlgBinOp.do -> tensor.MatMul -> gonum Sgemm (op_math.go:745-795, blas.go:54-56), with
 * the trans flags of op_math.go:752-768. Products are accumulated in double. */
void oracle_gemm_f32(int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda,
                     const float *B, int64_t ldb, float *C, int64_t ldc) {
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)(N > 0 ? N : 1));
#pragma omp for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
      for (int64_t j = 0; j < N; ++j) acc[j] = 0.0;
      if (!transB) {
        for (int64_t k = 0; k < K; ++k) {
          const double a = transA ? A[k * lda + i] : A[i * lda + k];
          const float *brow = B + k * ldb;
          for (int64_t j = 0; j < N; ++j) acc[j] += a * (double)brow[j];
        }
      } else {
        for (int64_t j = 0; j < N; ++j) {
          const float *brow = B + j * ldb;
          double s = 0.0;
          if (!transA)
            for (int64_t k = 0; k < K; ++k) s += (double)A[i * lda + k] * (double)brow[k];
          else
            for (int64_t k = 0; k < K; ++k) s += (double)A[k * lda + i] * (double)brow[k];
          acc[j] = s;
        }
      }
      for (int64_t j = 0; j < N; ++j) C[i * ldc + j] = (float)acc[j];
    }
    free(acc);
  }
}
void oracle_gemm_f64(int transA, int transB, int64_t M, int64_t N, int64_t K, const double *A, int64_t lda,
                     const double *B, int64_t ldb, double *C, int64_t ldc) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      long double s = 0;
      for (int64_t k = 0; k < K; ++k) {
        const double a = transA ? A[k * lda + i] : A[i * lda + k];
        const double b = transB ? B[j * ldb + k] : B[k * ldb + j];
        s += (long double)a * b;
      }
      C[i * ldc + j] = (double)s;
    }
}
/* The same contraction with float32 products and a float32 running sum in k order: what a
 * straightforward float32 BLAS does. Used only to show how far summation order alone moves
 * the result relative to the tolerance. */
void oracle_gemm_f32_naive(int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float s = 0.f;
      for (int64_t k = 0; k < K; ++k) s += A[i * K + k] * B[k * N + j];
      C[i * N + j] = s;
    }
}

/* y = A x or A^T x (A is M x N row-major): tensor.MatVecMul -> Sgemv
 * (cuda/linalg.go:47-107 for the flag handling; operatorLinAlg.go for the op). */
void oracle_gemv_f32(int transA, int64_t M, int64_t N, const float *A, int64_t lda, const float *x, float *y) {
  if (!transA) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
      double s = 0;
      for (int64_t j = 0; j < N; ++j) s += (double)A[i * lda + j] * (double)x[j];
      y[i] = (float)s;
    }
  } else {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < N; ++j) {
      double s = 0;
      for (int64_t i = 0; i < M; ++i) s += (double)A[i * lda + j] * (double)x[i];
      y[j] = (float)s;
    }
  }
}
void oracle_gemv_f64(int transA, int64_t M, int64_t N, const double *A, int64_t lda, const double *x,
                     double *y) {
  if (!transA) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M; ++i) {
      long double s = 0;
      for (int64_t j = 0; j < N; ++j) s += (long double)A[i * lda + j] * x[j];
      y[i] = (double)s;
    }
  } else {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < N; ++j) {
      long double s = 0;
      for (int64_t i = 0; i < M; ++i) s += (long double)A[i * lda + j] * x[i];
      y[j] = (double)s;
    }
  }
}
/* A[M,N] = x y^T, overwriting (tensor.Outer with reuse; cuda/linalg.go:245-265 row-major path). */
void oracle_outer_f32(int64_t M, int64_t N, const float *x, const float *y, float *A) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) A[i * N + j] = x[i] * y[j];
}
void oracle_outer_f64(int64_t M, int64_t N, const double *x, const double *y, double *A) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) A[i * N + j] = x[i] * y[j];
}

/* ---- nn ops ---------------------------------------------------------------------------- */

/* im2colOp.do / f32s (op_nn.go:317-444): input (B,C,H,W) -> col (B, Ho, Wo, C*kh*kw), inner
 * order channel, kernel row, kernel col; taps outside the image are 0.
 * Ho = (H + 2 padH - (dilH (kh-1) + 1)) / strideH + 1 (op_nn.go:311-315). */
void oracle_im2col_f32(const float *im, float *col, int64_t B, int64_t C, int64_t H, int64_t W, int kh, int kw,
                       int padH, int padW, int sH, int sW, int dH, int dW) {
  const int64_t Ho = (H + 2 * padH - (dH * (kh - 1) + 1)) / sH + 1;
  const int64_t Wo = (W + 2 * padW - (dW * (kw - 1) + 1)) / sW + 1;
  const int64_t kk = C * kh * kw;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < B; ++b) {
    const float *imb = im + b * C * H * W;
    float *colb = col + b * Ho * Wo * kk;
    int64_t idx = 0;
    for (int64_t oh = 0; oh < Ho; ++oh)
      for (int64_t ow = 0; ow < Wo; ++ow)
        for (int64_t c = 0; c < C; ++c)
          for (int r = 0; r < kh; ++r) {
            const int64_t ih = -padH + (int64_t)r * dH + oh * sH;
            for (int s = 0; s < kw; ++s) {
              const int64_t iw = -padW + (int64_t)s * dW + ow * sW;
              colb[idx++] = (ih < 0 || ih >= H || iw < 0 || iw >= W) ? 0.f : imb[c * H * W + ih * W + iw];
            }
          }
  }
}

/* Conv2d (nn.go:211-305): im2col, then (B*Ho*Wo, C*kh*kw) x filter(K, C*kh*kw)^T, then the
 * (B,Ho,Wo,K) result transposed to (B,K,Ho,Wo). The col buffer is not materialised here; the
 * sum runs over (c, r, s) in im2col order with a double accumulator. */
void oracle_conv2d_f32(const float *x, const float *w, float *y, int64_t B, int64_t C, int64_t H, int64_t W,
                       int64_t K, int kh, int kw, int padH, int padW, int sH, int sW, int dH, int dW) {
  const int64_t Ho = (H + 2 * padH - (dH * (kh - 1) + 1)) / sH + 1;
  const int64_t Wo = (W + 2 * padW - (dW * (kw - 1) + 1)) / sW + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t k = 0; k < K; ++k) {
      const float *xb = x + b * C * H * W;
      const float *wk = w + k * C * kh * kw;
      float *yk = y + (b * K + k) * Ho * Wo;
      for (int64_t oh = 0; oh < Ho; ++oh)
        for (int64_t ow = 0; ow < Wo; ++ow) {
          double s = 0;
          for (int64_t c = 0; c < C; ++c)
            for (int r = 0; r < kh; ++r) {
              const int64_t ih = -padH + (int64_t)r * dH + oh * sH;
              if (ih < 0 || ih >= H) continue;
              for (int q = 0; q < kw; ++q) {
                const int64_t iw = -padW + (int64_t)q * dW + ow * sW;
                if (iw < 0 || iw >= W) continue;
                s += (double)xb[c * H * W + ih * W + iw] * (double)wk[(c * kh + r) * kw + q];
              }
            }
          yk[oh * Wo + ow] = (float)s;
        }
    }
}

/* maxPoolOp.f32s (op_nn.go:858-907): accumulator starts at -MaxFloat32, strict '>' so the
 * first maximum in row-major window order wins; the window is clipped to the image; with
 * explicit 4-way padding the window origin uses the south/east pads (op_nn.go:870-875).
 * Output size (H + padN + padS - kh) / sH + 1 (op_nn.go:810-816). mask holds the winning
 * index inside the (H,W) plane, or -1. pad = {north, south, west, east}. */
void oracle_maxpool2d_f32(const float *x, float *y, int64_t *mask, int64_t B, int64_t C, int64_t H, int64_t W,
                          int kh, int kw, int padN, int padS, int padW_, int padE, int explicit_padding, int sH,
                          int sW) {
  const int64_t Ho = (H + padS + padN - (kh - 1) - 1) / sH + 1;
  const int64_t Wo = (W + padE + padW_ - (kw - 1) - 1) / sW + 1;
  const int64_t ph0 = explicit_padding ? padS : padN;
  const int64_t pw0 = explicit_padding ? padE : padW_;
#pragma omp parallel for schedule(static)
  for (int64_t bc = 0; bc < B * C; ++bc) {
    const float *in = x + bc * H * W;
    float *out = y + bc * Ho * Wo;
    int64_t *mk = mask ? mask + bc * Ho * Wo : 0;
    for (int64_t ph = 0; ph < Ho; ++ph)
      for (int64_t pw = 0; pw < Wo; ++pw) {
        int64_t hs = ph * sH - ph0, ws = pw * sW - pw0;
        int64_t he = hs + kh < H ? hs + kh : H, we = ws + kw < W ? ws + kw : W;
        if (hs < 0) hs = 0;
        if (ws < 0) ws = 0;
        float best = -FLT_MAX;
        int64_t arg = -1;
        for (int64_t hi = hs; hi < he; ++hi)
          for (int64_t wi = ws; wi < we; ++wi)
            if (in[hi * W + wi] > best) {
              best = in[hi * W + wi];
              arg = hi * W + wi;
            }
        out[ph * Wo + pw] = best;
        if (mk) mk[ph * Wo + pw] = arg;
      }
  }
}

/* maxPoolDiffOp.f32s / f64s (op_nn.go:1067-1121): the input gradient is zeroed, then every
 * pooled position adds its gradient to the input position its mask entry names, in (ph, pw)
 * order inside each (batch, channel) plane. The mask is the one the forward op recorded. A
 * mask entry of -1 (an empty window) is skipped here; the reference would index out of range. */
#define ORACLE_MAXPOOL_BWD(NAME, T)                                                                      \
  void NAME(const T *dy, const int64_t *mask, T *dx, int64_t planes, int64_t hw, int64_t howo) {         \
    _Pragma("omp parallel for schedule(static)") for (int64_t pl = 0; pl < planes; ++pl) {              \
      T *g = dx + pl * hw;                                                                               \
      for (int64_t i = 0; i < hw; ++i) g[i] = 0;                                                         \
      for (int64_t i = 0; i < howo; ++i) {                                                               \
        const int64_t at = mask[pl * howo + i];                                                          \
        if (at >= 0 && at < hw) g[at] += dy[pl * howo + i];                                              \
      }                                                                                                  \
    }                                                                                                    \
  }
ORACLE_MAXPOOL_BWD(oracle_maxpool2d_bwd_f32, float)
ORACLE_MAXPOOL_BWD(oracle_maxpool2d_bwd_f64, double)

/* col2imOp.f32s / f64s (op_nn.go:571-637): the image is zeroed, then col (B, Ho, Wo, C*kh*kw)
 * is walked in memory order (output row, output column, channel, kernel row, kernel column)
 * and every entry whose tap lies inside the image is added to that pixel. The additions of one
 * pixel therefore happen in ascending (output row, output column) order. */
#define ORACLE_COL2IM(NAME, T)                                                                           \
  void NAME(const T *col, T *im, int64_t B, int64_t C, int64_t H, int64_t W, int kh, int kw, int padH,   \
            int padW, int sH, int sW, int dH, int dW) {                                                  \
    const int64_t Ho = (H + 2 * padH - (dH * (kh - 1) + 1)) / sH + 1;                                    \
    const int64_t Wo = (W + 2 * padW - (dW * (kw - 1) + 1)) / sW + 1;                                    \
    const int64_t kk = C * kh * kw;                                                                      \
    _Pragma("omp parallel for schedule(static)") for (int64_t b = 0; b < B; ++b) {                      \
      T *imb = im + b * C * H * W;                                                                       \
      const T *colb = col + b * Ho * Wo * kk;                                                            \
      for (int64_t i = 0; i < C * H * W; ++i) imb[i] = 0;                                                \
      int64_t idx = 0;                                                                                   \
      for (int64_t oh = 0; oh < Ho; ++oh)                                                                \
        for (int64_t ow = 0; ow < Wo; ++ow)                                                              \
          for (int64_t c = 0; c < C; ++c)                                                                \
            for (int r = 0; r < kh; ++r) {                                                               \
              const int64_t ih = -padH + (int64_t)r * dH + oh * sH;                                      \
              for (int s = 0; s < kw; ++s, ++idx) {                                                      \
                const int64_t iw = -padW + (int64_t)s * dW + ow * sW;                                    \
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) imb[c * H * W + ih * W + iw] += colb[idx];   \
              }                                                                                          \
            }                                                                                            \
    }                                                                                                    \
  }
ORACLE_COL2IM(oracle_col2im_f32, float)
ORACLE_COL2IM(oracle_col2im_f64, double)

/* softmaxDiffOp.UsePreallocDo -> tensor.SoftMaxB / LogSoftMaxB (op_softmax.go:262-274), on a
 * tensor viewed as (outer, len, inner). gorgonia.org/tensor v0.9.23 is not part of the checkout;
 * these are the published derivatives, evaluated in double:
 *   softmax:      dx_i = y_i * (g_i - sum_j g_j y_j)
 *   log-softmax:  dx_i = g_i - exp(y_i) * sum_j g_j
 * PARITY UNPINNED: the reference's tests hold no vector for either (only forward outputs). */
#define ORACLE_SOFTMAX_BWD(NAME, T, ACC, EXPF)                                                           \
  void NAME(const T *y, const T *g, T *dx, int64_t outer, int64_t len, int64_t inner, int is_log) {      \
    _Pragma("omp parallel for schedule(static)") for (int64_t oi = 0; oi < outer * inner; ++oi) {       \
      const int64_t o = oi / inner, in = oi % inner;                                                     \
      const T *yp = y + o * len * inner + in, *gp = g + o * len * inner + in;                            \
      T *dp = dx + o * len * inner + in;                                                                 \
      ACC s = 0;                                                                                         \
      for (int64_t k = 0; k < len; ++k) s += is_log ? (ACC)gp[k * inner] : (ACC)gp[k * inner] * (ACC)yp[k * inner]; \
      for (int64_t k = 0; k < len; ++k) {                                                                \
        const ACC yy = yp[k * inner], gg = gp[k * inner];                                                \
        dp[k * inner] = (T)(is_log ? gg - EXPF(yy) * s : yy * (gg - s));                                 \
      }                                                                                                  \
    }                                                                                                    \
  }
ORACLE_SOFTMAX_BWD(oracle_softmax_bwd_f32, float, double, exp)
ORACLE_SOFTMAX_BWD(oracle_softmax_bwd_f64, double, long double, expl)

/* BatchNormOp.f32s / f64s with updateStats and calculateAlphaAndBeta (op_nn.go:1346-1640), input
 * (B, C, S) with S = the spatial size (1 for a matrix). Training: per channel, saveMean = sum / n
 * and saveVar = sum (x - mean)^2, both accumulated in the tensor's own type in (sample, position)
 * order; running = momentum * new + (1 - momentum) * running with the unbiased variance
 * saveVar / (n - 1); alpha = 1 / sqrt(saveVar / n + eps). Inference: alpha = 1 / sqrt(runningVar
 * + eps), mean = runningMean. Output = x * alpha + beta with beta = -mean * alpha, a product then a
 * sum. Scale and bias are separate graph ops (nn.go:430-436) and not part of this. */
#define ORACLE_BATCHNORM(NAME, T, SQRT)                                                                   \
  void NAME(const T *x, T *y, int64_t B, int64_t C, int64_t S, int training, double momentum_, double eps_, \
            T *running_mean, T *running_var, T *save_mean, T *save_var) {                                 \
    const T momentum = (T)momentum_, eps = (T)eps_;                                                       \
    const int64_t n = B * S;                                                                              \
    _Pragma("omp parallel for schedule(static)") for (int64_t c = 0; c < C; ++c) {                       \
      T mean, inv;                                                                                        \
      if (training) {                                                                                     \
        T m = 0, v = 0;                                                                                   \
        for (int64_t s = 0; s < B; ++s)                                                                   \
          for (int64_t d = 0; d < S; ++d) m += x[(s * C + c) * S + d];                                    \
        m /= (T)n;                                                                                        \
        for (int64_t s = 0; s < B; ++s)                                                                   \
          for (int64_t d = 0; d < S; ++d) {                                                               \
            const T xv = x[(s * C + c) * S + d];                                                          \
            v += (xv - m) * (xv - m);                                                                     \
          }                                                                                               \
        save_mean[c] = m;                                                                                 \
        save_var[c] = v;                                                                                  \
        running_mean[c] = momentum * m + ((T)1 - momentum) * running_mean[c];                             \
        running_var[c] = momentum * (v / (T)(n - 1)) + ((T)1 - momentum) * running_var[c];                \
        mean = m;                                                                                         \
        inv = (T)1 / SQRT(v / (T)n + eps);                                                                \
      } else {                                                                                            \
        mean = running_mean[c];                                                                           \
        inv = (T)1 / SQRT(running_var[c] + eps);                                                          \
      }                                                                                                   \
      const T beta = -mean * inv;                                                                         \
      for (int64_t s = 0; s < B; ++s)                                                                     \
        for (int64_t d = 0; d < S; ++d) {                                                                 \
          const T p = x[(s * C + c) * S + d] * inv;                                                       \
          y[(s * C + c) * S + d] = p + beta;                                                              \
        }                                                                                                 \
    }                                                                                                     \
  }
ORACLE_BATCHNORM(oracle_batchnorm_f32, float, sqrtf)
ORACLE_BATCHNORM(oracle_batchnorm_f64, double, sqrt)

/* batchnormDiffOp.f32s / f64s (op_nn.go:1727-1940): the input gradient of BatchNormOp. Per channel,
 * sum = sum dy and dotp = sum (x - mean) dy accumulated in the tensor's type in (sample, position)
 * order; invstd = 1 / sqrt(saveVar / n + eps); k = dotp * invstd^2 / n; gradMean = sum / n;
 *   training:  dx = (dy - gradMean - (x - mean) * k) * invstd     (S > 1)
 *              dx = (dy - (x - mean) * k - gradMean) * invstd     (S = 1: the matrix branch subtracts in
 *                                                                  the other order)
 *   inference: dx = dy * invstd, invstd from the saved variance when S > 1 and from the running
 *              variance when S = 1, as the two branches of the reference have it. */
#define ORACLE_BATCHNORM_BWD(NAME, T, SQRT)                                                               \
  void NAME(const T *x, const T *dy, T *dx, int64_t B, int64_t C, int64_t S, int training, double eps_,   \
            const T *running_var, const T *save_mean, const T *save_var) {                                \
    const T eps = (T)eps_;                                                                                \
    const int64_t n = B * S;                                                                              \
    _Pragma("omp parallel for schedule(static)") for (int64_t c = 0; c < C; ++c) {                       \
      T sum = 0, dotp = 0;                                                                                \
      const T mean = save_mean[c];                                                                        \
      for (int64_t s = 0; s < B; ++s)                                                                     \
        for (int64_t d = 0; d < S; ++d) {                                                                 \
          const int64_t i = (s * C + c) * S + d;                                                          \
          sum += dy[i];                                                                                   \
          dotp += S == 1 ? (x[i] - mean) * dy[i] : (x[i] * dy[i] - mean * dy[i]);                         \
        }                                                                                                 \
      T invstd = (T)1 / SQRT(save_var[c] / (T)n + eps);                                                   \
      if (!training && S == 1) invstd = (T)1 / SQRT(running_var[c] + eps);                                \
      const T k = (T)(dotp * invstd * invstd) / (T)n;                                                     \
      const T grad_mean = sum / (T)n;                                                                     \
      for (int64_t s = 0; s < B; ++s)                                                                     \
        for (int64_t d = 0; d < S; ++d) {                                                                 \
          const int64_t i = (s * C + c) * S + d;                                                          \
          if (!training) {                                                                                \
            dx[i] = dy[i] * invstd;                                                                       \
          } else {                                                                                        \
            const T t = (x[i] - mean) * k;                                                                \
            dx[i] = S == 1 ? (dy[i] - t - grad_mean) * invstd : (dy[i] - grad_mean - t) * invstd;         \
          }                                                                                               \
        }                                                                                                 \
    }                                                                                                     \
  }
ORACLE_BATCHNORM_BWD(oracle_batchnorm_bwd_f32, float, sqrtf)
ORACLE_BATCHNORM_BWD(oracle_batchnorm_bwd_f64, double, sqrt)

/* softmaxOp.Do -> tensor.SoftMax / LogSoftMax along `axis` of a tensor viewed as
 * (outer, len, inner) (op_softmax.go:99-128). exp(x - max) / sum, evaluated in double. */
void oracle_softmax_f32(const float *x, float *y, int64_t outer, int64_t len, int64_t inner, int is_log) {
#pragma omp parallel for schedule(static)
  for (int64_t oi = 0; oi < outer * inner; ++oi) {
    const int64_t o = oi / inner, in = oi % inner;
    const float *xp = x + o * len * inner + in;
    float *yp = y + o * len * inner + in;
    double mx = -INFINITY;
    for (int64_t k = 0; k < len; ++k)
      if ((double)xp[k * inner] > mx) mx = xp[k * inner];
    double s = 0;
    for (int64_t k = 0; k < len; ++k) s += exp((double)xp[k * inner] - mx);
    const double ls = log(s);
    for (int64_t k = 0; k < len; ++k) {
      const double d = (double)xp[k * inner] - mx;
      yp[k * inner] = (float)(is_log ? d - ls : exp(d) / s);
    }
  }
}
void oracle_softmax_f64(const double *x, double *y, int64_t outer, int64_t len, int64_t inner, int is_log) {
#pragma omp parallel for schedule(static)
  for (int64_t oi = 0; oi < outer * inner; ++oi) {
    const int64_t o = oi / inner, in = oi % inner;
    const double *xp = x + o * len * inner + in;
    double *yp = y + o * len * inner + in;
    double mx = -INFINITY;
    for (int64_t k = 0; k < len; ++k)
      if (xp[k * inner] > mx) mx = xp[k * inner];
    long double s = 0;
    for (int64_t k = 0; k < len; ++k) s += expl((long double)xp[k * inner] - mx);
    const long double ls = logl(s);
    for (int64_t k = 0; k < len; ++k) {
      const long double d = (long double)xp[k * inner] - mx;
      yp[k * inner] = (double)(is_log ? d - ls : expl(d) / s);
    }
  }
}

/* reductionDo -> tensor.Sum / tensor.Max along one axis (op_reduction.go:70-99), tensor
 * viewed as (outer, len, inner); kind 0 = sum, 1 = max. argmax (first maximum) as int64. */
void oracle_reduce_f32(int kind, const float *x, float *y, int64_t outer, int64_t len, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t oi = 0; oi < outer * inner; ++oi) {
    const int64_t o = oi / inner, in = oi % inner;
    const float *xp = x + o * len * inner + in;
    if (kind == 0) {
      double s = 0;
      for (int64_t k = 0; k < len; ++k) s += xp[k * inner];
      y[oi] = (float)s;
    } else {
      float m = xp[0];
      for (int64_t k = 1; k < len; ++k)
        if (xp[k * inner] > m) m = xp[k * inner];
      y[oi] = m;
    }
  }
}
void oracle_reduce_f64(int kind, const double *x, double *y, int64_t outer, int64_t len, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t oi = 0; oi < outer * inner; ++oi) {
    const int64_t o = oi / inner, in = oi % inner;
    const double *xp = x + o * len * inner + in;
    if (kind == 0) {
      long double s = 0;
      for (int64_t k = 0; k < len; ++k) s += xp[k * inner];
      y[oi] = (double)s;
    } else {
      double m = xp[0];
      for (int64_t k = 1; k < len; ++k)
        if (xp[k * inner] > m) m = xp[k * inner];
      y[oi] = m;
    }
  }
}
void oracle_argmax_f32(const float *x, int64_t *y, int64_t outer, int64_t len, int64_t inner) {
#pragma omp parallel for schedule(static)
  for (int64_t oi = 0; oi < outer * inner; ++oi) {
    const int64_t o = oi / inner, in = oi % inner;
    const float *xp = x + o * len * inner + in;
    int64_t arg = 0;
    float m = xp[0];
    for (int64_t k = 1; k < len; ++k)
      if (xp[k * inner] > m) {
        m = xp[k * inner];
        arg = k;
      }
    y[oi] = arg;
  }
}

/* transposeOp.Do -> tensor.Transpose (op_tensor.go:937-952): out dim d is in dim perm[d];
 * elem is the element size in bytes. */
void oracle_transpose(const void *x, void *y, int ndim, const int64_t *shape, const int *perm, int elem) {
  int64_t in_stride[8], out_shape[8], n = 1;
  int64_t s = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    in_stride[d] = s;
    s *= shape[d];
  }
  for (int d = 0; d < ndim; ++d) {
    out_shape[d] = shape[perm[d]];
    n *= out_shape[d];
  }
  const char *xi = (const char *)x;
  char *yo = (char *)y;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    int64_t rem = i, src = 0;
    for (int d = ndim - 1; d >= 0; --d) {
      const int64_t c = rem % out_shape[d];
      rem /= out_shape[d];
      src += c * in_stride[perm[d]];
    }
    memcpy(yo + i * elem, xi + src * elem, (size_t)elem);
  }
}

/* byIndicesOp.Do -> tensor.ByIndices along axis 0 (op_by_indices.go:90-97): out[i,:] = x[idx[i],:]. */
/* the same along an inner axis, tensor viewed as (outer, n_rows, row): y[o,i,:] = x[o,idx[i],:] */
void oracle_gather_axis(const void *x, const int64_t *idx, void *y, int64_t outer, int64_t n_rows, int64_t n_idx,
                        int64_t row_bytes) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < n_idx; ++i)
      memcpy((char *)y + (o * n_idx + i) * row_bytes, (const char *)x + (o * n_rows + idx[i]) * row_bytes,
             (size_t)row_bytes);
}
void oracle_gather_rows(const void *x, const int64_t *idx, void *y, int64_t n_idx, int64_t row_bytes) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n_idx; ++i)
    memcpy((char *)y + i * row_bytes, (const char *)x + idx[i] * row_bytes, (size_t)row_bytes);
}


/* ---- dropout: dropoutOp.do and dropoutDiffOp.UsePreallocDo (op_dropout.go:106-128,205-240) ------
 * r[i] comes from `uniforms` (the injected generator of the reference's own test) or from
 * Philox-4x32-10 (Salmon et al., SC'11) keyed by `seed`, counter = element index + offset: float32
 * takes word i % 4 of block i / 4 (top 24 bits), float64 the word pair 2 (i % 2), 2 (i % 2) + 1 of
 * block i / 2 (53 bits). */
static void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                          uint32_t out[4]) {
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

float oracle_philox_uniform_f32(uint64_t seed, uint64_t i) {
  uint32_t r[4];
  const uint64_t blk = i >> 2;
  philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
  return (float)(r[i & 3] >> 8) * 5.9604644775390625e-08f;
}

double oracle_philox_uniform_f64(uint64_t seed, uint64_t i) {
  uint32_t r[4];
  const uint64_t blk = i >> 1;
  philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), r);
  const uint32_t a = r[2 * (i & 1)], b = r[2 * (i & 1) + 1];
  return ((double)(a >> 5) * 67108864.0 + (double)(b >> 6)) * 1.1102230246251565e-16;
}

void oracle_dropout_f32(const float *x, float *y, int64_t n, double prob, const float *uniforms, uint64_t seed,
                        uint64_t offset) {
  const float keep = (float)(1.0 - prob);
  for (int64_t i = 0; i < n; ++i) {
    if (prob == 0.0) { y[i] = x[i]; continue; }       /* the op hands its input through (op_dropout.go:81-83) */
    const float r = uniforms ? uniforms[i] : oracle_philox_uniform_f32(seed, offset + (uint64_t)i);
    y[i] = r < keep ? x[i] / keep : 0.0f;            /* a fresh tensor holds zeros where nothing is written */
  }
}

void oracle_dropout_f64(const double *x, double *y, int64_t n, double prob, const double *uniforms, uint64_t seed,
                        uint64_t offset) {
  const double keep = 1.0 - prob;
  for (int64_t i = 0; i < n; ++i) {
    if (prob == 0.0) { y[i] = x[i]; continue; }
    const double r = uniforms ? uniforms[i] : oracle_philox_uniform_f64(seed, offset + (uint64_t)i);
    y[i] = r < keep ? x[i] / keep : 0.0;
  }
}

/* the reference divides by the drop probability and finds kept elements by their non-zero output */
void oracle_dropout_bwd_f32(const float *dy, const float *out, float *dx, int64_t n, double prob) {
  for (int64_t i = 0; i < n; ++i) dx[i] = (prob != 0 && out[i] != 0) ? dy[i] / (float)prob : 0.0f;
}

void oracle_dropout_bwd_f64(const double *dy, const double *out, double *dx, int64_t n, double prob) {
  for (int64_t i = 0; i < n; ++i) dx[i] = (prob != 0 && out[i] != 0) ? dy[i] / prob : 0.0;
}
