/*
 * knet_oracle.c -- CPU restatement of Knet.jl's CPU definitions of the memory-bound
 * training ops.  TEST INFRASTRUCTURE ONLY: this file is the checker that the CUDA
 * library is compared against (and the timed CPU baseline); nothing in the shipped
 * library or its host package may call it.
 *
 * Each function follows the Knet expression it cites, in the array's own precision and
 * with the same association of operations.  The file must be compiled with
 * -ffp-contract=off so that the compiler fuses nothing by itself: the only fused
 * multiply-adds are the explicit fma()/fmaf() calls that stand for BLAS axpy.
 *
 * Pins: the functions are checked in tests/ against the known answers that the
 * reference holds for this path (the nll docstring value, the accuracy identities,
 * softmax == exp(logsoftmax) with unit column sums, Rosenbrock convergence of the
 * optimizers, the dropout second-moment check).
 * PARITY UNPINNED for the scalar transcendental functions: Knet's CPU path uses Julia's
 * exp/tanh/log, whose bit patterns no reference test fixes and which cannot be run where
 * this file is built.  Here exp/tanh/log are the correctly rounded values: a Float32 one is
 * evaluated in double and rounded once, a Float64 one is the long double value rounded once
 * unless that value lies too close to a rounding boundary to decide, in which case the
 * 113-bit libquadmath value is rounded instead.
 * Sums along a dim are sequential in the array's precision (Julia's loop order without its
 * SIMD re-association), so a Float32 sum of n terms carries an error of order sqrt(n)*eps
 * of its own; tests that compare sums allow for it and also compare with the Float64 run.
 *
 * Array geometry for every "dims" operation: the array is seen as (inner, D, outer) in
 * column-major order, element (a,d,c) at a + inner*(d + D*c); the operation runs over d.
 * A matrix (C,B) with dims=1 is (1,C,B); with dims=2 it is (C,B,1) -> inner=C, D=B.
 */
#include <math.h>
#include <quadmath.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KO_API __attribute__((visibility("default")))

/* ---- scalar math in the array's precision ------------------------------------------ */
/* Loops over independent outputs can be split over host threads: every output is still computed
 * by one thread in the order written here, so the results do not depend on the thread count.
 * Without -fopenmp the pragmas are ignored (the checker itself is built serial; the timing legs
 * of the benchmark also build an OpenMP copy to report Knet's loops on all host cores). */
#ifdef _OPENMP
#define KO_PAR _Pragma("omp parallel for schedule(static)")
#define KO_PAR2 _Pragma("omp parallel for collapse(2) schedule(static)")
#else
#define KO_PAR
#define KO_PAR2
#endif

static inline float  ko_exp_f(float x)   { return (float)exp((double)x); }
static inline float  ko_log_f(float x)   { return (float)log((double)x); }
static inline float  ko_tanh_f(float x)  { return (float)tanh((double)x); }
static inline float  ko_sqrt_f(float x)  { return sqrtf(x); }
/* Float64: correctly rounded.  The 80-bit long double value (error below 1 unit of its 64-bit
 * significand) decides the rounding to 53 bits unless its low 11 bits lie within 4 units of the
 * halfway pattern, or the result is subnormal as a double; those cases (about one argument in
 * 200) are decided by the 113-bit libquadmath value. */
static inline int ko_ld_undecided(long double e) {
  union { long double v; struct { uint64_t mant; uint16_t se; } p; } u;
  u.v = e;
  const int ex = u.p.se & 0x7fff;
  if (ex == 0 || ex == 0x7fff) return 0;              /* zero, infinity, NaN */
  if (ex - 16383 < -1022) return 1;                   /* subnormal double */
  const unsigned m = (unsigned)(u.p.mant & 0x7ff);
  return m >= 0x400 - 4 && m <= 0x400 + 4;
}
static inline double ko_exp_d(double x)  { long double e = expl((long double)x);  return ko_ld_undecided(e) ? (double)expq((__float128)x)  : (double)e; }
static inline double ko_log_d(double x)  { long double e = logl((long double)x);  return ko_ld_undecided(e) ? (double)logq((__float128)x)  : (double)e; }
static inline double ko_tanh_d(double x) { long double e = tanhl((long double)x); return ko_ld_undecided(e) ? (double)tanhq((__float128)x) : (double)e; }
static inline double ko_sqrt_d(double x) { return sqrt(x); }
static inline float  ko_fma_f(float a, float b, float c)    { return fmaf(a, b, c); }
static inline double ko_fma_d(double a, double b, double c) { return fma(a, b, c); }

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

/* =====================================================================================
 * Everything below is instantiated twice: T=float (suffix f32) and T=double (f64).
 * ===================================================================================== */
#define DEFINE_ALL(T, S, M)                                                              \
                                                                                         \
/* -- activations: src/ops20/activation.jl:12,26,55; tanh is Base.tanh ---------------- */\
KO_API void CAT(ko_relu_, S)(int64_t n, const T *x, T *y) {                              \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = x[i] > (T)0 ? x[i] : (x[i] != x[i] ? x[i] : (T)0); \
}                                                                                        \
KO_API void CAT(ko_sigm_, S)(int64_t n, const T *x, T *y) {                              \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T xi = x[i];                                                                         \
    if (xi >= (T)0) y[i] = (T)1 / ((T)1 + CAT(ko_exp_, M)(-xi));                         \
    else { T z = CAT(ko_exp_, M)(xi); y[i] = z / ((T)1 + z); }                           \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_tanh_, S)(int64_t n, const T *x, T *y) {                              \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = CAT(ko_tanh_, M)(x[i]);                         \
}                                                                                        \
KO_API void CAT(ko_elu_, S)(int64_t n, const T *x, T *y) {                               \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = x[i] >= (T)0 ? x[i] : CAT(ko_exp_, M)(x[i]) - (T)1; \
}                                                                                        \
KO_API void CAT(ko_exp_, S)(int64_t n, const T *x, T *y) {                               \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = CAT(ko_exp_, M)(x[i]);                          \
}                                                                                        \
KO_API void CAT(ko_log_, S)(int64_t n, const T *x, T *y) {                               \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = CAT(ko_log_, M)(x[i]);                          \
}                                                                                        \
/* -- activation backward: activation.jl:13,27,56; ops20_gpu/activation.jl:11 --------- */\
KO_API void CAT(ko_reluback_, S)(int64_t n, const T *dy, const T *y, T *dx) {            \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) dx[i] = y[i] > (T)0 ? dy[i] : (T)0;                    \
}                                                                                        \
KO_API void CAT(ko_sigmback_, S)(int64_t n, const T *dy, const T *y, T *dx) {            \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) { T a = dy[i] * y[i]; T b = (T)1 - y[i]; dx[i] = a * b; } \
}                                                                                        \
KO_API void CAT(ko_tanhback_, S)(int64_t n, const T *dy, const T *y, T *dx) {            \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) { T yy = y[i] * y[i]; T b = (T)1 - yy; dx[i] = dy[i] * b; } \
}                                                                                        \
KO_API void CAT(ko_eluback_, S)(int64_t n, const T *dy, const T *y, T *dx) {             \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) dx[i] = y[i] >= (T)0 ? dy[i] : dy[i] * ((T)1 + y[i]);  \
}                                                                                        \
                                                                                         \
/* -- reductions over one dim (Julia Base semantics: sequential along the dim) -------- */\
/* op: 0 sum 1 prod 2 maximum 3 minimum 4 sumabs 5 sumabs2 6 maxabs 7 minabs 8 countnz */\
/*     (table: src/libknet8/ops.jl:144-156)                                            */\
static inline T CAT(ko_item_, S)(int op, T xi) {                                         \
  switch (op) {                                                                          \
    case 4: case 6: case 7: return xi < (T)0 ? -xi : xi;                                 \
    case 5: return xi * xi;                                                              \
    case 8: return xi != (T)0 ? (T)1 : (T)0;                                             \
    default: return xi;                                                                  \
  }                                                                                      \
}                                                                                        \
static inline T CAT(ko_init_, S)(int op) {                                               \
  switch (op) {                                                                          \
    case 1: return (T)1;                                                                 \
    case 2: return (T)(-INFINITY);                                                       \
    case 3: case 7: return (T)INFINITY;                                                  \
    default: return (T)0;                                                                \
  }                                                                                      \
}                                                                                        \
static inline T CAT(ko_merge_, S)(int op, T a, T x) {                                    \
  switch (op) {                                                                          \
    case 1: return a * x;                                                                \
    case 2: case 6: return a > x ? a : x;                                                \
    case 3: case 7: return a < x ? a : x;                                                \
    default: return a + x;                                                               \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_reduce_dim_, S)(int op, int64_t inner, int64_t D, int64_t outer,      \
                                   const T *x, T *y) {                                   \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++) {                                                \
      T acc = CAT(ko_init_, S)(op);                                                      \
      for (int64_t d = 0; d < D; d++)                                                    \
        acc = CAT(ko_merge_, S)(op, acc, CAT(ko_item_, S)(op, x[a + inner * (d + D * c)])); \
      y[a + inner * c] = acc;                                                            \
    }                                                                                    \
}                                                                                        \
/* full reduction: Julia's pairwise mapreduce, blocks of 1024 summed in order */         \
static T CAT(ko_pairwise_, S)(int op, const T *x, int64_t lo, int64_t hi) {              \
  if (hi - lo <= 1024) {                                                                 \
    T acc = CAT(ko_init_, S)(op);                                                        \
    for (int64_t i = lo; i < hi; i++) acc = CAT(ko_merge_, S)(op, acc, CAT(ko_item_, S)(op, x[i])); \
    return acc;                                                                          \
  }                                                                                      \
  int64_t mid = lo + ((hi - lo) >> 1);                                                   \
  T l = CAT(ko_pairwise_, S)(op, x, lo, mid);                                            \
  T r = CAT(ko_pairwise_, S)(op, x, mid, hi);                                            \
  return CAT(ko_merge_, S)(op, l, r);                                                    \
}                                                                                        \
KO_API T CAT(ko_reduce_all_, S)(int op, int64_t n, const T *x) {                         \
  return CAT(ko_pairwise_, S)(op, x, 0, n);                                              \
}                                                                                        \
                                                                                         \
/* -- softmax family: src/ops20/softmax.jl:42-74 --------------------------------------- */\
/* mode 0: softmax, 1: logsoftmax                                                      */\
KO_API void CAT(ko_softmax_fwd_, S)(int mode, int64_t inner, int64_t D, int64_t outer,   \
                                    const T *x, T *y) {                                  \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++) {                                                \
      const T *xp = x + a + inner * D * c; T *yp = y + a + inner * D * c;                \
      T mx = (T)(-INFINITY);                                                             \
      for (int64_t d = 0; d < D; d++) { T v = xp[inner * d]; mx = mx > v ? mx : v; }     \
      T s = (T)0;                                                                        \
      for (int64_t d = 0; d < D; d++) {                                                  \
        T x1 = xp[inner * d] - mx; T e = CAT(ko_exp_, M)(x1);                            \
        yp[inner * d] = mode ? x1 : e; s = s + e;                                        \
      }                                                                                  \
      if (mode) { T ls = CAT(ko_log_, M)(s);                                             \
        for (int64_t d = 0; d < D; d++) yp[inner * d] = yp[inner * d] - ls; }            \
      else { for (int64_t d = 0; d < D; d++) yp[inner * d] = yp[inner * d] / s; }        \
    }                                                                                    \
}                                                                                        \
/* softmax: y.*dy .- y.*sum(y.*dy); logsoftmax: dy - exp.(y).*sum(dy)  (softmax.jl:49-63) */\
KO_API void CAT(ko_softmax_bwd_, S)(int mode, int64_t inner, int64_t D, int64_t outer,   \
                                    const T *y, const T *dy, T *dx) {                    \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++) {                                                \
      int64_t o = a + inner * D * c;                                                     \
      T s = (T)0;                                                                        \
      for (int64_t d = 0; d < D; d++) {                                                  \
        int64_t i = o + inner * d; s = s + (mode ? dy[i] : y[i] * dy[i]);                \
      }                                                                                  \
      for (int64_t d = 0; d < D; d++) {                                                  \
        int64_t i = o + inner * d;                                                       \
        if (mode) dx[i] = dy[i] - CAT(ko_exp_, M)(y[i]) * s;                             \
        else { T p = y[i] * dy[i]; T q = y[i] * s; dx[i] = p - q; }                      \
      }                                                                                  \
    }                                                                                    \
}                                                                                        \
/* logsumexp: xmax + log(sum(exp(x-xmax))); bwd dy .* exp.(x .- y)  (softmax.jl:65-74) */\
KO_API void CAT(ko_logsumexp_fwd_, S)(int64_t inner, int64_t D, int64_t outer,           \
                                      const T *x, T *y) {                                \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++) {                                                \
      const T *xp = x + a + inner * D * c;                                               \
      T mx = (T)(-INFINITY);                                                             \
      for (int64_t d = 0; d < D; d++) { T v = xp[inner * d]; mx = mx > v ? mx : v; }     \
      T s = (T)0;                                                                        \
      for (int64_t d = 0; d < D; d++) s = s + CAT(ko_exp_, M)(xp[inner * d] - mx);       \
      y[a + inner * c] = mx + CAT(ko_log_, M)(s);                                        \
    }                                                                                    \
}                                                                                        \
KO_API void CAT(ko_logsumexp_bwd_, S)(int64_t inner, int64_t D, int64_t outer,           \
                                      const T *x, const T *y, const T *dy, T *dx) {      \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++)                                                  \
      for (int64_t d = 0; d < D; d++) {                                                  \
        int64_t i = a + inner * (d + D * c);                                             \
        dx[i] = dy[a + inner * c] * CAT(ko_exp_, M)(x[i] - y[a + inner * c]);            \
      }                                                                                  \
}                                                                                        \
                                                                                         \
/* -- nll / accuracy: src/ops20/loss.jl:37-62,116-140 ---------------------------------- */\
/* scores (R,K) column-major; dims=1: classes along rows, ninst=K; dims=2: ninst=R.    */\
/* labels 1-based, 0 = skip.  Returns -sum(lp) in *total and the count of used labels. */\
/* lp gathers logsoftmax at the 1-based linear index findindices() computes.           */\
KO_API int64_t CAT(ko_nll_, S)(int64_t R, int64_t K, int dims, const T *scores,          \
                               const int32_t *labels, T *total) {                        \
  int64_t ninst = dims == 1 ? K : R;                                                     \
  T *lsm = (T *)malloc(sizeof(T) * (size_t)(R * K > 0 ? R * K : 1));                     \
  T *lp = (T *)malloc(sizeof(T) * (size_t)(ninst > 0 ? ninst : 1));                      \
  if (dims == 1) CAT(ko_softmax_fwd_, S)(1, 1, R, K, scores, lsm);                       \
  else CAT(ko_softmax_fwd_, S)(1, R, K, 1, scores, lsm);                                 \
  int64_t cnt = 0;                                                                       \
  for (int64_t j = 1; j <= ninst; j++) {                                                 \
    int64_t l = labels[j - 1];                                                           \
    if (l == 0) continue;                                                                \
    int64_t idx = dims == 1 ? (j - 1) * R + l : (l - 1) * R + j;                         \
    lp[cnt++] = lsm[idx - 1];                                                            \
  }                                                                                      \
  *total = -CAT(ko_pairwise_, S)(0, lp, 0, cnt);                                         \
  free(lsm); free(lp);                                                                   \
  return cnt;                                                                            \
}                                                                                        \
/* gradient of nll wrt scores for output gradient dy of the averaged (average=1) or    */\
/* summed loss: AutoGrad's rules composed by hand: d(-sum(lp)/cnt) scatters -dy/cnt at */\
/* the label entries (ungetindex), then the logsoftmax rule dy - exp(y)*sum(dy).       */\
KO_API void CAT(ko_nll_bwd_, S)(int64_t R, int64_t K, int dims, int average,             \
                                const T *scores, const int32_t *labels, T dy, T *dx) {   \
  int64_t ninst = dims == 1 ? K : R; int64_t n = R * K;                                  \
  T *lsm = (T *)malloc(sizeof(T) * (size_t)(n > 0 ? n : 1));                             \
  T *g = (T *)calloc((size_t)(n > 0 ? n : 1), sizeof(T));                                \
  if (dims == 1) CAT(ko_softmax_fwd_, S)(1, 1, R, K, scores, lsm);                       \
  else CAT(ko_softmax_fwd_, S)(1, R, K, 1, scores, lsm);                                 \
  int64_t cnt = 0;                                                                       \
  for (int64_t j = 0; j < ninst; j++) if (labels[j] != 0) cnt++;                         \
  T gv = average ? -dy / (T)cnt : -dy;                                                   \
  for (int64_t j = 1; j <= ninst; j++) {                                                 \
    int64_t l = labels[j - 1]; if (l == 0) continue;                                     \
    int64_t idx = dims == 1 ? (j - 1) * R + l : (l - 1) * R + j;                         \
    g[idx - 1] += gv;                                                                    \
  }                                                                                      \
  if (dims == 1) CAT(ko_softmax_bwd_, S)(1, 1, R, K, lsm, g, dx);                        \
  else CAT(ko_softmax_bwd_, S)(1, R, K, 1, lsm, g, dx);                                  \
  free(lsm); free(g);                                                                    \
}                                                                                        \
/* argmax along d, first maximal element wins (Julia findmax); 1-based position in d.  */\
KO_API void CAT(ko_argmax_, S)(int64_t inner, int64_t D, int64_t outer, const T *x,      \
                               int32_t *idx) {                                           \
  KO_PAR2 \
  for (int64_t c = 0; c < outer; c++)                                                    \
    for (int64_t a = 0; a < inner; a++) {                                                \
      const T *xp = x + a + inner * D * c; T best = xp[0]; int64_t bi = 0;               \
      for (int64_t d = 1; d < D; d++) { T v = xp[inner * d]; if (v > best) { best = v; bi = d; } } \
      idx[a + inner * c] = (int32_t)(bi + 1);                                            \
    }                                                                                    \
}                                                                                        \
/* accuracy(scores,labels;dims): returns ncorrect, *count = used instances (loss.jl:54-62) */\
KO_API int64_t CAT(ko_accuracy_, S)(int64_t R, int64_t K, int dims, const T *scores,     \
                                    const int32_t *labels, int64_t *count) {             \
  int64_t ninst = dims == 1 ? K : R;                                                     \
  int32_t *am = (int32_t *)malloc(sizeof(int32_t) * (size_t)(ninst > 0 ? ninst : 1));    \
  if (dims == 1) CAT(ko_argmax_, S)(1, R, K, scores, am);                                \
  else CAT(ko_argmax_, S)(R, K, 1, scores, am);                                          \
  int64_t ok = 0, cnt = 0;                                                               \
  for (int64_t j = 0; j < ninst; j++) {                                                  \
    if (labels[j] == 0) continue;                                                        \
    cnt++; if (am[j] == labels[j]) ok++;                                                 \
  }                                                                                      \
  free(am); *count = cnt; return ok;                                                     \
}                                                                                        \
                                                                                         \
/* -- dropout with the uniforms supplied in y: src/ops20/dropout.jl:45-71 -------------- */\
KO_API void CAT(ko_dropout_, S)(int64_t n, double p_, const T *x, T *y) {                \
  T p = (T)p_; T q = (T)1 - p;                                                           \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) y[i] = y[i] > p ? x[i] / q : (T)0;                     \
}                                                                                        \
KO_API void CAT(ko_dropback_, S)(int64_t n, double p_, const T *y, const T *dy, T *dx) { \
  T p = (T)p_; T q = (T)1 - p;                                                           \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) dx[i] = y[i] == (T)0 ? (T)0 : dy[i] / q;               \
}                                                                                        \
                                                                                         \
/* -- update!: src/train20/update.jl:513-570.  lmul!(a::Float64, x) multiplies in      */\
/* Float64 and rounds to T; axpy!(a, x, y) converts a to T and is one fused multiply-  */\
/* add per element (BLAS axpy); "/" on an Array is a true division.                    */\
KO_API void CAT(ko_sgd_, S)(int64_t n, T *w, const T *g, double lr) {                    \
  T a = (T)(-lr);                                                                        \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) w[i] = CAT(ko_fma_, M)(a, g[i], w[i]);                 \
}                                                                                        \
KO_API void CAT(ko_momentum_, S)(int64_t n, T *w, const T *g, T *v, double lr, double gamma) { \
  T a = (T)(-lr);                                                                        \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T vi = (T)(gamma * (double)v[i]);                                                    \
    vi = CAT(ko_fma_, M)(a, g[i], vi);                                                   \
    v[i] = vi; w[i] = CAT(ko_fma_, M)((T)1, vi, w[i]);                                   \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_nesterov_, S)(int64_t n, T *w, const T *g, T *v, double lr, double gamma) { \
  T a = (T)(-lr); T b = (T)(1 + gamma);                                                  \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T vi = (T)(gamma * (double)v[i]);                                                    \
    T wi = CAT(ko_fma_, M)((T)(-1), vi, w[i]);                                           \
    vi = CAT(ko_fma_, M)(a, g[i], vi);                                                   \
    v[i] = vi; w[i] = CAT(ko_fma_, M)(b, vi, wi);                                        \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_adagrad_, S)(int64_t n, T *w, const T *g, T *G, double lr, double eps) { \
  T a = (T)(-lr); T e = (T)eps;                                                          \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T gg = g[i] * g[i]; T Gi = CAT(ko_fma_, M)((T)1, gg, G[i]); G[i] = Gi;               \
    T u = g[i] / CAT(ko_sqrt_, M)(Gi + e);                                               \
    w[i] = CAT(ko_fma_, M)(a, u, w[i]);                                                  \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_rmsprop_, S)(int64_t n, T *w, const T *g, T *G, double lr, double rho, double eps) { \
  T a = (T)(-lr); T e = (T)eps; T r1 = (T)(1 - rho);                                     \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T Gi = (T)(rho * (double)G[i]); T gg = g[i] * g[i];                                  \
    Gi = CAT(ko_fma_, M)(r1, gg, Gi); G[i] = Gi;                                         \
    T u = g[i] / CAT(ko_sqrt_, M)(Gi + e);                                               \
    w[i] = CAT(ko_fma_, M)(a, u, w[i]);                                                  \
  }                                                                                      \
}                                                                                        \
KO_API void CAT(ko_adadelta_, S)(int64_t n, T *w, const T *g, T *G, T *delta, double lr, double rho, double eps) { \
  T a = (T)(-lr); T e = (T)eps; T r1 = (T)(1 - rho);                                     \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T Gi = (T)(rho * (double)G[i]); T gg = g[i] * g[i];                                  \
    Gi = CAT(ko_fma_, M)(r1, gg, Gi); G[i] = Gi;                                         \
    T num = g[i] * CAT(ko_sqrt_, M)(delta[i] + e);                                       \
    T dw = num / CAT(ko_sqrt_, M)(Gi + e);                                               \
    T di = (T)(rho * (double)delta[i]); T dd = dw * dw;                                  \
    delta[i] = CAT(ko_fma_, M)(r1, dd, di);                                              \
    w[i] = CAT(ko_fma_, M)(a, dw, w[i]);                                                 \
  }                                                                                      \
}                                                                                        \
/* Adam: t is the step count AFTER the increment (update.jl:562).                      */\
KO_API void CAT(ko_adam_, S)(int64_t n, T *w, const T *g, T *m, T *v, double lr,         \
                             double beta1, double beta2, double eps, int t) {            \
  T a = (T)(-lr); T e = (T)eps;                                                          \
  T c1 = (T)(1 - beta1); T c2 = (T)(1 - beta2);                                          \
  T b1t = (T)(1 - pow(beta1, (double)t)); T b2t = (T)(1 - pow(beta2, (double)t));        \
  KO_PAR \
  for (int64_t i = 0; i < n; i++) {                                                      \
    T mi = (T)(beta1 * (double)m[i]);                                                    \
    mi = CAT(ko_fma_, M)(c1, g[i], mi);                                                  \
    T vi = (T)(beta2 * (double)v[i]); T gg = g[i] * g[i];                                \
    vi = CAT(ko_fma_, M)(c2, gg, vi);                                                    \
    m[i] = mi; v[i] = vi;                                                                \
    T mh = mi / b1t; T vh = vi / b2t;                                                    \
    T den = CAT(ko_sqrt_, M)(vh) + e;                                                    \
    T u = mh / den;                                                                      \
    w[i] = CAT(ko_fma_, M)(a, u, w[i]);                                                  \
  }                                                                                      \
}                                                                                        \
                                                                                         \
/* -- dense matrix products for the MLP oracle (column-major, plain triple loops) ----- */\
/* C(m,n) = op(A)(m,k) * op(B)(k,n); ta/tb: 0 = as stored, 1 = transposed              */\
KO_API void CAT(ko_gemm_, S)(int ta, int tb, int64_t m, int64_t n, int64_t k,            \
                             const T *A, const T *B, T *C) {                             \
  int64_t lda = ta ? k : m, ldb = tb ? n : k;                                            \
  for (int64_t j = 0; j < n; j++)                                                        \
    for (int64_t i = 0; i < m; i++) {                                                    \
      T acc = (T)0;                                                                      \
      for (int64_t l = 0; l < k; l++) {                                                  \
        T a = ta ? A[l + lda * i] : A[i + lda * l];                                      \
        T b = tb ? B[j + ldb * l] : B[l + ldb * j];                                      \
        acc = acc + a * b;                                                               \
      }                                                                                  \
      C[i + m * j] = acc;                                                                \
    }                                                                                    \
}

DEFINE_ALL(float, f32, f)
DEFINE_ALL(double, f64, d)

/* xavier_uniform (src/train20/distributions.jl:35-52): u ~ U[0,1) drawn in Float64 by the
 * caller; s = sqrt(6/(fanin+fanout)) with fanout = rows, fanin = cols; w = 2s*u - s in
 * Float64, converted to the array type by param() (src/train20/param.jl:22-24). */
KO_API void ko_xavier_uniform(int64_t rows, int64_t cols, const double *u, double *w) {
  double s = 1.0 * sqrt(6.0 / (double)(cols + rows));
  for (int64_t i = 0; i < rows * cols; i++) w[i] = (2 * s) * u[i] - s;
}
