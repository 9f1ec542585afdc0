/*
 * knet_sm100.h -- C ABI of libknet_sm100.so, a B200 (sm_100a) implementation of the
 * memory-bound kernels behind Knet.jl's `@knet8` ccalls, plus fused entry points for the
 * call sites that Knet serves today with cuDNN, cuBLAS axpy/scal chains or host loops.
 *
 * Conventions (the ones Knet's Julia side already follows, src/libknet8/LibKnet8.jl:50-62):
 *   - plain device pointers and sizes; arrays are dense and column-major; the caller owns
 *     and pre-allocates every buffer; the library keeps no pointer after a call returns;
 *   - every function exists as `name(...)`, which uses the per-thread default stream, and
 *     as `name_stream(..., cudaStream_t)`, the only form Julia calls;
 *   - S = 32 is Float32 (float), S = 64 is Float64 (double);
 *   - index arrays are 1-based Int32 (src/knetarrays/getindex.jl:291-297);
 *   - n <= 0 is a no-op (src/libknet8/cuda1.jl:29);
 *   - section A functions return void like the ones they replace; section B functions
 *     return int: 0 ok, <0 argument error (KNET_E*), >0 a cudaError_t value.
 * Pointers need only be aligned to the element size (KnetArray views carry element
 * offsets, src/knetarrays/getindex.jl:153-159); 16-byte aligned pointers get the fast path.
 * An output may be the very same pointer as an input; partially overlapping buffers are
 * not supported.
 */
#ifndef KNET_SM100_H
#define KNET_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if !defined(__DRIVER_TYPES_H__) && !defined(__CUDA_RUNTIME_H__)
typedef struct CUstream_st *cudaStream_t;
#endif

#ifndef KNET_API
#define KNET_API
#endif

#define KNET_OK 0
#define KNET_EINVAL (-1)     /* null pointer, negative size, unknown op or dims */
#define KNET_ESIZE (-2)      /* size beyond what the entry point supports */
#define KNET_EWORKSPACE (-3) /* workspace missing or too small */
#define KNET_EALIGN (-4)     /* pointer not aligned to its element size */
#define KNET_ENCCL (-5)      /* section C: NCCL could not be loaded */
#define KNET_ETIMEOUT (-6)   /* section C: the other ranks did not answer before the deadline */
#define KNET_ECUBLAS (-7)    /* section D: cuBLAS could not be loaded */
#define KNET_EUNSUPPORTED (-8) /* section D: the loaded cuBLAS does not offer the requested mode */

/* ---- op lists (name = the symbol stem Knet uses, src/libknet8/ops.jl) ------------------- */
/* unary ops, ops.jl:6-81 */
#define KNET_UNARY_OPS(X) \
  X(abs2) X(abs) X(acos) X(acosh) X(asin) X(asinh) X(atan) X(atanh) X(cbrt) X(ceil) X(cos) \
  X(cosh) X(cospi) X(erf) X(erfc) X(erfcinv) X(erfcx) X(erfinv) X(exp) X(exp10) X(exp2) \
  X(expm1) X(floor) X(j0) X(j1) X(gamma_impl) X(lgamma) X(digamma_impl) X(trigamma_impl) X(log) X(log10) \
  X(log1p) X(log2) \
  X(neg) X(one) X(round) X(sign) X(sin) X(sinh) X(sinpi) X(sqrt) X(tan) X(tanh) X(tanh_) \
  X(trunc) X(y0) X(y1) X(zero) X(invx) X(elu) X(gelu) X(hardsigmoid) X(hardswish) X(relu) \
  X(selu) X(sigm) X(swish)
/* binary ops, ops.jl:87-100 */
#define KNET_BINARY_OPS(X) \
  X(add) X(sub) X(mul) X(div) X(pow) X(max) X(min) X(eq) X(ne) X(gt) X(ge) X(lt) X(le)
/* two-argument activation backward forms (x = dy, y = y), ops.jl:114-122 */
#define KNET_ACTBACK2_OPS(X) \
  X(invxback) X(eluback) X(geluback) X(reluback) X(seluback) X(sigmback) X(tanhback) X(swishback)
/* three-argument backward forms (x, y, dy), ops.jl:125-136 */
#define KNET_ACTBACK3_OPS(X) \
  X(eluback) X(geluback) X(hardsigmoidback) X(hardswishback) X(seluback) X(sigmback) \
  X(tanh_back) X(swishback)
/* reductions, ops.jl:144-156 */
#define KNET_REDUCTION_OPS(X) \
  X(sum) X(prod) X(maximum) X(minimum) X(sumabs) X(sumabs2) X(maxabs) X(minabs) X(countnz)

#define KNET_BOTH_TYPES(M, f) M(f, 32, float) M(f, 64, double)

/* =====================================================================================
 * A. Entry points with the names and argument lists of libknet8
 * ===================================================================================== */

/* y[i] = f(x[i]).  Replaces src/libknet8/cuda1.jl:13-44 ({f}_S, {f}_S_stream). */
#define KNET_DECL_UNARY(f, S, T)                             \
  KNET_API void f##_##S(int n, const T *x, T *y);            \
  KNET_API void f##_##S##_stream(int n, const T *x, T *y, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_UNARY, f)
KNET_UNARY_OPS(KNET_X)
#undef KNET_X

/* relu with keyword arguments and its backward.  Replaces src/libknet8/relu.jl:3-43. */
#define KNET_DECL_RELU1(f, S, T)                                                            \
  KNET_API void relu_##S##_1(int n, T max_value, T negative_slope, T threshold, const T *x, \
                             T *y);                                                         \
  KNET_API void relu_##S##_1_stream(int n, T max_value, T negative_slope, T threshold,      \
                                    const T *x, T *y, cudaStream_t s);                      \
  KNET_API void reluback_##S##_1(int n, T max_value, T negative_slope, T threshold,         \
                                 const T *x, const T *y, const T *dy, T *dx);               \
  KNET_API void reluback_##S##_1_stream(int n, T max_value, T negative_slope, T threshold,  \
                                        const T *x, const T *y, const T *dy, T *dx,         \
                                        cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_RELU1, relu)

/* y[i] = x for all i.  Replaces fill_S, src/libknet8/cuda1.jl:82-107. */
#define KNET_DECL_FILL(f, S, T)                 \
  KNET_API void fill_##S(int n, T x, T *y);     \
  KNET_API void fill_##S##_stream(int n, T x, T *y, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_FILL, fill)

/* z[i] = f(xi, y[i]) with a scalar first operand.  Replaces src/libknet8/cuda01.jl:6-30. */
#define KNET_DECL_01(f, S, T)                                    \
  KNET_API void f##_##S##_01(int n, T xi, const T *y, T *z);     \
  KNET_API void f##_##S##_01_stream(int n, T xi, const T *y, T *z, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_01, f)
KNET_BINARY_OPS(KNET_X)
#undef KNET_X

/* z[i] = f(x[i], y[i]), same-size arrays; for the backward forms x = dy and y = y.
 * Replaces src/libknet8/cuda11.jl:7-32. */
#define KNET_DECL_11(f, S, T)                                          \
  KNET_API void f##_##S##_11(int n, const T *x, const T *y, T *z);     \
  KNET_API void f##_##S##_11_stream(int n, const T *x, const T *y, T *z, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_11, f)
KNET_BINARY_OPS(KNET_X)
KNET_ACTBACK2_OPS(KNET_X)
#undef KNET_X

/* dx[i] = g(x[i], y[i], dy[i]).  Replaces src/libknet8/cuda111.jl:7-33. */
#define KNET_DECL_111(f, S, T)                                                        \
  KNET_API void f##_##S##_111(int n, const T *x, const T *y, const T *dy, T *dx);     \
  KNET_API void f##_##S##_111_stream(int n, const T *x, const T *y, const T *dy, T *dx, \
                                     cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_111, f)
KNET_ACTBACK3_OPS(KNET_X)
#undef KNET_X

/* Broadcast where each operand is full-size, a scalar, or a vector along one dim:
 * xi = nx==n ? x[i] : sx==1 ? x[i%nx] : nx==1 ? x[0] : x[(i/sx)%nx], same for y.
 * Replaces src/libknet8/cuda12.jl:13-38. */
#define KNET_DECL_12(f, S, T)                                                                \
  KNET_API void f##_##S##_12(int n, const T *x, int sx, int nx, const T *y, int sy, int ny,  \
                             T *z);                                                          \
  KNET_API void f##_##S##_12_stream(int n, const T *x, int sx, int nx, const T *y, int sy,   \
                                    int ny, T *z, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_12, f)
KNET_BINARY_OPS(KNET_X)
#undef KNET_X

/* Vector of B_N elements along a non-first dim of a dense array of A_N elements:
 * z[j*dimstride + k*nextstride + i] = f(big, vec[j]) (_x_y: x is the array, y the vector;
 * _y_x: x is the array, y the vector, and the result is f(vec, big)).
 * Replaces src/libknet8/cuda13.jl:37-188. */
#define KNET_DECL_13(f, S, T)                                                               \
  KNET_API void f##_##S##_13_x_y(const T *x, const T *y, T *z, int brdcastdimstride,        \
                                 int brdcastnextstride, int multidimsize, int A_N, int B_N); \
  KNET_API void f##_##S##_13_x_y_stream(const T *x, const T *y, T *z, int brdcastdimstride, \
                                        int brdcastnextstride, int multidimsize, int A_N,   \
                                        int B_N, cudaStream_t s);                           \
  KNET_API void f##_##S##_13_y_x(const T *x, const T *y, T *z, int brdcastdimstride,        \
                                 int brdcastnextstride, int multidimsize, int A_N, int B_N); \
  KNET_API void f##_##S##_13_y_x_stream(const T *x, const T *y, T *z, int brdcastdimstride, \
                                        int brdcastnextstride, int multidimsize, int A_N,   \
                                        int B_N, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_13, f)
KNET_BINARY_OPS(KNET_X)
#undef KNET_X

/* General 3-, 4- and 5-d broadcast with per-dimension strides passed by value (0 on a
 * broadcast dim).  Replaces src/libknet8/cuda16.jl:5-103. */
#define KNET_DECL_16(f, S, T)                                                                 \
  KNET_API void f##_##S##_16_3(const T *x, const T *y, T *z, int sx0, int sx1, int sx2,        \
                               int sy0, int sy1, int sy2, int sz0, int sz1, int sz2, int Nz);  \
  KNET_API void f##_##S##_16_3_stream(const T *x, const T *y, T *z, int sx0, int sx1, int sx2, \
                                      int sy0, int sy1, int sy2, int sz0, int sz1, int sz2,    \
                                      int Nz, cudaStream_t s);                                 \
  KNET_API void f##_##S##_16_4(const T *x, const T *y, T *z, int sx0, int sx1, int sx2,        \
                               int sx3, int sy0, int sy1, int sy2, int sy3, int sz0, int sz1,  \
                               int sz2, int sz3, int Nz);                                      \
  KNET_API void f##_##S##_16_4_stream(const T *x, const T *y, T *z, int sx0, int sx1, int sx2, \
                                      int sx3, int sy0, int sy1, int sy2, int sy3, int sz0,    \
                                      int sz1, int sz2, int sz3, int Nz, cudaStream_t s);      \
  KNET_API void f##_##S##_16_5(const T *x, const T *y, T *z, int sx0, int sx1, int sx2,        \
                               int sx3, int sx4, int sy0, int sy1, int sy2, int sy3, int sy4,  \
                               int sz0, int sz1, int sz2, int sz3, int sz4, int Nz);           \
  KNET_API void f##_##S##_16_5_stream(const T *x, const T *y, T *z, int sx0, int sx1, int sx2, \
                                      int sx3, int sx4, int sy0, int sy1, int sy2, int sy3,    \
                                      int sy4, int sz0, int sz1, int sz2, int sz3, int sz4,    \
                                      int Nz, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_16, f)
KNET_BINARY_OPS(KNET_X)
#undef KNET_X

/* Reductions.  _20: whole array to a scalar returned by value after the stream has been
 * synchronised (src/libknet8/cuda20.jl:10-111); _21: x[i] accumulates into y[(i/sy)%ny]
 * (cuda21.jl:6-83); _22: one middle dim of an N-d array, s1 = its stride, s2 = the next
 * stride, xd1 = its size - 1 (cuda22.jl:6-72).
 * The _21 forms with sy == 1 (a matrix reduced over its second dim) run in two stages when the
 * matrix has fewer than about 1000 rows and at least 8 MiB, or fewer than about 4000 rows and at
 * least 64 MiB: the partial results of the first
 * stage live in a stream-ordered allocation (at most a few MiB, freed on the same stream) from
 * a memory pool that the library creates per device on first use.  Nothing synchronises, calls
 * on different streams share nothing, and the calls can be captured into a graph once the pool
 * exists (a first call made during a capture takes the single-launch path instead).  The
 * environment variable KNET_SM100_ROWS_NOSPLIT=1 turns the two-stage path off. */
#define KNET_DECL_RED(f, S, T)                                                               \
  KNET_API T f##_##S##_20(int n, const T *x);                                                \
  KNET_API T f##_##S##_20_stream(int n, const T *x, cudaStream_t s);                         \
  KNET_API void f##_##S##_21(int nx, const T *x, int sy, int ny, T *y);                      \
  KNET_API void f##_##S##_21_stream(int nx, const T *x, int sy, int ny, T *y, cudaStream_t s); \
  KNET_API void f##_##S##_22(int nx, int xd1, const T *x, int s1, int s2, int ny, T *y);     \
  KNET_API void f##_##S##_22_stream(int nx, int xd1, const T *x, int s1, int s2, int ny,     \
                                    T *y, cudaStream_t s);
#define KNET_X(f) KNET_BOTH_TYPES(KNET_DECL_RED, f)
KNET_REDUCTION_OPS(KNET_X)
#undef KNET_X

/* Dropout with the uniforms already in y: y = y>p ? x/(1-p) : 0, and its backward
 * dx = y==0 ? 0 : dy/(1-p).  Replaces dropout_S/dropback_S, src/libknet8/cuda1.jl:454-500;
 * the scale is a division as in Knet's CPU loop (src/ops20/dropout.jl:45-71). */
#define KNET_DECL_DROPOUT(f, S, T)                                                        \
  KNET_API void dropout_##S(int n, T p, const T *x, T *y);                                \
  KNET_API void dropout_##S##_stream(int n, T p, const T *x, T *y, cudaStream_t s);       \
  KNET_API void dropback_##S(int n, T p, const T *x, const T *y, const T *dy, T *dx);     \
  KNET_API void dropback_##S##_stream(int n, T p, const T *x, const T *y, const T *dy,    \
                                      T *dx, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_DROPOUT, dropout)

/* Entry gather / scatter with 1-based linear indices: getents y[i] = x[ents[i]-1];
 * setents x[ents[i]-1] = y[i]; addents x[ents[i]-1] += y[i] (atomic); setent1 stores one
 * scalar.  Replaces src/libknet8/cuda1.jl:342-369,419-449. */
#define KNET_DECL_ENTS(f, S, T)                                                            \
  KNET_API void getents_##S(int n, const int *ents, const T *x, T *y);                     \
  KNET_API void getents_##S##_stream(int n, const int *ents, const T *x, T *y, cudaStream_t s); \
  KNET_API void setents_##S(int n, const int *ents, T *x, const T *y);                     \
  KNET_API void setents_##S##_stream(int n, const int *ents, T *x, const T *y, cudaStream_t s); \
  KNET_API void addents_##S(int n, const int *ents, T *x, const T *y);                     \
  KNET_API void addents_##S##_stream(int n, const int *ents, T *x, const T *y, cudaStream_t s); \
  KNET_API void setent1_##S(int n, const int *ents, T *x, T y);                            \
  KNET_API void setent1_##S##_stream(int n, const int *ents, T *x, T y, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_ENTS, ents)

/* Whole columns / rows of a column-major (xrows, xcols) matrix x picked by 1-based Int32
 * indices.  Columns: y is (xrows, ncols); getcols y[:,j] = x[:,cols[j]], setcols
 * x[:,cols[j]] = y[:,j], addcols x[:,cols[j]] += y[:,j] (atomic, repeated indices add up),
 * setcol1 x[:,cols[j]] = scalar.  Rows: y is (nrows, xcols) and the same four with
 * x[rows[i],:].  Indices are not range-checked here (the caller does, as
 * src/knetarrays/getindex.jl:277-287).  Replaces src/libknet8/cuda1.jl:246-341,371-418;
 * callers src/knetarrays/getindex.jl:235-271 and src/autograd_gpu/addto.jl:67-82. */
#define KNET_DECL_COLSROWS(f, S, T)                                                              \
  KNET_API void getcols_##S(int xrows, int xcols, int ncols, const int *cols, const T *x, T *y); \
  KNET_API void getcols_##S##_stream(int xrows, int xcols, int ncols, const int *cols,           \
                                     const T *x, T *y, cudaStream_t s);                          \
  KNET_API void setcols_##S(int xrows, int xcols, int ncols, const int *cols, T *x, const T *y); \
  KNET_API void setcols_##S##_stream(int xrows, int xcols, int ncols, const int *cols, T *x,     \
                                     const T *y, cudaStream_t s);                                \
  KNET_API void addcols_##S(int xrows, int xcols, int ncols, const int *cols, T *x, const T *y); \
  KNET_API void addcols_##S##_stream(int xrows, int xcols, int ncols, const int *cols, T *x,     \
                                     const T *y, cudaStream_t s);                                \
  KNET_API void setcol1_##S(int xrows, int xcols, int ncols, const int *cols, T *x, T y);        \
  KNET_API void setcol1_##S##_stream(int xrows, int xcols, int ncols, const int *cols, T *x,     \
                                     T y, cudaStream_t s);                                       \
  KNET_API void getrows_##S(int xrows, int xcols, int nrows, const int *rows, const T *x, T *y); \
  KNET_API void getrows_##S##_stream(int xrows, int xcols, int nrows, const int *rows,           \
                                     const T *x, T *y, cudaStream_t s);                          \
  KNET_API void setrows_##S(int xrows, int xcols, int nrows, const int *rows, T *x, const T *y); \
  KNET_API void setrows_##S##_stream(int xrows, int xcols, int nrows, const int *rows, T *x,     \
                                     const T *y, cudaStream_t s);                                \
  KNET_API void addrows_##S(int xrows, int xcols, int nrows, const int *rows, T *x, const T *y); \
  KNET_API void addrows_##S##_stream(int xrows, int xcols, int nrows, const int *rows, T *x,     \
                                     const T *y, cudaStream_t s);                                \
  KNET_API void setrow1_##S(int xrows, int xcols, int nrows, const int *rows, T *x, T y);        \
  KNET_API void setrow1_##S##_stream(int xrows, int xcols, int nrows, const int *rows, T *x,     \
                                     T y, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_COLSROWS, colsrows)

/* Pitched 2-d block moves behind range indexing A[i1:i2, j1:j2].  xcopy moves ncols runs of
 * nrows BYTES, run c from x + c*incx to y + c*incy (pitches in bytes); xfill stores the
 * scalar into ncols runs of nrows ELEMENTS with pitch incy elements.  Replace
 * src/libknet8/cuda1.jl:108-165; callers src/knetarrays/getindex.jl:645-703. */
KNET_API void xcopy(int nrows, int ncols, const void *x, int incx, void *y, int incy);
KNET_API void xcopy_stream(int nrows, int ncols, const void *x, int incx, void *y, int incy,
                           cudaStream_t s);
#define KNET_DECL_XFILL(f, S, T)                                                     \
  KNET_API void xfill_##S(int nrows, int ncols, T x, T *y, int incy);                \
  KNET_API void xfill_##S##_stream(int nrows, int ncols, T x, T *y, int incy, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_XFILL, xfill)

/* Concatenate ncols device vectors of nrows elements into the columns of y (nrows, ncols);
 * x is a HOST array of ncols device pointers.  The pointers travel in kernel parameters, a
 * group per launch, so nothing is allocated or copied (the reference cudaMallocs a pointer
 * table per call).  Replaces icat_S, src/libknet8/cuda1.jl:168-214. */
#define KNET_DECL_ICAT(f, S, T)                                               \
  KNET_API void icat_##S(int nrows, int ncols, T **x, T *y);                  \
  KNET_API void icat_##S##_stream(int nrows, int ncols, T **x, T *y, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_ICAT, icat)

/* =====================================================================================
 * B. Fused entry points (int status).  "dims" geometry: the array is seen as
 * (inner, D, outer), element (a,d,c) at a + inner*(d + D*c), and the op runs over d.
 * A (C,B) matrix with dims=1 is (1,C,B); with dims=2 it is (C,B,1).
 * ===================================================================================== */

/* softmax / logsoftmax forward and backward over one dim, in place allowed (y may be x,
 * dx may be dy).  Replace cudnnSoftmaxForward/Backward and the two geam transposes of the
 * dims=2 case, src/ops20_gpu/softmax.jl:10-59; math of src/ops20/softmax.jl:42-63. */
#define KNET_DECL_SOFTMAX(f, S, T)                                                           \
  KNET_API int knet_softmax_fwd_##S(const T *x, T *y, int64_t inner, int64_t D,              \
                                    int64_t outer, cudaStream_t s);                          \
  KNET_API int knet_logsoftmax_fwd_##S(const T *x, T *y, int64_t inner, int64_t D,           \
                                       int64_t outer, cudaStream_t s);                       \
  KNET_API int knet_softmax_bwd_##S(const T *y, const T *dy, T *dx, int64_t inner,           \
                                    int64_t D, int64_t outer, cudaStream_t s);               \
  KNET_API int knet_logsoftmax_bwd_##S(const T *y, const T *dy, T *dx, int64_t inner,        \
                                       int64_t D, int64_t outer, cudaStream_t s);            \
  /* y[a,c] = log sum_d exp(x[a,d,c]); dx = dy[a,c]*exp(x - y[a,c]).  Replaces the six-   */ \
  /* kernel generic path of src/ops20/softmax.jl:65-74.                                    */ \
  KNET_API int knet_logsumexp_fwd_##S(const T *x, T *y, int64_t inner, int64_t D,            \
                                      int64_t outer, cudaStream_t s);                        \
  KNET_API int knet_logsumexp_bwd_##S(const T *x, const T *y, const T *dy, T *dx,            \
                                      int64_t inner, int64_t D, int64_t outer, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_SOFTMAX, softmax)

/* nll(scores, labels; dims) on a (R,K) score matrix: classes along dim `dims` (1 or 2),
 * labels 1-based Int32 on the device, 0 = skip the instance.
 * fwd: *total = -sum of logsoftmax at the label entries, *count = instances used;
 *      `per_instance` is caller scratch of one T per instance (it receives each
 *      instance's -log p).  Replaces findindices + logsoftmax + getents + sum_S_20,
 *      src/ops20/loss.jl:37-41,116-140.
 * bwd: dscores = (softmax(scores) - onehot(label)) * scale on used instances, 0 on skipped
 *      ones, where scale = dy/(*count) if average else dy; `count` is the device value
 *      fwd wrote (ignored if average == 0).  Replaces addents_S + cudnnSoftmaxBackward,
 *      src/autograd_gpu/getindex.jl:5-18, addto.jl:59-65, ops20_gpu/softmax.jl:51-58. */
#define KNET_DECL_NLL(f, S, T)                                                                \
  KNET_API int knet_nll_fwd_##S(const T *scores, const int32_t *labels, int64_t R, int64_t K, \
                                int dims, T *total, int32_t *count, T *per_instance,          \
                                cudaStream_t s);                                              \
  KNET_API int knet_nll_bwd_##S(const T *scores, const int32_t *labels, int64_t R, int64_t K, \
                                int dims, int average, T dy, const int32_t *count,            \
                                T *dscores, cudaStream_t s);                                  \
  /* 1-based position of the first maximum along d (Julia findmax/argmax); replaces the   */  \
  /* host copy of src/knetarrays/reduction.jl:92-96.                                      */  \
  KNET_API int knet_argmax_##S(const T *x, int32_t *idx, int64_t inner, int64_t D,            \
                               int64_t outer, cudaStream_t s);                                \
  /* result[0] = instances whose argmax equals the label, result[1] = instances used;     */  \
  /* replaces the host computation of src/ops20/loss.jl:54-62.                            */  \
  KNET_API int knet_accuracy_##S(const T *scores, const int32_t *labels, int64_t R,           \
                                 int64_t K, int dims, int32_t *result, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_NLL, nll)

/* Whole-array reduction to a device scalar without a synchronisation or an allocation.
 * op: 0 sum 1 prod 2 maximum 3 minimum 4 sumabs 5 sumabs2 6 maxabs 7 minabs 8 countnz.
 * `workspace` is caller scratch of knet_reduce_workspace_bytes() bytes, 256-byte aligned;
 * calls that share a workspace must be ordered on one stream.  The stream-ordered form
 * of {f}_S_20 (src/libknet8/cuda20.jl:83-104). */
KNET_API size_t knet_reduce_workspace_bytes(void);
#define KNET_DECL_REDUCE_DEV(f, S, T)                                                      \
  KNET_API int knet_reduce_##S(int op, int64_t n, const T *x, T *result, void *workspace,  \
                               size_t workspace_bytes, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_REDUCE_DEV, reduce)

/* knet_reduce_32 for callers that can neither lend a workspace nor let the library allocate
 * one (a runtime whose own memory pool owns the GPU, a loop that allocates nothing after
 * start-up): same ops, same result, with the partial results kept in a 4 KiB array that is
 * part of the library image on every GPU.  It has no counterpart in libknet8.
 * Limits and rules: n <= KNET_REDUCE_NOALLOC_MAX_N, else KNET_ESIZE; Float32 only; the
 * array is shared by all calls on a device, so calls that may overlap on the GPU (different
 * streams without ordering) must not be issued; the first call on each device looks up the
 * array's address and should happen before any stream capture begins.  The call itself
 * allocates nothing and synchronises nothing. */
#define KNET_REDUCE_NOALLOC_MAX_N 2147483647
KNET_API int knet_reduce_noalloc_32(int op, int64_t n, const float *x, float *result,
                                    cudaStream_t s);

/* Dropout with an in-kernel counter-based generator (Philox4x32-10 keyed by seed): a counter
 * yields 32 bytes of output, so element i uses counter offset + i/8 for Float32 (16 random
 * bits per element, u = bits * 2^-16) and offset + i/4 for Float64 (32 bits, u = word * 2^-32);
 * a call over n elements consumes ceil(n/8) resp. ceil(n/4) counters.
 * y = u>p ? x/(1-p) : 0 with u in [0,1).  Saves the separate rand! pass of
 * src/ops20_gpu/dropout.jl:12-17.  knet_dropout_uniform_S writes the same uniforms, so that a
 * mask can be reproduced. */
#define KNET_DECL_PHILOX(f, S, T)                                                            \
  KNET_API int knet_dropout_philox_##S(int64_t n, T p, uint64_t seed, uint64_t offset,       \
                                       const T *x, T *y, cudaStream_t s);                    \
  KNET_API int knet_dropout_uniform_##S(int64_t n, uint64_t seed, uint64_t offset, T *u,     \
                                        cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_PHILOX, philox)

/* Fused layer pieces for y = dropout(relu(z .+ b)) on a (N,B) column-major z, b of N:
 * fwd writes y (z may be y) with the generator above; p == 0 leaves dropout out.
 * bwd: dz = reluback(dropback(dy)) from y alone: dz = y==0 ? 0 : dy/(1-p), because y == 0
 *      marks an element that was dropped or clipped.  Replace add_S_12 + relu_S + rand! +
 *      dropout_S and dropback_S + reluback_S_11 (call stack of src/train20/train.jl:26).
 * bias_bwd: the same dz (which may be the dy buffer) and, in the same pass, the bias
 *      gradient db[r] = sum over the B columns of dz[r,:] (deterministic order); replaces
 *      dropback_S + reluback_S_11 followed by sum_S_21 with sy == 1
 *      (src/ops20/dropout.jl:29-42, src/ops20/activation.jl:28,
 *      src/knetarrays/reduction.jl:42-57 -> src/libknet8/cuda21.jl:32-36).  B == 0 gives db = 0. */
#define KNET_DECL_LAYER(f, S, T)                                                             \
  KNET_API int knet_bias_relu_dropout_fwd_##S(const T *z, const T *b, T *y, int64_t N,       \
                                              int64_t B, T p, uint64_t seed, uint64_t offset, \
                                              cudaStream_t s);                               \
  KNET_API int knet_relu_dropout_bwd_##S(const T *y, const T *dy, T *dz, int64_t n, T p,     \
                                         cudaStream_t s);                                    \
  KNET_API int knet_relu_dropout_bias_bwd_##S(const T *y, const T *dy, T *dz, T *db,         \
                                              int64_t N, int64_t B, T p, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_LAYER, layer)

/* update!(w, g, opt) in one pass, in Knet's CPU operation order (src/train20/update.jl:
 * 513-570): a Float64 factor times a state array is formed in Float64 and rounded (lmul!),
 * axpy! is one fused multiply-add with the factor rounded to T, "/" is a true division.
 * Hyper-parameters are passed as double, exactly as the optimizer structs hold them.
 * `gscale` multiplies g on load when it is not 1 (the 1/world factor of a data-parallel
 * mean).  `t` is Adam's step count after its increment (1 on the first call).
 * Replace the cublasSaxpy/Sscal + broadcast chains of update.jl:513-570. */
#define KNET_DECL_OPT(f, S, T)                                                                \
  KNET_API int knet_sgd_##S(int64_t n, T *w, const T *g, double lr, double gscale,            \
                            cudaStream_t s);                                                  \
  KNET_API int knet_momentum_##S(int64_t n, T *w, const T *g, T *v, double lr, double gamma,  \
                                 double gscale, cudaStream_t s);                              \
  KNET_API int knet_nesterov_##S(int64_t n, T *w, const T *g, T *v, double lr, double gamma,  \
                                 double gscale, cudaStream_t s);                              \
  KNET_API int knet_adagrad_##S(int64_t n, T *w, const T *g, T *G, double lr, double eps,     \
                                double gscale, cudaStream_t s);                               \
  KNET_API int knet_rmsprop_##S(int64_t n, T *w, const T *g, T *G, double lr, double rho,     \
                                double eps, double gscale, cudaStream_t s);                   \
  KNET_API int knet_adadelta_##S(int64_t n, T *w, const T *g, T *G, T *delta, double lr,      \
                                 double rho, double eps, double gscale, cudaStream_t s);      \
  KNET_API int knet_adam_##S(int64_t n, T *w, const T *g, T *m, T *v, double lr,              \
                             double beta1, double beta2, double eps, int t, double gscale,    \
                             cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_OPT, opt)

/* Multi-tensor forms: one launch updates every array of a parameter set.  `table` is a
 * device array of `ntensors` descriptors; p[] = {w, g, state1, state2} (unused entries
 * null); first_chunk[i] = sum over j<i of ceil(n[j]/KNET_MULTI_CHUNK), and total_chunks is
 * that sum over all tensors.  knet_multi_plan fills first_chunk on the host and returns
 * total_chunks.  Replace the per-Param loop of src/train20/train.jl:27-32. */
#define KNET_MULTI_CHUNK 8192
typedef struct knet_tensor_desc {
  void *p[4];
  int64_t n;
  int64_t first_chunk;
} knet_tensor_desc;
KNET_API int64_t knet_multi_plan(knet_tensor_desc *host_table, int ntensors);
#define KNET_DECL_MULTI(f, S, T)                                                               \
  KNET_API int knet_sgd_multi_##S(const knet_tensor_desc *table, int ntensors,                 \
                                  int64_t total_chunks, double lr, double gscale,              \
                                  cudaStream_t s);                                             \
  KNET_API int knet_momentum_multi_##S(const knet_tensor_desc *table, int ntensors,            \
                                       int64_t total_chunks, double lr, double gamma,          \
                                       double gscale, cudaStream_t s);                         \
  KNET_API int knet_adam_multi_##S(const knet_tensor_desc *table, int ntensors,                \
                                   int64_t total_chunks, double lr, double beta1,              \
                                   double beta2, double eps, int t, double gscale,             \
                                   cudaStream_t s);                                            \
  /* Adam for a captured CUDA graph: the only step-dependent scalars, 1 - beta1^t and      */  \
  /* 1 - beta2^t, are read from bias_corr[0..1] in device memory when the kernel runs.     */  \
  /* knet_adam_bias_corr_S computes them on the host exactly as knet_adam_multi_S does, so */  \
  /* a copy node fed from pinned host memory keeps replays bit-identical to eager steps.   */  \
  KNET_API int knet_adam_multi_g_##S(const knet_tensor_desc *table, int ntensors,              \
                                     int64_t total_chunks, double lr, double beta1,            \
                                     double beta2, double eps, const T *bias_corr,             \
                                     double gscale, cudaStream_t s);                           \
  KNET_API void knet_adam_bias_corr_##S(double beta1, double beta2, int t, T *host_out);        \
  /* Per-array gradient clipping (gclip!, src/train20/update.jl:572-583) without the host     */ \
  /* round trip of norm(g): knet_gclip_factors_S writes factors[i] = gclip / norm_i when      */ \
  /* norm_i = |gscale| * sqrt(sum g_i^2) exceeds gclip and 1 otherwise (two launches, fixed    */ \
  /* summation order; `partials` is scratch of total_chunks elements), and the _c forms of    */ \
  /* the multi-tensor updates replace g on load by lmul!(factors[i], g).  The norm is summed  */ \
  /* per 8192-element chunk, so it can differ from sumabs2_S_20's in the last bits.           */ \
  KNET_API int knet_gclip_factors_##S(const knet_tensor_desc *table, int ntensors,              \
                                      int64_t total_chunks, double gclip, double gscale,        \
                                      T *partials, double *factors, cudaStream_t s);            \
  KNET_API int knet_sgd_multi_c_##S(const knet_tensor_desc *table, int ntensors,                \
                                    int64_t total_chunks, double lr, double gscale,             \
                                    const double *factors, cudaStream_t s);                     \
  KNET_API int knet_momentum_multi_c_##S(const knet_tensor_desc *table, int ntensors,           \
                                         int64_t total_chunks, double lr, double gamma,         \
                                         double gscale, const double *factors, cudaStream_t s); \
  KNET_API int knet_adam_multi_c_##S(const knet_tensor_desc *table, int ntensors,               \
                                     int64_t total_chunks, double lr, double beta1,             \
                                     double beta2, double eps, int t, double gscale,            \
                                     const double *factors, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_MULTI, multi)

/* =====================================================================================
 * C. Data-parallel collectives (one process per GPU; NCCL over NVLink, loaded at run time).
 * Knet has no multi-GPU path, so these have no counterpart in the reference: they are what a
 * Julia host needs around update! (src/train20/train.jl:27-32) to run the batch-sharded
 * step, without an NCCL binding of its own.  All return the status codes above; positive
 * values here are 1000 + the ncclResult_t.  KN -5 = NCCL could not be loaded.
 *
 *   rank 0:   knet_dp_unique_id(id)          then hands the 128 bytes to the other ranks
 *   all:      knet_dp_init(id, rank, world, timeout_ms, &comm)   after cudaSetDevice
 *   per step: knet_dp_allreduce_sum_S(comm, buf, n, stream)                (in place)
 *             or knet_dp_reduce_scatter_sum_S / knet_dp_allgather_S for a sharded update
 *   end:      knet_dp_destroy(comm)
 *
 * The communicator is created non-blocking and every call polls with a host deadline
 * (timeout_ms of knet_dp_init): a peer that never joins makes the call return -6 (timeout)
 * after aborting the communicator; it never hangs the host.
 * ===================================================================================== */
#define KNET_DP_ID_BYTES 128
KNET_API int knet_dp_unique_id(void *id128);
KNET_API int knet_dp_init(const void *id128, int rank, int world, int timeout_ms, void **comm);
KNET_API int knet_dp_rank(void *comm);
KNET_API int knet_dp_world(void *comm);
KNET_API int knet_dp_destroy(void *comm);
#define KNET_DECL_DP(f, S, T)                                                                    \
  KNET_API int knet_dp_allreduce_sum_##S(void *comm, T *buf, int64_t n, cudaStream_t s);         \
  KNET_API int knet_dp_reduce_scatter_sum_##S(void *comm, const T *send, T *recv,                \
                                              int64_t n_per_rank, cudaStream_t s);               \
  KNET_API int knet_dp_allgather_##S(void *comm, const T *send, T *recv, int64_t n_per_rank,     \
                                     cudaStream_t s);                                            \
  KNET_API int knet_dp_broadcast_##S(void *comm, T *buf, int64_t n, int root, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_DP, dp)

/* =====================================================================================
 * Section D - matrix products.  Replaces the cuBLAS calls of gemm!(transA, transB, alpha,
 * A, B, beta, C) for KnetArray (src/knetarrays/linalg.jl:27-55: cublasSgemm_v2 /
 * cublasDgemm_v2 through CUDA.jl), which serve `*`, A_mul_Bt and At_mul_B (linalg.jl:11-17).
 * Column-major: C (m,n) = alpha * op(A) (m,k) * op(B) (k,n) + beta * C; transX is 0 for 'N'
 * and 1 for 'T'; ldX are leading dimensions in elements.  The products are cuBLAS kernels
 * (cuBLAS is opened with dlopen when the first handle is created; KNET_SM100_CUBLAS_LIB
 * names another copy); a handle belongs to the host thread and device that created it,
 * like CUDA.jl's task-local CUBLAS.handle().
 *
 * mode (Float32 only; Float64 takes 0):
 *   0  plain FP32 arithmetic, what the reference runs;
 *   1  cuBLAS's FP32 emulation on the BF16 tensor cores (each operand split into three
 *      BF16 terms, nine partial products accumulated in FP32), used whenever cuBLAS can;
 *   2  the same, leaving the choice per call to cuBLAS's own heuristics.
 * Modes 1 and 2 need cuBLAS 12.9 or later and answer KNET_EUNSUPPORTED otherwise.
 * workspace is optional scratch for cuBLAS (256-byte aligned; NULL and 0 keep the handle's
 * own), which must outlive the work enqueued with it.  Errors: negative as above, cuBLAS's
 * status r as 2000 + r.
 * ===================================================================================== */
KNET_API int knet_gemm_create(void **handle);
KNET_API int knet_gemm_destroy(void *handle);
KNET_API int knet_gemm_version(void *handle);   /* cublasGetVersion: 10000*major + 100*minor + patch */
KNET_API int knet_gemm_emulation(void *handle); /* 1 when modes 1 and 2 are offered, else 0 */
#define KNET_DECL_GEMM(f, S, T)                                                                  \
  KNET_API int knet_gemm_##S##_S(void *handle, int transA, int transB, int64_t m, int64_t n,     \
                                 int64_t k, T alpha, const T *A, int64_t lda, const T *B,        \
                                 int64_t ldb, T beta, T *C, int64_t ldc, int mode,               \
                                 void *workspace, size_t workspace_bytes, cudaStream_t s);
KNET_BOTH_TYPES(KNET_DECL_GEMM, gemm)

/* Library identification: the compute capability the kernels were built for (100). */
KNET_API int knet_sm100_arch(void);

/* Waits inside the kernels (on bulk copies into shared memory) are bounded; one that gives
 * up sets a sticky device flag and the kernel carries on to its end.  Returns 1 and clears
 * the flag if that happened since the last call, 0 if not, -1 if the flag cannot be read.
 * Synchronises the device.  libknet8 has no counterpart: its kernels never wait. */
KNET_API int knet_device_status(void);

/* Exercises that mechanism without a fault: a one-CTA kernel announces 32 bytes on an mbarrier
 * and copies 16, so its first wait (limited to `spins` polls, 1..2^20) gives up and raises the
 * flag; the kernel then completes the barrier itself, sees its copy land and returns.
 * out6 (device): {first wait gave up, second wait completed, the 4 copied words 11,22,33,44}.
 * For tests and for a host that wants to check the status path at start-up; no counterpart
 * in libknet8. */
KNET_API int knet_debug_wait_probe(uint32_t spins, uint32_t *out6, cudaStream_t s);

#ifdef __cplusplus
}
#endif
#endif /* KNET_SM100_H */
