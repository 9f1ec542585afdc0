// Pointwise entry points: unary ops, scalar-operand and same-size binary ops, activation
// backward forms, relu with keyword arguments, fill, dropout with supplied uniforms, and
// the 1-based entry gather/scatter.  Every kernel is an instance of kn::ew_kernel
// (16-byte streaming loads and stores, several loads in flight per thread).
#include "common.cuh"
#include "ops.cuh"

namespace kn {

template <typename T, typename Op> struct Ew1 {
  Op op;
  __device__ __forceinline__ void operator()(const T (&a)[1], T (&r)[1]) const { r[0] = op(a[0]); }
};
// Float64 exp, sigm, elu, selu: the two exps of a 16-byte group are evaluated together
// (exp_cr64_pair), then Knet's operations in Knet's order as in the scalar functors of ops.cuh.
template <int WHICH> struct Ew1Exp64 {   // 0 exp, 1 sigm, 2 elu, 3 selu
  static constexpr bool kGroup = true;
  static __device__ __forceinline__ double finish(double x, double z) {
    if (WHICH == 0) return z;
    if (WHICH == 1) return x != x ? x : (x >= 0 ? 1.0 : z) / (1.0 + z);
    if (WHICH == 2) return x >= 0 ? x : (x != x ? x : z - 1.0);
    return x >= 0 ? 1.0507009873554805 * x : (x != x ? x : 1.7580993408473773 * (z - 1.0));
  }
  static __device__ __forceinline__ double arg(double x) { return WHICH == 1 ? -fabs(x) : x; }
  __device__ __forceinline__ void operator()(const double (&a)[1], double (&r)[1]) const {
    r[0] = finish(a[0], Math<double>::exp(arg(a[0])));
  }
  template <int VEC>
  __device__ __forceinline__ void group(const Pack<double, VEC> (&in)[1], Pack<double, VEC> (&out)[1]) const {
    if constexpr (VEC == 2) {
      double z0, z1;
      exp_cr64_pair(arg(in[0].v[0]), arg(in[0].v[1]), z0, z1);
      out[0].v[0] = finish(in[0].v[0], z0);
      out[0].v[1] = finish(in[0].v[1], z1);
    } else {        // element-wise kernel for operands that do not share their 16-byte offset
#pragma unroll
      for (int e = 0; e < VEC; e++) out[0].v[e] = finish(in[0].v[e], Math<double>::exp(arg(in[0].v[e])));
    }
  }
};
template <> struct Ew1<double, op::U_exp<double>> : Ew1Exp64<0> {};
template <> struct Ew1<double, op::U_sigm<double>> : Ew1Exp64<1> {};
template <> struct Ew1<double, op::U_elu<double>> : Ew1Exp64<2> {};
template <> struct Ew1<double, op::U_selu<double>> : Ew1Exp64<3> {};

template <typename T, typename Op> struct Ew2 {
  Op op;
  __device__ __forceinline__ void operator()(const T (&a)[2], T (&r)[1]) const { r[0] = op(a[0], a[1]); }
};
template <typename T, typename Op> struct EwS1 {  // scalar first operand
  Op op;
  T xi;
  __device__ __forceinline__ void operator()(const T (&a)[1], T (&r)[1]) const { r[0] = op(xi, a[0]); }
};
// Float32 s ./ y: one special-case test per 16-byte group (div_group, math.cuh).  The same-shape
// x ./ y keeps the compiler's division: with two full-size inputs in flight the group form needs
// more registers than it saves in instructions, and capped at the registers of the other
// two-input kernels it merely equals the compiler's form (both measured).
template <> struct EwS1<float, op::B_div<float>> {
  op::B_div<float> op;
  float xi;
  static constexpr bool kGroup = true;
  __device__ __forceinline__ void operator()(const float (&a)[1], float (&r)[1]) const { r[0] = xi / a[0]; }
  template <int VEC>
  __device__ __forceinline__ void group(const Pack<float, VEC> (&in)[1], Pack<float, VEC> (&out)[1]) const {
    float num[VEC];
#pragma unroll
    for (int e = 0; e < VEC; e++) num[e] = xi;
    div_group<VEC>(num, in[0].v, out[0].v);
  }
};
template <typename T, typename Op> struct Ew3 {
  Op op;
  __device__ __forceinline__ void operator()(const T (&a)[3], T (&r)[1]) const { r[0] = op(a[0], a[1], a[2]); }
};
template <typename T> struct EwFill {
  T x;
  __device__ __forceinline__ void operator()(const T (&)[1], T (&r)[1]) const { r[0] = x; }
};
// relu(x; max_value, negative_slope, threshold), src/ops21/activation.jl, relu.jl:8-15
template <typename T> struct EwRelu1 {
  T maxv, slope, thr;
  __device__ __forceinline__ void operator()(const T (&a)[1], T (&r)[1]) const {
    const T x = a[0];
    r[0] = x >= maxv ? maxv : x >= thr ? x : slope == 0 ? (T)0 : slope * (x - thr);
  }
};
template <typename T> struct EwReluBack1 {  // inputs (x, dy)
  T maxv, slope, thr;
  __device__ __forceinline__ void operator()(const T (&a)[2], T (&r)[1]) const {
    const T x = a[0];
    r[0] = a[1] * (x >= maxv ? (T)0 : x >= thr ? (T)1 : slope);
  }
};
// dropout: inputs (x, u) -> y; Knet's CPU loop divides by q = 1-p (src/ops20/dropout.jl:49-57)
template <typename T> struct EwDropout {
  T p, q;
  __device__ __forceinline__ void operator()(const T (&a)[2], T (&r)[1]) const {
    r[0] = a[1] > p ? a[0] / q : (T)0;
  }
};
template <typename T> struct EwDropback {  // inputs (y, dy) -> dx
  T q;
  __device__ __forceinline__ void operator()(const T (&a)[2], T (&r)[1]) const {
    r[0] = a[0] == (T)0 ? (T)0 : a[1] / q;
  }
};

template <typename T, typename Op> void run_unary(int n, const T* x, T* y, cudaStream_t s) {
  EwPtrs<T, 1, 1> p{{x}, {y}};
  ew_launch<T, 1, 1>(Ew1<T, Op>{}, p, n, s);
}
template <typename T, typename Op> void run_01(int n, T xi, const T* y, T* z, cudaStream_t s) {
  EwPtrs<T, 1, 1> p{{y}, {z}};
  ew_launch<T, 1, 1>(EwS1<T, Op>{Op(), xi}, p, n, s);
}
template <typename T, typename Op> void run_11(int n, const T* x, const T* y, T* z, cudaStream_t s) {
  EwPtrs<T, 2, 1> p{{x, y}, {z}};
  ew_launch<T, 2, 1>(Ew2<T, Op>{Op()}, p, n, s);
}
template <typename T, typename Op>
void run_111(int n, const T* x, const T* y, const T* dy, T* dx, cudaStream_t s) {
  EwPtrs<T, 3, 1> p{{x, y, dy}, {dx}};
  ew_launch<T, 3, 1>(Ew3<T, Op>{Op()}, p, n, s);
}

// ---- entry gather / scatter -------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(256) ents_kernel(int n, const int* __restrict__ ents, T* x, T* y, T y1) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t e = (int64_t)ents[i] - 1;
    if (MODE == 0) y[i] = x[e];
    else if (MODE == 1) x[e] = y[i];
    else if (MODE == 2) atomicAdd(&x[e], y[i]);
    else x[e] = y1;
  }
}
template <typename T, int MODE>
void run_ents(int n, const int* ents, T* x, T* y, T y1, cudaStream_t s) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  ents_kernel<T, MODE><<<blocks, 256, 0, s>>>(n, ents, x, y, y1);
}

}  // namespace kn

using namespace kn;

#define KN_DEF_UNARY(f, S, T)                                                        \
  KN_EXPORT void f##_##S##_stream(int n, const T* x, T* y, cudaStream_t s) {         \
    run_unary<T, op::U_##f<T>>(n, x, y, s);                                          \
  }                                                                                  \
  KN_EXPORT void f##_##S(int n, const T* x, T* y) { f##_##S##_stream(n, x, y, cudaStreamPerThread); }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_UNARY, f)
KNET_UNARY_OPS(KN_X)
#undef KN_X

#define KN_DEF_01(f, S, T)                                                              \
  KN_EXPORT void f##_##S##_01_stream(int n, T xi, const T* y, T* z, cudaStream_t s) {   \
    run_01<T, op::B_##f<T>>(n, xi, y, z, s);                                            \
  }                                                                                     \
  KN_EXPORT void f##_##S##_01(int n, T xi, const T* y, T* z) {                          \
    f##_##S##_01_stream(n, xi, y, z, cudaStreamPerThread);                              \
  }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_01, f)
KNET_BINARY_OPS(KN_X)
#undef KN_X

#define KN_DEF_11(f, S, T)                                                                   \
  KN_EXPORT void f##_##S##_11_stream(int n, const T* x, const T* y, T* z, cudaStream_t s) {  \
    run_11<T, op::B_##f<T>>(n, x, y, z, s);                                                  \
  }                                                                                          \
  KN_EXPORT void f##_##S##_11(int n, const T* x, const T* y, T* z) {                         \
    f##_##S##_11_stream(n, x, y, z, cudaStreamPerThread);                                    \
  }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_11, f)
KNET_BINARY_OPS(KN_X)
KNET_ACTBACK2_OPS(KN_X)
#undef KN_X

#define KN_DEF_111(f, S, T)                                                                  \
  KN_EXPORT void f##_##S##_111_stream(int n, const T* x, const T* y, const T* dy, T* dx,     \
                                      cudaStream_t s) {                                      \
    run_111<T, op::T_##f<T>>(n, x, y, dy, dx, s);                                            \
  }                                                                                          \
  KN_EXPORT void f##_##S##_111(int n, const T* x, const T* y, const T* dy, T* dx) {          \
    f##_##S##_111_stream(n, x, y, dy, dx, cudaStreamPerThread);                              \
  }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_111, f)
KNET_ACTBACK3_OPS(KN_X)
#undef KN_X

#define KN_DEF_MISC(f, S, T)                                                                    \
  KN_EXPORT void relu_##S##_1_stream(int n, T maxv, T slope, T thr, const T* x, T* y,           \
                                     cudaStream_t s) {                                          \
    EwPtrs<T, 1, 1> p{{x}, {y}};                                                                \
    ew_launch<T, 1, 1>(EwRelu1<T>{maxv, slope, thr}, p, n, s);                                  \
  }                                                                                             \
  KN_EXPORT void relu_##S##_1(int n, T maxv, T slope, T thr, const T* x, T* y) {                \
    relu_##S##_1_stream(n, maxv, slope, thr, x, y, cudaStreamPerThread);                        \
  }                                                                                             \
  KN_EXPORT void reluback_##S##_1_stream(int n, T maxv, T slope, T thr, const T* x, const T* y, \
                                         const T* dy, T* dx, cudaStream_t s) {                  \
    (void)y;                                                                                    \
    EwPtrs<T, 2, 1> p{{x, dy}, {dx}};                                                           \
    ew_launch<T, 2, 1>(EwReluBack1<T>{maxv, slope, thr}, p, n, s);                              \
  }                                                                                             \
  KN_EXPORT void reluback_##S##_1(int n, T maxv, T slope, T thr, const T* x, const T* y,        \
                                  const T* dy, T* dx) {                                         \
    reluback_##S##_1_stream(n, maxv, slope, thr, x, y, dy, dx, cudaStreamPerThread);            \
  }                                                                                             \
  KN_EXPORT void fill_##S##_stream(int n, T x, T* y, cudaStream_t s) {                          \
    EwPtrs<T, 0, 1> p{{nullptr}, {y}};                                                          \
    ew_launch<T, 0, 1>(EwFill<T>{x}, p, n, s);                                                  \
  }                                                                                             \
  KN_EXPORT void fill_##S(int n, T x, T* y) { fill_##S##_stream(n, x, y, cudaStreamPerThread); } \
  KN_EXPORT void dropout_##S##_stream(int n, T p, const T* x, T* y, cudaStream_t s) {           \
    EwPtrs<T, 2, 1> pp{{x, y}, {y}};                                                            \
    ew_launch<T, 2, 1>(EwDropout<T>{p, (T)1 - p}, pp, n, s);                                    \
  }                                                                                             \
  KN_EXPORT void dropout_##S(int n, T p, const T* x, T* y) {                                    \
    dropout_##S##_stream(n, p, x, y, cudaStreamPerThread);                                      \
  }                                                                                             \
  KN_EXPORT void dropback_##S##_stream(int n, T p, const T* x, const T* y, const T* dy, T* dx,  \
                                       cudaStream_t s) {                                        \
    (void)x;                                                                                    \
    EwPtrs<T, 2, 1> pp{{y, dy}, {dx}};                                                          \
    ew_launch<T, 2, 1>(EwDropback<T>{(T)1 - p}, pp, n, s);                                      \
  }                                                                                             \
  KN_EXPORT void dropback_##S(int n, T p, const T* x, const T* y, const T* dy, T* dx) {         \
    dropback_##S##_stream(n, p, x, y, dy, dx, cudaStreamPerThread);                             \
  }                                                                                             \
  KN_EXPORT void getents_##S##_stream(int n, const int* e, const T* x, T* y, cudaStream_t s) {  \
    run_ents<T, 0>(n, e, const_cast<T*>(x), y, (T)0, s);                                        \
  }                                                                                             \
  KN_EXPORT void getents_##S(int n, const int* e, const T* x, T* y) {                           \
    getents_##S##_stream(n, e, x, y, cudaStreamPerThread);                                      \
  }                                                                                             \
  KN_EXPORT void setents_##S##_stream(int n, const int* e, T* x, const T* y, cudaStream_t s) {  \
    run_ents<T, 1>(n, e, x, const_cast<T*>(y), (T)0, s);                                        \
  }                                                                                             \
  KN_EXPORT void setents_##S(int n, const int* e, T* x, const T* y) {                           \
    setents_##S##_stream(n, e, x, y, cudaStreamPerThread);                                      \
  }                                                                                             \
  KN_EXPORT void addents_##S##_stream(int n, const int* e, T* x, const T* y, cudaStream_t s) {  \
    run_ents<T, 2>(n, e, x, const_cast<T*>(y), (T)0, s);                                        \
  }                                                                                             \
  KN_EXPORT void addents_##S(int n, const int* e, T* x, const T* y) {                           \
    addents_##S##_stream(n, e, x, y, cudaStreamPerThread);                                      \
  }                                                                                             \
  KN_EXPORT void setent1_##S##_stream(int n, const int* e, T* x, T y, cudaStream_t s) {         \
    run_ents<T, 3>(n, e, x, nullptr, y, s);                                                     \
  }                                                                                             \
  KN_EXPORT void setent1_##S(int n, const int* e, T* x, T y) {                                  \
    setent1_##S##_stream(n, e, x, y, cudaStreamPerThread);                                      \
  }
KNET_BOTH_TYPES(KN_DEF_MISC, misc)

KN_EXPORT int knet_sm100_arch(void) { return 100; }
