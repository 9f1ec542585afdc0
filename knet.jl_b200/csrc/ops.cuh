// Scalar definitions of every pointwise op, one struct per symbol stem, shared by the
// same-size, scalar-operand and broadcast kernels.  The expressions follow Knet's CPU
// definitions (src/ops20/activation.jl, src/ops21/activation.jl) where those exist and the
// op table (src/libknet8/ops.jl) otherwise.  The library is compiled with -fmad=false, so
// a*b+c below is two roundings unless it is written as an explicit fma.
#pragma once
#include "math.cuh"

namespace kn {
namespace op {

#define KN_UNARY(name, expr)                                          \
  template <typename T> struct U_##name {                             \
    __device__ __forceinline__ T operator()(T xi) const { return expr; } \
  };

// helpers that pick the float or double flavour of a libm function
#define KN_LIBM1(fn)                                                              \
  __device__ __forceinline__ float m_##fn(float x) { return ::fn##f(x); }         \
  __device__ __forceinline__ double m_##fn(double x) { return ::fn(x); }
KN_LIBM1(acos) KN_LIBM1(acosh) KN_LIBM1(asin) KN_LIBM1(asinh) KN_LIBM1(atan) KN_LIBM1(atanh)
KN_LIBM1(cbrt) KN_LIBM1(ceil) KN_LIBM1(cos) KN_LIBM1(cosh) KN_LIBM1(cospi) KN_LIBM1(erf)
KN_LIBM1(erfc) KN_LIBM1(erfcinv) KN_LIBM1(erfcx) KN_LIBM1(erfinv) KN_LIBM1(exp10) KN_LIBM1(exp2)
KN_LIBM1(expm1) KN_LIBM1(floor) KN_LIBM1(j0) KN_LIBM1(j1) KN_LIBM1(tgamma) KN_LIBM1(lgamma)
KN_LIBM1(log10) KN_LIBM1(log1p) KN_LIBM1(log2) KN_LIBM1(rint) KN_LIBM1(sin) KN_LIBM1(sinh)
KN_LIBM1(sinpi) KN_LIBM1(tan) KN_LIBM1(trunc) KN_LIBM1(y0) KN_LIBM1(y1)
#undef KN_LIBM1
__device__ __forceinline__ float m_pow(float a, float b) { return ::powf(a, b); }
__device__ __forceinline__ double m_pow(double a, double b) { return ::pow(a, b); }

// digamma and trigamma (ops.jl:37-38; the CPU path is SpecialFunctions.jl): the classical scheme -
// reflection for x < 0, the recurrence f(x) = f(x+1) -/+ 1/x^k up to x >= 10, then the
// asymptotic series in 1/x^2 with Bernoulli-number coefficients, evaluated in the array's type.
// Poles: digamma(0) = -inf, NaN at the negative integers; trigamma = +inf at every pole.
template <typename T> __device__ __forceinline__ T pi_v() { return (T)3.14159265358979323846; }
template <typename T> __device__ T digamma_t(T x) {
  T refl = (T)0;
  if (x <= (T)0) {
    if (x == (T)0) return -Math<T>::inf();
    const T f = x - m_floor(x);
    if (f == (T)0) return (T)NAN;
    // psi(x) = psi(1-x) - pi/tan(pi x); tan(pi x) from the fractional part, nearest integer removed
    const T g = f > (T)0.5 ? f - (T)1 : f;
    refl = g == (T)0.5 ? (T)0 : -pi_v<T>() / m_tan(pi_v<T>() * g);
    x = (T)1 - x;
  }
  T acc = (T)0;
  while (x < (T)10) {
    acc -= (T)1 / x;
    x += (T)1;
  }
  const T z = (T)1 / (x * x);
  // sum_{k>=1} B_2k / (2k x^2k): 1/12, -1/120, 1/252, -1/240, 1/132, -691/32760, 1/12
  T s;
  if (sizeof(T) == 4) {
    s = z * ((T)(1.0 / 12) + z * ((T)(-1.0 / 120) + z * ((T)(1.0 / 252) + z * (T)(-1.0 / 240))));
  } else {
    s = z * ((T)(1.0 / 12) + z * ((T)(-1.0 / 120) + z * ((T)(1.0 / 252) + z * ((T)(-1.0 / 240) + z * ((T)(1.0 / 132) +
        z * ((T)(-691.0 / 32760) + z * (T)(1.0 / 12)))))));
  }
  return Math<T>::log(x) - (T)0.5 / x - s + acc + refl;
}
template <typename T> __device__ T trigamma_t(T x) {
  T refl = (T)0, sign = (T)1;
  if (x <= (T)0) {
    const T f = x - m_floor(x);
    if (f == (T)0) return Math<T>::inf();
    // psi1(x) = pi^2 / sin^2(pi x) - psi1(1-x)
    const T sn = m_sinpi(f);
    refl = pi_v<T>() * pi_v<T>() / (sn * sn);
    sign = (T)-1;
    x = (T)1 - x;
  }
  T acc = (T)0;
  while (x < (T)10) {
    acc += (T)1 / (x * x);
    x += (T)1;
  }
  const T r = (T)1 / x, z = r * r;
  // 1/x + 1/(2x^2) + sum_{k>=1} B_2k / x^(2k+1): 1/6, -1/30, 1/42, -1/30, 5/66, -691/2730, 7/6
  T s;
  if (sizeof(T) == 4) {
    s = (T)(1.0 / 6) + z * ((T)(-1.0 / 30) + z * ((T)(1.0 / 42) + z * (T)(-1.0 / 30)));
  } else {
    s = (T)(1.0 / 6) + z * ((T)(-1.0 / 30) + z * ((T)(1.0 / 42) + z * ((T)(-1.0 / 30) + z * ((T)(5.0 / 66) +
        z * ((T)(-691.0 / 2730) + z * (T)(7.0 / 6))))));
  }
  const T tail = r + (T)0.5 * z + r * z * s;
  return refl + sign * (tail + acc);
}

KN_UNARY(abs2, xi * xi)
KN_UNARY(abs, (xi < 0 ? -xi : xi))
KN_UNARY(acos, m_acos(xi))
KN_UNARY(acosh, m_acosh(xi))
KN_UNARY(asin, m_asin(xi))
KN_UNARY(asinh, m_asinh(xi))
KN_UNARY(atan, m_atan(xi))
KN_UNARY(atanh, m_atanh(xi))
KN_UNARY(cbrt, m_cbrt(xi))
KN_UNARY(ceil, m_ceil(xi))
KN_UNARY(cos, m_cos(xi))
KN_UNARY(cosh, m_cosh(xi))
KN_UNARY(cospi, m_cospi(xi))
KN_UNARY(erf, m_erf(xi))
KN_UNARY(erfc, m_erfc(xi))
KN_UNARY(erfcinv, m_erfcinv(xi))
KN_UNARY(erfcx, m_erfcx(xi))
KN_UNARY(erfinv, m_erfinv(xi))
KN_UNARY(exp, Math<T>::exp(xi))
KN_UNARY(exp10, m_exp10(xi))
KN_UNARY(exp2, m_exp2(xi))
KN_UNARY(expm1, m_expm1(xi))
KN_UNARY(floor, m_floor(xi))
KN_UNARY(j0, m_j0(xi))
KN_UNARY(j1, m_j1(xi))
KN_UNARY(gamma_impl, m_tgamma(xi))
KN_UNARY(digamma_impl, digamma_t<T>(xi))
KN_UNARY(trigamma_impl, trigamma_t<T>(xi))
KN_UNARY(lgamma, m_lgamma(xi))
KN_UNARY(log, Math<T>::log(xi))
KN_UNARY(log10, m_log10(xi))
KN_UNARY(log1p, m_log1p(xi))
KN_UNARY(log2, m_log2(xi))
KN_UNARY(neg, -xi)
KN_UNARY(one, (T)1)
KN_UNARY(round, m_rint(xi))  // Julia's round: ties to even
KN_UNARY(sign, (xi > 0 ? (T)1 : xi < 0 ? (T)-1 : xi))
KN_UNARY(sin, m_sin(xi))
KN_UNARY(sinh, m_sinh(xi))
KN_UNARY(sinpi, m_sinpi(xi))
KN_UNARY(sqrt, Math<T>::sqrt(xi))
KN_UNARY(tan, m_tan(xi))
KN_UNARY(tanh, Math<T>::tanh(xi))
KN_UNARY(tanh_, Math<T>::tanh(xi))
KN_UNARY(trunc, m_trunc(xi))
KN_UNARY(y0, m_y0(xi))
KN_UNARY(y1, m_y1(xi))
KN_UNARY(zero, (T)0)
KN_UNARY(invx, (T)1 / xi)
// elu(x) = x >= 0 ? x : exp(x)-1, with the cancellation (src/ops20/activation.jl:12)
KN_UNARY(elu, (xi >= 0 ? xi : Math<T>::exp(xi) - (T)1))
// gelu, hardsigmoid, hardswish, swish: src/ops21/activation.jl, ops.jl:74-80
KN_UNARY(gelu, (T)0.5 * xi * ((T)1 + m_erf(xi / (T)1.4142135623730951)))
KN_UNARY(hardsigmoid, (xi <= -3 ? (T)0 : xi >= 3 ? (T)1 : (xi + 3) / 6))
KN_UNARY(hardswish, (xi <= -3 ? (T)0 : xi >= 3 ? xi : xi * (xi + 3) / 6))
// relu(x) = max(x,0): NaN propagates, -0 gives +0 (src/ops20/activation.jl:26)
KN_UNARY(relu, (xi > 0 ? xi : (xi != xi ? xi : (T)0)))
// selu (src/ops20/activation.jl:39)
KN_UNARY(selu, (xi >= 0 ? (T)1.0507009873554805 * xi
                        : (T)1.7580993408473773 * (Math<T>::exp(xi) - (T)1)))
#undef KN_UNARY

// Float32 elu and selu: only the non-positive side needs exp, so its argument is min(x, 0)
// (one clamp, no branch on NaN; NaN is patched in at the end) - the kernels are bound by
// instruction issue, not by HBM.
template <> struct U_elu<float> {
  __device__ __forceinline__ float operator()(float xi) const {
    const float z = exp_cr_nonpos(fminf(xi, 0.0f));
    const float y = xi >= 0.0f ? xi : z - 1.0f;
    return xi != xi ? xi : y;
  }
};
template <> struct U_selu<float> {
  __device__ __forceinline__ float operator()(float xi) const {
    const float z = exp_cr_nonpos(fminf(xi, 0.0f));
    const float y = xi >= 0.0f ? 1.0507009873554805f * xi : 1.7580993408473773f * (z - 1.0f);
    return xi != xi ? xi : y;
  }
};

// sigm(x) = x>=0 ? 1/(1+exp(-x)) : (z=exp(x); z/(1+z))  (src/ops20/activation.jl:55).
// Both branches need exp(-|x|), so it is evaluated once.
template <typename T> struct U_sigm {
  __device__ __forceinline__ T operator()(T xi) const {
    if (xi != xi) return xi;
    const T z = Math<T>::exp(xi >= 0 ? -xi : xi);
    const T num = xi >= 0 ? (T)1 : z;  // one division serves both branches
    return num / ((T)1 + z);
  }
};
// Float32: the kernel is bound by instruction issue, not by HBM, so the same arithmetic is
// spelled with fewer instructions: exp of -|x| needs one clamp, and the quotient of a value
// in [0,1] by one in [1,2] needs no range checks.
template <> struct U_sigm<float> {
  __device__ __forceinline__ float operator()(float xi) const {
    const float z = exp_cr_nonpos_nan(-fabsf(xi));     // NaN stays NaN through everything below
    const float num = xi >= 0.0f ? 1.0f : z;
    return div_rn_inrange(num, 1.0f + z);
  }
};
template <typename T> struct U_swish {
  __device__ __forceinline__ T operator()(T xi) const {
    if (xi != xi) return xi;
    const T z = Math<T>::exp(xi >= 0 ? -xi : xi);
    return xi >= 0 ? xi / ((T)1 + z) : xi * z / ((T)1 + z);
  }
};

// ---- binary -------------------------------------------------------------------------------
#define KN_BINARY(name, expr)                                                \
  template <typename T> struct B_##name {                                    \
    __device__ __forceinline__ T operator()(T xi, T yi) const { return expr; } \
  };
KN_BINARY(add, xi + yi)
KN_BINARY(sub, xi - yi)
KN_BINARY(mul, xi * yi)
KN_BINARY(div, xi / yi)
KN_BINARY(pow, m_pow(xi, yi))
KN_BINARY(max, (xi > yi ? xi : yi))
KN_BINARY(min, (xi < yi ? xi : yi))
KN_BINARY(eq, (T)(xi == yi))
KN_BINARY(ne, (T)(xi != yi))
KN_BINARY(gt, (T)(xi > yi))
KN_BINARY(ge, (T)(xi >= yi))
KN_BINARY(lt, (T)(xi < yi))
KN_BINARY(le, (T)(xi <= yi))
// backward forms with xi = dy, yi = y (src/ops20/activation.jl:13,27,40,56;
// src/ops20_gpu/activation.jl:11; geluback/swishback take yi = dy, xi = x as in ops.jl:116,122)
KN_BINARY(invxback, (-xi * yi * yi))
KN_BINARY(eluback, (yi >= 0 ? xi : xi * ((T)1 + yi)))
KN_BINARY(reluback, (yi > 0 ? xi : (T)0))
KN_BINARY(seluback, (yi >= 0 ? xi * (T)1.0507009873554805 : xi * (yi + (T)1.7580993408473773)))
KN_BINARY(sigmback, (xi * yi * ((T)1 - yi)))
KN_BINARY(tanhback, (xi * ((T)1 - yi * yi)))
#undef KN_BINARY

template <typename T> __device__ __forceinline__ T gelu_grad(T x) {
  const T cdf = (T)0.5 * ((T)1 + m_erf(x / (T)1.4142135623730951));
  const T pdf = Math<T>::exp(-x * x / 2) / (T)2.5066282746310002;
  return cdf + x * pdf;
}
template <typename T> __device__ __forceinline__ T swish_grad(T x) {
  if (x >= 0) {
    const T e = Math<T>::exp(-x);
    return (x * e + e + 1) / ((e + 1) * (e + 1));
  }
  const T e = Math<T>::exp(x);
  return e * (e + x + 1) / ((e + 1) * (e + 1));
}
template <typename T> struct B_geluback {
  __device__ __forceinline__ T operator()(T xi, T yi) const { return yi * gelu_grad(xi); }
};
template <typename T> struct B_swishback {
  __device__ __forceinline__ T operator()(T xi, T yi) const { return yi * swish_grad(xi); }
};

// ---- three-argument backward forms g(x, y, dy) (src/ops21/activation.jl; ops.jl:125-136) ----
#define KN_TERNARY(name, expr)                                                   \
  template <typename T> struct T_##name {                                        \
    __device__ __forceinline__ T operator()(T x, T y, T dy) const { return expr; } \
  };
KN_TERNARY(eluback, (y >= 0 ? dy : dy * ((T)1 + y)))
KN_TERNARY(geluback, dy * gelu_grad(x))
KN_TERNARY(hardsigmoidback, dy * (x <= -3 ? (T)0 : x >= 3 ? (T)0 : (T)(1.0 / 6.0)))
KN_TERNARY(hardswishback, dy * (x <= -3 ? (T)0 : x >= 3 ? (T)1 : (x / (T)3 + (T)0.5)))
KN_TERNARY(seluback, (y >= 0 ? (T)1.0507009873554805 * dy : dy * ((T)1.7580993408473773 + y)))
KN_TERNARY(sigmback, (dy * y * ((T)1 - y)))
KN_TERNARY(tanh_back, (dy * ((T)1 - y * y)))
KN_TERNARY(swishback, dy * swish_grad(x))
#undef KN_TERNARY

}  // namespace op
}  // namespace kn
