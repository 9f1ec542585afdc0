// Correctly rounded Float64 exp.
//
// Knet's sigm, elu, selu and swish feed exp into further roundings (src/ops20/activation.jl:12,39,
// 55), so a 1-ulp difference in exp can become 2 ulp in the result; matching a CPU evaluation to
// 1 ulp therefore needs the same exp on both sides, and the only implementation-independent
// choice is the correctly rounded one.  exp_cr64 returns it:
//
//   fast path   x = k*ln2/64 + r; exp(r) and the table entry 2^(j/64) are carried as unevaluated
//               sums of two doubles, about 27 FP64 instructions, relative error below 2^-66;
//   test        if the two ends of the error interval round to the same double, that is the
//               result (Ziv's test; it fails for about one argument in 800);
//   slow path   the same reduction with a third part of ln2/64 and a double-double Taylor sum,
//               relative error below 2^-100.
//
// Every operation is an IEEE add, multiply or fused multiply-add, so the host build of this
// header (used by the tests as a model of the kernel) gives bit-identical results.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

#include "exp64_table.inc"

#if defined(__CUDACC__)
#define KN_HD __host__ __device__ __forceinline__
// the rare slow path stays out of line, so that it does not weigh on the registers of the fast path
#define KN_HD_SLOW static __host__ __device__ __noinline__
#else
#define KN_HD inline
#define KN_HD_SLOW inline
#endif

namespace kn {
namespace x64 {

#if defined(__CUDACC__)
static __device__ __align__(16) const double kExp64Table[128] = {KN_EXP64_TABLE};
#endif
#if defined(__CUDA_ARCH__)
#define KN_EXP64_T(i) kn::x64::kExp64Table[i]
KN_HD double fma_(double a, double b, double c) { return __fma_rn(a, b, c); }
KN_HD double add_(double a, double b) { return __dadd_rn(a, b); }
KN_HD double mul_(double a, double b) { return __dmul_rn(a, b); }
KN_HD int32_t lo32(double a) { return __double2loint(a); }
KN_HD double scale2(double y, int m) {   // y * 2^m for a normal result
  return __hiloint2double(__double2hiint(y) + m * 1048576, __double2loint(y));
}
#else
static const double kExp64TableHost[128] = {KN_EXP64_TABLE};
#define KN_EXP64_T(i) kn::x64::kExp64TableHost[i]
KN_HD double fma_(double a, double b, double c) { return std::fma(a, b, c); }
KN_HD double add_(double a, double b) { volatile double r = a + b; return r; }
KN_HD double mul_(double a, double b) { volatile double r = a * b; return r; }
KN_HD int32_t lo32(double a) {
  uint64_t u;
  std::memcpy(&u, &a, 8);
  return (int32_t)(uint32_t)u;
}
KN_HD double scale2(double y, int m) {
  uint64_t u;
  std::memcpy(&u, &y, 8);
  u += (uint64_t)(int64_t)m << 52;
  std::memcpy(&y, &u, 8);
  return y;
}
#endif

struct DD {
  double h, l;
};
// s + e = a + b exactly
KN_HD DD two_sum(double a, double b) {
  const double s = add_(a, b), bb = add_(s, -a);
  return DD{s, add_(add_(a, -add_(s, -bb)), add_(b, -bb))};
}
// the same for |a| >= |b|
KN_HD DD fast_two_sum(double a, double b) {
  const double s = add_(a, b);
  return DD{s, add_(b, -add_(s, -a))};
}
KN_HD DD dd_mul(DD a, DD b) {
  const double p = mul_(a.h, b.h);
  double e = fma_(a.h, b.h, -p);
  e = fma_(a.h, b.l, e);
  e = fma_(a.l, b.h, e);
  return fast_two_sum(p, e);
}
KN_HD DD dd_add(DD a, DD b) {   // no cancellation between a and b in this file
  DD s = two_sum(a.h, b.h);
  s.l = add_(s.l, add_(a.l, b.l));
  return fast_two_sum(s.h, s.l);
}

// The reduction shared by both paths: k = round(a * 64/ln2), r1 = a - k*L1 (exact).
struct Reduced {
  double kd, r1, th, tl;
  int m;
};
KN_HD Reduced reduce(double a) {
  const double t = fma_(a, KN_EXP64_INV, 0x1.8p52);   // low bits = round(a * 64/ln2)
  const int32_t k = lo32(t);
  Reduced q;
  q.kd = add_(t, -0x1.8p52);
  q.r1 = fma_(-q.kd, KN_EXP64_L1, a);                 // exact
  q.m = k >> 6;
#if defined(__CUDA_ARCH__)
  const double2 tt = *reinterpret_cast<const double2*>(&kExp64Table[2 * (k & 63)]);   // one 16-byte load
  q.th = tt.x;
  q.tl = tt.y;
#else
  q.th = KN_EXP64_T(2 * (k & 63));
  q.tl = KN_EXP64_T(2 * (k & 63) + 1);
#endif
  return q;
}

// Fast path for -708 <= a <= 709: true and the correctly rounded exp(a) in y when the rounding could
// be decided, false otherwise (y is then only an approximation).  Branch-free, so that several
// arguments can be evaluated side by side.
KN_HD bool exp_cr64_fast(double a, double& y) {
  const Reduced q0 = reduce(a);
  // r = r1 - kd*L2 = rr + dl with rr the nearest double and dl the rest;
  // exp(r) = 1 + rr + [dl + rr^2 (1/2 + rr/6 + ... + rr^6/8!)]
  const double rr = fma_(-q0.kd, KN_EXP64_L2, q0.r1);
  const double dl = fma_(-q0.kd, KN_EXP64_L2, add_(q0.r1, -rr));
  const double rr2 = mul_(rr, rr);
  double P = fma_(rr, KN_EXP64_C8, KN_EXP64_C7H);
  P = fma_(P, rr, KN_EXP64_C6H);
  P = fma_(P, rr, KN_EXP64_C5H);
  P = fma_(P, rr, KN_EXP64_C4H);
  P = fma_(P, rr, KN_EXP64_C3H);
  P = fma_(P, rr, 0.5);
  const double q = fma_(rr2, P, dl);
  const double s_hi = add_(1.0, rr);
  const double s_lo = add_(rr, -add_(s_hi, -1.0));
  const double c = add_(s_lo, q);
  const double p_hi = mul_(q0.th, s_hi);
  double tail = fma_(q0.th, s_hi, -p_hi);
  tail = fma_(q0.th, c, tail);
  tail = fma_(q0.tl, s_hi, tail);
  // the error of p_hi + tail is below 2^-66 p_hi and p_hi < 2.03: if both ends of tail +- 2^-63
  // round to the same double, that double is the correctly rounded result
  const double y1 = add_(p_hi, add_(tail, 0x1p-63)), y2 = add_(p_hi, add_(tail, -0x1p-63));
  y = scale2(y1, q0.m);
  return y1 == y2;
}

// Slow path for the same range: r as a double-double with the third part of ln2/64, Taylor sum in
// double-double; relative error below 2^-100.
KN_HD_SLOW double exp_cr64_slow(double a) {
  const Reduced q0 = reduce(a);
  const double kd = q0.kd;
  const double t2h = mul_(kd, KN_EXP64_L2);
  const double t2l = fma_(kd, KN_EXP64_L2, -t2h);     // kd*L2 = t2h + t2l exactly
  DD r = two_sum(q0.r1, -t2h);
  r.l = add_(r.l, add_(-t2l, -mul_(kd, KN_EXP64_L3)));
  r = fast_two_sum(r.h, r.l);
  double H = fma_(r.h, KN_EXP64_C13, KN_EXP64_C12);   // terms n >= 8 are below 2^-75: plain doubles do
  H = fma_(H, r.h, KN_EXP64_C11);
  H = fma_(H, r.h, KN_EXP64_C10);
  H = fma_(H, r.h, KN_EXP64_C9);
  H = fma_(H, r.h, KN_EXP64_C8);
  DD S{H, 0.0};
  S = dd_add(dd_mul(S, r), DD{KN_EXP64_C7H, KN_EXP64_C7L});
  S = dd_add(dd_mul(S, r), DD{KN_EXP64_C6H, KN_EXP64_C6L});
  S = dd_add(dd_mul(S, r), DD{KN_EXP64_C5H, KN_EXP64_C5L});
  S = dd_add(dd_mul(S, r), DD{KN_EXP64_C4H, KN_EXP64_C4L});
  S = dd_add(dd_mul(S, r), DD{KN_EXP64_C3H, KN_EXP64_C3L});
  S = dd_add(dd_mul(S, r), DD{0.5, 0.0});
  S = dd_add(dd_mul(S, r), DD{1.0, 0.0});
  S = dd_add(dd_mul(S, r), DD{1.0, 0.0});
  const DD y = dd_mul(S, DD{q0.th, q0.tl});
  return scale2(y.h, q0.m);
}

// exp(a) for -708 <= a <= 709, correctly rounded.
KN_HD double exp_cr64_inrange(double a) {
  double y;
  if (exp_cr64_fast(a, y)) return y;
#ifdef KN_EXP64_COUNT_SLOW
  KN_EXP64_COUNT_SLOW;
#endif
  return exp_cr64_slow(a);
}

}  // namespace x64
}  // namespace kn
