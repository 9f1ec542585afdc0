// Broadcasting binary kernels behind the _12, _13 and _16 entry points.
//
// One kernel serves every "operand is full-size, a scalar, or a vector along one dim" case
// (src/knetarrays/binary.jl:152-212 decides the (s,n) pair of each operand).  The output is
// written with 16-byte stores; for each 16-byte group the operand index is decoded once
// (one 32-bit divide at most), not once per element, and a vector operand is read through
// L1/L2 where it stays resident because it is tiny next to the output.
#include "common.cuh"
#include "ops.cuh"

namespace kn {

enum : int { OPD_FULL = 0, OPD_SCALAR = 1, OPD_MOD = 2, OPD_DIV = 3 };

template <typename T> struct Operand {
  const T* p;
  int mode;
  int vec_ok;   // FULL/MOD: 16-byte loads are legal
  FastDiv s;    // DIV: inner stride
  FastDiv n;    // MOD/DIV: vector length
};

template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> load_operand(const Operand<T>& o, uint32_t i) {
  Pack<T, VEC> r;
  if (o.mode == OPD_FULL) {
    if (VEC > 1 && o.vec_ok) return ld_stream<T, VEC>(o.p + i);
#pragma unroll
    for (int e = 0; e < VEC; e++) r.v[e] = __ldcs(o.p + i + e);
  } else if (o.mode == OPD_SCALAR) {
    const T v = __ldg(o.p);
#pragma unroll
    for (int e = 0; e < VEC; e++) r.v[e] = v;
  } else if (o.mode == OPD_MOD) {
    uint32_t j = mod_fast(i, o.n);
    if (VEC > 1 && o.vec_ok) {
      // n is a multiple of VEC and i is too, so the group does not wrap
      const float4 t = __ldg(reinterpret_cast<const float4*>(o.p + j));
      *reinterpret_cast<float4*>(&r) = t;
      return r;
    }
#pragma unroll
    for (int e = 0; e < VEC; e++) {
      r.v[e] = __ldg(o.p + j);
      if (++j >= o.n.d) j = 0;
    }
  } else {
    if (o.s.d % VEC == 0) {
      const T v = __ldg(o.p + mod_fast(div_fast(i, o.s), o.n));
#pragma unroll
      for (int e = 0; e < VEC; e++) r.v[e] = v;
    } else {
#pragma unroll
      for (int e = 0; e < VEC; e++) r.v[e] = __ldg(o.p + mod_fast(div_fast(i + e, o.s), o.n));
    }
  }
  return r;
}

// ---- the operation on one group ---------------------------------------------------------------
template <typename T, typename Op, int VEC>
__device__ __forceinline__ Pack<T, VEC> apply_pack(Op op, const Pack<T, VEC>& a, const Pack<T, VEC>& b) {
  Pack<T, VEC> r;
#pragma unroll
  for (int e = 0; e < VEC; e++) r.v[e] = op(a.v[e], b.v[e]);
  return r;
}

// Float32 division goes through div_group (math.cuh): one special-case test per group.
template <int VEC>
__device__ __forceinline__ Pack<float, VEC> apply_pack(op::B_div<float>, const Pack<float, VEC>& a,
                                                       const Pack<float, VEC>& b) {
  Pack<float, VEC> r;
  div_group<VEC>(a.v, b.v, r.v);
  return r;
}

constexpr int kBcThreads = 256;
constexpr int kBcUnroll = 4;

template <typename T, typename Op, int VEC>
__global__ void __launch_bounds__(kBcThreads, sizeof(T) == 4 ? 5 : 1)   // Float32: five CTAs per SM (48 registers)
bcast12_kernel(Op op, Operand<T> x, Operand<T> y, T* __restrict__ z, uint32_t nvec, uint32_t n) {
  const uint64_t base = (uint64_t)blockIdx.x * (kBcThreads * kBcUnroll) + threadIdx.x;
  Pack<T, VEC> a[kBcUnroll], b[kBcUnroll];
#pragma unroll
  for (int u = 0; u < kBcUnroll; u++) {
    const uint64_t iv = base + (uint64_t)u * kBcThreads;
    if (iv < nvec) {
      a[u] = load_operand<T, VEC>(x, (uint32_t)(iv * VEC));
      b[u] = load_operand<T, VEC>(y, (uint32_t)(iv * VEC));
    }
  }
#pragma unroll
  for (int u = 0; u < kBcUnroll; u++) {
    const uint64_t iv = base + (uint64_t)u * kBcThreads;
    if (iv < nvec) {
      st_stream<T, VEC>(z + iv * VEC, apply_pack(op, a[u], b[u]));
    }
  }
  if (VEC > 1 && blockIdx.x == 0) {
    const uint32_t i = nvec * VEC + threadIdx.x;
    if (i < n) {
      const Pack<T, 1> a1 = load_operand<T, 1>(x, i), b1 = load_operand<T, 1>(y, i);
      z[i] = op(a1.v[0], b1.v[0]);
    }
  }
}

template <typename T> Operand<T> make_operand(const T* p, int n, int s_, int n_) {
  Operand<T> o;
  o.p = p;
  o.s = fast_div((uint32_t)(s_ > 0 ? s_ : 1));
  o.n = fast_div((uint32_t)(n_ > 0 ? n_ : 1));
  const bool aligned = ((uintptr_t)p & 15) == 0;
  constexpr int VEC = VecN<T>::value;
  if (n_ == n) { o.mode = OPD_FULL; o.vec_ok = aligned; }
  else if (s_ == 1) { o.mode = OPD_MOD; o.vec_ok = aligned && (n_ % VEC == 0); }
  else if (n_ == 1) { o.mode = OPD_SCALAR; o.vec_ok = 0; }
  else { o.mode = OPD_DIV; o.vec_ok = 0; }
  return o;
}

template <typename T, typename Op>
void run_12(int n, const T* x, int sx, int nx, const T* y, int sy, int ny, T* z, cudaStream_t st) {
  if (n <= 0) return;
  constexpr int VEC = VecN<T>::value;
  const Operand<T> ox = make_operand<T>(x, n, sx, nx), oy = make_operand<T>(y, n, sy, ny);
  if (((uintptr_t)z & 15) == 0) {
    const uint32_t nvec = (uint32_t)n / VEC;
    uint32_t blocks = (nvec + kBcThreads * kBcUnroll - 1) / (kBcThreads * kBcUnroll);
    if (blocks == 0) blocks = 1;
    bcast12_kernel<T, Op, VEC><<<blocks, kBcThreads, 0, st>>>(Op(), ox, oy, z, nvec, (uint32_t)n);
  } else {
    const uint32_t blocks = ((uint32_t)n + kBcThreads * kBcUnroll - 1) / (kBcThreads * kBcUnroll);
    bcast12_kernel<T, Op, 1><<<blocks, kBcThreads, 0, st>>>(Op(), ox, oy, z, (uint32_t)n, (uint32_t)n);
  }
}

// _13: vector of B_N elements along a dim with stride `ds` in a dense array of A_N elements.
// For a dense array the element at linear index i belongs to vector entry (i/ds) % B_N, so
// the call is the DIV case of the kernel above.  swap = 1 computes f(vec, big).
template <typename T, typename Op>
void run_13(const T* big, const T* vec, T* z, int ds, int A_N, int B_N, bool swap, cudaStream_t st) {
  if (A_N <= 0) return;
  if (swap) run_12<T, Op>(A_N, vec, ds, B_N, big, 1, A_N, z, st);
  else run_12<T, Op>(A_N, big, 1, A_N, vec, ds, B_N, z, st);
}

// _16: general strided broadcast of up to 5 dims.  Coordinates are decoded once per 16-byte
// group of z when the first dim is a multiple of the group.
template <int ND> struct Strides { int sx[ND], sy[ND], sz[ND]; };

template <int ND> struct StrideDivs { FastDiv fz[ND]; };   // multiply-high reciprocals of Strides::sz

template <typename T, typename Op, int ND, int VEC>
__global__ void __launch_bounds__(256)
bcast16_kernel(Op op, const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ z,
               Strides<ND> s, StrideDivs<ND> sd, uint32_t nvec) {
  for (uint64_t iv = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; iv < nvec;
       iv += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t rem = (uint32_t)(iv * VEC);
    uint32_t ix = 0, iy = 0;
#pragma unroll
    for (int d = ND - 1; d >= 0; d--) {
      const uint32_t c = div_fast(rem, sd.fz[d]);      // the element count is an int: rem < 2^31
      rem -= c * (uint32_t)s.sz[d];
      ix += c * (uint32_t)s.sx[d];
      iy += c * (uint32_t)s.sy[d];
    }
    Pack<T, VEC> r;
#pragma unroll
    for (int e = 0; e < VEC; e++)
      r.v[e] = op(__ldg(x + ix + e * s.sx[0]), __ldg(y + iy + e * s.sy[0]));
    st_stream<T, VEC>(z + iv * VEC, r);
  }
}

template <typename T, typename Op, int ND>
void run_16(const T* x, const T* y, T* z, const Strides<ND>& s, int Nz, cudaStream_t st) {
  if (Nz <= 0) return;
  constexpr int VEC = VecN<T>::value;
  // size of the first dim = stride of the second one
  const bool vec = ((uintptr_t)z & 15) == 0 && s.sz[0] == 1 && (s.sz[1] % VEC) == 0 && (Nz % VEC) == 0;
  const int cap = sm_count() * 16;
  StrideDivs<ND> sd;
  for (int d = 0; d < ND; d++) sd.fz[d] = fast_div((uint32_t)(s.sz[d] > 0 ? s.sz[d] : 1));
  if (vec) {
    const uint32_t nvec = (uint32_t)Nz / VEC;
    int blocks = (int)((nvec + 255) / 256);
    if (blocks > cap) blocks = cap;
    bcast16_kernel<T, Op, ND, VEC><<<blocks, 256, 0, st>>>(Op(), x, y, z, s, sd, nvec);
  } else {
    int blocks = (int)(((uint32_t)Nz + 255) / 256);
    if (blocks > cap) blocks = cap;
    bcast16_kernel<T, Op, ND, 1><<<blocks, 256, 0, st>>>(Op(), x, y, z, s, sd, (uint32_t)Nz);
  }
}

}  // namespace kn

using namespace kn;

#define KN_DEF_BCAST(f, S, T)                                                                    \
  KN_EXPORT void f##_##S##_12_stream(int n, const T* x, int sx, int nx, const T* y, int sy,      \
                                     int ny, T* z, cudaStream_t s) {                             \
    run_12<T, op::B_##f<T>>(n, x, sx, nx, y, sy, ny, z, s);                                      \
  }                                                                                              \
  KN_EXPORT void f##_##S##_12(int n, const T* x, int sx, int nx, const T* y, int sy, int ny,     \
                              T* z) {                                                            \
    f##_##S##_12_stream(n, x, sx, nx, y, sy, ny, z, cudaStreamPerThread);                        \
  }                                                                                              \
  KN_EXPORT void f##_##S##_13_x_y_stream(const T* x, const T* y, T* z, int ds, int ns, int md,   \
                                         int A_N, int B_N, cudaStream_t s) {                     \
    (void)ns; (void)md;                                                                          \
    run_13<T, op::B_##f<T>>(x, y, z, ds, A_N, B_N, false, s);                                    \
  }                                                                                              \
  KN_EXPORT void f##_##S##_13_x_y(const T* x, const T* y, T* z, int ds, int ns, int md, int A_N, \
                                  int B_N) {                                                     \
    f##_##S##_13_x_y_stream(x, y, z, ds, ns, md, A_N, B_N, cudaStreamPerThread);                 \
  }                                                                                              \
  KN_EXPORT void f##_##S##_13_y_x_stream(const T* x, const T* y, T* z, int ds, int ns, int md,   \
                                         int A_N, int B_N, cudaStream_t s) {                     \
    (void)ns; (void)md;                                                                          \
    run_13<T, op::B_##f<T>>(x, y, z, ds, A_N, B_N, true, s);                                     \
  }                                                                                              \
  KN_EXPORT void f##_##S##_13_y_x(const T* x, const T* y, T* z, int ds, int ns, int md, int A_N, \
                                  int B_N) {                                                     \
    f##_##S##_13_y_x_stream(x, y, z, ds, ns, md, A_N, B_N, cudaStreamPerThread);                 \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_3_stream(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,  \
                                       int sy0, int sy1, int sy2, int sz0, int sz1, int sz2,     \
                                       int Nz, cudaStream_t s) {                                 \
    Strides<3> st{{sx0, sx1, sx2}, {sy0, sy1, sy2}, {sz0, sz1, sz2}};                            \
    run_16<T, op::B_##f<T>, 3>(x, y, z, st, Nz, s);                                              \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_3(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,         \
                                int sy0, int sy1, int sy2, int sz0, int sz1, int sz2, int Nz) {  \
    f##_##S##_16_3_stream(x, y, z, sx0, sx1, sx2, sy0, sy1, sy2, sz0, sz1, sz2, Nz,              \
                          cudaStreamPerThread);                                                  \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_4_stream(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,  \
                                       int sx3, int sy0, int sy1, int sy2, int sy3, int sz0,     \
                                       int sz1, int sz2, int sz3, int Nz, cudaStream_t s) {      \
    Strides<4> st{{sx0, sx1, sx2, sx3}, {sy0, sy1, sy2, sy3}, {sz0, sz1, sz2, sz3}};             \
    run_16<T, op::B_##f<T>, 4>(x, y, z, st, Nz, s);                                              \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_4(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,         \
                                int sx3, int sy0, int sy1, int sy2, int sy3, int sz0, int sz1,   \
                                int sz2, int sz3, int Nz) {                                      \
    f##_##S##_16_4_stream(x, y, z, sx0, sx1, sx2, sx3, sy0, sy1, sy2, sy3, sz0, sz1, sz2, sz3,   \
                          Nz, cudaStreamPerThread);                                              \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_5_stream(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,  \
                                       int sx3, int sx4, int sy0, int sy1, int sy2, int sy3,     \
                                       int sy4, int sz0, int sz1, int sz2, int sz3, int sz4,     \
                                       int Nz, cudaStream_t s) {                                 \
    Strides<5> st{{sx0, sx1, sx2, sx3, sx4}, {sy0, sy1, sy2, sy3, sy4},                          \
                  {sz0, sz1, sz2, sz3, sz4}};                                                    \
    run_16<T, op::B_##f<T>, 5>(x, y, z, st, Nz, s);                                              \
  }                                                                                              \
  KN_EXPORT void f##_##S##_16_5(const T* x, const T* y, T* z, int sx0, int sx1, int sx2,         \
                                int sx3, int sx4, int sy0, int sy1, int sy2, int sy3, int sy4,   \
                                int sz0, int sz1, int sz2, int sz3, int sz4, int Nz) {           \
    f##_##S##_16_5_stream(x, y, z, sx0, sx1, sx2, sx3, sx4, sy0, sy1, sy2, sy3, sy4, sz0, sz1,   \
                          sz2, sz3, sz4, Nz, cudaStreamPerThread);                               \
  }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_BCAST, f)
KNET_BINARY_OPS(KN_X)
#undef KN_X
