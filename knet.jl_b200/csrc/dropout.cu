// Dropout with an in-kernel counter-based generator, and the fused hidden-layer pieces
// y = dropout(relu(z .+ b)) forward and dz = reluback(dropback(dy)) backward.
//
// The generator is Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as
// easy as 1, 2, 3", SC'11): key = the 64-bit seed, counter = offset + group index, one call
// yields four 32-bit words = 32 bytes of output: a group is 8 consecutive Float32 elements
// (element e takes 16 bits, the low half of word e/2 for even e, the high half for odd e,
// u = bits * 2^-16) or 4 consecutive Float64 elements (u = word * 2^-32).  A dropout decision
// needs no more resolution than that, and the ten rounds - about sixty integer instructions -
// are then paid once per 32 bytes, which keeps the kernels on the HBM roofline.
// The decision rule is Knet's: keep when u > p, scale by a division with q = 1 - p
// (src/ops20/dropout.jl:45-57).
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "math.cuh"
#include "reduce.cuh"

namespace kn {

struct U4 {
  uint32_t v[4];
};

// The ten round keys depend on the seed only: the host computes them once per launch and
// they reach the kernel through the parameter bank, which saves twenty adds per call.
struct PhiloxKeys {
  uint32_t k0[10], k1[10];
};
inline PhiloxKeys philox_keys(uint64_t seed) {
  PhiloxKeys k;
  uint32_t a = (uint32_t)seed, b = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; r++) {
    k.k0[r] = a;
    k.k1[r] = b;
    a += 0x9E3779B9u;
    b += 0xBB67AE85u;
  }
  return k;
}

__device__ __forceinline__ U4 philox4x32_10(uint64_t counter, const PhiloxKeys& k) {
  uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; r++) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k.k0[r], n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k.k1[r];
    c0 = n0; c1 = (uint32_t)p1; c2 = n2; c3 = (uint32_t)p0;
  }
  return U4{{c0, c1, c2, c3}};
}

template <typename T> struct Uniform;
template <> struct Uniform<float> {
  enum { GROUP = 8 };
  static __device__ __forceinline__ uint32_t bits(const U4& r, int e) { return (e & 1) ? (r.v[e >> 1] >> 16) : (r.v[e >> 1] & 0xffffu); }
  static __device__ __forceinline__ void make(const U4& r, float (&u)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e++) u[e] = (float)bits(r, e) * 0x1p-16f;
  }
  // u > p without forming u: u = k * 2^-16 with the integer k, so u > p exactly when
  // k > floor(p * 2^16) (`thr`, computed on the host)
  static __device__ __forceinline__ void keep(const U4& r, uint64_t thr, bool (&k)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e++) k[e] = bits(r, e) > (uint32_t)thr;
  }
  static uint64_t threshold(float p) { return (uint64_t)std::floor((double)p * 65536.0); }
};
template <> struct Uniform<double> {
  enum { GROUP = 4 };
  static __device__ __forceinline__ void make(const U4& r, double (&u)[4]) {
#pragma unroll
    for (int e = 0; e < 4; e++) u[e] = (double)r.v[e] * 0x1p-32;
  }
  // the same with the 32-bit integer k = word and thr = floor(p * 2^32)
  static __device__ __forceinline__ void keep(const U4& r, uint64_t thr, bool (&k)[4]) {
#pragma unroll
    for (int e = 0; e < 4; e++) k[e] = r.v[e] > (uint32_t)thr;
  }
  static uint64_t threshold(double p) { return (uint64_t)std::floor(std::ldexp(p, 32)); }
};

// MODE 0: y = dropout(x); 1: u only; 2: y = dropout(relu(x + b[row])); 3: y = relu(x + b[row])
// Scale of the kept elements: x / q as Knet's CPU loop does; when q is a power of two the
// product with 1/q is the same number and costs one instruction instead of a division.
template <typename T> struct KeepScale {
  T q, rq;
  int exact_rq;
  uint64_t thr;   // Uniform<T>::threshold(p)
  __device__ __forceinline__ T operator()(T x) const { return exact_rq ? x * rq : x / q; }
};

// n % d for n < 2^31 by a multiply-high with a host-computed reciprocal (Granlund-Montgomery
// round-up method: s = ceil(log2 d), m = floor(2^32 (2^s - d) / d) + 1, q = (mulhi(m, n) + n) >> s;
// the sum cannot overflow because n < 2^31).  Four instructions instead of a 32-bit division.
struct FastMod {
  uint32_t d, m, s;
  uint32_t bvec;   // the bias vector can be read as whole 16-byte groups (set by the launcher)
};
inline FastMod fast_mod(uint32_t d) {
  FastMod f{d, 0u, 0u, 0u};
  while ((1ull << f.s) < d) f.s++;
  f.m = (uint32_t)((((1ull << f.s) - d) << 32) / d + 1);
  return f;
}
__device__ __forceinline__ uint32_t mod_fast(uint32_t n, const FastMod& f) {
  const uint32_t q = (__umulhi(f.m, n) + n) >> f.s;
  return n - q * f.d;
}

// I is the index type: 32-bit whenever the element count allows (the bias row then comes from
// the multiply-high modulo above).
template <typename T, int MODE, bool VECIO, typename I>
__global__ void __launch_bounds__(256)
philox_kernel(const T* __restrict__ x, const T* __restrict__ b, T* __restrict__ y, I n, I N, T p,
              KeepScale<T> scale, PhiloxKeys keys, uint64_t offset, const uint64_t* __restrict__ offset_dev,
              FastMod fm) {
  constexpr int G = Uniform<T>::GROUP, VE = VecN<T>::value;   // a group is two 16-byte packs
  if (offset_dev) offset += __ldg(offset_dev);   // replayed graphs: the step's part of the counter lives on the device
  const I ngroups = (n + (G - 1)) / G;
  const I stride = (I)gridDim.x * blockDim.x;
  for (I gi = (I)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += stride) {
    const I i0 = gi * G;
    T xv[G], r[G], u[G];
    const bool full = i0 + G <= n;
    if (MODE != 1) {   // the loads go first: the generator's integer work hides their latency
      if (VECIO && full) {
#pragma unroll
        for (int h = 0; h < G / VE; h++) {
          const Pack<T, VE> t = ld_stream<T, VE>(x + i0 + h * VE);
#pragma unroll
          for (int e = 0; e < VE; e++) xv[h * VE + e] = t.v[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < G; e++) xv[e] = i0 + e < n ? x[i0 + e] : (T)0;
      }
    }
    bool kp[G];
    if (MODE == 1) Uniform<T>::make(philox4x32_10(offset + gi, keys), u);
    else if (MODE != 3) Uniform<T>::keep(philox4x32_10(offset + gi, keys), scale.thr, kp);
    if (MODE >= 2) {
      I row = sizeof(I) == 4 ? (I)mod_fast((uint32_t)i0, fm) : i0 % N;
      T bv[G];
      if (fm.bvec) {     // N is a multiple of the group and b is 16-byte aligned: the group never wraps
#pragma unroll
        for (int h = 0; h < G / VE; h++) {
          const Pack<T, VE> t = *reinterpret_cast<const Pack<T, VE>*>(b + row + h * VE);
#pragma unroll
          for (int e = 0; e < VE; e++) bv[h * VE + e] = t.v[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < G; e++) {
          bv[e] = __ldg(b + row);
          if (++row >= N) row = 0;
        }
      }
#pragma unroll
      for (int e = 0; e < G; e++) {
        const T t = xv[e] + bv[e];
        xv[e] = !(t <= (T)0) ? t : (T)0;   // max(t, 0) that lets NaN through: one compare
      }
    }
#pragma unroll
    for (int e = 0; e < G; e++) {
      if (MODE == 1) r[e] = u[e];
      else if (MODE == 3) r[e] = xv[e];
      else r[e] = kp[e] ? scale(xv[e]) : (T)0;
    }
    if (VECIO && full) {
#pragma unroll
      for (int h = 0; h < G / VE; h++) {
        Pack<T, VE> t;
#pragma unroll
        for (int e = 0; e < VE; e++) t.v[e] = r[h * VE + e];
        st_stream<T, VE>(y + i0 + h * VE, t);
      }
    } else {
#pragma unroll
      for (int e = 0; e < G; e++)
        if (i0 + e < n) y[i0 + e] = r[e];
    }
  }
}

template <typename T> inline KeepScale<T> keep_scale(T p) {
  const T q = (T)1 - p;
  int ex = 0;
  const double m = std::frexp((double)q, &ex);
  return KeepScale<T>{q, (T)1 / q, m == 0.5 ? 1 : 0, Uniform<T>::threshold(p)};
}

template <typename T, int MODE>
int run_philox(const T* x, const T* b, T* y, int64_t n, int64_t N, T p, uint64_t seed, uint64_t offset,
               cudaStream_t st, const uint64_t* offset_dev = nullptr) {
  if (n < 0) return KN_EINVAL;
  if (n == 0) return KN_OK;
  constexpr int G = Uniform<T>::GROUP;
  const uint64_t ngroups = ((uint64_t)n + G - 1) / G;
  uint64_t blocks = (ngroups + 255) / 256;
  static const int per_sm = [] {
    const char* e = getenv("KNET_SM100_PHILOX_CTAS_PER_SM");   // tuning knob; 0 = one group per thread
    return e ? atoi(e) : 64;
  }();
  const uint64_t cap = per_sm > 0 ? (uint64_t)sm_count() * per_sm : 0x7fffffffull;
  if (blocks > cap) blocks = cap;
  const bool vec = (((uintptr_t)y | (uintptr_t)x) & 15) == 0;
  const KeepScale<T> sc = keep_scale<T>(p);
  const PhiloxKeys keys = philox_keys(seed);
  const int64_t rows = N > 0 ? N : 1;
  const unsigned g = (unsigned)blocks;
  FastMod fm = fast_mod((uint32_t)(rows < ((int64_t)1 << 31) ? rows : 1));
  fm.bvec = (MODE >= 2 && b && rows % G == 0 && ((uintptr_t)b & 15) == 0) ? 1u : 0u;
  if (n < ((int64_t)1 << 31)) {   // indices, and index + group size, fit 32 bits
    if (vec) philox_kernel<T, MODE, true, uint32_t><<<g, 256, 0, st>>>(x, b, y, (uint32_t)n, (uint32_t)rows, p, sc, keys, offset, offset_dev, fm);
    else philox_kernel<T, MODE, false, uint32_t><<<g, 256, 0, st>>>(x, b, y, (uint32_t)n, (uint32_t)rows, p, sc, keys, offset, offset_dev, fm);
  } else {
    if (vec) philox_kernel<T, MODE, true, uint64_t><<<g, 256, 0, st>>>(x, b, y, (uint64_t)n, (uint64_t)rows, p, sc, keys, offset, offset_dev, fm);
    else philox_kernel<T, MODE, false, uint64_t><<<g, 256, 0, st>>>(x, b, y, (uint64_t)n, (uint64_t)rows, p, sc, keys, offset, offset_dev, fm);
  }
  return launch_status();
}

// dz = y == 0 ? 0 : dy / q  (q = 1 - p; p = 0 gives reluback, since y = relu(.) >= 0)
// EXACT: q is a power of two, so dy * (1/q) is the same number as dy / q and costs one instruction
template <typename T, bool EXACT> struct ReluDropBack {
  T q, rq;
  __device__ __forceinline__ void operator()(const T (&a)[2], T (&r)[1]) const {
    r[0] = a[0] == (T)0 ? (T)0 : (EXACT ? a[1] * rq : a[1] / q);
  }
};

// ---- dz = reluback(dropback(dy)) and db = sum(dz, dims=2) in one pass ---------------------------
// y, dy, dz are (rows, cols) column-major.  A warp owns 32*RV adjacent rows and walks columns
// (one 16-byte load of y and of dy per thread and column when RV > 1), so every access is
// coalesced and each thread sums the dz it has just written.  Columns are spread over the
// blockDim.y warps of a CTA and over the CTAs of a thread-block cluster; the warps' sums meet
// in shared memory and the CTAs' sums in distributed shared memory, both in a fixed order,
// so db is deterministic.  dz may be the same buffer as dy.
constexpr int kBwdWY = 8;

// EXACT: 1 - p is a power of two, so dy * (1/q) is the same number as dy / q
template <typename T, int RV, bool EXACT>
__global__ void __launch_bounds__(32 * kBwdWY, 4)
relu_drop_bias_bwd_kernel(const T* __restrict__ y, const T* dy, T* dz, T* __restrict__ db, uint32_t rows,
                          uint32_t cols, uint32_t cs, T q, T rq) {
  __shared__ T part[kBwdWY][32 * RV];
  __shared__ T total[32 * RV];
  const uint32_t lx = threadIdx.x, ly = threadIdx.y;
  const uint32_t row0 = (blockIdx.x * 32 + lx) * RV;
  const bool valid = row0 < rows;
  // The CTAs of a cluster take blocks of 4*kBwdWY consecutive columns in turn (block b belongs to
  // CTA b % cs), so that at any time the cluster reads one contiguous region that moves through the
  // arrays, like a linear sweep, instead of cs regions a power of two apart.
  constexpr uint32_t BLK = 4 * kBwdWY;
  T acc[2][RV];
#pragma unroll
  for (int e = 0; e < RV; e++) acc[0][e] = acc[1][e] = (T)0;
  auto one = [&](T yv, T g) -> T { return yv == (T)0 ? (T)0 : (EXACT ? g * rq : g / q); };
  if (valid) {
    for (uint32_t b0 = blockIdx.y * BLK; b0 < cols; b0 += cs * BLK) {
      const uint32_t c = b0 + ly;
      if (b0 + BLK <= cols) {
        Pack<T, RV> yv[4], gv[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const uint64_t off = (uint64_t)(c + k * kBwdWY) * rows + row0;
          yv[k] = ld_stream<T, RV>(y + off);
          gv[k] = ld_stream<T, RV>(dy + off);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
          Pack<T, RV> r;
#pragma unroll
          for (int e = 0; e < RV; e++) {
            r.v[e] = one(yv[k].v[e], gv[k].v[e]);
            acc[k & 1][e] += r.v[e];
          }
          st_stream<T, RV>(dz + (uint64_t)(c + k * kBwdWY) * rows + row0, r);
        }
      } else {
        for (uint32_t cc = c; cc < cols; cc += kBwdWY) {
          const uint64_t off = (uint64_t)cc * rows + row0;
          const Pack<T, RV> yv = ld_stream<T, RV>(y + off), gv = ld_stream<T, RV>(dy + off);
          Pack<T, RV> r;
#pragma unroll
          for (int e = 0; e < RV; e++) {
            r.v[e] = one(yv.v[e], gv.v[e]);
            acc[0][e] += r.v[e];
          }
          st_stream<T, RV>(dz + off, r);
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < RV; e++) part[ly][lx * RV + e] = acc[0][e] + acc[1][e];
  __syncthreads();
  if (ly == 0) {
#pragma unroll
    for (int e = 0; e < RV; e++) {
      T a = part[0][lx * RV + e];
#pragma unroll
      for (int k = 1; k < kBwdWY; k++) a += part[k][lx * RV + e];
      total[lx * RV + e] = a;
    }
  }
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (blockIdx.y % cs == 0 && ly == 0 && valid) {
#pragma unroll
      for (int e = 0; e < RV; e++) {
        T a = total[lx * RV + e];
        for (uint32_t r = 1; r < cs; r++) a += cluster.map_shared_rank(total, r)[lx * RV + e];
        db[row0 + e] = a;
      }
    }
    cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
  } else if (ly == 0 && valid) {
#pragma unroll
    for (int e = 0; e < RV; e++) db[row0 + e] = total[lx * RV + e];
  }
}

template <typename T>
int run_relu_drop_bias_bwd(const T* y, const T* dy, T* dz, T* db, int64_t N, int64_t B, T p, cudaStream_t st) {
  if (N < 0 || B < 0) return KN_EINVAL;
  if (N == 0) return KN_OK;
  if (N >= ((int64_t)1 << 31) || B >= ((int64_t)1 << 31)) return KN_ESIZE;
  if (!db || (B > 0 && (!y || !dy || !dz))) return KN_EINVAL;
  if (!(p >= 0 && p < 1)) return KN_EINVAL;
  constexpr int VEC = VecN<T>::value;
  const KeepScale<T> sc = keep_scale<T>(p);
  const uint32_t rows = (uint32_t)N, cols = (uint32_t)B;
  static const int forced_cs = [] {
    const char* e = getenv("KNET_SM100_BWD_CS");   // tuning knob
    return e ? atoi(e) : 0;
  }();
  auto ok = [&](uint32_t rv) {
    return rv == 1 || ((((uintptr_t)y | (uintptr_t)dy | (uintptr_t)dz) % (rv * sizeof(T))) == 0 && rows % rv == 0);
  };
  const RowsGeom g = rows_geometry(rows, cols, 1, VEC, kBwdWY, ok, forced_cs);
  const uint32_t cs = g.cs;
  const dim3 block(32, kBwdWY), grid(g.tiles, cs, 1);
  auto k = sc.exact_rq ? relu_drop_bias_bwd_kernel<T, 1, true> : relu_drop_bias_bwd_kernel<T, 1, false>;
  if (g.rv == VEC) k = sc.exact_rq ? relu_drop_bias_bwd_kernel<T, VEC, true> : relu_drop_bias_bwd_kernel<T, VEC, false>;
  else if (g.rv == 2) k = sc.exact_rq ? relu_drop_bias_bwd_kernel<T, (VEC >= 2 ? 2 : 1), true> : relu_drop_bias_bwd_kernel<T, (VEC >= 2 ? 2 : 1), false>;
  const cudaError_t e = launch_cluster(k, grid, block, 0, st, cs, y, dy, dz, db, rows, cols, cs, sc.q, sc.rq);
  return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace kn

using namespace kn;

#define KN_DEF_PHILOX(f, S, T)                                                                        \
  KN_EXPORT int knet_dropout_philox_##S(int64_t n, T p, uint64_t seed, uint64_t offset, const T* x,   \
                                        T* y, cudaStream_t s) {                                       \
    if (n > 0 && (!x || !y)) return KN_EINVAL;                                                        \
    if (!(p >= 0 && p < 1)) return KN_EINVAL;                                                         \
    return run_philox<T, 0>(x, nullptr, y, n, 1, p, seed, offset, s);                                 \
  }                                                                                                   \
  KN_EXPORT int knet_dropout_uniform_##S(int64_t n, uint64_t seed, uint64_t offset, T* u,             \
                                         cudaStream_t s) {                                            \
    if (n > 0 && !u) return KN_EINVAL;                                                                \
    return run_philox<T, 1>(nullptr, nullptr, u, n, 1, (T)0, seed, offset, s);                        \
  }                                                                                                   \
  KN_EXPORT int knet_bias_relu_dropout_fwd_##S(const T* z, const T* b, T* y, int64_t N, int64_t B,    \
                                               T p, uint64_t seed, uint64_t offset, cudaStream_t s) { \
    if (N < 0 || B < 0) return KN_EINVAL;                                                             \
    if (N * B > 0 && (!z || !b || !y)) return KN_EINVAL;                                              \
    if (!(p >= 0 && p < 1)) return KN_EINVAL;                                                         \
    if (p == 0) return run_philox<T, 3>(z, b, y, N * B, N, p, seed, offset, s);                       \
    return run_philox<T, 2>(z, b, y, N * B, N, p, seed, offset, s);                                   \
  }                                                                                                   \
  KN_EXPORT int knet_bias_relu_dropout_fwd_g_##S(const T* z, const T* b, T* y, int64_t N, int64_t B,  \
                                                 T p, uint64_t seed, uint64_t offset,                 \
                                                 const uint64_t* offset_dev, cudaStream_t s) {        \
    if (N < 0 || B < 0) return KN_EINVAL;                                                             \
    if (N * B > 0 && (!z || !b || !y)) return KN_EINVAL;                                              \
    if (!(p >= 0 && p < 1)) return KN_EINVAL;                                                         \
    if (p == 0) return run_philox<T, 3>(z, b, y, N * B, N, p, seed, offset, s);                       \
    return run_philox<T, 2>(z, b, y, N * B, N, p, seed, offset, s, offset_dev);                       \
  }                                                                                                   \
  KN_EXPORT int knet_relu_dropout_bwd_##S(const T* y, const T* dy, T* dz, int64_t n, T p,             \
                                          cudaStream_t s) {                                           \
    if (n < 0 || (n > 0 && (!y || !dy || !dz))) return KN_EINVAL;                                     \
    if (!(p >= 0 && p < 1)) return KN_EINVAL;                                                         \
    EwPtrs<T, 2, 1> pp{{y, dy}, {dz}};                                                                \
    const KeepScale<T> sc = keep_scale<T>(p);                                                         \
    if (sc.exact_rq) ew_launch<T, 2, 1>(ReluDropBack<T, true>{sc.q, sc.rq}, pp, n, s);                \
    else ew_launch<T, 2, 1>(ReluDropBack<T, false>{sc.q, sc.rq}, pp, n, s);                           \
    return launch_status();                                                                           \
  }                                                                                                   \
  KN_EXPORT int knet_relu_dropout_bias_bwd_##S(const T* y, const T* dy, T* dz, T* db, int64_t N,      \
                                               int64_t B, T p, cudaStream_t s) {                      \
    return run_relu_drop_bias_bwd<T>(y, dy, dz, db, N, B, p, s);                                      \
  }
KNET_BOTH_TYPES(KN_DEF_PHILOX, philox)
