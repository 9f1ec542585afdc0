// update!(w, g, opt) as one read-modify-write pass per parameter array, and multi-tensor
// forms that cover a whole parameter set in one launch.
//
// The arithmetic follows Knet's CPU operation order (src/train20/update.jl:513-570), so the
// results are bit-identical to a CPU that rounds the same way: lmul!(a::Float64, x) is a
// Float64 product rounded to T, axpy!(a, x, y) is one fused multiply-add with a rounded to
// T, Array "/" is an IEEE division, sqrt is IEEE.  HBM traffic is the algorithmic minimum:
// SGD 3, Momentum 5, Adam 7 words per parameter.
#include <cmath>

#include <type_traits>

#include "common.cuh"
#include "math.cuh"
#include "reduce.cuh"

namespace kn {

// Float64 factor times a T value, rounded once to T (Julia: x .= a .* x with a::Float64)
template <typename T> __device__ __forceinline__ T lmul(double a, T x) { return (T)(a * (double)x); }

template <typename T> struct GScale {
  T gs;
  int on;
  __device__ __forceinline__ T operator()(T g) const { return on ? g * gs : g; }
};

// p[] = {w, g, s1, s2}; each functor updates the entries it owns in place
template <typename T> struct SgdF {
  enum { NP = 2, WMASK = 0x1 };
  T a; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    p[0] = Math<T>::fma(a, gs(p[1]), p[0]);
  }
};
template <typename T> struct MomentumF {
  enum { NP = 3, WMASK = 0x5 };
  T a; double gamma; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    T v = lmul<T>(gamma, p[2]);
    v = Math<T>::fma(a, gs(p[1]), v);
    p[2] = v;
    p[0] = Math<T>::fma((T)1, v, p[0]);
  }
};
template <typename T> struct NesterovF {
  enum { NP = 3, WMASK = 0x5 };
  T a, b; double gamma; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    T v = lmul<T>(gamma, p[2]);
    const T w = Math<T>::fma((T)-1, v, p[0]);
    v = Math<T>::fma(a, gs(p[1]), v);
    p[2] = v;
    p[0] = Math<T>::fma(b, v, w);
  }
};
template <typename T> struct AdagradF {
  enum { NP = 3, WMASK = 0x5 };
  T a, e; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    const T g = gs(p[1]);
    const T G = Math<T>::fma((T)1, g * g, p[2]);
    p[2] = G;
    p[0] = Math<T>::fma(a, g / Math<T>::sqrt(G + e), p[0]);
  }
};
template <typename T> struct RmspropF {
  enum { NP = 3, WMASK = 0x5 };
  T a, e, r1; double rho; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    const T g = gs(p[1]);
    T G = lmul<T>(rho, p[2]);
    G = Math<T>::fma(r1, g * g, G);
    p[2] = G;
    p[0] = Math<T>::fma(a, g / Math<T>::sqrt(G + e), p[0]);
  }
};
template <typename T> struct AdadeltaF {
  enum { NP = 4, WMASK = 0xD };
  T a, e, r1; double rho; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    const T g = gs(p[1]);
    T G = lmul<T>(rho, p[2]);
    G = Math<T>::fma(r1, g * g, G);
    p[2] = G;
    const T num = g * Math<T>::sqrt(p[3] + e);
    const T dw = num / Math<T>::sqrt(G + e);
    const T d = lmul<T>(rho, p[3]);
    p[3] = Math<T>::fma(r1, dw * dw, d);
    p[0] = Math<T>::fma(a, dw, p[0]);
  }
};
template <typename T> struct AdamF {
  enum { NP = 4, WMASK = 0xD };
  T a, e, c1, c2, b1t, b2t; double beta1, beta2; GScale<T> gs;
  __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    const T g = gs(p[1]);
    T m = lmul<T>(beta1, p[2]);
    m = Math<T>::fma(c1, g, m);
    T v = lmul<T>(beta2, p[3]);
    v = Math<T>::fma(c2, g * g, v);
    p[2] = m;
    p[3] = v;
    const T mh = m / b1t, vh = v / b2t;
    const T u = mh / (Math<T>::sqrt(vh) + e);
    p[0] = Math<T>::fma(a, u, p[0]);
  }
};

// Adam whose bias corrections 1 - beta^t are read from device memory when the kernel starts,
// so that a captured CUDA graph can be replayed with a new t: the host refreshes the two
// numbers (computed exactly as make_adam does) through a copy node of the same graph.
template <typename T> struct AdamDevF {
  enum { NP = 4, WMASK = 0xD };
  AdamF<T> f;
  const T* bias_corr;   // device: {1 - beta1^t, 1 - beta2^t} rounded to T
};

// Functor as the kernel uses it: itself, or Adam with its device-side scalars loaded.
template <typename F> __device__ __forceinline__ const F& resolve(const F& f) { return f; }
template <typename T> __device__ __forceinline__ AdamF<T> resolve(const AdamDevF<T>& d) {
  AdamF<T> f = d.f;
  f.b1t = __ldg(d.bias_corr);
  f.b2t = __ldg(d.bias_corr + 1);
  return f;
}

constexpr int kOptThreads = 256;

template <typename T, typename F, int VEC>
__device__ __forceinline__ void opt_range(const F& f, T* (&ptr)[4], uint32_t head, uint32_t nvec) {
  constexpr int NP = F::NP;
  // two vectors per pointer in flight per thread
  uint32_t v = threadIdx.x;
  for (; v + kOptThreads < nvec; v += 2 * kOptThreads) {
    Pack<T, VEC> a[2][NP];
#pragma unroll
    for (int u = 0; u < 2; u++)
#pragma unroll
      for (int k = 0; k < NP; k++) a[u][k] = ld_stream<T, VEC>(ptr[k] + head + (size_t)(v + u * kOptThreads) * VEC);
#pragma unroll
    for (int u = 0; u < 2; u++) {
#pragma unroll
      for (int e = 0; e < VEC; e++) {
        T p[NP];
#pragma unroll
        for (int k = 0; k < NP; k++) p[k] = a[u][k].v[e];
        f(p);
#pragma unroll
        for (int k = 0; k < NP; k++) a[u][k].v[e] = p[k];
      }
#pragma unroll
      for (int k = 0; k < NP; k++)
        if (F::WMASK & (1 << k)) st_stream<T, VEC>(ptr[k] + head + (size_t)(v + u * kOptThreads) * VEC, a[u][k]);
    }
  }
  for (; v < nvec; v += kOptThreads) {
    Pack<T, VEC> a[NP];
#pragma unroll
    for (int k = 0; k < NP; k++) a[k] = ld_stream<T, VEC>(ptr[k] + head + (size_t)v * VEC);
#pragma unroll
    for (int e = 0; e < VEC; e++) {
      T p[NP];
#pragma unroll
      for (int k = 0; k < NP; k++) p[k] = a[k].v[e];
      f(p);
#pragma unroll
      for (int k = 0; k < NP; k++) a[k].v[e] = p[k];
    }
#pragma unroll
    for (int k = 0; k < NP; k++)
      if (F::WMASK & (1 << k)) st_stream<T, VEC>(ptr[k] + head + (size_t)v * VEC, a[k]);
  }
}

// One chunk (at most KNET_MULTI_CHUNK elements starting at chunk * KNET_MULTI_CHUNK) of one tensor.
template <typename T, typename F>
__device__ __forceinline__ void opt_chunk(const F& f, const knet_tensor_desc& d, int64_t chunk) {
  constexpr int NP = F::NP;
  constexpr uint32_t VEC = VecN<T>::value;
  const int64_t start = chunk * KNET_MULTI_CHUNK;
  if (start >= d.n) return;
  const uint32_t cnt = (uint32_t)min((int64_t)KNET_MULTI_CHUNK, d.n - start);
  T* ptr[4] = {nullptr, nullptr, nullptr, nullptr};
  bool same = true;
  const uint32_t off = (uint32_t)((uintptr_t)(reinterpret_cast<T*>(d.p[0]) + start) & 15);
#pragma unroll
  for (int k = 0; k < NP; k++) {
    ptr[k] = reinterpret_cast<T*>(d.p[k]) + start;
    same &= ((uint32_t)((uintptr_t)ptr[k] & 15) == off);
  }
  if (same) {
    uint32_t head = off ? (16 - off) / (uint32_t)sizeof(T) : 0;
    if (head > cnt) head = cnt;
    const uint32_t nvec = (cnt - head) / VEC;
    opt_range<T, F, VEC>(f, ptr, head, nvec);
    const uint32_t tail0 = head + nvec * VEC;
    const uint32_t nrag = head + (cnt - tail0);
    if (threadIdx.x < nrag) {
      const uint32_t i = threadIdx.x < head ? threadIdx.x : tail0 + (threadIdx.x - head);
      T p[NP];
#pragma unroll
      for (int k = 0; k < NP; k++) p[k] = ptr[k][i];
      f(p);
#pragma unroll
      for (int k = 0; k < NP; k++)
        if (F::WMASK & (1 << k)) ptr[k][i] = p[k];
    }
  } else {
    opt_range<T, F, 1>(f, ptr, 0, cnt);
  }
}

// The tensor and the chunk inside it that block `b` of a multi-tensor launch works on.
__device__ __forceinline__ int find_tensor(const knet_tensor_desc* __restrict__ table, int ntensors, int64_t b, int* s_t) {
  for (int t = threadIdx.x; t < ntensors; t += blockDim.x) {
    const int64_t lo = table[t].first_chunk;
    const int64_t hi = t + 1 < ntensors ? table[t + 1].first_chunk : INT64_MAX;
    if (lo <= b && b < hi) *s_t = t;
  }
  __syncthreads();
  return *s_t;
}

// Per-array gradient clipping folded into the update (gclip!, src/train20/update.jl:572-583):
// the gradient is replaced on load by lmul!(factor, g), factor = gclip / norm(g) when the norm
// exceeds gclip and 1 otherwise, read from a per-tensor device array.
template <typename F> struct ClipF {
  enum { NP = F::NP, WMASK = F::WMASK };
  F f;
  double factor;
  template <typename T> __device__ __forceinline__ void operator()(T (&p)[NP]) const {
    if (factor != 1.0) p[1] = lmul<T>(factor, p[1]);
    f(p);
  }
};

template <typename T, typename F0>
__global__ void __launch_bounds__(kOptThreads)
opt_kernel(F0 f0, const knet_tensor_desc* __restrict__ table, int ntensors, knet_tensor_desc single) {
  const auto f = resolve(f0);
  typedef typename std::remove_cv<typename std::remove_reference<decltype(f)>::type>::type F;
  __shared__ int s_t;
  if (table == nullptr) {
    opt_chunk<T, F>(f, single, blockIdx.x);
  } else {
    const knet_tensor_desc d = table[find_tensor(table, ntensors, blockIdx.x, &s_t)];
    opt_chunk<T, F>(f, d, (int64_t)blockIdx.x - d.first_chunk);
  }
}

// The same with a per-tensor factor on the gradient (multi-tensor form only).
template <typename T, typename F0>
__global__ void __launch_bounds__(kOptThreads)
opt_clip_kernel(F0 f0, const knet_tensor_desc* __restrict__ table, int ntensors, const double* __restrict__ factors) {
  const auto f = resolve(f0);
  typedef typename std::remove_cv<typename std::remove_reference<decltype(f)>::type>::type F;
  __shared__ int s_t;
  const int t = find_tensor(table, ntensors, blockIdx.x, &s_t);
  const knet_tensor_desc d = table[t];
  opt_chunk<T, ClipF<F>>(ClipF<F>{f, factors[t]}, d, (int64_t)blockIdx.x - d.first_chunk);
}

template <typename T, typename F>
int run_single(const F& f, int64_t n, void* w, const void* g, void* s1, void* s2, cudaStream_t st) {
  if (n < 0) return KN_EINVAL;
  if (n == 0) return KN_OK;
  void* need[4] = {w, const_cast<void*>(g), s1, s2};
  for (int k = 0; k < F::NP; k++) {
    if (!need[k]) return KN_EINVAL;
    if ((uintptr_t)need[k] % sizeof(T)) return KN_EALIGN;
  }
  knet_tensor_desc d;
  for (int k = 0; k < 4; k++) d.p[k] = need[k];
  d.n = n;
  d.first_chunk = 0;
  const int64_t chunks = (n + KNET_MULTI_CHUNK - 1) / KNET_MULTI_CHUNK;
  if (chunks > 0x7fffffff) return KN_ESIZE;
  opt_kernel<T, F><<<(unsigned)chunks, kOptThreads, 0, st>>>(f, nullptr, 1, d);
  return launch_status();
}

template <typename T, typename F>
int run_multi(const F& f, const knet_tensor_desc* table, int ntensors, int64_t total_chunks, cudaStream_t st) {
  if (ntensors < 0 || total_chunks < 0) return KN_EINVAL;
  if (ntensors == 0 || total_chunks == 0) return KN_OK;
  if (!table) return KN_EINVAL;
  if (total_chunks > 0x7fffffff) return KN_ESIZE;
  opt_kernel<T, F><<<(unsigned)total_chunks, kOptThreads, 0, st>>>(f, table, ntensors, knet_tensor_desc{});
  return launch_status();
}

template <typename T, typename F>
int run_multi_clip(const F& f, const knet_tensor_desc* table, int ntensors, int64_t total_chunks,
                   const double* factors, cudaStream_t st) {
  if (ntensors < 0 || total_chunks < 0) return KN_EINVAL;
  if (ntensors == 0 || total_chunks == 0) return KN_OK;
  if (!table || !factors) return KN_EINVAL;
  if (total_chunks > 0x7fffffff) return KN_ESIZE;
  opt_clip_kernel<T, F><<<(unsigned)total_chunks, kOptThreads, 0, st>>>(f, table, ntensors, factors);
  return launch_status();
}

// ---- per-array gradient norms and clipping factors, without a host round trip ---------------------
// Stage 1: one block per chunk sums g^2 over its chunk.  Stage 2: one block per tensor adds the
// partial sums of its chunks in a fixed order, takes the root, scales by |gscale| and writes
// factor = norm > gclip ? gclip / norm : 1.  Deterministic: no atomics.
template <typename T>
__global__ void __launch_bounds__(kOptThreads)
sumsq_chunks_kernel(const knet_tensor_desc* __restrict__ table, int ntensors, T* __restrict__ partials) {
  __shared__ int s_t;
  __shared__ T red[32];
  const knet_tensor_desc d = table[find_tensor(table, ntensors, blockIdx.x, &s_t)];
  const int64_t start = ((int64_t)blockIdx.x - d.first_chunk) * KNET_MULTI_CHUNK;
  const uint32_t cnt = start < d.n ? (uint32_t)min((int64_t)KNET_MULTI_CHUNK, d.n - start) : 0u;
  const T* g = reinterpret_cast<const T*>(d.p[1]) + start;
  T acc = (T)0;
  segment_visit<T>(g, cnt, threadIdx.x, kOptThreads, [&](T v, uint32_t) { acc += v * v; });
  acc = block_reduce(acc, [](T a, T b) { return a + b; }, (T)0, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

template <typename T>
__global__ void __launch_bounds__(kOptThreads)
clip_factors_kernel(const knet_tensor_desc* __restrict__ table, int ntensors, int64_t total_chunks,
                    const T* __restrict__ partials, double gclip, double gscale, double* __restrict__ factors) {
  __shared__ T red[32];
  const int t = blockIdx.x;
  const int64_t lo = table[t].first_chunk, hi = t + 1 < ntensors ? table[t + 1].first_chunk : total_chunks;
  T acc = (T)0;
  for (int64_t c = lo + threadIdx.x; c < hi; c += kOptThreads) acc += partials[c];
  acc = block_reduce(acc, [](T a, T b) { return a + b; }, (T)0, red);
  if (threadIdx.x == 0) {
    const T gnorm = Math<T>::sqrt(acc) * (T)fabs(gscale);
    factors[t] = (double)gnorm > gclip ? gclip / (double)gnorm : 1.0;
  }
}

template <typename T>
int run_clip_factors(const knet_tensor_desc* table, int ntensors, int64_t total_chunks, double gclip, double gscale,
                     T* partials, double* factors, cudaStream_t st) {
  if (ntensors < 0 || total_chunks < 0 || !(gclip > 0)) return KN_EINVAL;
  if (ntensors == 0) return KN_OK;
  if (!table || !factors || (total_chunks > 0 && !partials)) return KN_EINVAL;
  if (total_chunks > 0x7fffffff) return KN_ESIZE;
  if (total_chunks > 0) sumsq_chunks_kernel<T><<<(unsigned)total_chunks, kOptThreads, 0, st>>>(table, ntensors, partials);
  clip_factors_kernel<T><<<(unsigned)ntensors, kOptThreads, 0, st>>>(table, ntensors, total_chunks, partials, gclip,
                                                                  gscale, factors);
  return launch_status();
}

template <typename T> GScale<T> make_gs(double gscale) { return GScale<T>{(T)gscale, gscale != 1.0}; }

template <typename T> AdamF<T> make_adam(double lr, double beta1, double beta2, double eps, int t, double gscale) {
  AdamF<T> f;
  f.a = (T)(-lr);
  f.e = (T)eps;
  f.c1 = (T)(1 - beta1);
  f.c2 = (T)(1 - beta2);
  f.b1t = (T)(1 - std::pow(beta1, (double)t));
  f.b2t = (T)(1 - std::pow(beta2, (double)t));
  f.beta1 = beta1;
  f.beta2 = beta2;
  f.gs = make_gs<T>(gscale);
  return f;
}

}  // namespace kn

using namespace kn;

KN_EXPORT int64_t knet_multi_plan(knet_tensor_desc* host_table, int ntensors) {
  if (!host_table || ntensors < 0) return KN_EINVAL;
  int64_t c = 0;
  for (int i = 0; i < ntensors; i++) {
    if (host_table[i].n < 0) return KN_EINVAL;
    host_table[i].first_chunk = c;
    c += (host_table[i].n + KNET_MULTI_CHUNK - 1) / KNET_MULTI_CHUNK;
  }
  return c;
}

#define KN_DEF_OPT(f_, S, T)                                                                         \
  KN_EXPORT int knet_sgd_##S(int64_t n, T* w, const T* g, double lr, double gscale, cudaStream_t s) { \
    return run_single<T>(SgdF<T>{(T)(-lr), make_gs<T>(gscale)}, n, w, g, nullptr, nullptr, s);       \
  }                                                                                                  \
  KN_EXPORT int knet_momentum_##S(int64_t n, T* w, const T* g, T* v, double lr, double gamma,        \
                                  double gscale, cudaStream_t s) {                                   \
    return run_single<T>(MomentumF<T>{(T)(-lr), gamma, make_gs<T>(gscale)}, n, w, g, v, nullptr, s); \
  }                                                                                                  \
  KN_EXPORT int knet_nesterov_##S(int64_t n, T* w, const T* g, T* v, double lr, double gamma,        \
                                  double gscale, cudaStream_t s) {                                   \
    return run_single<T>(NesterovF<T>{(T)(-lr), (T)(1 + gamma), gamma, make_gs<T>(gscale)}, n, w, g, \
                         v, nullptr, s);                                                             \
  }                                                                                                  \
  KN_EXPORT int knet_adagrad_##S(int64_t n, T* w, const T* g, T* G, double lr, double eps,           \
                                 double gscale, cudaStream_t s) {                                    \
    return run_single<T>(AdagradF<T>{(T)(-lr), (T)eps, make_gs<T>(gscale)}, n, w, g, G, nullptr, s); \
  }                                                                                                  \
  KN_EXPORT int knet_rmsprop_##S(int64_t n, T* w, const T* g, T* G, double lr, double rho,           \
                                 double eps, double gscale, cudaStream_t s) {                        \
    return run_single<T>(RmspropF<T>{(T)(-lr), (T)eps, (T)(1 - rho), rho, make_gs<T>(gscale)}, n, w, \
                         g, G, nullptr, s);                                                          \
  }                                                                                                  \
  KN_EXPORT int knet_adadelta_##S(int64_t n, T* w, const T* g, T* G, T* delta, double lr,            \
                                  double rho, double eps, double gscale, cudaStream_t s) {           \
    return run_single<T>(AdadeltaF<T>{(T)(-lr), (T)eps, (T)(1 - rho), rho, make_gs<T>(gscale)}, n,   \
                         w, g, G, delta, s);                                                         \
  }                                                                                                  \
  KN_EXPORT int knet_adam_##S(int64_t n, T* w, const T* g, T* m, T* v, double lr, double beta1,      \
                              double beta2, double eps, int t, double gscale, cudaStream_t s) {      \
    if (t < 1) return KN_EINVAL;                                                                     \
    return run_single<T>(make_adam<T>(lr, beta1, beta2, eps, t, gscale), n, w, g, m, v, s);          \
  }                                                                                                  \
  KN_EXPORT int knet_sgd_multi_##S(const knet_tensor_desc* table, int ntensors,                      \
                                   int64_t total_chunks, double lr, double gscale,                   \
                                   cudaStream_t s) {                                                 \
    return run_multi<T>(SgdF<T>{(T)(-lr), make_gs<T>(gscale)}, table, ntensors, total_chunks, s);    \
  }                                                                                                  \
  KN_EXPORT int knet_momentum_multi_##S(const knet_tensor_desc* table, int ntensors,                 \
                                        int64_t total_chunks, double lr, double gamma,               \
                                        double gscale, cudaStream_t s) {                             \
    return run_multi<T>(MomentumF<T>{(T)(-lr), gamma, make_gs<T>(gscale)}, table, ntensors,          \
                        total_chunks, s);                                                            \
  }                                                                                                  \
  KN_EXPORT int knet_adam_multi_##S(const knet_tensor_desc* table, int ntensors,                     \
                                    int64_t total_chunks, double lr, double beta1, double beta2,     \
                                    double eps, int t, double gscale, cudaStream_t s) {              \
    if (t < 1) return KN_EINVAL;                                                                     \
    return run_multi<T>(make_adam<T>(lr, beta1, beta2, eps, t, gscale), table, ntensors,             \
                        total_chunks, s);                                                            \
  }                                                                                                  \
  KN_EXPORT int knet_adam_multi_g_##S(const knet_tensor_desc* table, int ntensors,                   \
                                      int64_t total_chunks, double lr, double beta1, double beta2,   \
                                      double eps, const T* bias_corr, double gscale,                 \
                                      cudaStream_t s) {                                              \
    if (!bias_corr) return KN_EINVAL;                                                                \
    return run_multi<T>(AdamDevF<T>{make_adam<T>(lr, beta1, beta2, eps, 1, gscale), bias_corr},      \
                        table, ntensors, total_chunks, s);                                           \
  }                                                                                                  \
  KN_EXPORT int knet_gclip_factors_##S(const knet_tensor_desc* table, int ntensors,                  \
                                       int64_t total_chunks, double gclip, double gscale,            \
                                       T* partials, double* factors, cudaStream_t s) {               \
    return run_clip_factors<T>(table, ntensors, total_chunks, gclip, gscale, partials, factors, s);  \
  }                                                                                                  \
  KN_EXPORT int knet_sgd_multi_c_##S(const knet_tensor_desc* table, int ntensors,                    \
                                     int64_t total_chunks, double lr, double gscale,                 \
                                     const double* factors, cudaStream_t s) {                        \
    return run_multi_clip<T>(SgdF<T>{(T)(-lr), make_gs<T>(gscale)}, table, ntensors, total_chunks,   \
                             factors, s);                                                            \
  }                                                                                                  \
  KN_EXPORT int knet_momentum_multi_c_##S(const knet_tensor_desc* table, int ntensors,               \
                                          int64_t total_chunks, double lr, double gamma,             \
                                          double gscale, const double* factors, cudaStream_t s) {    \
    return run_multi_clip<T>(MomentumF<T>{(T)(-lr), gamma, make_gs<T>(gscale)}, table, ntensors,     \
                             total_chunks, factors, s);                                              \
  }                                                                                                  \
  KN_EXPORT int knet_adam_multi_c_##S(const knet_tensor_desc* table, int ntensors,                   \
                                      int64_t total_chunks, double lr, double beta1, double beta2,   \
                                      double eps, int t, double gscale, const double* factors,       \
                                      cudaStream_t s) {                                              \
    if (t < 1) return KN_EINVAL;                                                                     \
    return run_multi_clip<T>(make_adam<T>(lr, beta1, beta2, eps, t, gscale), table, ntensors,        \
                             total_chunks, factors, s);                                              \
  }                                                                                                  \
  KN_EXPORT void knet_adam_bias_corr_##S(double beta1, double beta2, int t, T* host_out) {           \
    const AdamF<T> f = make_adam<T>(0.0, beta1, beta2, 0.0, t, 1.0);                                 \
    host_out[0] = f.b1t;                                                                             \
    host_out[1] = f.b2t;                                                                             \
  }
KNET_BOTH_TYPES(KN_DEF_OPT, opt)
