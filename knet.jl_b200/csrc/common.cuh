// Shared helpers for libknet_sm100: 128-bit streaming accesses, launch geometry, and the
// elementwise engine every pointwise kernel (activations, their backward forms, dropout,
// optimizers) is an instance of.  Written for sm_100a only.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <type_traits>

#define KNET_API __attribute__((visibility("default")))
#include "../../include/knet_sm100.h"

#define KN_EXPORT extern "C" __attribute__((visibility("default")))

namespace kn {

// Status codes of the int-returning entry points: 0 ok, negative = bad argument,
// positive = the cudaError_t of the failed runtime call.
enum : int { KN_OK = 0, KN_EINVAL = -1, KN_ESIZE = -2, KN_EWORKSPACE = -3, KN_EALIGN = -4 };

inline int sm_count() {
  // One query per device; the table is only ever written with the same value.
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

inline int launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  return e == cudaSuccess ? KN_OK : (int)e;
}

// ---- 16-byte packs ----------------------------------------------------------------------
template <typename T, int N> struct alignas(sizeof(T) * N) Pack { T v[N]; };

template <typename T> struct VecN { enum { value = 16 / sizeof(T) }; };

template <typename T, int N>
__device__ __forceinline__ Pack<T, N> ld_stream(const T* p) {
  Pack<T, N> r;
  if constexpr (sizeof(T) * N == 16) {
    float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    *reinterpret_cast<float4*>(&r) = t;
  } else if constexpr (sizeof(T) * N == 8) {
    float2 t = __ldcs(reinterpret_cast<const float2*>(p));
    *reinterpret_cast<float2*>(&r) = t;
  } else {
    r.v[0] = __ldcs(p);
  }
  return r;
}
template <typename T, int N>
__device__ __forceinline__ void st_stream(T* p, const Pack<T, N>& v) {
  if constexpr (sizeof(T) * N == 16) {
    __stcs(reinterpret_cast<float4*>(p), *reinterpret_cast<const float4*>(&v));
  } else if constexpr (sizeof(T) * N == 8) {
    __stcs(reinterpret_cast<float2*>(p), *reinterpret_cast<const float2*>(&v));
  } else {
    __stcs(p, v.v[0]);
  }
}

// i / d for i < 2^31 by a multiply-high with a host-computed reciprocal (Granlund-Montgomery
// round-up method: sh = ceil(log2 d), m = floor(2^32 (2^sh - d) / d) + 1,
// q = (mulhi(m, i) + i) >> sh; the sum cannot overflow because i < 2^31).  A 32-bit division
// costs several transcendental-unit instructions, which the division kernels need themselves.
struct FastDiv {
  uint32_t d, m, sh;
};
inline FastDiv fast_div(uint32_t d) {
  FastDiv f{d, 0u, 0u};
  while ((1ull << f.sh) < d) f.sh++;
  f.m = (uint32_t)((((1ull << f.sh) - d) << 32) / d + 1);
  return f;
}
__device__ __forceinline__ uint32_t div_fast(uint32_t i, const FastDiv& f) { return (__umulhi(f.m, i) + i) >> f.sh; }
__device__ __forceinline__ uint32_t mod_fast(uint32_t i, const FastDiv& f) { return i - div_fast(i, f) * f.d; }

// ---- elementwise engine -------------------------------------------------------------------
// out[k][i] = f(in[0][i], ..., in[NIN-1][i]) for i in [0,n).  An output may be the same
// pointer as an input (in-place); partial overlaps are not supported.
template <typename T, int NIN, int NOUT> struct EwPtrs {
  const T* in[NIN > 0 ? NIN : 1];
  T* out[NOUT];
};

constexpr int kEwThreads = 256;

// A functor may declare `static constexpr bool kGroup = true` and a member
// group(const Pack<T,VEC> (&in)[NIN], Pack<T,VEC> (&out)[NOUT]) to handle a 16-byte group at once.
template <typename F, typename = void> struct EwHasGroup : std::false_type {};
template <typename F> struct EwHasGroup<F, std::void_t<decltype(F::kGroup)>> : std::true_type {};

// Body: 16-byte accesses starting at element `head`; head/tail elements are done one by one
// by the first block.  VEC == 1 is the fallback for pointers that do not share an alignment.
template <typename T, int NIN, int NOUT, int VEC, int UNROLL, typename F>
__global__ void __launch_bounds__(kEwThreads)
ew_kernel(F f, EwPtrs<T, NIN, NOUT> p, uint32_t head, uint64_t nvec, uint64_t n) {
  const uint64_t base = (uint64_t)blockIdx.x * (kEwThreads * UNROLL) + threadIdx.x;
  Pack<T, VEC> in[UNROLL][NIN > 0 ? NIN : 1];
#pragma unroll
  for (int u = 0; u < UNROLL; u++) {
    const uint64_t iv = base + (uint64_t)u * kEwThreads;
    if (iv < nvec) {
#pragma unroll
      for (int k = 0; k < NIN; k++) in[u][k] = ld_stream<T, VEC>(p.in[k] + head + iv * VEC);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; u++) {
    const uint64_t iv = base + (uint64_t)u * kEwThreads;
    if (iv < nvec) {
      Pack<T, VEC> out[NOUT];
      if constexpr (EwHasGroup<F>::value) {
        f.group(in[u], out);      // the functor works on the whole 16-byte group
      } else {
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          T a[NIN > 0 ? NIN : 1], r[NOUT];
#pragma unroll
          for (int k = 0; k < NIN; k++) a[k] = in[u][k].v[e];
          f(a, r);
#pragma unroll
          for (int k = 0; k < NOUT; k++) out[k].v[e] = r[k];
        }
      }
#pragma unroll
      for (int k = 0; k < NOUT; k++) st_stream<T, VEC>(p.out[k] + head + iv * VEC, out[k]);
    }
  }
  if (VEC > 1 && blockIdx.x == 0) {
    // ragged ends: [0,head) and [head + nvec*VEC, n)
    const uint64_t tail0 = head + nvec * VEC;
    const uint64_t nrag = head + (n - tail0);
    if (threadIdx.x < nrag) {
      const uint64_t i = threadIdx.x < head ? threadIdx.x : tail0 + (threadIdx.x - head);
      T a[NIN > 0 ? NIN : 1], r[NOUT];
#pragma unroll
      for (int k = 0; k < NIN; k++) a[k] = p.in[k][i];
      f(a, r);
#pragma unroll
      for (int k = 0; k < NOUT; k++) p.out[k][i] = r[k];
    }
  }
}

template <typename T, int NIN, int NOUT, typename F>
inline void ew_launch(F f, const EwPtrs<T, NIN, NOUT>& p, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  constexpr int VEC = VecN<T>::value;
  // Loads in flight per thread: UNROLL * NIN 16-byte vectors; keep that near 8.
  constexpr int UNROLL = (NIN <= 1) ? 4 : (NIN == 2 ? 4 : 2);
  // All pointers must share the same offset inside a 16-byte line for the vector path.
  uintptr_t off = (uintptr_t)p.out[0] & 15;
  bool same = true;
  for (int k = 0; k < NIN; k++) same &= (((uintptr_t)p.in[k] & 15) == off);
  for (int k = 0; k < NOUT; k++) same &= (((uintptr_t)p.out[k] & 15) == off);
  same &= (off % sizeof(T)) == 0;
  if (same) {
    uint64_t head = off ? (16 - off) / sizeof(T) : 0;
    if (head > (uint64_t)n) head = (uint64_t)n;
    const uint64_t nvec = ((uint64_t)n - head) / VEC;
    uint64_t blocks = (nvec + (uint64_t)kEwThreads * UNROLL - 1) / ((uint64_t)kEwThreads * UNROLL);
    if (blocks == 0) blocks = 1;
    ew_kernel<T, NIN, NOUT, VEC, UNROLL, F>
        <<<(unsigned)blocks, kEwThreads, 0, st>>>(f, p, (uint32_t)head, nvec, (uint64_t)n);
  } else {
    constexpr int U1 = 8;
    const uint64_t blocks = ((uint64_t)n + (uint64_t)kEwThreads * U1 - 1) / ((uint64_t)kEwThreads * U1);
    ew_kernel<T, NIN, NOUT, 1, U1, F>
        <<<(unsigned)blocks, kEwThreads, 0, st>>>(f, p, 0u, (uint64_t)n, (uint64_t)n);
  }
}

// ---- warp / block reductions ----------------------------------------------------------------
template <typename T, typename Op>
__device__ __forceinline__ T warp_reduce(T v, Op op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Result valid in every thread.  `smem` must hold 32 values; blockDim.x is a multiple of 32.
template <typename T, typename Op>
__device__ __forceinline__ T block_reduce(T v, Op op, T ident, T* smem) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_reduce(v, op);
  __syncthreads();  // protects smem reuse between consecutive calls
  if (lane == 0) smem[w] = v;
  __syncthreads();
  T r = lane < nw ? smem[lane] : ident;
  r = warp_reduce(r, op);
  return r;
}

}  // namespace kn
