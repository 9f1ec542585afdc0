// softmax / logsoftmax / logsumexp forward and backward, and the fused nll loss, over one
// dim of an array seen as (inner, D, outer).
//
// inner == 1 ("segments", e.g. a (C,B) score matrix with classes along dim 1): every
// instance is a contiguous run of D numbers.  Short runs get a thread or a warp and are
// re-read through L1.  Long runs are staged once in shared memory by a CTA, or by a
// thread-block cluster whose CTAs each hold a slice and exchange their (max, sum) through
// distributed shared memory, so DRAM sees each input exactly once (2 n s bytes forward,
// 3 n s backward) whatever D is, up to 8 slices.
// inner > 1 ("rows", e.g. dims=2): a warp covers 32 adjacent instances per load, the D axis
// is split over threadIdx.y and optionally a cluster; reductions (logsumexp, nll) are single
// pass, the normalising ops read their input a second time.
#include <cstdlib>

#include "reduce.cuh"

namespace kn {

enum : int { FWD_SOFTMAX = 0, FWD_LOGSOFTMAX = 1, FWD_LSE = 2, FWD_NLL = 3, FWD_NLLBWD = 4 };
enum : int { BWD_SOFTMAX = 0, BWD_LOGSOFTMAX = 1 };

// running maximum m and sum of exp(x - m)
template <typename T> struct MS {
  T m, s;
};
template <typename T> __device__ __forceinline__ MS<T> ms_init() { return MS<T>{-Math<T>::inf(), (T)0}; }
template <typename T> __device__ __forceinline__ void ms_push(MS<T>& a, T v) {
  if (v <= a.m) {
    if (v != -Math<T>::inf()) a.s += Math<T>::exp_neg(v - a.m);  // exp(-inf) = 0
  } else {
    a.s = a.s * Math<T>::exp_neg(a.m - v) + (T)1;  // exp(-inf) = 0 on the first element
    a.m = v;
  }
}
// K packs of N values at once (N even): one rescale of the running sum for all of them, the
// maxima in three-input form, the exponentials and their sum two at a time through the
// packed f32x2 forms.  No branch on the data apart from the all -inf case.
template <typename T, int N, int K>
__device__ __forceinline__ void ms_push_packs(MS<T>& a, const Pack<T, N> (&p)[K]) {
  T m = a.m;
#pragma unroll
  for (int k = 0; k < K; k++)
#pragma unroll
    for (int e = 0; e < N; e += 2) m = fmax(fmax(m, p[k].v[e]), p[k].v[e + 1]);
  if (m == -Math<T>::inf()) return;  // nothing but -inf so far: no contribution
  const Two<T> neg = two(-m);
  Two<T> acc = two((T)0);
#pragma unroll
  for (int k = 0; k < K; k++)
#pragma unroll
    for (int e = 0; e < N; e += 2) acc = add2(acc, exp_neg2(add2(Two<T>{p[k].v[e], p[k].v[e + 1]}, neg)));
  a.s = a.s * Math<T>::exp_neg(a.m - m) + (acc.a + acc.b);   // exp(-inf) = 0 on the first finite value
  a.m = m;
}
template <typename T, int N> __device__ __forceinline__ void ms_push_pack(MS<T>& a, const Pack<T, N>& p) {
  const Pack<T, N> one[1] = {p};
  ms_push_packs<T, N, 1>(a, one);
}
template <typename T> __device__ __forceinline__ MS<T> ms_merge(MS<T> a, MS<T> b) {
  if (b.s == (T)0) return a;
  if (a.s == (T)0) return b;
  const T m = a.m > b.m ? a.m : b.m;
  return MS<T>{m, a.s * Math<T>::exp_fast(a.m - m) + b.s * Math<T>::exp_fast(b.m - m)};
}
template <typename T> __device__ __forceinline__ MS<T> ms_shfl_xor(MS<T> a, int o) {
  return MS<T>{__shfl_xor_sync(0xffffffffu, a.m, o), __shfl_xor_sync(0xffffffffu, a.s, o)};
}
template <typename T> __device__ __forceinline__ MS<T> ms_warp(MS<T> a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = ms_merge(a, ms_shfl_xor(a, o));
  return a;
}

// Per-instance extras of the nll modes.
template <typename T> struct NllArgs {
  const int32_t* labels;   // 1-based, 0 = skip
  T* per_instance;         // FWD_NLL: receives lse - x[label] (0 when skipped)
  const int32_t* count;    // FWD_NLLBWD with average
  T dy;
  int average;
};

template <typename T, int MODE>
__device__ __forceinline__ T fwd_value(T v, T m, T s, T logs, T scale, bool is_label) {
  // 1/s is loop-invariant at every call site; the per-element cost is one multiply
  if (MODE == FWD_SOFTMAX) return Math<T>::exp_neg(v - m) * ((T)1 / s);
  if (MODE == FWD_LOGSOFTMAX) return (v - m) - logs;
  // FWD_NLLBWD: (softmax - onehot) * scale
  const T p = Math<T>::exp_neg(v - m) * ((T)1 / s);
  return (is_label ? p - (T)1 : p) * scale;
}

template <typename T>
__device__ __forceinline__ T nll_scale(const NllArgs<T>& a) {
  return a.average ? a.dy / (T)(*a.count) : a.dy;
}

// ---- store a contiguous run with 128-bit stores; f(index) gives the value -----------------------
template <typename T, typename F>
__device__ __forceinline__ void segment_store(T* __restrict__ p, uint32_t len, uint32_t tid, uint32_t nthr, F&& f) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t head = (uint32_t)(((16u - (uint32_t)((uintptr_t)p & 15u)) & 15u) / sizeof(T));
  if (head > len) head = len;
  const uint32_t nvec = (len - head) / VEC;
  const uint32_t tail0 = head + nvec * VEC;
  if (tid < head) p[tid] = f(tid);
  for (uint32_t v = tid; v < nvec; v += nthr) {
    Pack<T, VEC> r;
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) r.v[e] = f(head + v * VEC + e);
    st_stream<T, VEC>(p + head + (size_t)v * VEC, r);
  }
  if (tail0 + tid < len) p[tail0 + tid] = f(tail0 + tid);
}

// =====================================================================================
// segments, short runs: G threads (1 or 32) per instance, input re-read through L1
// =====================================================================================
template <typename T, int MODE, int G>
__global__ void __launch_bounds__(256)
seg_small_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, NllArgs<T> na) {
  const uint32_t seg = (uint32_t)(((uint64_t)blockIdx.x * 256 + threadIdx.x) / G);
  if (seg >= nseg) return;
  const uint32_t lane = threadIdx.x % G;
  const T* xp = x + (uint64_t)seg * D;
  MS<T> ms = ms_init<T>();
  if (G == 1) {
    for (uint32_t d = 0; d < D; d++) ms_push(ms, __ldg(xp + d));
  } else {
    segment_visit_vec4<T>(xp, D, lane, G, [&](const Pack<T, VecN<T>::value> (&p)[4]) { ms_push_packs(ms, p); },
                          [&](const Pack<T, VecN<T>::value>& p) { ms_push_pack(ms, p); }, [&](T v) { ms_push(ms, v); });
    ms = ms_warp(ms);
  }
  const T logs = Math<T>::log(ms.s);
  if (MODE == FWD_LSE) {
    if (lane == 0) y[seg] = ms.m + logs;
    return;
  }
  int32_t label = 0;
  if (MODE == FWD_NLL || MODE == FWD_NLLBWD) label = na.labels[seg];
  if (MODE == FWD_NLL) {
    if (lane == 0) na.per_instance[seg] = label == 0 ? (T)0 : (ms.m + logs) - xp[label - 1];
    return;
  }
  T scale = (T)0;
  if (MODE == FWD_NLLBWD) scale = label == 0 ? (T)0 : nll_scale(na);
  T* yp = y + (uint64_t)seg * D;
  if (G == 1) {
    for (uint32_t d = 0; d < D; d++)
      yp[d] = fwd_value<T, MODE>(xp[d], ms.m, ms.s, logs, scale, (int32_t)(d + 1) == label);
  } else {
    segment_store<T>(yp, D, lane, G, [&](uint32_t d) {
      return fwd_value<T, MODE>(xp[d], ms.m, ms.s, logs, scale, (int32_t)(d + 1) == label);
    });
  }
}

template <typename T, int MODE, int G>
__global__ void __launch_bounds__(256)
seg_small_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D, uint32_t nseg) {
  const uint32_t seg = (uint32_t)(((uint64_t)blockIdx.x * 256 + threadIdx.x) / G);
  if (seg >= nseg) return;
  const uint32_t lane = threadIdx.x % G;
  const T* yp = y + (uint64_t)seg * D;
  const T* gp = dy + (uint64_t)seg * D;
  T acc = (T)0;
  for (uint32_t d = lane; d < D; d += G) acc += MODE == BWD_SOFTMAX ? yp[d] * gp[d] : gp[d];
  if (G > 1) acc = warp_reduce(acc, [](T a, T b) { return a + b; });
  T* xp = dx + (uint64_t)seg * D;
  for (uint32_t d = lane; d < D; d += G) {
    const T yv = yp[d], gv = gp[d];
    xp[d] = MODE == BWD_SOFTMAX ? yv * gv - yv * acc : gv - Math<T>::exp_neg(yv) * acc;
  }
}

// =====================================================================================
// segments, short Float32 runs held in registers: a group of G = 8, 16 or 32 lanes per
// instance, the whole run loaded once with 16-byte accesses (NP packs per lane); maximum,
// sum and the output come from registers.  The run may start anywhere inside a 16-byte line:
// packs are taken from the aligned address below it, and the (at most two) packs that
// straddle an end of the run are handled element by element.  All arrays of a call must
// share their offset within a 16-byte line.  Float64 uses these kernels for forward runs of
// up to 128 elements only (fewer merge steps than a whole warp per instance needs); beyond
// that its exponentials bound the time and the registers spent on the run cost more in
// occupancy than the second read through L1 does.
// =====================================================================================
template <typename T, int NP, int G>
__device__ __forceinline__ void group_run_load(const T* __restrict__ base, uint32_t mis, uint32_t total, uint32_t lane,
                                               Pack<T, VecN<T>::value> (&v)[NP], T fill) {
  constexpr uint32_t VEC = VecN<T>::value;
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
    if (e0 >= mis && e0 + VEC <= total) {
      v[j] = ld_stream<T, VEC>(base + e0);
    } else {
#pragma unroll
      for (uint32_t e = 0; e < VEC; e++) {
        const uint32_t i = e0 + e;
        v[j].v[e] = (i >= mis && i < total) ? __ldg(base + i) : fill;
      }
    }
  }
}
template <typename T, int NP, int G, typename F>
__device__ __forceinline__ void group_run_store(T* __restrict__ base, uint32_t mis, uint32_t total, uint32_t lane, F&& f) {
  constexpr uint32_t VEC = VecN<T>::value;
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
    if (e0 >= mis && e0 + VEC <= total) {
      Pack<T, VEC> r;
#pragma unroll
      for (uint32_t e = 0; e < VEC; e++) r.v[e] = f(j, e, e0 + e - mis);
      st_stream<T, VEC>(base + e0, r);
    } else {
#pragma unroll
      for (uint32_t e = 0; e < VEC; e++) {
        const uint32_t i = e0 + e;
        if (i >= mis && i < total) base[i] = f(j, e, i - mis);
      }
    }
  }
}

// Groups past the last instance keep running with an empty run (no load, no store): every lane of
// the warp takes part in the shuffles.
template <typename T, int MODE, int NP, int G>
__global__ void __launch_bounds__(256)
seg_group_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, NllArgs<T> na) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t seg = (uint32_t)(((uint64_t)blockIdx.x * 256 + threadIdx.x) / G);
  const bool live = seg < nseg;
  if (!live) seg = 0;
  const uint32_t lane = threadIdx.x % G;
  const T* xp = x + (uint64_t)seg * D;
  const uint32_t mis = (uint32_t)(((uintptr_t)xp & 15u) / sizeof(T));
  const uint32_t total = mis + (live ? D : 0);
  Pack<T, VEC> v[NP];
  group_run_load<T, NP, G>(xp - mis, mis, total, lane, v, -Math<T>::inf());
  // the group's maximum first (shuffles of one number), then every lane sums exp(v - m) against it:
  // merging per-lane (max, sum) pairs instead costs two exponentials per lane and shuffle step, as
  // many as the run itself has for short runs (logsumexp of 64-element runs: 31 us against 20 us for
  // their plain sum)
  T m = -Math<T>::inf();
#pragma unroll
  for (int j = 0; j < NP; j++)
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) m = fmax(m, v[j].v[e]);
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
  MS<T> ms{m, (T)0};
  ms_push_packs<T, (int)VEC, NP>(ms, v);       // every value <= m: a plain sum; positions outside the run hold -inf: exp = 0
  T s = ms.s;
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const T logs = Math<T>::log(s);
  if (!live) return;
  if (MODE == FWD_LSE) {
    if (lane == 0) y[seg] = m + logs;
    return;
  }
  int32_t label = 0;
  if (MODE == FWD_NLL || MODE == FWD_NLLBWD) label = na.labels[seg];
  if (MODE == FWD_NLL) {
    if (lane == 0) na.per_instance[seg] = label == 0 ? (T)0 : (m + logs) - xp[label - 1];
    return;
  }
  T scale = (T)0;
  if (MODE == FWD_NLLBWD) scale = label == 0 ? (T)0 : nll_scale(na);
  T* yp = y + (uint64_t)seg * D;
  group_run_store<T, NP, G>(yp - mis, mis, total, lane, [&](int j, uint32_t e, uint32_t d) {
    return fwd_value<T, MODE>(v[j].v[e], m, s, logs, scale, (int32_t)(d + 1) == label);
  });
}

template <typename T, int MODE, int NP, int G>
__global__ void __launch_bounds__(256)
seg_group_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D, uint32_t nseg) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t seg = (uint32_t)(((uint64_t)blockIdx.x * 256 + threadIdx.x) / G);
  const bool live = seg < nseg;
  if (!live) seg = 0;
  const uint32_t lane = threadIdx.x % G;
  const T* yp = y + (uint64_t)seg * D;
  const uint32_t mis = (uint32_t)(((uintptr_t)yp & 15u) / sizeof(T));
  const uint32_t total = mis + (live ? D : 0);
  Pack<T, VEC> a[NP], g[NP];
  group_run_load<T, NP, G>(yp - mis, mis, total, lane, a, (T)0);
  group_run_load<T, NP, G>(dy + (uint64_t)seg * D - mis, mis, total, lane, g, (T)0);
  T acc = (T)0;
#pragma unroll
  for (int j = 0; j < NP; j++)
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) acc += MODE == BWD_SOFTMAX ? a[j].v[e] * g[j].v[e] : g[j].v[e];   // 0 outside the run
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  group_run_store<T, NP, G>(dx + (uint64_t)seg * D - mis, mis, total, lane, [&](int j, uint32_t e, uint32_t) {
    const T yv = a[j].v[e], gv = g[j].v[e];
    return MODE == BWD_SOFTMAX ? yv * gv - yv * acc : gv - Math<T>::exp_neg(yv) * acc;
  });
}

// Float64 takes the lane-group kernels for forward runs of up to 128 elements only.
template <typename T> inline GroupGeom softmax_group_geometry(const void* p, int64_t D, bool backward) {
  if (sizeof(T) == 4) return group_geometry<T>(p, D, backward ? 8 : 16);
  if (backward) return {0, 0};
  const GroupGeom g = group_geometry<T>(p, D, 4);
  return g.g == 32 ? GroupGeom{0, 0} : g;
}

// =====================================================================================
// segments, long runs: one CTA, or a cluster of `cs` CTAs, per instance; slice staged in
// shared memory (STAGE) or, for reductions and oversize runs, streamed.
// =====================================================================================
constexpr int kSegSoftThreads = 512;

template <typename T>
__device__ __forceinline__ MS<T> ms_block(MS<T> a, MS<T>* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  a = ms_warp(a);
  __syncthreads();
  if (lane == 0) red[w] = a;
  __syncthreads();
  MS<T> r = lane < nw ? red[lane] : ms_init<T>();
  return ms_warp(r);
}

template <typename T, int MODE, bool STAGE>
__global__ void __launch_bounds__(kSegSoftThreads)
seg_big_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t cs, NllArgs<T> na) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* buf = reinterpret_cast<T*>(smem_raw);
  __shared__ MS<T> red[32];
  __shared__ MS<T> mine;
  const uint32_t seg = blockIdx.x;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, blockIdx.y * slice), a1 = min(D, a0 + slice), len = a1 - a0;
  const T* xp = x + (uint64_t)seg * D + a0;
  MS<T> ms = ms_init<T>();
  if (STAGE) {
    // pass over DRAM: stage and find the maximum; pass over shared memory: sum of exp
    T mx = -Math<T>::inf();
    segment_visit<T>(xp, len, threadIdx.x, kSegSoftThreads, [&](T v, uint32_t i) {
      buf[i] = v;
      mx = v > mx ? v : mx;
    });
    mx = block_reduce(mx, [](T a, T b) { return a > b ? a : b; }, -Math<T>::inf(), reinterpret_cast<T*>(red));
    T s = (T)0;
    for (uint32_t i = threadIdx.x; i < len; i += kSegSoftThreads) s += Math<T>::exp_fast(buf[i] - mx);
    s = block_reduce(s, [](T a, T b) { return a + b; }, (T)0, reinterpret_cast<T*>(red));
    ms = MS<T>{mx, s};
  } else {
    segment_visit_vec4<T>(xp, len, threadIdx.x, kSegSoftThreads,
                          [&](const Pack<T, VecN<T>::value> (&p)[4]) { ms_push_packs(ms, p); },
                          [&](const Pack<T, VecN<T>::value>& p) { ms_push_pack(ms, p); }, [&](T v) { ms_push(ms, v); });
    ms = ms_block(ms, red);
  }
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) mine = ms;
    cluster.sync();
    MS<T> tot = ms_init<T>();
    for (uint32_t r = 0; r < cs; r++) tot = ms_merge(tot, *cluster.map_shared_rank(&mine, r));
    cluster.sync();
    ms = tot;
  }
  const T logs = Math<T>::log(ms.s);
  if (MODE == FWD_LSE) {
    if (threadIdx.x == 0 && blockIdx.y == 0) y[seg] = ms.m + logs;
    return;
  }
  int32_t label = 0;
  if (MODE == FWD_NLL || MODE == FWD_NLLBWD) label = na.labels[seg];
  if (MODE == FWD_NLL) {
    if (threadIdx.x == 0 && blockIdx.y == 0)
      na.per_instance[seg] = label == 0 ? (T)0 : (ms.m + logs) - x[(uint64_t)seg * D + (label - 1)];
    return;
  }
  T scale = (T)0;
  if (MODE == FWD_NLLBWD) scale = label == 0 ? (T)0 : nll_scale(na);
  T* yp = y + (uint64_t)seg * D + a0;
  const int32_t lab_local = label - 1 - (int32_t)a0;
  segment_store<T>(yp, len, threadIdx.x, kSegSoftThreads, [&](uint32_t i) {
    const T v = STAGE ? buf[i] : xp[i];
    return fwd_value<T, MODE>(v, ms.m, ms.s, logs, scale, (int32_t)i == lab_local);
  });
}

template <typename T, int MODE, bool STAGE>
__global__ void __launch_bounds__(kSegSoftThreads)
seg_big_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D, uint32_t cs) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ T red[32];
  __shared__ T mine;
  const uint32_t seg = blockIdx.x;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, blockIdx.y * slice), a1 = min(D, a0 + slice), len = a1 - a0;
  T* ybuf = reinterpret_cast<T*>(smem_raw);
  T* gbuf = ybuf + slice;
  const T* yp = y + (uint64_t)seg * D + a0;
  const T* gp = dy + (uint64_t)seg * D + a0;
  T acc = (T)0;
  if (STAGE) {
    segment_visit<T>(yp, len, threadIdx.x, kSegSoftThreads, [&](T v, uint32_t i) { ybuf[i] = v; });
    segment_visit<T>(gp, len, threadIdx.x, kSegSoftThreads, [&](T v, uint32_t i) { gbuf[i] = v; });
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < len; i += kSegSoftThreads)
      acc += MODE == BWD_SOFTMAX ? ybuf[i] * gbuf[i] : gbuf[i];
  } else {
    for (uint32_t i = threadIdx.x; i < len; i += kSegSoftThreads)
      acc += MODE == BWD_SOFTMAX ? yp[i] * gp[i] : gp[i];
  }
  acc = block_reduce(acc, [](T a, T b) { return a + b; }, (T)0, red);
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) mine = acc;
    cluster.sync();
    T tot = (T)0;
    for (uint32_t r = 0; r < cs; r++) tot += *cluster.map_shared_rank(&mine, r);
    cluster.sync();
    acc = tot;
  }
  T* xp = dx + (uint64_t)seg * D + a0;
  segment_store<T>(xp, len, threadIdx.x, kSegSoftThreads, [&](uint32_t i) {
    const T yv = STAGE ? ybuf[i] : yp[i], gv = STAGE ? gbuf[i] : gp[i];
    return MODE == BWD_SOFTMAX ? yv * gv - yv * acc : gv - Math<T>::exp_neg(yv) * acc;
  });
}

// =====================================================================================
// rows layout (inner > 1)
// =====================================================================================
// A CTA of 32 x WY threads owns 32*RV adjacent instances (rows); thread (lx, ly) owns RV of them
// and the columns ly, ly+WY, ... of the CTA's slice of the D axis (a cluster splits D when there
// are too few row tiles to fill the GPU).  A thread loads NP columns at a time (NP independent
// loads of RV elements in flight).  When the slice has at most WY*NP columns the values stay in
// registers for the output pass; longer slices are read a second time (plain loads in the first
// pass, so that L2 keeps what it can).  Measured on 32768 x 1000 Float32 (fractions of the copy
// rate on 2n / 3n bytes): forward 0.70, backward 0.68, against 0.37 / 0.53 with one row and four
// 4-byte loads per thread.  Holding whole slices in registers through clusters (NP = 16, cluster
// of 4 or 8) measured worse: one CTA of 512 threads per SM, gang-scheduled, 0.43 at best.
constexpr int kRowSoftWY = 16;          // warps per CTA of the normalising kernels (8 and 4 measured slower)
constexpr int kRowReduceWY = 16;        // and of the reduce-only kernel
constexpr int kRowPacksFwd = 8, kRowPacksBwd = 8;   // 4 columns per round measured 0-20 % slower in either kernel

template <typename T, int N> __device__ __forceinline__ Pack<T, N> ld_keep_l2(const T* p) {
  Pack<T, N> r;
  if constexpr (sizeof(T) * N == 16) *reinterpret_cast<float4*>(&r) = *reinterpret_cast<const float4*>(p);
  else if constexpr (sizeof(T) * N == 8) *reinterpret_cast<float2*>(&r) = *reinterpret_cast<const float2*>(p);
  else r.v[0] = *p;
  return r;
}

template <typename T, int MODE, int RV>
__global__ void __launch_bounds__(32 * kRowSoftWY, (sizeof(T) == 4 ? 2 : 1))
rows_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t inner, uint32_t D, uint32_t dper,
                uint32_t cs, NllArgs<T> na) {
  static_assert(MODE == FWD_SOFTMAX || MODE == FWD_LOGSOFTMAX || MODE == FWD_NLLBWD, "normalising modes");
  constexpr int WY = kRowSoftWY, NP = kRowPacksFwd;
  __shared__ MS<T> part[WY][32 * RV];
  __shared__ MS<T> total[32 * RV];
  __shared__ MS<T> merged[32 * RV];
  const uint32_t lx = threadIdx.x, ly = threadIdx.y;
  const uint32_t a = (blockIdx.x * 32 + lx) * RV;
  const bool valid = a < inner;
  const uint64_t base = (uint64_t)blockIdx.z * inner * D + a;
  const uint32_t d0 = min(D, blockIdx.y * dper), d1 = min(D, d0 + dper);
  const bool single = d1 - d0 <= (uint32_t)(WY * NP);
  Pack<T, RV> v[NP];
  MS<T> ms[RV];
#pragma unroll
  for (int e = 0; e < RV; e++) ms[e] = ms_init<T>();
  auto load_round = [&](uint32_t r0, bool keep) {
#pragma unroll
    for (int k = 0; k < NP; k++) {
      const uint32_t d = r0 + ly + k * WY;
      if (d < d1) {
        const T* p = x + base + (uint64_t)d * inner;
        v[k] = keep ? ld_keep_l2<T, RV>(p) : ld_stream<T, RV>(p);
      } else {
#pragma unroll
        for (int e = 0; e < RV; e++) v[k].v[e] = -Math<T>::inf();
      }
    }
  };
  auto push_round = [&]() {
#pragma unroll
    for (int e = 0; e < RV; e++) {
      Pack<T, NP> col;
#pragma unroll
      for (int k = 0; k < NP; k++) col.v[k] = v[k].v[e];
      ms_push_pack<T, NP>(ms[e], col);
    }
  };
  if (valid) {
    if (single) {
      load_round(d0, false);
      push_round();
    } else {
      for (uint32_t r0 = d0; r0 < d1; r0 += WY * NP) {
        load_round(r0, true);
        push_round();
      }
    }
  }
#pragma unroll
  for (int e = 0; e < RV; e++) part[ly][lx * RV + e] = ms[e];
  __syncthreads();
  if (ly < RV) {          // warp e merges the column groups of row e of every thread
    MS<T> t = part[0][lx * RV + ly];
#pragma unroll
    for (int k = 1; k < WY; k++) t = ms_merge(t, part[k][lx * RV + ly]);
    total[lx * RV + ly] = t;
  }
  MS<T> fin[RV];
  if (cs > 1) {
    // one warp per row slot fetches the other CTAs' partials (remote shared memory is slow: RV warps
    // read it, not all sixteen), everyone then reads the merged table locally
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (ly < RV) {
      MS<T> t = ms_init<T>();
      for (uint32_t r = 0; r < cs; r++) t = ms_merge(t, cluster.map_shared_rank(total, r)[lx * RV + ly]);
      merged[lx * RV + ly] = t;
    }
    cluster.sync();   // also orders merged[] within the CTA; peers keep total[] alive until here
#pragma unroll
    for (int e = 0; e < RV; e++) fin[e] = merged[lx * RV + e];
  } else {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < RV; e++) fin[e] = total[lx * RV + e];
  }
  if (!valid) return;
  const uint64_t inst = (uint64_t)blockIdx.z * inner + a;
  T logs[RV];
#pragma unroll
  for (int e = 0; e < RV; e++) logs[e] = Math<T>::log(fin[e].s);
  int32_t label[RV];
  T scale[RV];
#pragma unroll
  for (int e = 0; e < RV; e++) {
    label[e] = MODE == FWD_NLLBWD ? na.labels[inst + e] : 0;
    scale[e] = (MODE == FWD_NLLBWD && label[e] != 0) ? nll_scale(na) : (T)0;
  }
  auto store_round = [&](uint32_t r0) {
#pragma unroll
    for (int k = 0; k < NP; k++) {
      const uint32_t d = r0 + ly + k * WY;
      if (d < d1) {
        Pack<T, RV> r;
#pragma unroll
        for (int e = 0; e < RV; e++)
          r.v[e] = fwd_value<T, MODE>(v[k].v[e], fin[e].m, fin[e].s, logs[e], scale[e], (int32_t)(d + 1) == label[e]);
        st_stream<T, RV>(y + base + (uint64_t)d * inner, r);
      }
    }
  };
  if (single) {
    store_round(d0);
  } else {
    for (uint32_t r0 = d0; r0 < d1; r0 += WY * NP) {
      load_round(r0, false);
      store_round(r0);
    }
  }
}

template <typename T, int MODE, int RV>
__global__ void __launch_bounds__(32 * kRowSoftWY)
rows_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t inner,
                uint32_t D, uint32_t dper, uint32_t cs) {
  constexpr int WY = kRowSoftWY, NP = kRowPacksBwd;
  __shared__ T part[WY][32 * RV];
  __shared__ T total[32 * RV];
  __shared__ T merged[32 * RV];
  const uint32_t lx = threadIdx.x, ly = threadIdx.y;
  const uint32_t a = (blockIdx.x * 32 + lx) * RV;
  const bool valid = a < inner;
  const uint64_t base = (uint64_t)blockIdx.z * inner * D + a;
  const uint32_t d0 = min(D, blockIdx.y * dper), d1 = min(D, d0 + dper);
  const bool single = d1 - d0 <= (uint32_t)(WY * NP);
  Pack<T, RV> yv[NP], gv[NP];
  T acc[RV];
#pragma unroll
  for (int e = 0; e < RV; e++) acc[e] = (T)0;
  auto load_round = [&](uint32_t r0, bool keep) {
#pragma unroll
    for (int k = 0; k < NP; k++) {
      const uint32_t d = r0 + ly + k * WY;
      if (d < d1) {
        const uint64_t i = base + (uint64_t)d * inner;
        yv[k] = keep ? ld_keep_l2<T, RV>(y + i) : ld_stream<T, RV>(y + i);
        gv[k] = keep ? ld_keep_l2<T, RV>(dy + i) : ld_stream<T, RV>(dy + i);
      } else {
#pragma unroll
        for (int e = 0; e < RV; e++) yv[k].v[e] = gv[k].v[e] = (T)0;
      }
    }
  };
  auto push_round = [&]() {
#pragma unroll
    for (int k = 0; k < NP; k++)
#pragma unroll
      for (int e = 0; e < RV; e++) acc[e] += MODE == BWD_SOFTMAX ? yv[k].v[e] * gv[k].v[e] : gv[k].v[e];
  };
  if (valid) {
    if (single) {
      load_round(d0, false);
      push_round();
    } else {
      for (uint32_t r0 = d0; r0 < d1; r0 += WY * NP) {
        load_round(r0, true);
        push_round();
      }
    }
  }
#pragma unroll
  for (int e = 0; e < RV; e++) part[ly][lx * RV + e] = acc[e];
  __syncthreads();
  if (ly < RV) {
    T t = part[0][lx * RV + ly];
#pragma unroll
    for (int k = 1; k < WY; k++) t += part[k][lx * RV + ly];
    total[lx * RV + ly] = t;
  }
  T fin[RV];
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (ly < RV) {
      T t = (T)0;
      for (uint32_t r = 0; r < cs; r++) t += cluster.map_shared_rank(total, r)[lx * RV + ly];
      merged[lx * RV + ly] = t;
    }
    cluster.sync();
#pragma unroll
    for (int e = 0; e < RV; e++) fin[e] = merged[lx * RV + e];
  } else {
    __syncthreads();
#pragma unroll
    for (int e = 0; e < RV; e++) fin[e] = total[lx * RV + e];
  }
  if (!valid) return;
  auto store_round = [&](uint32_t r0) {
#pragma unroll
    for (int k = 0; k < NP; k++) {
      const uint32_t d = r0 + ly + k * WY;
      if (d < d1) {
        Pack<T, RV> r;
#pragma unroll
        for (int e = 0; e < RV; e++) {
          const T a1 = yv[k].v[e], g1 = gv[k].v[e];
          r.v[e] = MODE == BWD_SOFTMAX ? a1 * g1 - a1 * fin[e] : g1 - Math<T>::exp_neg(a1) * fin[e];
        }
        st_stream<T, RV>(dx + base + (uint64_t)d * inner, r);
      }
    }
  };
  if (single) {
    store_round(d0);
  } else {
    for (uint32_t r0 = d0; r0 < d1; r0 += WY * NP) {
      load_round(r0, false);
      store_round(r0);
    }
  }
}

// logsumexp and the nll loss need one pass and write one number per instance: one row per thread
// and four loads in flight measured faster there than the wide form above (8192 x 4096 Float32:
// 0.66 against 0.44 of the copy rate), so the reduce-only modes keep this kernel.
template <typename T, int MODE>
__global__ void __launch_bounds__(32 * kRowReduceWY)
rows_reduce_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t inner, uint32_t D, uint32_t dper,
                   uint32_t cs, NllArgs<T> na) {
  static_assert(MODE == FWD_LSE || MODE == FWD_NLL, "reduce-only modes");
  __shared__ MS<T> part[kRowReduceWY][32];
  __shared__ MS<T> total[32];
  const uint32_t lx = threadIdx.x, ly = threadIdx.y;
  const uint32_t a = blockIdx.x * 32 + lx;
  const bool valid = a < inner;
  const uint64_t base = (uint64_t)blockIdx.z * inner * D + a;
  const uint32_t d0 = min(D, blockIdx.y * dper), d1 = min(D, d0 + dper);
  MS<T> ms = ms_init<T>();
  if (valid) {
    uint32_t d = d0 + ly;
    for (; d + 3 * kRowReduceWY < d1; d += 4 * kRowReduceWY) {
      Pack<T, 4> v;
#pragma unroll
      for (int k = 0; k < 4; k++) v.v[k] = __ldcs(x + base + (uint64_t)(d + k * kRowReduceWY) * inner);
      ms_push_pack(ms, v);
    }
    for (; d < d1; d += kRowReduceWY) ms_push(ms, __ldcs(x + base + (uint64_t)d * inner));
  }
  part[ly][lx] = ms;
  __syncthreads();
  if (ly == 0) {
    MS<T> t = part[0][lx];
    for (int k = 1; k < kRowReduceWY; k++) t = ms_merge(t, part[k][lx]);
    total[lx] = t;
  }
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (blockIdx.y == 0 && ly == 0) {
      MS<T> t = total[lx];
      for (uint32_t r = 1; r < cs; r++) t = ms_merge(t, cluster.map_shared_rank(total, r)[lx]);
      total[lx] = t;
    }
    cluster.sync();   // peers keep their table alive until rank 0 has read it
  }
  if (!(valid && ly == 0 && blockIdx.y == 0)) return;
  const MS<T> fin = total[lx];
  const T lse = fin.m + Math<T>::log(fin.s);
  const uint64_t inst = (uint64_t)blockIdx.z * inner + a;
  if (MODE == FWD_LSE) {
    y[inst] = lse;
  } else {
    const int32_t label = na.labels[inst];
    na.per_instance[inst] = label == 0 ? (T)0 : lse - x[base + (uint64_t)(label - 1) * inner];
  }
}

// Geometry of the rows kernels: the widest row vector (16 bytes down to one element) that the pointers
// and `inner` allow and that still gives about two CTAs per SM with a cluster of 4 (wider vectors
// behind clusters of 8 measured slower on 4096 rows); then the smallest cluster that reaches that count.
struct RowSoftGeom {
  uint32_t rv, tiles, cs, dper;
};
template <typename T>
inline RowSoftGeom rows_soft_geometry(uintptr_t ptr_bits, int64_t inner, int64_t D, int64_t outer, int sms) {
  constexpr uint32_t VEC = VecN<T>::value;
  RowSoftGeom g{1u, (uint32_t)((inner + 31) / 32), 1u, 0u};
  for (uint32_t rv = VEC; rv > 1; rv /= 2) {
    if (inner % rv != 0 || (ptr_bits % (rv * sizeof(T))) != 0) continue;
    const uint64_t tiles = (uint64_t)((inner + 32 * rv - 1) / (32 * rv));
    if (tiles * (uint64_t)outer * 4 >= (uint64_t)2 * sms) {
      g.rv = rv;
      g.tiles = (uint32_t)tiles;
      break;
    }
  }
  static const int forced_rv = [] { const char* e = getenv("KNET_SM100_ROWSOFT_RV"); return e ? atoi(e) : 0; }();   // tuning knobs
  static const int forced_cs = [] { const char* e = getenv("KNET_SM100_ROWSOFT_CS"); return e ? atoi(e) : 0; }();
  if ((forced_rv == 1 || forced_rv == 2 || forced_rv == 4) && (uint32_t)forced_rv <= g.rv) {
    g.rv = (uint32_t)forced_rv;
    g.tiles = (uint32_t)((inner + 32 * g.rv - 1) / (32 * g.rv));
  }
  if (forced_cs == 1 || forced_cs == 2 || forced_cs == 4 || forced_cs == 8) {
    g.cs = (uint32_t)forced_cs;
    g.dper = (uint32_t)((D + g.cs - 1) / g.cs);
    return g;
  }
  while (g.cs < 8 && D >= (int64_t)4 * kRowSoftWY * g.cs && (uint64_t)g.tiles * outer * g.cs < (uint64_t)2 * sms)
    g.cs *= 2;
  g.dper = (uint32_t)((D + g.cs - 1) / g.cs);
  return g;
}

}  // namespace kn

#include "softmax_tma.cuh"

namespace kn {

// ---- launch logic --------------------------------------------------------------------------------
// Threads per CTA of the staged kernels, as threads*10 + 2 (two stages).  The environment
// variables KNET_SM100_TMA_FWD (1282 | 2562) and KNET_SM100_TMA_BWD (2562 | 5122) override the
// defaults for tuning runs.
inline int tma_variant(const char* env, int dflt) {
  const char* e = getenv(env);
  const int req = e ? atoi(e) : 0;
  switch (req) {
    case 1282: case 1283: case 1284: case 2562: case 2563: case 2564: case 5122: case 5123: return req;
    default: return dflt;
  }
}
inline int tma_fwd_variant() { return tma_variant("KNET_SM100_TMA_FWD", 2562); }
// How the CTAs of a cluster exchange their partial results: 1 = remote stores that signal the
// receiver's mbarrier (st.async), 0 = plain remote stores and a cluster-wide barrier.
// KNET_SM100_TMA_XCHG overrides for tuning runs.
inline uint32_t tma_xchg() {
  static const uint32_t v = [] {
    const char* e = getenv("KNET_SM100_TMA_XCHG");
    return e ? (uint32_t)atoi(e) : 1u;
  }();
  return v;
}

template <typename K> inline void allow_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

inline bool fits_u32(int64_t v) { return v >= 0 && v < ((int64_t)1 << 32); }

template <typename T, int MODE>
int run_fwd(const T* x, T* y, int64_t inner, int64_t D, int64_t outer, NllArgs<T> na, cudaStream_t st) {
  if (inner < 0 || D < 0 || outer < 0) return KN_EINVAL;
  if (inner == 0 || D == 0 || outer == 0) return KN_OK;
  if (!fits_u32(inner) || !fits_u32(D) || !fits_u32(outer) || !fits_u32(inner * outer)) return KN_ESIZE;
  const int sms = sm_count();
  if (inner == 1) {
    const uint32_t nseg = (uint32_t)outer;
    if (D <= 32) {
      seg_small_fwd_kernel<T, MODE, 1><<<(nseg + 255) / 256, 256, 0, st>>>(x, y, (uint32_t)D, nseg, na);
    } else if (D <= 2048 && nseg >= (uint32_t)sms) {
      // register-resident form when x and y share their 16-byte offset
      const bool same = y == nullptr || (((uintptr_t)x ^ (uintptr_t)y) & 15) == 0;
      const GroupGeom gg = same ? softmax_group_geometry<T>(x, D, false) : GroupGeom{0, 0};
      const unsigned g = (nseg + 7) / 8;
      bool done = false;
#define KN_GROUP_FWD(G_, NP_)                                                                            \
  if (gg.g == G_ && gg.np == NP_) {                                                                      \
    seg_group_fwd_kernel<T, MODE, NP_, G_><<<(unsigned)(((uint64_t)nseg * G_ + 255) / 256), 256, 0, st>>>(x, y, (uint32_t)D, nseg, na); \
    done = true;                                                                                         \
  }
      KN_GROUP_FWD(8, 2) KN_GROUP_FWD(8, 4) KN_GROUP_FWD(16, 4)
      if constexpr (sizeof(T) == 4) {
        KN_GROUP_FWD(32, 4) KN_GROUP_FWD(32, 8) KN_GROUP_FWD(32, 16)
      }
#undef KN_GROUP_FWD
      if (!done)
        seg_small_fwd_kernel<T, MODE, 32><<<g, 256, 0, st>>>(x, y, (uint32_t)D, nseg, na);
    } else {
      constexpr bool reduce_only = (MODE == FWD_LSE || MODE == FWD_NLL);
      // normalising ops: staged once in shared memory by bulk copies, NS-deep pipeline
      constexpr int M2 = reduce_only ? FWD_SOFTMAX : MODE;
      // 256 threads per CTA unless KNET_SM100_TMA_FWD=128 (tuning runs); each thread keeps at
      // most 16 packs of 16 bytes in registers, which bounds the slice a CTA can take
      const int nthr = tma_fwd_variant() / 10 == 128 ? 128 : 256;
      const size_t max_slice = (size_t)16 * 16 * nthr;
      TmaPlan p{};
      if (!reduce_only) p = plan_tma<T>((uint64_t)D, nseg, 1, nthr, 2, sms, max_slice);
      if (p.ok) {
        const uint64_t slice = ((uint64_t)D + p.cs - 1) / p.cs, nvec = slice / VecN<T>::value;
        const uint64_t per_lane = ((nvec + nthr / 32 - 1) / (nthr / 32) + 31) / 32;   // packs per thread
        auto go = [&](auto kernel) {
          allow_smem(kernel, p.smem);
          p.clusters = min(p.clusters, (uint32_t)max_active_clusters(kernel, dim3(nthr), p.smem, p.cs));
          launch_cluster(kernel, dim3(p.clusters, p.cs), dim3(nthr), p.smem, st, p.cs, x, y, (uint32_t)D, nseg,
                         p.cs, p.stage_elems, na, tma_xchg());
        };
        if (nthr == 128) {
          if (per_lane <= 4) go(seg_tma_fwd_kernel<T, M2, 128, 4>);
          else if (per_lane <= 8) go(seg_tma_fwd_kernel<T, M2, 128, 8>);
          else if (per_lane <= 13) go(seg_tma_fwd_kernel<T, M2, 128, 13>);
          else go(seg_tma_fwd_kernel<T, M2, 128, 16>);
        } else {
          if (per_lane <= 4) go(seg_tma_fwd_kernel<T, M2, 256, 4>);
          else if (per_lane <= 8) go(seg_tma_fwd_kernel<T, M2, 256, 8>);
          else if (per_lane <= 13) go(seg_tma_fwd_kernel<T, M2, 256, 13>);   // a 50257-long run over 4 CTAs
          else go(seg_tma_fwd_kernel<T, M2, 256, 16>);
        }
      } else {
        // reductions (one streaming pass) and runs too long to stage (a second read)
        const uint32_t cs = seg_cluster_size(nseg, (uint64_t)D);
        launch_cluster(seg_big_fwd_kernel<T, MODE, false>, dim3(nseg, cs), dim3(kSegSoftThreads), 0, st, cs,
                       x, y, (uint32_t)D, cs, na);
      }
    }
  } else {
    if (outer > 65535) return KN_ESIZE;
    if constexpr (MODE == FWD_LSE || MODE == FWD_NLL) {
      const uint32_t tiles = (uint32_t)((inner + 31) / 32);
      uint32_t cs = 1;
      while (cs < 8 && (uint64_t)tiles * outer * cs < (uint64_t)2 * sms && D >= (int64_t)4 * kRowReduceWY * cs) cs *= 2;
      const uint32_t dper = (uint32_t)((D + cs - 1) / cs);
      launch_cluster(rows_reduce_kernel<T, MODE>, dim3(tiles, cs, (uint32_t)outer), dim3(32, kRowReduceWY), 0, st, cs,
                     x, y, (uint32_t)inner, (uint32_t)D, dper, cs, na);
    } else {
      const uintptr_t bits = (uintptr_t)x | (uintptr_t)y;
      const RowSoftGeom g = rows_soft_geometry<T>(bits, inner, D, outer, sms);
      auto k = rows_fwd_kernel<T, MODE, 1>;
      if (g.rv == VecN<T>::value) k = rows_fwd_kernel<T, MODE, VecN<T>::value>;
      else if (g.rv == 2) k = rows_fwd_kernel<T, MODE, (VecN<T>::value >= 2 ? 2 : 1)>;
      launch_cluster(k, dim3(g.tiles, g.cs, (uint32_t)outer), dim3(32, kRowSoftWY), 0, st, g.cs,
                     x, y, (uint32_t)inner, (uint32_t)D, g.dper, g.cs, na);
    }
  }
  return launch_status();
}

template <typename T, int MODE>
int run_bwd(const T* y, const T* dy, T* dx, int64_t inner, int64_t D, int64_t outer, cudaStream_t st) {
  if (inner < 0 || D < 0 || outer < 0) return KN_EINVAL;
  if (inner == 0 || D == 0 || outer == 0) return KN_OK;
  if (!fits_u32(inner) || !fits_u32(D) || !fits_u32(outer) || !fits_u32(inner * outer)) return KN_ESIZE;
  const int sms = sm_count();
  if (inner == 1) {
    const uint32_t nseg = (uint32_t)outer;
    if (D <= 32) {
      seg_small_bwd_kernel<T, MODE, 1><<<(nseg + 255) / 256, 256, 0, st>>>(y, dy, dx, (uint32_t)D, nseg);
    } else if (D <= 2048 && nseg >= (uint32_t)sms) {
      // register-resident form: y and dy of a run in 2 x 8 packs per lane at most
      const bool same = ((((uintptr_t)y ^ (uintptr_t)dy) | ((uintptr_t)y ^ (uintptr_t)dx)) & 15) == 0;
      const GroupGeom gg = same ? softmax_group_geometry<T>(y, D, true) : GroupGeom{0, 0};
      const unsigned g = (nseg + 7) / 8;
      bool done = false;
#define KN_GROUP_BWD(G_, NP_)                                                                            \
  if (gg.g == G_ && gg.np == NP_) {                                                                      \
    seg_group_bwd_kernel<T, MODE, NP_, G_><<<(unsigned)(((uint64_t)nseg * G_ + 255) / 256), 256, 0, st>>>(y, dy, dx, (uint32_t)D, nseg); \
    done = true;                                                                                         \
  }
      if constexpr (sizeof(T) == 4) {
        KN_GROUP_BWD(8, 2) KN_GROUP_BWD(8, 4) KN_GROUP_BWD(16, 4) KN_GROUP_BWD(32, 4) KN_GROUP_BWD(32, 8)
      }
#undef KN_GROUP_BWD
      if (!done)
        seg_small_bwd_kernel<T, MODE, 32><<<g, 256, 0, st>>>(y, dy, dx, (uint32_t)D, nseg);
    } else {
      // 256 threads per CTA for slices below 32 KB, 512 above (measured: 512 threads with half
      // the packs per thread win 1-2 % there and lose 8 % on 16 KB slices); KNET_SM100_TMA_BWD =
      // 2562 | 5122 forces one of them.  One CTA per SM either way (200 KB of stage buffers).
      const int forced = tma_variant("KNET_SM100_TMA_BWD", 0) / 10;
      int nthr = forced == 512 ? 512 : 256;
      const size_t max_slice = (size_t)64 * 1024;      // 16 packs x 256 threads = 8 packs x 512 threads
      TmaPlan p = plan_tma<T>((uint64_t)D, nseg, 2, nthr, 2, sms, max_slice);
      if (p.ok && forced == 0 && (((uint64_t)D + p.cs - 1) / p.cs) * sizeof(T) >= 32 * 1024) {
        nthr = 512;
        p = plan_tma<T>((uint64_t)D, nseg, 2, nthr, 2, sms, max_slice);
      }
      if (p.ok) {
        const uint64_t slice = ((uint64_t)D + p.cs - 1) / p.cs, nvec = slice / VecN<T>::value;
        const uint64_t per_lane = ((nvec + nthr / 32 - 1) / (nthr / 32) + 31) / 32;   // packs per thread and array
        auto go = [&](auto kernel) {
          allow_smem(kernel, p.smem);
          p.clusters = min(p.clusters, (uint32_t)max_active_clusters(kernel, dim3(nthr), p.smem, p.cs));
          launch_cluster(kernel, dim3(p.clusters, p.cs), dim3(nthr), p.smem, st, p.cs, y, dy, dx, (uint32_t)D,
                         nseg, p.cs, p.stage_elems, tma_xchg());
        };
        if (nthr == 512) {
          if (per_lane <= 4) go(seg_tma_bwd_kernel<T, MODE, 512, 4>);     // 32 KB slices: 4 packs per thread
          else go(seg_tma_bwd_kernel<T, MODE, 512, 8>);
        } else {
          if (per_lane <= 4) go(seg_tma_bwd_kernel<T, MODE, 256, 4>);
          else if (per_lane <= 8) go(seg_tma_bwd_kernel<T, MODE, 256, 8>);
          else if (per_lane <= 13) go(seg_tma_bwd_kernel<T, MODE, 256, 13>);
          else go(seg_tma_bwd_kernel<T, MODE, 256, 16>);
        }
      } else {
        uint32_t cs = 1;
        while (cs < 8 && (uint64_t)nseg * cs < (uint64_t)2 * sms && D / (cs * 2) >= 4096) cs *= 2;
        launch_cluster(seg_big_bwd_kernel<T, MODE, false>, dim3(nseg, cs), dim3(kSegSoftThreads), 0, st, cs,
                       y, dy, dx, (uint32_t)D, cs);
      }
    }
  } else {
    if (outer > 65535) return KN_ESIZE;
    const uintptr_t bits = (uintptr_t)y | (uintptr_t)dy | (uintptr_t)dx;
    const RowSoftGeom g = rows_soft_geometry<T>(bits, inner, D, outer, sms);
    auto k = rows_bwd_kernel<T, MODE, 1>;
    if (g.rv == VecN<T>::value) k = rows_bwd_kernel<T, MODE, VecN<T>::value>;
    else if (g.rv == 2) k = rows_bwd_kernel<T, MODE, (VecN<T>::value >= 2 ? 2 : 1)>;
    launch_cluster(k, dim3(g.tiles, g.cs, (uint32_t)outer), dim3(32, kRowSoftWY), 0, st, g.cs,
                   y, dy, dx, (uint32_t)inner, (uint32_t)D, g.dper, g.cs);
  }
  return launch_status();
}

// ---- logsumexp backward: dx = dy[a,c] * exp(x - y[a,c]) -------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
lse_bwd_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
               uint32_t inner, uint32_t D, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    uint64_t j;
    if (inner == 1) j = i / D;
    else { const uint64_t q = i / inner; j = (i - q * inner) + (q / D) * inner; }
    __stcs(dx + i, __ldg(dy + j) * Math<T>::exp_fast(__ldcs(x + i) - __ldg(y + j)));
  }
}

// ---- nll: final sum over the per-instance losses, argmax, accuracy --------------------------------
// One CTA, or for many instances a cluster of `cs` CTAs that each sum a contiguous slice and hand
// their partial to rank 0 through distributed shared memory (fixed order: repeatable bit for bit).
template <typename T>
__global__ void __launch_bounds__(1024)
nll_finish_kernel(const T* __restrict__ per_instance, const int32_t* __restrict__ labels, uint32_t ninst,
                  T* total, int32_t* count, uint32_t cs) {
  __shared__ T red[32];
  __shared__ int redi[32];
  __shared__ T part_sum;
  __shared__ int part_cnt;
  const uint32_t per = (ninst + cs - 1) / cs;
  const uint32_t lo = min(blockIdx.y * per, ninst), hi = min(lo + per, ninst);
  T a[4] = {(T)0, (T)0, (T)0, (T)0};
  int c[4] = {0, 0, 0, 0};
  uint32_t j = lo + threadIdx.x;
  for (; j + 7 * 1024 < hi; j += 8 * 1024) {     // eight independent loads of each array in flight
    int32_t l[8];
    T v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) { l[k] = __ldg(labels + j + k * 1024); v[k] = __ldg(per_instance + j + k * 1024); }
#pragma unroll
    for (int k = 0; k < 8; k++) if (l[k] != 0) { a[k & 3] += v[k]; c[k & 3]++; }
  }
  for (; j < hi; j += 1024)
    if (labels[j] != 0) { a[0] += per_instance[j]; c[0]++; }
  T acc = (a[0] + a[1]) + (a[2] + a[3]);
  int cnt = (c[0] + c[1]) + (c[2] + c[3]);
  acc = block_reduce(acc, [](T p, T q) { return p + q; }, (T)0, red);
  cnt = block_reduce(cnt, [](int p, int q) { return p + q; }, 0, redi);
  if (cs == 1) {
    if (threadIdx.x == 0) { *total = acc; *count = cnt; }
    return;
  }
  if (threadIdx.x == 0) { part_sum = acc; part_cnt = cnt; }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  if (blockIdx.y == 0 && threadIdx.x == 0) {
    for (uint32_t r = 1; r < cs; r++) {
      acc += *cluster.map_shared_rank(&part_sum, r);
      cnt += *cluster.map_shared_rank(&part_cnt, r);
    }
    *total = acc;
    *count = cnt;
  }
  cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}
// 16384 instances per CTA, up to a cluster of 8
inline unsigned nll_finish_cluster(int64_t ninst) {
  unsigned cs = 1;
  while (cs < 8 && (int64_t)cs * 16384 < ninst) cs *= 2;
  return cs;
}

template <typename T> struct VI {
  T v;
  uint32_t i;
};
template <typename T> __device__ __forceinline__ VI<T> vi_merge(VI<T> a, VI<T> b) {
  // the first maximal element wins, as Julia's findmax does
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

template <typename T> __device__ __forceinline__ VI<T> vi_shfl_xor(VI<T> a, int o) {
  return VI<T>{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
}

// Accuracy counts (instances with a label, hits) are kept per thread while a CTA walks its share of
// the instances and reach the two global counters once per CTA: atomics on one address run at
// about one per nanosecond, which bounded the time when every instance (or every warp) sent its own
// (4 M instances of 10 classes: 2.9 ms with two atomics per instance, 0.9 ms with two per warp).
struct AccCount {
  int counted = 0, hit = 0;
};
template <typename T>
__device__ __forceinline__ void argmax_record(VI<T> best, bool writer, uint64_t inst, int32_t* __restrict__ idx,
                                              const int32_t* __restrict__ labels, bool want_acc, AccCount& acc) {
  if (!writer) return;
  if (best.i == 0xffffffffu) best.i = 0;  // all NaN or -inf: first element
  if (idx) idx[inst] = (int32_t)(best.i + 1);
  if (want_acc) {
    const int32_t l = labels[inst];
    if (l != 0) {
      acc.counted++;
      acc.hit += l == (int32_t)(best.i + 1);
    }
  }
}
// every thread of the CTA calls this once, after its last instance
__device__ __forceinline__ void acc_flush(AccCount acc, int32_t* __restrict__ acc_result) {
  __shared__ int s_counted, s_hit;
  if (threadIdx.x == 0) s_counted = s_hit = 0;
  __syncthreads();
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    acc.counted += __shfl_xor_sync(0xffffffffu, acc.counted, o);
    acc.hit += __shfl_xor_sync(0xffffffffu, acc.hit, o);
  }
  if ((threadIdx.x & 31) == 0 && acc.counted) {
    atomicAdd(&s_counted, acc.counted);
    atomicAdd(&s_hit, acc.hit);
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_counted) {
    atomicAdd(acc_result + 1, s_counted);
    if (s_hit) atomicAdd(acc_result, s_hit);
  }
}

// segments, runs of up to 2048 Float32 / 1024 Float64 elements: a group of G lanes per instance loads
// the whole run at once (see reduce_seg_group_kernel); a CTA takes 256/G instances per round
template <typename T, int NP, int G>
__global__ void __launch_bounds__(256)
argmax_group_kernel(const T* __restrict__ x, int32_t* __restrict__ idx, uint32_t D, uint32_t ninst,
                    const int32_t* __restrict__ labels, int32_t* __restrict__ acc_result) {
  constexpr uint32_t VEC = VecN<T>::value, PER = 256 / G;
  const uint32_t lane = threadIdx.x % G, slot = threadIdx.x / G;
  const uint64_t rounds = ((uint64_t)ninst + PER - 1) / PER;
  AccCount acc;
  for (uint64_t r = blockIdx.x; r < rounds; r += gridDim.x) {   // the same trip count for every thread of the CTA
    uint64_t inst = r * PER + slot;
    const bool live = inst < ninst;
    if (!live) inst = 0;
    const T* p = x + inst * D;
    const uint32_t mis = (uint32_t)(((uintptr_t)p & 15u) / sizeof(T));
    const uint32_t total = mis + (live ? D : 0);
    const T* base = p - mis;
    Pack<T, VEC> v[NP];
#pragma unroll
    for (int j = 0; j < NP; j++) {
      const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
      if (e0 >= mis && e0 + VEC <= total) v[j] = ld_stream<T, VEC>(base + e0);
    }
    VI<T> best{-Math<T>::inf(), 0xffffffffu};
#pragma unroll
    for (int j = 0; j < NP; j++) {
      const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
      if (e0 >= mis && e0 + VEC <= total) {
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) best = vi_merge(best, VI<T>{v[j].v[e], e0 + e - mis});
      } else {
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) {
          const uint32_t i = e0 + e;
          if (i >= mis && i < total) best = vi_merge(best, VI<T>{__ldg(base + i), i - mis});
        }
      }
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) best = vi_merge(best, vi_shfl_xor(best, o));
    argmax_record<T>(best, live && lane == 0, inst, idx, labels, acc_result != nullptr, acc);
  }
  if (acc_result) acc_flush(acc, acc_result);
}

// segments, runs of up to 32 elements (ten classes, say): one thread per instance; a warp's 32 runs are
// one contiguous stretch of memory, which L1 holds while the threads walk it
template <typename T>
__global__ void __launch_bounds__(256)
argmax_thread_kernel(const T* __restrict__ x, int32_t* __restrict__ idx, uint32_t D, uint32_t ninst,
                     const int32_t* __restrict__ labels, int32_t* __restrict__ acc_result) {
  const uint64_t rounds = ((uint64_t)ninst + 255) / 256;
  AccCount acc;
  for (uint64_t r = blockIdx.x; r < rounds; r += gridDim.x) {
    const uint64_t inst = r * 256 + threadIdx.x;
    const bool live = inst < ninst;
    VI<T> best{-Math<T>::inf(), 0xffffffffu};
    if (live) {
      const T* p = x + inst * D;
#pragma unroll 4
      for (uint32_t d = 0; d < D; d++) best = vi_merge(best, VI<T>{__ldg(p + d), d});
    }
    argmax_record<T>(best, live, inst, idx, labels, acc_result != nullptr, acc);
  }
  if (acc_result) acc_flush(acc, acc_result);
}

// segments, long runs: one CTA per instance and round, four 16-byte loads in flight per thread
template <typename T>
__global__ void __launch_bounds__(256)
argmax_block_kernel(const T* __restrict__ x, int32_t* __restrict__ idx, uint32_t D, uint32_t ninst,
                    const int32_t* __restrict__ labels, int32_t* __restrict__ acc_result) {
  __shared__ T sv[8];
  __shared__ uint32_t si[8];
  AccCount acc;
  for (uint32_t inst = blockIdx.x; inst < ninst; inst += gridDim.x) {
    VI<T> best{-Math<T>::inf(), 0xffffffffu};
    segment_visit<T>(x + (uint64_t)inst * D, D, threadIdx.x, 256,
                     [&](T v, uint32_t i) { best = vi_merge(best, VI<T>{v, i}); });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = vi_merge(best, vi_shfl_xor(best, o));
    __syncthreads();   // the previous round's table has been read
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best.v; si[threadIdx.x >> 5] = best.i; }
    __syncthreads();
    if (threadIdx.x < 32) {
      best = threadIdx.x < 8 ? VI<T>{sv[threadIdx.x], si[threadIdx.x]} : VI<T>{-Math<T>::inf(), 0xffffffffu};
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) best = vi_merge(best, vi_shfl_xor(best, o));
      argmax_record<T>(best, threadIdx.x == 0, inst, idx, labels, acc_result != nullptr, acc);
    }
  }
  if (acc_result) acc_flush(acc, acc_result);
}

// rows layout: a CTA of 32 x 8 threads takes 32 adjacent instances per round, the columns spread over
// its 8 warps with eight strided loads in flight per thread; warp 0 merges and records
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const T* __restrict__ x, int32_t* __restrict__ idx, uint32_t inner, uint32_t D, uint32_t outer,
                   const int32_t* __restrict__ labels, int32_t* __restrict__ acc_result) {
  __shared__ T sv[8][32];
  __shared__ uint32_t si[8][32];
  const uint32_t lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
  const uint32_t tiles = (inner + 31) / 32;
  const uint64_t rounds = (uint64_t)tiles * outer;
  AccCount acc;
  for (uint64_t r = blockIdx.x; r < rounds; r += gridDim.x) {
    const uint32_t c = (uint32_t)(r / tiles), a = (uint32_t)(r % tiles) * 32 + lx;
    const bool live = a < inner;
    const T* p = x + (uint64_t)c * inner * D + (live ? a : 0);
    VI<T> best{-Math<T>::inf(), 0xffffffffu};
    if (live) {
      uint32_t d = ly;
      for (; d + 56 < D; d += 64) {
        T v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __ldcs(p + (uint64_t)(d + 8 * k) * inner);
#pragma unroll
        for (int k = 0; k < 8; k++) best = vi_merge(best, VI<T>{v[k], d + 8 * k});
      }
      for (; d < D; d += 8) best = vi_merge(best, VI<T>{__ldcs(p + (uint64_t)d * inner), d});
    }
    __syncthreads();   // the previous round's table has been read
    sv[ly][lx] = best.v;
    si[ly][lx] = best.i;
    __syncthreads();
    if (ly == 0) {
#pragma unroll
      for (int k = 1; k < 8; k++) best = vi_merge(best, VI<T>{sv[k][lx], si[k][lx]});
      argmax_record<T>(best, live, (uint64_t)c * inner + a, idx, labels, acc_result != nullptr, acc);
    }
  }
  if (acc_result) acc_flush(acc, acc_result);
}

template <typename T>
int run_argmax(const T* x, int32_t* idx, int64_t inner, int64_t D, int64_t outer, const int32_t* labels,
               int32_t* acc_result, cudaStream_t st) {
  if (inner < 0 || D < 0 || outer < 0) return KN_EINVAL;
  if (inner == 0 || D == 0 || outer == 0) return KN_OK;
  if (!fits_u32(inner) || !fits_u32(D) || !fits_u32(outer) || !fits_u32(inner * outer)) return KN_ESIZE;
  const uint32_t ninst = (uint32_t)(inner * outer);
  const uint64_t cap = (uint64_t)sm_count() * 16;        // CTAs walk their share of the instances
  auto grid = [&](uint64_t rounds) { return (unsigned)(rounds < cap ? rounds : cap); };
  if (inner != 1) {
    const uint64_t rounds = (uint64_t)((inner + 31) / 32) * (uint64_t)outer;
    argmax_rows_kernel<T><<<grid(rounds), 256, 0, st>>>(x, idx, (uint32_t)inner, (uint32_t)D, (uint32_t)outer, labels, acc_result);
    return launch_status();
  }
  if (D <= 32) {
    argmax_thread_kernel<T><<<grid(((uint64_t)ninst + 255) / 256), 256, 0, st>>>(x, idx, (uint32_t)D, ninst, labels, acc_result);
    return launch_status();
  }
  const GroupGeom gg = group_geometry<T>(x, D, 16);
  bool done = false;
#define KN_GROUP_ARGMAX(G_, NP_)                                                                           \
  if (gg.g == G_ && gg.np == NP_) {                                                                        \
    argmax_group_kernel<T, NP_, G_><<<grid(((uint64_t)ninst * G_ + 255) / 256), 256, 0, st>>>(             \
        x, idx, (uint32_t)D, ninst, labels, acc_result);                                                   \
    done = true;                                                                                           \
  }
  KN_GROUP_ARGMAX(8, 2) KN_GROUP_ARGMAX(8, 4) KN_GROUP_ARGMAX(16, 4) KN_GROUP_ARGMAX(32, 4) KN_GROUP_ARGMAX(32, 8)
  KN_GROUP_ARGMAX(32, 16)
#undef KN_GROUP_ARGMAX
  if (!done) argmax_block_kernel<T><<<grid(ninst), 256, 0, st>>>(x, idx, (uint32_t)D, ninst, labels, acc_result);
  return launch_status();
}

// (R,K) score matrix, classes along `dims`: dims=1 -> (1,R,K); dims=2 -> (R,K,1)
inline bool nll_geometry(int64_t R, int64_t K, int dims, int64_t* inner, int64_t* D, int64_t* outer) {
  if (R < 0 || K < 0) return false;
  if (dims == 1) { *inner = 1; *D = R; *outer = K; return true; }
  if (dims == 2) { *inner = R; *D = K; *outer = 1; return true; }
  return false;
}

}  // namespace kn

using namespace kn;

namespace kn {
int index_wait_flag_read_clear();   // index.cu: the flag of the staged row kernels and of the wait probe
}

KN_EXPORT int knet_device_status(void) {
  const int a = wait_flag_read_clear(), b = index_wait_flag_read_clear();
  if (a < 0 || b < 0) return -1;
  return (a | b) ? 1 : 0;
}

#define KN_DEF_SOFTMAX(f, S, T)                                                                     \
  KN_EXPORT int knet_softmax_fwd_##S(const T* x, T* y, int64_t inner, int64_t D, int64_t outer,      \
                                     cudaStream_t s) {                                               \
    if (!x || !y) return KN_EINVAL;                                                                  \
    return run_fwd<T, FWD_SOFTMAX>(x, y, inner, D, outer, NllArgs<T>{}, s);                          \
  }                                                                                                  \
  KN_EXPORT int knet_logsoftmax_fwd_##S(const T* x, T* y, int64_t inner, int64_t D, int64_t outer,   \
                                        cudaStream_t s) {                                            \
    if (!x || !y) return KN_EINVAL;                                                                  \
    return run_fwd<T, FWD_LOGSOFTMAX>(x, y, inner, D, outer, NllArgs<T>{}, s);                       \
  }                                                                                                  \
  KN_EXPORT int knet_softmax_bwd_##S(const T* y, const T* dy, T* dx, int64_t inner, int64_t D,       \
                                     int64_t outer, cudaStream_t s) {                                \
    if (!y || !dy || !dx) return KN_EINVAL;                                                          \
    return run_bwd<T, BWD_SOFTMAX>(y, dy, dx, inner, D, outer, s);                                   \
  }                                                                                                  \
  KN_EXPORT int knet_logsoftmax_bwd_##S(const T* y, const T* dy, T* dx, int64_t inner, int64_t D,    \
                                        int64_t outer, cudaStream_t s) {                             \
    if (!y || !dy || !dx) return KN_EINVAL;                                                          \
    return run_bwd<T, BWD_LOGSOFTMAX>(y, dy, dx, inner, D, outer, s);                                \
  }                                                                                                  \
  KN_EXPORT int knet_logsumexp_fwd_##S(const T* x, T* y, int64_t inner, int64_t D, int64_t outer,    \
                                       cudaStream_t s) {                                             \
    if (!x || !y) return KN_EINVAL;                                                                  \
    return run_fwd<T, FWD_LSE>(x, y, inner, D, outer, NllArgs<T>{}, s);                              \
  }                                                                                                  \
  KN_EXPORT int knet_logsumexp_bwd_##S(const T* x, const T* y, const T* dy, T* dx, int64_t inner,    \
                                       int64_t D, int64_t outer, cudaStream_t s) {                   \
    if (!x || !y || !dy || !dx || inner < 0 || D < 0 || outer < 0) return KN_EINVAL;                 \
    if (!fits_u32(inner) || !fits_u32(D)) return KN_ESIZE;                                           \
    const uint64_t n = (uint64_t)inner * D * outer;                                                  \
    if (n == 0) return KN_OK;                                                                        \
    uint64_t blocks = (n + 255) / 256;                                                               \
    const uint64_t cap = (uint64_t)sm_count() * 32;                                                  \
    if (blocks > cap) blocks = cap;                                                                  \
    lse_bwd_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(x, y, dy, dx, (uint32_t)inner, (uint32_t)D, n); \
    return launch_status();                                                                          \
  }
KNET_BOTH_TYPES(KN_DEF_SOFTMAX, softmax)

#define KN_DEF_NLL(f, S, T)                                                                          \
  KN_EXPORT int knet_nll_fwd_##S(const T* scores, const int32_t* labels, int64_t R, int64_t K,       \
                                 int dims, T* total, int32_t* count, T* per_instance,                \
                                 cudaStream_t s) {                                                   \
    int64_t inner, D, outer;                                                                         \
    if (!scores || !labels || !total || !count) return KN_EINVAL;                                    \
    if (!nll_geometry(R, K, dims, &inner, &D, &outer)) return KN_EINVAL;                             \
    if (!per_instance) return KN_EWORKSPACE;                                                         \
    NllArgs<T> na{labels, per_instance, nullptr, (T)1, 0};                                           \
    int rc = run_fwd<T, FWD_NLL>(scores, nullptr, inner, D, outer, na, s);                           \
    if (rc != KN_OK) return rc;                                                                      \
    const int64_t ninst = D == 0 ? 0 : inner * outer;                                                \
    const unsigned fcs = nll_finish_cluster(ninst);                                                  \
    cudaError_t e = launch_cluster(nll_finish_kernel<T>, dim3(1, fcs, 1), dim3(1024), 0, s, fcs,     \
                                   (const T*)per_instance, labels, (uint32_t)ninst, total, count, fcs); \
    if (e != cudaSuccess) return (int)e;                                                             \
    return launch_status();                                                                          \
  }                                                                                                  \
  KN_EXPORT int knet_nll_bwd_##S(const T* scores, const int32_t* labels, int64_t R, int64_t K,       \
                                 int dims, int average, T dy, const int32_t* count, T* dscores,      \
                                 cudaStream_t s) {                                                   \
    int64_t inner, D, outer;                                                                         \
    if (!scores || !labels || !dscores || (average && !count)) return KN_EINVAL;                     \
    if (!nll_geometry(R, K, dims, &inner, &D, &outer)) return KN_EINVAL;                             \
    NllArgs<T> na{labels, nullptr, count, dy, average};                                              \
    return run_fwd<T, FWD_NLLBWD>(scores, dscores, inner, D, outer, na, s);                          \
  }                                                                                                  \
  KN_EXPORT int knet_argmax_##S(const T* x, int32_t* idx, int64_t inner, int64_t D, int64_t outer,   \
                                cudaStream_t s) {                                                    \
    if (!x || !idx) return KN_EINVAL;                                                                \
    return run_argmax<T>(x, idx, inner, D, outer, nullptr, nullptr, s);                              \
  }                                                                                                  \
  KN_EXPORT int knet_accuracy_##S(const T* scores, const int32_t* labels, int64_t R, int64_t K,      \
                                  int dims, int32_t* result, cudaStream_t s) {                       \
    int64_t inner, D, outer;                                                                         \
    if (!scores || !labels || !result) return KN_EINVAL;                                             \
    if (!nll_geometry(R, K, dims, &inner, &D, &outer)) return KN_EINVAL;                             \
    cudaError_t e = cudaMemsetAsync(result, 0, 2 * sizeof(int32_t), s);                              \
    if (e != cudaSuccess) return (int)e;                                                             \
    return run_argmax<T>(scores, nullptr, inner, D, outer, labels, result, s);                       \
  }
KNET_BOTH_TYPES(KN_DEF_NLL, nll)
