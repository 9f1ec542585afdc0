// Building blocks shared by the reduction and softmax kernels: reduction functors, a
// vectorised walk over one contiguous segment, and thread-block-cluster helpers
// (distributed shared memory) used when one output needs more than one CTA.
#pragma once
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"
#include "math.cuh"

namespace kn {
namespace cg = cooperative_groups;

// item/merge/init of src/libknet8/ops.jl:144-156
template <typename T> struct R_sum     { static __device__ __forceinline__ T item(T x) { return x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a + x; }
                                         static __device__ __forceinline__ T init() { return (T)0; } };
template <typename T> struct R_prod    { static __device__ __forceinline__ T item(T x) { return x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a * x; }
                                         static __device__ __forceinline__ T init() { return (T)1; } };
template <typename T> struct R_maximum { static __device__ __forceinline__ T item(T x) { return x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a > x ? a : x; }
                                         static __device__ __forceinline__ T init() { return -Math<T>::inf(); } };
template <typename T> struct R_minimum { static __device__ __forceinline__ T item(T x) { return x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a < x ? a : x; }
                                         static __device__ __forceinline__ T init() { return Math<T>::inf(); } };
template <typename T> struct R_sumabs  { static __device__ __forceinline__ T item(T x) { return x < 0 ? -x : x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a + x; }
                                         static __device__ __forceinline__ T init() { return (T)0; } };
template <typename T> struct R_sumabs2 { static __device__ __forceinline__ T item(T x) { return x * x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a + x; }
                                         static __device__ __forceinline__ T init() { return (T)0; } };
template <typename T> struct R_maxabs  { static __device__ __forceinline__ T item(T x) { return x < 0 ? -x : x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a > x ? a : x; }
                                         static __device__ __forceinline__ T init() { return (T)0; } };
template <typename T> struct R_minabs  { static __device__ __forceinline__ T item(T x) { return x < 0 ? -x : x; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a < x ? a : x; }
                                         static __device__ __forceinline__ T init() { return Math<T>::inf(); } };
template <typename T> struct R_countnz { static __device__ __forceinline__ T item(T x) { return x != 0 ? (T)1 : (T)0; }
                                         static __device__ __forceinline__ T merge(T a, T x) { return a + x; }
                                         static __device__ __forceinline__ T init() { return (T)0; } };

// Visit every element of the contiguous segment p[0..len) exactly once, spread over `nthr`
// threads (this thread is `tid`): unaligned head and tail one by one, the 16-byte aligned
// body with 128-bit loads, four of them in flight per thread.  f(value, index).
template <typename T, typename F>
__device__ __forceinline__ void segment_visit(const T* __restrict__ p, uint32_t len, uint32_t tid,
                                              uint32_t nthr, F&& f) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t head = (uint32_t)(((16u - (uint32_t)((uintptr_t)p & 15u)) & 15u) / sizeof(T));
  if (head > len) head = len;
  const uint32_t nvec = (len - head) / VEC;
  const uint32_t tail0 = head + nvec * VEC;
  if (tid < head) f(p[tid], tid);
  const T* q = p + head;
  uint32_t v = tid;
  for (; v + 3 * nthr < nvec; v += 4 * nthr) {
    Pack<T, VEC> a0 = ld_stream<T, VEC>(q + (size_t)v * VEC);
    Pack<T, VEC> a1 = ld_stream<T, VEC>(q + (size_t)(v + nthr) * VEC);
    Pack<T, VEC> a2 = ld_stream<T, VEC>(q + (size_t)(v + 2 * nthr) * VEC);
    Pack<T, VEC> a3 = ld_stream<T, VEC>(q + (size_t)(v + 3 * nthr) * VEC);
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) f(a0.v[e], head + v * VEC + e);
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) f(a1.v[e], head + (v + nthr) * VEC + e);
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) f(a2.v[e], head + (v + 2 * nthr) * VEC + e);
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) f(a3.v[e], head + (v + 3 * nthr) * VEC + e);
  }
  for (; v < nvec; v += nthr) {
    Pack<T, VEC> a0 = ld_stream<T, VEC>(q + (size_t)v * VEC);
#pragma unroll
    for (uint32_t e = 0; e < VEC; e++) f(a0.v[e], head + v * VEC + e);
  }
  if (tail0 + tid < len) f(p[tail0 + tid], tail0 + tid);
}

// Same walk, but the aligned body is handed over one 16-byte pack at a time: fv(pack) for
// the body, fs(value) for the ragged ends.
template <typename T, typename FV, typename FS>
__device__ __forceinline__ void segment_visit_vec(const T* __restrict__ p, uint32_t len, uint32_t tid,
                                                  uint32_t nthr, FV&& fv, FS&& fs) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t head = (uint32_t)(((16u - (uint32_t)((uintptr_t)p & 15u)) & 15u) / sizeof(T));
  if (head > len) head = len;
  const uint32_t nvec = (len - head) / VEC;
  const uint32_t tail0 = head + nvec * VEC;
  if (tid < head) fs(p[tid]);
  const T* q = p + head;
  uint32_t v = tid;
  for (; v + 3 * nthr < nvec; v += 4 * nthr) {
    const Pack<T, VEC> a0 = ld_stream<T, VEC>(q + (size_t)v * VEC);
    const Pack<T, VEC> a1 = ld_stream<T, VEC>(q + (size_t)(v + nthr) * VEC);
    const Pack<T, VEC> a2 = ld_stream<T, VEC>(q + (size_t)(v + 2 * nthr) * VEC);
    const Pack<T, VEC> a3 = ld_stream<T, VEC>(q + (size_t)(v + 3 * nthr) * VEC);
    fv(a0); fv(a1); fv(a2); fv(a3);
  }
  for (; v < nvec; v += nthr) fv(ld_stream<T, VEC>(q + (size_t)v * VEC));
  if (tail0 + tid < len) fs(p[tail0 + tid]);
}

// The same walk handing over four packs at a time (fv4), single packs for the remainder (fv).
template <typename T, typename FV4, typename FV, typename FS>
__device__ __forceinline__ void segment_visit_vec4(const T* __restrict__ p, uint32_t len, uint32_t tid,
                                                   uint32_t nthr, FV4&& fv4, FV&& fv, FS&& fs) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t head = (uint32_t)(((16u - (uint32_t)((uintptr_t)p & 15u)) & 15u) / sizeof(T));
  if (head > len) head = len;
  const uint32_t nvec = (len - head) / VEC;
  const uint32_t tail0 = head + nvec * VEC;
  if (tid < head) fs(p[tid]);
  const T* q = p + head;
  uint32_t v = tid;
  for (; v + 3 * nthr < nvec; v += 4 * nthr) {
    Pack<T, VEC> a[4];
#pragma unroll
    for (int k = 0; k < 4; k++) a[k] = ld_stream<T, VEC>(q + (size_t)(v + k * nthr) * VEC);
    fv4(a);
  }
  for (; v < nvec; v += nthr) fv(ld_stream<T, VEC>(q + (size_t)v * VEC));
  if (tail0 + tid < len) fs(p[tail0 + tid]);
}

// Geometry of the "rows" kernels (a warp owns 32*rv adjacent rows, columns are spread over the
// warps of a CTA and the CTAs of a cluster).  Measured on B200 over row counts from 1024 to 32768:
// these kernels run at the copy rate when the grid has about 1.7 CTAs of 256 threads per SM and
// lose 5-10 % with twice as many and 25 % with half as many.  So: the widest row vector `rv`
// (elements per thread and column; candidates VEC, VEC/2, ..., 1, each subject to `ok(rv)`) whose
// tile count still allows that many CTAs with a cluster of 8, then the smallest cluster that
// reaches it.
struct RowsGeom {
  uint32_t rv, tiles, cs;
};
template <typename OK>
inline RowsGeom rows_geometry(uint32_t rows, uint32_t cols, uint32_t nbatch, uint32_t vec, uint32_t wy, OK ok,
                              int forced_cs, bool un_by_rv = false) {
  const uint64_t target = (uint64_t)sm_count() * 17 / 10;
  RowsGeom g{1u, (rows + 31) / 32, 1u};
  for (uint32_t rv = vec; rv >= 1; rv /= 2) {
    if (!ok(rv)) continue;
    const uint32_t tiles = (rows + 32 * rv - 1) / (32 * rv);
    if ((uint64_t)tiles * nbatch * 8 >= target || rv == 1) {
      g.rv = rv;
      g.tiles = tiles;
      break;
    }
  }
  // columns a CTA takes per turn: 8 per warp, or 8*vec/rv where the kernel keeps 128 bytes per thread in flight
  const uint32_t blk = (un_by_rv ? 8u * vec / g.rv : 8u) * wy;
  while (g.cs < 8 && (uint64_t)g.tiles * nbatch * g.cs < target && cols >= blk * g.cs) g.cs *= 2;
  if (forced_cs == 1 || forced_cs == 2 || forced_cs == 4 || forced_cs == 8) g.cs = (uint32_t)forced_cs;
  return g;
}

// Short contiguous runs handled by a group of G = 8, 16 or 32 lanes that holds the run in NP packs of
// 16 bytes per lane: lanes and packs for runs of D elements of the array at p.  Runs start on a
// 16-byte line when the array does and D is a multiple of the pack, else up to VEC-1 elements past
// one; the packs are counted from the line below the start.  np = 0: the run does not fit max_np packs.
struct GroupGeom {
  int g, np;
};
template <typename T> inline GroupGeom group_geometry(const void* p, int64_t D, int max_np) {
  constexpr int VEC = VecN<T>::value;
  const int64_t mis = (((uintptr_t)p & 15) == 0 && D % VEC == 0) ? 0 : VEC - 1;
  const int64_t packs = (D + mis + VEC - 1) / VEC;
  GroupGeom g{0, 0};
  if (packs <= 16) g = {8, 2};
  else if (packs <= 32) g = {8, 4};
  else if (packs <= 64) g = {16, 4};
  else if (packs <= 128) g = {32, 4};
  else if (packs <= 256) g = {32, 8};
  else if (packs <= 512) g = {32, 16};
  if (g.np > max_np) g = {0, 0};
  return g;
}

// Cluster split of the "segments" kernels (one CTA, or a cluster of CTAs, per contiguous run): runs
// are split only until the grid has `KNET_SM100_SEG_CTAS_PER_SM` (default 2) CTAs per SM, and only
// while a CTA keeps at least 4096 elements.  Splitting further was measured and loses: 512 runs of
// 50257 Float32 take 20.4 us unsplit, 24.2 / 30.6 / 50.3 us over clusters of 2 / 4 / 8 (the cluster
// launch and its two barriers cost more than the shorter tail gains).
inline uint32_t seg_cluster_size(uint64_t nseg, uint64_t len) {
  static const int per_sm = [] {
    const char* e = getenv("KNET_SM100_SEG_CTAS_PER_SM");   // tuning knob
    const int v = e ? atoi(e) : 2;
    return v > 0 ? v : 2;
  }();
  uint32_t cs = 1;
  while (cs < 8 && nseg * cs < (uint64_t)per_sm * sm_count() && len / (cs * 2) >= 4096) cs *= 2;
  return cs;
}

// How many clusters of `cs` CTAs (along y) of this kernel the device can hold at once; a
// persistent kernel must not launch more, or the surplus runs as a second wave.
template <typename... KArgs>
inline int max_active_clusters(void (*kernel)(KArgs...), dim3 block, size_t smem, unsigned cs) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1, cs, 1);
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cs;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(kernel), &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = 1;
  }
  return n;
}

// Launch with a thread-block cluster of `cs` CTAs along grid dimension y.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t st, unsigned cs, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cs;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace kn
