// Long contiguous runs (a (C,B) score matrix with C in the tens of thousands): persistent
// thread-block clusters with bulk-copy (TMA) staging.
//
// A cluster of `cs` CTAs owns one instance at a time; CTA r holds slice r of the run in
// shared memory.  Each CTA keeps two stage buffers: while it reduces and writes instance i,
// the bulk copy of instance i + (number of clusters) is already in flight, so HBM reads never
// wait for the arithmetic.  One thread issues one bulk copy per slice (the 16-byte aligned
// interior; the few ragged elements at either end are loaded by ordinary loads) and an
// mbarrier counts the bytes.  The slice is placed in shared memory at the same offset inside
// a 16-byte line as it has in global memory, which is what makes the aligned interior a
// legal bulk copy for any run length.  The (max, sum) pairs of the slices meet through
// distributed shared memory with one cluster barrier per instance.  DRAM sees every input
// once and every output once.
//
// Included by softmax.cu after MS, NllArgs, fwd_value and segment_store are defined.
#pragma once
#include "tma.cuh"

namespace kn {

// Set when a bounded wait on a bulk copy gives up; read (and cleared) by knet_device_status.
__device__ int g_wait_timeout_flag = 0;

template <typename T> struct SliceGeom {
  uint32_t sh, head, body;  // shared-memory shift, ragged head elements, aligned interior elements
};

template <typename T>
__device__ __forceinline__ SliceGeom<T> slice_geom(const T* gp, uint32_t len) {
  constexpr uint32_t VEC = VecN<T>::value;
  SliceGeom<T> g;
  g.sh = (uint32_t)(((uintptr_t)gp & 15u) / sizeof(T));
  g.head = (VEC - g.sh) % VEC;
  if (g.head > len) g.head = len;
  g.body = ((len - g.head) / VEC) * VEC;
  return g;
}

// ragged ends of a slice by ordinary loads (element i goes to buf[sh + i])
template <typename T>
__device__ __forceinline__ void load_ragged(const T* gp, uint32_t len, const SliceGeom<T>& g, T* buf) {
  const uint32_t tid = threadIdx.x;
  if (tid < g.head) buf[g.sh + tid] = gp[tid];
  const uint32_t tail0 = g.head + g.body;
  if (tid < len - tail0) buf[g.sh + tail0 + tid] = gp[tail0 + tid];
}

constexpr int kTmaFwdThreads = 256;
constexpr int kTmaBwdThreads = 512;

template <typename T, int MODE>
__global__ void __launch_bounds__(kTmaFwdThreads)
seg_tma_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, uint32_t cs,
                   uint32_t stage_elems, NllArgs<T> na) {
  constexpr uint32_t NT = kTmaFwdThreads;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* stage[2] = {reinterpret_cast<T*>(smem_raw), reinterpret_cast<T*>(smem_raw) + stage_elems};
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ MS<T> red[32];
  __shared__ MS<T> slot[2];
  const uint32_t tid = threadIdx.x;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, blockIdx.y * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    mbar_init_fence();
  }
  __syncthreads();

  auto issue = [&](uint32_t seg, uint32_t s) {
    const T* gp = x + (uint64_t)seg * D + a0;
    const SliceGeom<T> g = slice_geom(gp, len);
    if (tid == 0) {
      mbar_arrive_expect_tx(&bar[s], g.body * (uint32_t)sizeof(T));
      if (g.body) bulk_copy_g2s(stage[s] + g.sh + g.head, gp + g.head, g.body * (uint32_t)sizeof(T), &bar[s]);
    }
    load_ragged(gp, len, g, stage[s]);
  };

  uint32_t seg = blockIdx.x;
  if (seg < nseg) issue(seg, 0);
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t s = it & 1;
    if (seg + gridDim.x < nseg) issue(seg + gridDim.x, s ^ 1);
    if (!mbar_wait_bounded(&bar[s], (it >> 1) & 1) && tid == 0) atomicExch(&g_wait_timeout_flag, 1);
    __syncthreads();  // ragged elements stored by other threads
    const T* gp = x + (uint64_t)seg * D + a0;
    const uint32_t sh = (uint32_t)(((uintptr_t)gp & 15u) / sizeof(T));
    T* buf = stage[s] + sh;
    // local maximum, then local sum of exp(x - max); softmax keeps the exponentials
    T mx = -Math<T>::inf();
    for (uint32_t i = tid; i < len; i += NT) { const T v = buf[i]; mx = v > mx ? v : mx; }
    mx = block_reduce(mx, [](T a, T b) { return a > b ? a : b; }, -Math<T>::inf(), reinterpret_cast<T*>(red));
    T sum = (T)0;
    for (uint32_t i = tid; i < len; i += NT) {
      const T e = Math<T>::exp_fast(buf[i] - mx);
      if (MODE == FWD_SOFTMAX || MODE == FWD_NLLBWD) buf[i] = e;
      sum += e;
    }
    sum = block_reduce(sum, [](T a, T b) { return a + b; }, (T)0, reinterpret_cast<T*>(red));
    MS<T> ms{mx, sum};
    if (len == 0) ms = ms_init<T>();
    T rescale = (T)1;  // exp(local max - global max), applied to the stored exponentials
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (tid == 0) slot[s] = ms;
      cluster.sync();
      MS<T> tot = ms_init<T>();
      for (uint32_t r = 0; r < cs; r++) tot = ms_merge(tot, *cluster.map_shared_rank(&slot[s], r));
      rescale = Math<T>::exp_fast(mx - tot.m);
      ms = tot;
    }
    const T logs = Math<T>::log(ms.s);
    int32_t label = 0;
    T scale = (T)0;
    if (MODE == FWD_NLLBWD) {
      label = na.labels[seg];
      scale = label == 0 ? (T)0 : nll_scale(na);
    }
    const int32_t lab_local = label - 1 - (int32_t)a0;
    T* yp = y + (uint64_t)seg * D + a0;
    segment_store<T>(yp, len, tid, NT, [&](uint32_t i) {
      const T v = buf[i];
      if (MODE == FWD_LOGSOFTMAX) return (v - ms.m) - logs;
      const T p = v * rescale / ms.s;
      if (MODE == FWD_SOFTMAX) return p;
      return ((int32_t)i == lab_local ? p - (T)1 : p) * scale;
    });
    __syncthreads();  // everyone is done with this stage before the next copy lands in it
  }
  if (cs > 1) cg::this_cluster().sync();  // peers may still be reading this CTA's slot
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kTmaBwdThreads)
seg_tma_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D,
                   uint32_t nseg, uint32_t cs, uint32_t stage_elems) {
  constexpr uint32_t NT = kTmaBwdThreads;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* base = reinterpret_cast<T*>(smem_raw);
  T* ystage[2] = {base, base + 2 * stage_elems};
  T* gstage[2] = {base + stage_elems, base + 3 * stage_elems};
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ T red[32];
  __shared__ T slot[2];
  const uint32_t tid = threadIdx.x;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, blockIdx.y * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    mbar_init_fence();
  }
  __syncthreads();

  auto issue = [&](uint32_t seg, uint32_t s) {
    const T* yp = y + (uint64_t)seg * D + a0;
    const T* gp = dy + (uint64_t)seg * D + a0;
    const SliceGeom<T> gy = slice_geom(yp, len), gg = slice_geom(gp, len);
    if (tid == 0) {
      mbar_arrive_expect_tx(&bar[s], (gy.body + gg.body) * (uint32_t)sizeof(T));
      if (gy.body) bulk_copy_g2s(ystage[s] + gy.sh + gy.head, yp + gy.head, gy.body * (uint32_t)sizeof(T), &bar[s]);
      if (gg.body) bulk_copy_g2s(gstage[s] + gg.sh + gg.head, gp + gg.head, gg.body * (uint32_t)sizeof(T), &bar[s]);
    }
    load_ragged(yp, len, gy, ystage[s]);
    load_ragged(gp, len, gg, gstage[s]);
  };

  uint32_t seg = blockIdx.x;
  if (seg < nseg) issue(seg, 0);
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t s = it & 1;
    if (seg + gridDim.x < nseg) issue(seg + gridDim.x, s ^ 1);
    if (!mbar_wait_bounded(&bar[s], (it >> 1) & 1) && tid == 0) atomicExch(&g_wait_timeout_flag, 1);
    __syncthreads();
    const T* yp = y + (uint64_t)seg * D + a0;
    const T* gp = dy + (uint64_t)seg * D + a0;
    const T* ybuf = ystage[s] + (uint32_t)(((uintptr_t)yp & 15u) / sizeof(T));
    const T* gbuf = gstage[s] + (uint32_t)(((uintptr_t)gp & 15u) / sizeof(T));
    T acc = (T)0;
    for (uint32_t i = tid; i < len; i += NT) acc += MODE == BWD_SOFTMAX ? ybuf[i] * gbuf[i] : gbuf[i];
    acc = block_reduce(acc, [](T a, T b) { return a + b; }, (T)0, red);
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (tid == 0) slot[s] = acc;
      cluster.sync();
      T tot = (T)0;
      for (uint32_t r = 0; r < cs; r++) tot += *cluster.map_shared_rank(&slot[s], r);
      acc = tot;
    }
    T* xp = dx + (uint64_t)seg * D + a0;
    segment_store<T>(xp, len, tid, NT, [&](uint32_t i) {
      const T yv = ybuf[i], gv = gbuf[i];
      return MODE == BWD_SOFTMAX ? yv * gv - yv * acc : gv - Math<T>::exp_fast(yv) * acc;
    });
    __syncthreads();
  }
  if (cs > 1) cg::this_cluster().sync();
}

// Geometry of a staged launch: cluster size, elements per stage buffer, dynamic shared
// memory and persistent grid.  `arrays` = stage buffers per stage (1 forward, 2 backward).
struct TmaPlan {
  bool ok;
  uint32_t cs, stage_elems, clusters;
  size_t smem;
};

template <typename T>
inline TmaPlan plan_tma(uint64_t D, uint32_t nseg, int arrays, int threads, int sms) {
  TmaPlan p{};
  const size_t target = (arrays == 1 ? 32 : 25) * 1024;   // preferred bytes per stage buffer
  const size_t limit = 200 * 1024;                        // dynamic shared memory we are willing to ask for
  uint32_t cs = 1;
  while (cs < 8 && ((D + cs - 1) / cs) * sizeof(T) > target) cs *= 2;
  // few instances: split further so that every SM gets work
  while (cs < 8 && (uint64_t)nseg * cs < (uint64_t)2 * sms && D / (cs * 2) >= 2048) cs *= 2;
  const uint64_t slice = (D + cs - 1) / cs;
  const uint64_t stage_elems = (slice + 2 * VecN<T>::value + 31) / 32 * 32;   // room for the shift, 128-byte multiple
  const size_t smem = (size_t)stage_elems * sizeof(T) * 2 * arrays;
  if (smem > limit) return p;
  const int by_smem = (int)((227 * 1024) / (smem + 1024));
  const int by_threads = 2048 / threads;
  const int per_sm = by_smem < by_threads ? by_smem : by_threads;
  if (per_sm < 1) return p;
  uint32_t clusters = (uint32_t)((sms * per_sm) / cs);
  if (clusters < 1) clusters = 1;
  if (clusters > nseg) clusters = nseg;
  p.ok = true;
  p.cs = cs;
  p.stage_elems = (uint32_t)stage_elems;
  p.clusters = clusters;
  p.smem = smem;
  return p;
}

}  // namespace kn
