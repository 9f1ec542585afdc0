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
// legal bulk copy for any run length, and lets every pass over the slice use 128-bit
// shared-memory accesses.  The (max, sum) pairs of the slices meet through distributed
// shared memory with one cluster barrier per instance.  DRAM sees every input once and
// every output once; the arithmetic is about eight instructions per element.
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

// Walk a staged slice: fv(pack&, index of its first element) over the aligned interior with
// 128-bit shared-memory accesses (written back when WRITE), fs(value&, index) over the ends.
// `buf` points at element 0; buf + g.head is 16-byte aligned.
template <typename T, bool WRITE, int NT, typename FV, typename FS>
__device__ __forceinline__ void slice_walk(T* buf, uint32_t len, const SliceGeom<T>& g, FV&& fv, FS&& fs) {
  constexpr uint32_t VEC = VecN<T>::value;
  const uint32_t tid = threadIdx.x;
  Pack<T, VEC>* vb = reinterpret_cast<Pack<T, VEC>*>(buf + g.head);
  const uint32_t nvec = g.body / VEC;
#pragma unroll 2
  for (uint32_t v = tid; v < nvec; v += NT) {
    Pack<T, VEC> p = vb[v];
    fv(p, g.head + v * VEC);
    if (WRITE) vb[v] = p;
  }
  if (tid < g.head) fs(buf[tid], tid);
  const uint32_t tail0 = g.head + g.body;
  if (tid < len - tail0) fs(buf[tail0 + tid], tail0 + tid);
}

// CTA-wide reduction with one barrier: warp results go to `part` (one slot per warp, used for
// this reduction only within an iteration) and every thread combines them in the same order.
template <typename T, int NT, typename Op>
__device__ __forceinline__ T cta_reduce(T v, Op op, T* part) {
  v = warp_reduce(v, op);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  T r = part[0];
#pragma unroll
  for (int w = 1; w < NT / 32; w++) r = op(r, part[w]);
  return r;
}

constexpr int kTmaFwdThreads = 256;
constexpr int kTmaBwdThreads = 512;

template <typename T, int MODE>
__global__ void __launch_bounds__(kTmaFwdThreads)
seg_tma_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, uint32_t cs,
                   uint32_t stage_elems, NllArgs<T> na) {
  constexpr uint32_t NT = kTmaFwdThreads;
  constexpr uint32_t VEC = VecN<T>::value;
  constexpr bool KEEP = (MODE == FWD_SOFTMAX || MODE == FWD_NLLBWD);  // exponentials stay in the stage
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* const stage0 = reinterpret_cast<T*>(smem_raw);   // stage s starts at stage0 + s*stage_elems
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ T red_max[NT / 32], red_sum[NT / 32];
  __shared__ MS<T> slot[2];
  __shared__ MS<T> fin;
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
      if (g.body)
        bulk_copy_g2s(stage0 + s * stage_elems + g.sh + g.head, gp + g.head, g.body * (uint32_t)sizeof(T), &bar[s]);
    }
    load_ragged(gp, len, g, stage0 + s * stage_elems);
  };

  uint32_t seg = blockIdx.x;
  if (seg < nseg) issue(seg, 0);
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t s = it & 1;
    if (seg + gridDim.x < nseg) issue(seg + gridDim.x, s ^ 1);
    if (!mbar_wait_bounded(&bar[s], (it >> 1) & 1) && tid == 0) atomicExch(&g_wait_timeout_flag, 1);
    __syncthreads();  // ragged elements stored by other threads
    const T* gp = x + (uint64_t)seg * D + a0;
    const SliceGeom<T> g = slice_geom(gp, len);
    T* buf = stage0 + s * stage_elems + g.sh;
    // local maximum
    T mx = -Math<T>::inf();
    slice_walk<T, false, NT>(buf, len, g,
        [&](Pack<T, VEC>& p, uint32_t) {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++) mx = p.v[e] > mx ? p.v[e] : mx;
        },
        [&](T& v, uint32_t) { mx = v > mx ? v : mx; });
    mx = cta_reduce<T, NT>(mx, [](T a, T b) { return a > b ? a : b; }, red_max);
    // local sum of exp(x - max); softmax keeps the exponentials in place
    T sum = (T)0;
    slice_walk<T, KEEP, NT>(buf, len, g,
        [&](Pack<T, VEC>& p, uint32_t) {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++) {
            const T ex = Math<T>::exp_neg(p.v[e] - mx);
            if (KEEP) p.v[e] = ex;
            sum += ex;
          }
        },
        [&](T& v, uint32_t) {
          const T ex = Math<T>::exp_neg(v - mx);
          if (KEEP) v = ex;
          sum += ex;
        });
    sum = cta_reduce<T, NT>(sum, [](T a, T b) { return a + b; }, red_sum);
    MS<T> ms{mx, sum};
    if (len == 0) ms = ms_init<T>();
    T rescale = (T)1;  // exp(local max - global max), applied to the stored exponentials
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (tid == 0) slot[s] = ms;
      cluster.sync();
      if (tid < 32) {  // one warp fetches the peers' pairs through distributed shared memory
        MS<T> v = tid < cs ? *cluster.map_shared_rank(&slot[s], tid) : ms_init<T>();
        v = ms_warp(v);
        if (tid == 0) fin = v;
      }
      __syncthreads();
      const MS<T> tot = fin;
      rescale = Math<T>::exp_neg(mx - tot.m);
      ms = tot;
    }
    const T logs = Math<T>::log(ms.s);
    const T pk = rescale / ms.s;  // stored exponential -> probability
    int32_t label = 0;
    T scale = (T)0;
    if (MODE == FWD_NLLBWD) {
      label = na.labels[seg];
      scale = label == 0 ? (T)0 : nll_scale(na);
    }
    const uint32_t lab_local = (uint32_t)(label - 1 - (int32_t)a0);  // wraps to "never" for label 0
    auto value = [&](T v, uint32_t i) -> T {
      if (MODE == FWD_LOGSOFTMAX) return (v - ms.m) - logs;
      const T p = v * pk;
      if (MODE == FWD_SOFTMAX) return p;
      return ((label != 0 && i == lab_local) ? p - (T)1 : p) * scale;
    };
    T* yp = y + (uint64_t)seg * D + a0;
    if ((((uintptr_t)yp ^ (uintptr_t)gp) & 15u) == 0) {
      // output shares the input's alignment: 128-bit loads from the stage, 128-bit stores
      slice_walk<T, false, NT>(buf, len, g,
          [&](Pack<T, VEC>& p, uint32_t i0) {
            Pack<T, VEC> o;
#pragma unroll
            for (uint32_t e = 0; e < VEC; e++) o.v[e] = value(p.v[e], i0 + e);
            st_stream<T, VEC>(yp + i0, o);
          },
          [&](T& v, uint32_t i) { yp[i] = value(v, i); });
    } else {
      segment_store<T>(yp, len, tid, NT, [&](uint32_t i) { return value(buf[i], i); });
    }
    __syncthreads();  // everyone is done with this stage before the next copy lands in it
  }
  if (cs > 1) cg::this_cluster().sync();  // peers may still be reading this CTA's slot
}

template <typename T, int MODE>
__global__ void __launch_bounds__(kTmaBwdThreads)
seg_tma_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D,
                   uint32_t nseg, uint32_t cs, uint32_t stage_elems) {
  constexpr uint32_t NT = kTmaBwdThreads;
  constexpr uint32_t VEC = VecN<T>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* base = reinterpret_cast<T*>(smem_raw);
  // stage s: y slice at base + 2*s*stage_elems, dy slice one stage_elems further
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ T red[NT / 32];
  __shared__ T slot[2];
  __shared__ T fin;
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
      T* ys = base + 2 * s * stage_elems;
      if (gy.body) bulk_copy_g2s(ys + gy.sh + gy.head, yp + gy.head, gy.body * (uint32_t)sizeof(T), &bar[s]);
      if (gg.body)
        bulk_copy_g2s(ys + stage_elems + gg.sh + gg.head, gp + gg.head, gg.body * (uint32_t)sizeof(T), &bar[s]);
    }
    load_ragged(yp, len, gy, base + 2 * s * stage_elems);
    load_ragged(gp, len, gg, base + 2 * s * stage_elems + stage_elems);
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
    T* xp = dx + (uint64_t)seg * D + a0;
    const SliceGeom<T> gy = slice_geom(yp, len), gg = slice_geom(gp, len);
    const T* ybuf = base + 2 * s * stage_elems + gy.sh;
    const T* gbuf = base + 2 * s * stage_elems + stage_elems + gg.sh;
    // all three arrays on the same offset inside a 16-byte line: paired 128-bit accesses
    const bool aligned = gy.sh == gg.sh && ((((uintptr_t)xp ^ (uintptr_t)yp) & 15u) == 0);
    const Pack<T, VEC>* yv = reinterpret_cast<const Pack<T, VEC>*>(ybuf + gy.head);
    const Pack<T, VEC>* gv = reinterpret_cast<const Pack<T, VEC>*>(gbuf + gy.head);
    const uint32_t nvec = gy.body / VEC, tail0 = gy.head + gy.body;
    T acc = (T)0;
    if (aligned) {
#pragma unroll 2
      for (uint32_t v = tid; v < nvec; v += NT) {
        const Pack<T, VEC> a = yv[v], b = gv[v];
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) acc += MODE == BWD_SOFTMAX ? a.v[e] * b.v[e] : b.v[e];
      }
      if (tid < gy.head) acc += MODE == BWD_SOFTMAX ? ybuf[tid] * gbuf[tid] : gbuf[tid];
      if (tid < len - tail0) acc += MODE == BWD_SOFTMAX ? ybuf[tail0 + tid] * gbuf[tail0 + tid] : gbuf[tail0 + tid];
    } else {
      for (uint32_t i = tid; i < len; i += NT) acc += MODE == BWD_SOFTMAX ? ybuf[i] * gbuf[i] : gbuf[i];
    }
    acc = cta_reduce<T, NT>(acc, [](T a, T b) { return a + b; }, red);
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (tid == 0) slot[s] = acc;
      cluster.sync();
      if (tid < 32) {
        T v = tid < cs ? *cluster.map_shared_rank(&slot[s], tid) : (T)0;
        v = warp_reduce(v, [](T a, T b) { return a + b; });
        if (tid == 0) fin = v;
      }
      __syncthreads();
      acc = fin;
    }
    auto value = [&](T a, T b) -> T {
      return MODE == BWD_SOFTMAX ? a * b - a * acc : b - Math<T>::exp_neg(a) * acc;
    };
    if (aligned) {
#pragma unroll 2
      for (uint32_t v = tid; v < nvec; v += NT) {
        const Pack<T, VEC> a = yv[v], b = gv[v];
        Pack<T, VEC> o;
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) o.v[e] = value(a.v[e], b.v[e]);
        st_stream<T, VEC>(xp + gy.head + v * VEC, o);
      }
      if (tid < gy.head) xp[tid] = value(ybuf[tid], gbuf[tid]);
      if (tid < len - tail0) xp[tail0 + tid] = value(ybuf[tail0 + tid], gbuf[tail0 + tid]);
    } else {
      segment_store<T>(xp, len, tid, NT, [&](uint32_t i) { return value(ybuf[i], gbuf[i]); });
    }
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
