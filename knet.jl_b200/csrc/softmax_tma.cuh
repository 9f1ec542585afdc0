// Long contiguous runs (a (C,B) score matrix with C in the tens of thousands): persistent
// thread-block clusters with bulk-copy (TMA) staging.
//
// A cluster of `cs` CTAs owns one instance at a time; CTA r holds slice r of the run in
// shared memory.  Each CTA keeps NS stage buffers: while it reduces and writes instance i,
// the bulk copies of the next NS-1 instances of its cluster are already in flight, so HBM
// reads never wait for the arithmetic.  One thread issues one bulk copy per slice (the
// 16-byte aligned interior; the few ragged elements at either end travel through registers)
// and an mbarrier counts the bytes.  The slice is placed in shared memory at the same offset
// inside a 16-byte line as it has in global memory, which is what makes the aligned interior
// a legal bulk copy for any run length, and lets every pass use 128-bit shared-memory
// accesses.
//
// Inside a CTA every warp owns a contiguous part of the slice and reduces it on its own
// (maximum, then sum of exponentials relative to that maximum), so the only CTA-wide
// barriers of an iteration are the exchange and the hand-back of the stage.  The exchange is
// a push: each warp writes its (max, sum) pair into the slot tables of all CTAs of the
// cluster through distributed shared memory, one cluster barrier makes them visible, and
// the first warp of each CTA folds the table locally.  DRAM sees every input once and
// every output once; the arithmetic is about ten instructions per element.
//
// Included by softmax.cu after MS, NllArgs and segment_store are defined.
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

// The ragged ends of a slice, fetched into registers when the bulk copy is issued and put
// into the stage at the end of the iteration, so that their latency hides behind the
// arithmetic instead of holding up the first warp.  At most VEC-1 elements at either end.
template <typename T> struct Ragged {
  T h, t;
};
template <typename T>
__device__ __forceinline__ Ragged<T> ragged_fetch(const T* gp, uint32_t len, const SliceGeom<T>& g) {
  const uint32_t tid = threadIdx.x, tail0 = g.head + g.body;
  Ragged<T> r{(T)0, (T)0};
  if (tid < g.head) r.h = gp[tid];
  if (tid < len - tail0) r.t = gp[tail0 + tid];
  return r;
}
template <typename T>
__device__ __forceinline__ void ragged_commit(const Ragged<T>& r, uint32_t len, const SliceGeom<T>& g, T* stage) {
  const uint32_t tid = threadIdx.x, tail0 = g.head + g.body;
  if (tid < g.head) stage[g.sh + tid] = r.h;
  if (tid < len - tail0) stage[g.sh + tail0 + tid] = r.t;
}

// The part of a staged slice that one warp owns: packs [v0, v1) of the aligned interior;
// warp 0 also owns the ragged ends (lanes below `head`, lanes below len - tail0).
struct WarpPart {
  uint32_t v0, v1;
};
template <int NT>
__device__ __forceinline__ WarpPart warp_part(uint32_t nvec) {
  constexpr uint32_t NW = NT / 32;
  const uint32_t w = threadIdx.x >> 5, chunk = (nvec + NW - 1) / NW;
  WarpPart p;
  p.v0 = min(nvec, w * chunk);
  p.v1 = min(nvec, p.v0 + chunk);
  return p;
}

// Walk this warp's part: fv(pack&, index of its first element) with 128-bit shared-memory
// accesses (written back when WRITE), fs(value&, index) for the ragged ends.  `buf` points at
// element 0 of the slice; buf + g.head is 16-byte aligned.
template <typename T, bool WRITE, typename FV, typename FS>
__device__ __forceinline__ void part_walk(T* buf, uint32_t len, const SliceGeom<T>& g, const WarpPart& wp, FV&& fv,
                                          FS&& fs) {
  constexpr uint32_t VEC = VecN<T>::value;
  const uint32_t tid = threadIdx.x, lane = tid & 31;
  Pack<T, VEC>* vb = reinterpret_cast<Pack<T, VEC>*>(buf + g.head);
#pragma unroll 2
  for (uint32_t v = wp.v0 + lane; v < wp.v1; v += 32) {
    Pack<T, VEC> p = vb[v];
    fv(p, g.head + v * VEC);
    if (WRITE) vb[v] = p;
  }
  const uint32_t tail0 = g.head + g.body;
  if (tid < g.head) fs(buf[tid], tid);
  if (tid < len - tail0) fs(buf[tail0 + tid], tail0 + tid);
}

// ---- forward: softmax, logsoftmax, and the nll gradient (softmax - onehot) * scale ------------
// NTHR threads per CTA, NS stage buffers (copies run NS-1 instances ahead of the arithmetic)
template <typename T, int MODE, int NTHR, int NS>
__global__ void __launch_bounds__(NTHR)
seg_tma_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, uint32_t cs,
                   uint32_t stage_elems, NllArgs<T> na) {
  constexpr uint32_t NT = NTHR, NW = NT / 32, MAXCS = 8;
  constexpr uint32_t VEC = VecN<T>::value;
  constexpr bool KEEP = (MODE == FWD_SOFTMAX || MODE == FWD_NLLBWD);  // exponentials stay in the stage
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* const stage0 = reinterpret_cast<T*>(smem_raw);   // stage s starts at stage0 + s*stage_elems
  __shared__ __align__(8) uint64_t bar[NS];
  __shared__ MS<T> table[2][MAXCS * NW];   // (max, sum) of every warp of every CTA of the cluster
  __shared__ MS<T> fin;
  const uint32_t tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const uint32_t rank = blockIdx.y;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, rank * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    for (int j = 0; j < NS; j++) mbar_init(&bar[j], 1);
    mbar_init_fence();
  }
  __syncthreads();

  // arm the barrier, start the bulk copy of the aligned interior, fetch the ragged ends
  auto issue = [&](uint32_t seg, uint32_t s, SliceGeom<T>& g) -> Ragged<T> {
    const T* gp = x + (uint64_t)seg * D + a0;
    g = slice_geom(gp, len);
    if (tid == 0) {
      mbar_arrive_expect_tx(&bar[s], g.body * (uint32_t)sizeof(T));
      if (g.body)
        bulk_copy_g2s(stage0 + s * stage_elems + g.sh + g.head, gp + g.head, g.body * (uint32_t)sizeof(T), &bar[s]);
    }
    return ragged_fetch(gp, len, g);
  };

  uint32_t seg = blockIdx.x;
  for (uint32_t j = 0; j + 1 < NS; j++)
    if (seg + j * gridDim.x < nseg) {
      SliceGeom<T> g0;
      const Ragged<T> r0 = issue(seg + j * gridDim.x, j, g0);
      ragged_commit(r0, len, g0, stage0 + j * stage_elems);
    }
  __syncthreads();
  uint32_t s = 0, ph = 0;  // stage of this iteration and the parity of its barrier phase
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    // the stage freed at the end of the previous iteration takes the copy NS-1 instances ahead
    const uint32_t pre = seg + (NS - 1) * gridDim.x, spre = s == 0 ? NS - 1 : s - 1;
    SliceGeom<T> gpre{};
    Ragged<T> rpre{};
    if (pre < nseg) rpre = issue(pre, spre, gpre);
    if (!mbar_wait_bounded(&bar[s], ph) && tid == 0) atomicExch(&g_wait_timeout_flag, 1);
    const T* gp = x + (uint64_t)seg * D + a0;
    const SliceGeom<T> g = slice_geom(gp, len);
    T* buf = stage0 + s * stage_elems + g.sh;
    const WarpPart wp = warp_part<NT>(g.body / VEC);
    const uint32_t tb = it & 1;  // slot table of this iteration

    // this warp's maximum, then its sum of exp(x - that maximum)
    T mx = -Math<T>::inf();
    part_walk<T, false>(buf, len, g, wp,
        [&](Pack<T, VEC>& p, uint32_t) {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++) mx = p.v[e] > mx ? p.v[e] : mx;
        },
        [&](T& v, uint32_t) { mx = v > mx ? v : mx; });
    mx = warp_reduce(mx, [](T a, T b) { return a > b ? a : b; });
    T sum = (T)0;
    part_walk<T, KEEP>(buf, len, g, wp,
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
    sum = warp_reduce(sum, [](T a, T b) { return a + b; });
    if (mx == -Math<T>::inf()) sum = (T)0;  // an empty part: exp(-inf + inf) is not a number

    // push this warp's pair to every CTA of the cluster, one barrier, fold the table locally
    const MS<T> mine{mx, sum};
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (lane < cs) *cluster.map_shared_rank(&table[tb][rank * NW + w], lane) = mine;
      cluster.sync();
    } else {
      if (lane == 0) table[tb][w] = mine;
      __syncthreads();
    }
    if (w == 0) {
      MS<T> v = ms_init<T>();
      for (uint32_t i = lane; i < cs * NW; i += 32) v = ms_merge(v, table[tb][i]);
      v = ms_warp(v);
      if (lane == 0) fin = v;
    }
    __syncthreads();
    const MS<T> ms = fin;
    const T logs = Math<T>::log(ms.s);
    const T pk = Math<T>::exp_neg(mx - ms.m) / ms.s;  // this warp's stored exponential -> probability
    int32_t label = 0;
    T scale = (T)0;
    if (MODE == FWD_NLLBWD) {
      label = na.labels[seg];
      scale = label == 0 ? (T)0 : nll_scale(na);
    }
    const uint32_t lab_local = (uint32_t)(label - 1 - (int32_t)a0);
    auto value = [&](T v, uint32_t i) -> T {
      if (MODE == FWD_LOGSOFTMAX) return (v - ms.m) - logs;
      const T p = v * pk;
      if (MODE == FWD_SOFTMAX) return p;
      return ((label != 0 && i == lab_local) ? p - (T)1 : p) * scale;
    };
    T* yp = y + (uint64_t)seg * D + a0;
    if ((((uintptr_t)yp ^ (uintptr_t)gp) & 15u) == 0) {
      // output shares the input's alignment: 128-bit loads from the stage, 128-bit stores
      part_walk<T, false>(buf, len, g, wp,
          [&](Pack<T, VEC>& p, uint32_t i0) {
            Pack<T, VEC> o;
#pragma unroll
            for (uint32_t e = 0; e < VEC; e++) o.v[e] = value(p.v[e], i0 + e);
            st_stream<T, VEC>(yp + i0, o);
          },
          [&](T& v, uint32_t i) { yp[i] = value(v, i); });
    } else {
      // element by element in the owner's order (the stored exponentials are per warp)
      part_walk<T, false>(buf, len, g, wp,
          [&](Pack<T, VEC>& p, uint32_t i0) {
#pragma unroll
            for (uint32_t e = 0; e < VEC; e++) yp[i0 + e] = value(p.v[e], i0 + e);
          },
          [&](T& v, uint32_t i) { yp[i] = value(v, i); });
    }
    if (pre < nseg) ragged_commit(rpre, len, gpre, stage0 + spre * stage_elems);
    __syncthreads();  // this stage is free for the next copy; the ragged ends above are visible
    if (++s == NS) { s = 0; ph ^= 1; }
  }
  if (cs > 1) cg::this_cluster().sync();  // no CTA leaves while peers may still push into its table
}

// ---- backward: softmax y.*dy .- y.*sum(y.*dy), logsoftmax dy - exp.(y).*sum(dy) ---------------
template <typename T, int MODE, int NTHR, int NS>
__global__ void __launch_bounds__(NTHR)
seg_tma_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D,
                   uint32_t nseg, uint32_t cs, uint32_t stage_elems) {
  constexpr uint32_t NT = NTHR, NW = NT / 32, MAXCS = 8;
  constexpr uint32_t VEC = VecN<T>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // stage s: y slice at base + 2*s*stage_elems, dy slice one stage_elems further
  T* const base = reinterpret_cast<T*>(smem_raw);
  __shared__ __align__(8) uint64_t bar[NS];
  __shared__ T table[2][MAXCS * NW];
  __shared__ T fin;
  const uint32_t tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const uint32_t rank = blockIdx.y;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, rank * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    for (int j = 0; j < NS; j++) mbar_init(&bar[j], 1);
    mbar_init_fence();
  }
  __syncthreads();

  struct Rag2 {
    Ragged<T> y, g;
    SliceGeom<T> gy, gg;
  };
  auto issue = [&](uint32_t seg, uint32_t s) -> Rag2 {
    const T* yp = y + (uint64_t)seg * D + a0;
    const T* gp = dy + (uint64_t)seg * D + a0;
    Rag2 r;
    r.gy = slice_geom(yp, len);
    r.gg = slice_geom(gp, len);
    if (tid == 0) {
      T* ys = base + 2 * s * stage_elems;
      mbar_arrive_expect_tx(&bar[s], (r.gy.body + r.gg.body) * (uint32_t)sizeof(T));
      if (r.gy.body)
        bulk_copy_g2s(ys + r.gy.sh + r.gy.head, yp + r.gy.head, r.gy.body * (uint32_t)sizeof(T), &bar[s]);
      if (r.gg.body)
        bulk_copy_g2s(ys + stage_elems + r.gg.sh + r.gg.head, gp + r.gg.head, r.gg.body * (uint32_t)sizeof(T),
                      &bar[s]);
    }
    r.y = ragged_fetch(yp, len, r.gy);
    r.g = ragged_fetch(gp, len, r.gg);
    return r;
  };
  auto commit = [&](const Rag2& r, uint32_t s) {
    ragged_commit(r.y, len, r.gy, base + 2 * s * stage_elems);
    ragged_commit(r.g, len, r.gg, base + 2 * s * stage_elems + stage_elems);
  };

  uint32_t seg = blockIdx.x;
  for (uint32_t j = 0; j + 1 < NS; j++)
    if (seg + j * gridDim.x < nseg) commit(issue(seg + j * gridDim.x, j), j);
  __syncthreads();
  uint32_t s = 0, ph = 0;
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t pre = seg + (NS - 1) * gridDim.x, spre = s == 0 ? NS - 1 : s - 1;
    Rag2 rpre{};
    if (pre < nseg) rpre = issue(pre, spre);
    if (!mbar_wait_bounded(&bar[s], ph) && tid == 0) atomicExch(&g_wait_timeout_flag, 1);
    const T* yp = y + (uint64_t)seg * D + a0;
    const T* gp = dy + (uint64_t)seg * D + a0;
    T* xp = dx + (uint64_t)seg * D + a0;
    const SliceGeom<T> gy = slice_geom(yp, len), gg = slice_geom(gp, len);
    const T* ybuf = base + 2 * s * stage_elems + gy.sh;
    const T* gbuf = base + 2 * s * stage_elems + stage_elems + gg.sh;
    const uint32_t tb = it & 1;
    // all three arrays on the same offset inside a 16-byte line: paired 128-bit accesses
    const bool aligned = gy.sh == gg.sh && ((((uintptr_t)xp ^ (uintptr_t)yp) & 15u) == 0);
    const Pack<T, VEC>* yv = reinterpret_cast<const Pack<T, VEC>*>(ybuf + gy.head);
    const Pack<T, VEC>* gv = reinterpret_cast<const Pack<T, VEC>*>(gbuf + gy.head);
    const uint32_t nvec = gy.body / VEC, tail0 = gy.head + gy.body;
    const WarpPart wp = warp_part<NT>(nvec);
    T acc = (T)0;
    if (aligned) {
#pragma unroll 2
      for (uint32_t v = wp.v0 + lane; v < wp.v1; v += 32) {
        const Pack<T, VEC> a = yv[v], b = gv[v];
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) acc += MODE == BWD_SOFTMAX ? a.v[e] * b.v[e] : b.v[e];
      }
      if (tid < gy.head) acc += MODE == BWD_SOFTMAX ? ybuf[tid] * gbuf[tid] : gbuf[tid];
      if (tid < len - tail0) acc += MODE == BWD_SOFTMAX ? ybuf[tail0 + tid] * gbuf[tail0 + tid] : gbuf[tail0 + tid];
    } else {
      for (uint32_t i = tid; i < len; i += NT) acc += MODE == BWD_SOFTMAX ? ybuf[i] * gbuf[i] : gbuf[i];
    }
    acc = warp_reduce(acc, [](T a, T b) { return a + b; });
    if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (lane < cs) *cluster.map_shared_rank(&table[tb][rank * NW + w], lane) = acc;
      cluster.sync();
    } else {
      if (lane == 0) table[tb][w] = acc;
      __syncthreads();
    }
    if (w == 0) {
      T v = (T)0;
      for (uint32_t i = lane; i < cs * NW; i += 32) v += table[tb][i];
      v = warp_reduce(v, [](T a, T b) { return a + b; });
      if (lane == 0) fin = v;
    }
    __syncthreads();
    const T tot = fin;
    auto value = [&](T a, T b) -> T {
      return MODE == BWD_SOFTMAX ? a * b - a * tot : b - Math<T>::exp_neg(a) * tot;
    };
    if (aligned) {
#pragma unroll 2
      for (uint32_t v = wp.v0 + lane; v < wp.v1; v += 32) {
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
    if (pre < nseg) commit(rpre, spre);
    __syncthreads();
    if (++s == NS) { s = 0; ph ^= 1; }
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
inline TmaPlan plan_tma(uint64_t D, uint32_t nseg, int arrays, int threads, int stages, int sms) {
  TmaPlan p{};
  // preferred bytes per stage buffer: measured best on B200 for forward and backward alike
  // (larger slices amortise the per-instance barriers; the copies keep HBM busy meanwhile)
  size_t target = 52 * 1024;
  if (const char* e = getenv("KNET_SM100_TMA_TARGET_KB")) target = (size_t)atoi(e) * 1024;   // tuning runs
  const size_t limit = 220 * 1024;                        // dynamic shared memory we are willing to ask for
  uint32_t cs = 1;
  while (cs < 8 && ((D + cs - 1) / cs) * sizeof(T) > target) cs *= 2;
  // few instances: split further so that every SM gets work
  while (cs < 8 && (uint64_t)nseg * cs < (uint64_t)2 * sms && D / (cs * 2) >= 2048) cs *= 2;
  const uint64_t slice = (D + cs - 1) / cs;
  const uint64_t stage_elems = (slice + 2 * VecN<T>::value + 31) / 32 * 32;   // room for the shift, 128-byte multiple
  const size_t smem = (size_t)stage_elems * sizeof(T) * stages * arrays;
  if (smem > limit) return p;
  const int by_smem = (int)((227 * 1024) / (smem + 2048));
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
