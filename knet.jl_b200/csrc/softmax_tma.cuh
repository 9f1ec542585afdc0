// Long contiguous runs (a (C,B) score matrix with C in the tens of thousands): persistent
// thread-block clusters with bulk-copy (TMA) staging.
//
// A cluster of `cs` CTAs owns one instance at a time; CTA r holds slice r of the run in
// shared memory.  Each CTA has two stage buffers: while it works on instance i, the bulk copy
// of its cluster's next instance is already in flight, so HBM reads never wait for the
// arithmetic (measured: 2-3 % of a CTA's time is spent waiting for a copy).  One thread issues
// one bulk copy per slice (the 16-byte aligned interior; the few ragged elements at either
// end travel through registers) and an mbarrier counts the bytes.  The slice is placed in
// shared memory at the same offset inside a 16-byte line as it has in global memory, which
// is what makes the aligned interior a legal bulk copy for any run length and lets the
// threads fetch it with 128-bit shared-memory loads.
//
// Inside a CTA every warp owns a contiguous part of the slice; each thread moves its share
// of that part into registers once and all passes run on registers (these kernels are bound
// by instruction issue, not by HBM, once the copies are overlapped).  The only rendezvous of
// an iteration is the exchange, a push: each warp sends its partial result into the slot
// tables of all CTAs of the cluster with st.async, whose bytes are counted by an mbarrier of
// the receiving CTA; a warp continues when its own CTA's barrier has seen all cs x warps
// results, and folds the table for itself.  There is no cluster-wide barrier in the loop (the
// older exchange, plain remote stores + cluster barrier, is kept behind a launch flag), and the
// same completion also orders the reuse of the stage buffers.  DRAM sees every input once and
// every output once.
//
// Included by softmax.cu after MS, NllArgs and segment_store are defined.
#pragma once
#include "tma.cuh"

namespace kn {

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

// ---- forward: softmax, logsoftmax, and the nll gradient (softmax - onehot) * scale ------------
// Two stage buffers per CTA.  Once a slice has landed, every thread moves its share of it
// (at most PPT 16-byte packs, strided over its warp's part) from shared memory into
// registers with independent 128-bit loads, and all three passes (maximum, sum of
// exponentials, output) run on registers: shared memory is read once, and the stage is
// free for the next bulk copy as soon as the CTA passes the exchange barrier.  The ragged
// ends never touch shared memory: the registers that fetched them at issue time are carried
// into the next iteration.
// Two CTAs of 256 threads per SM for every PPT: letting the short-slice instantiations run three
// or four CTAs per SM (64-80 registers) was measured slower, not faster.
template <typename T, int MODE, int NTHR, int PPT>
__global__ void __launch_bounds__(NTHR, 512 / NTHR)
seg_tma_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t D, uint32_t nseg, uint32_t cs,
                   uint32_t stage_elems, NllArgs<T> na, uint32_t xchg_async) {
  constexpr uint32_t NT = NTHR, NW = NT / 32, MAXCS = 8, NS = 2;
  constexpr uint32_t VEC = VecN<T>::value;
  constexpr bool KEEP = (MODE == FWD_SOFTMAX || MODE == FWD_NLLBWD);  // exponentials replace the values
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* const stage0 = reinterpret_cast<T*>(smem_raw);   // stage s starts at stage0 + s*stage_elems
  __shared__ __align__(8) uint64_t bar[NS];
  __shared__ __align__(8) uint64_t xbar[2];                // counts the bytes pushed into table[0|1]
  __shared__ __align__(16) MS<T> table[2][MAXCS * NW];     // (max, sum) of every warp of every CTA of the cluster
  const uint32_t tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const uint32_t rank = blockIdx.y;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, rank * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    for (int j = 0; j < (int)NS; j++) mbar_init(&bar[j], 1);
    for (int j = 0; j < 2; j++) mbar_init(&xbar[j], 1);
    mbar_init_fence();
  }
  __syncthreads();
  const bool push_async = xchg_async != 0 && cs > 1;
  if (push_async) cg::this_cluster().sync();   // peers' barriers are initialised before anyone pushes

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
  SliceGeom<T> g{};
  Ragged<T> rag{};
  if (seg < nseg) rag = issue(seg, 0, g);
  // nll gradient: the scale is the same for every instance, and the label of an instance is
  // fetched one iteration ahead like the ragged ends, so no iteration waits for global memory
  int32_t label = 0;
  T nll_sc = (T)0;
  if (MODE == FWD_NLLBWD) {
    nll_sc = nll_scale(na);
    if (seg < nseg) label = na.labels[seg];
  }
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t s = it & 1, ph = (it >> 1) & 1, tb = it & 1;
    // the other stage was read into registers before the exchange barrier of the previous iteration
    const uint32_t nxt = seg + gridDim.x;
    SliceGeom<T> gnext{};
    Ragged<T> ragnext{};
    if (nxt < nseg) ragnext = issue(nxt, s ^ 1, gnext);
    if (push_async && tid == 0) mbar_arrive_expect_tx(&xbar[tb], cs * NW * (uint32_t)sizeof(MS<T>));
    int32_t label_next = 0;
    if (MODE == FWD_NLLBWD && nxt < nseg) label_next = na.labels[nxt];
    if (!mbar_wait_bounded(&bar[s], ph) && tid == 0) note_wait_timeout();
    const T* gp = x + (uint64_t)seg * D + a0;
    const WarpPart wp = warp_part<NT>(g.body / VEC);
    const uint32_t tail0 = g.head + g.body;
    const bool has_h = tid < g.head, has_t = tid < len - tail0;
    const Pack<T, VEC>* vb = reinterpret_cast<const Pack<T, VEC>*>(stage0 + s * stage_elems + g.sh + g.head);
    Pack<T, VEC> r[PPT];
#pragma unroll
    for (int k = 0; k < PPT; k++) {
      const uint32_t v = wp.v0 + lane + 32u * k;
      if (v < wp.v1) {
        r[k] = vb[v];
      } else {
#pragma unroll
        for (uint32_t e = 0; e < VEC; e++) r[k].v[e] = -Math<T>::inf();
      }
    }
    T rh = has_h ? rag.h : -Math<T>::inf(), rt = has_t ? rag.t : -Math<T>::inf();

    // this warp's maximum, then its sum of exp(x - that maximum)
    T mx = fmax(rh, rt);
#pragma unroll
    for (int k = 0; k < PPT; k++) {      // written as nested two-operand maxima so that three-input forms can be used
      T pm = r[k].v[0];
#pragma unroll
      for (uint32_t e = 1; e + 1 < VEC; e += 2) pm = fmax(fmax(pm, r[k].v[e]), r[k].v[e + 1]);
      mx = (VEC % 2 == 0) ? fmax(fmax(mx, pm), r[k].v[VEC - 1]) : fmax(mx, pm);
    }
    mx = warp_reduce(mx, [](T a, T b) { return a > b ? a : b; });
    // two elements per instruction where the type has packed arithmetic (Two<float>)
    Two<T> acc[VEC / 2];
#pragma unroll
    for (uint32_t e = 0; e < VEC / 2; e++) acc[e] = two((T)0);
    const Two<T> neg_mx = two(-mx);
#pragma unroll
    for (int k = 0; k < PPT; k++)
#pragma unroll
      for (uint32_t e = 0; e < VEC; e += 2) {
        const Two<T> ex = exp_neg2(add2(Two<T>{r[k].v[e], r[k].v[e + 1]}, neg_mx));   // exp(-inf) = 0 for the padding
        if (KEEP) { r[k].v[e] = ex.a; r[k].v[e + 1] = ex.b; }
        acc[e / 2] = add2(acc[e / 2], ex);
      }
    {
      const Two<T> ex = exp_neg2(add2(Two<T>{rh, rt}, neg_mx));
      if (KEEP) { rh = ex.a; rt = ex.b; }
      acc[0] = add2(acc[0], ex);
    }
    T sum = acc[0].a + acc[0].b;
#pragma unroll
    for (uint32_t e = 1; e < VEC / 2; e++) sum += acc[e].a + acc[e].b;
    sum = warp_reduce(sum, [](T a, T b) { return a + b; });
    if (mx == -Math<T>::inf()) sum = (T)0;  // an empty part: exp(-inf + inf) is not a number

    // push this warp's pair to every CTA of the cluster; one barrier; every warp folds the table
    const MS<T> mine{mx, sum};
    if (push_async) {
      // each pair travels with a byte count for the receiving CTA's barrier: no cluster-wide barrier;
      // a warp goes on as soon as all cs*NW pairs of this instance have reached its own CTA
      if (lane < cs) {
        const uint32_t dst = mapa_u32(&table[tb][rank * NW + w], lane), dbar = mapa_u32(&xbar[tb], lane);
        if constexpr (sizeof(T) == 4) {
          st_async_b64(dst, ((uint64_t)__float_as_uint((float)mine.s) << 32) | __float_as_uint((float)mine.m), dbar);
        } else {
          st_async_v2b64(dst, (uint64_t)__double_as_longlong((double)mine.m), (uint64_t)__double_as_longlong((double)mine.s), dbar);
        }
      }
      if (!mbar_wait_cluster_bounded(&xbar[tb], ph) && lane == 0) note_wait_timeout();
    } else if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (lane < cs) *cluster.map_shared_rank(&table[tb][rank * NW + w], lane) = mine;
      cluster.sync();
    } else {
      if (lane == 0) table[tb][w] = mine;
      __syncthreads();
    }
    // (every warp does this for itself: about forty instructions, and no second barrier):
    // the maximum over the table, then the sums rescaled to it; empty parts hold (-inf, 0)
    MS<T> ms;
    {
      T m = -Math<T>::inf();
      for (uint32_t i = lane; i < cs * NW; i += 32) m = fmax(m, table[tb][i].m);
      m = warp_reduce(m, [](T a, T b) { return a > b ? a : b; });
      T part = (T)0;
      for (uint32_t i = lane; i < cs * NW; i += 32) {
        const MS<T> e = table[tb][i];
        if (e.s != (T)0) part += e.s * Math<T>::exp_neg(e.m - m);
      }
      ms.m = m;
      ms.s = warp_reduce(part, [](T a, T b) { return a + b; });
    }
    const T logs = Math<T>::log(ms.s);
    const T pk = Math<T>::exp_neg(mx - ms.m) / ms.s;  // this warp's stored exponential -> probability
    const T scale = (MODE == FWD_NLLBWD && label != 0) ? nll_sc : (T)0;
    const uint32_t lab_local = (uint32_t)(label - 1 - (int32_t)a0);
    auto value = [&](T v, uint32_t i) -> T {
      if (MODE == FWD_LOGSOFTMAX) return (v - ms.m) - logs;
      const T p = v * pk;
      if (MODE == FWD_SOFTMAX) return p;
      return ((label != 0 && i == lab_local) ? p - (T)1 : p) * scale;
    };
    T* yp = y + (uint64_t)seg * D + a0;
    const bool vec_out = (((uintptr_t)yp ^ (uintptr_t)gp) & 15u) == 0;   // output shares the input's alignment
    // the same arithmetic as value(), two elements at a time; the label's element is patched afterwards
    const Two<T> neg_m = two(-ms.m), neg_logs = two(-logs), pk2 = two(pk), scale2 = two(scale);
#pragma unroll
    for (int k = 0; k < PPT; k++) {
      const uint32_t v = wp.v0 + lane + 32u * k;
      if (v < wp.v1) {
        const uint32_t i0 = g.head + v * VEC;
        Pack<T, VEC> o;
#pragma unroll
        for (uint32_t e = 0; e < VEC; e += 2) {
          Two<T> t{r[k].v[e], r[k].v[e + 1]};
          if (MODE == FWD_LOGSOFTMAX) t = add2(add2(t, neg_m), neg_logs);
          else t = mul2(t, pk2);
          if (MODE == FWD_NLLBWD) t = mul2(t, scale2);
          o.v[e] = t.a;
          o.v[e + 1] = t.b;
        }
        if (MODE == FWD_NLLBWD && label != 0 && lab_local - i0 < VEC) {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++)
            if (i0 + e == lab_local) o.v[e] = value(r[k].v[e], i0 + e);
        }
        if (vec_out) {
          st_stream<T, VEC>(yp + i0, o);
        } else {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++) yp[i0 + e] = o.v[e];
        }
      }
    }
    if (has_h) yp[tid] = value(rh, tid);
    if (has_t) yp[tail0 + tid] = value(rt, tail0 + tid);
    g = gnext;
    rag = ragnext;
    label = label_next;
  }
  if (cs > 1) cg::this_cluster().sync();  // no CTA leaves while peers may still push into its table
}

// ---- backward: softmax y.*dy .- y.*sum(y.*dy), logsoftmax dy - exp.(y).*sum(dy) ---------------
// The same scheme with two staged inputs.  When y, dy and dx share their offset inside a
// 16-byte line (always, for whole arrays) each thread keeps its packs of y and dy in
// registers for both passes; otherwise the passes walk shared memory element by element and
// the stage is handed back by a CTA barrier at the end of the iteration.
template <typename T, int MODE, int NTHR, int PPT>
__global__ void __launch_bounds__(NTHR, 1)
seg_tma_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, uint32_t D,
                   uint32_t nseg, uint32_t cs, uint32_t stage_elems, uint32_t xchg_async) {
  constexpr uint32_t NT = NTHR, NW = NT / 32, MAXCS = 8, NS = 2;
  constexpr uint32_t VEC = VecN<T>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // stage s: y slice at base + 2*s*stage_elems, dy slice one stage_elems further
  T* const base = reinterpret_cast<T*>(smem_raw);
  __shared__ __align__(8) uint64_t bar[NS];
  __shared__ __align__(8) uint64_t xbar[2];            // counts the bytes pushed into table[0|1]
  __shared__ __align__(8) T table[2][MAXCS * NW];
  const uint32_t tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const uint32_t rank = blockIdx.y;
  const uint32_t slice = (D + cs - 1) / cs;
  const uint32_t a0 = min(D, rank * slice), len = min(D, a0 + slice) - a0;
  if (tid == 0) {
    for (int j = 0; j < (int)NS; j++) mbar_init(&bar[j], 1);
    for (int j = 0; j < 2; j++) mbar_init(&xbar[j], 1);
    mbar_init_fence();
  }
  __syncthreads();
  const bool push_async = xchg_async != 0 && cs > 1;
  if (push_async) cg::this_cluster().sync();   // peers' barriers are initialised before anyone pushes

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

  uint32_t seg = blockIdx.x;
  Rag2 cur{};
  if (seg < nseg) cur = issue(seg, 0);
  for (uint32_t it = 0; seg < nseg; seg += gridDim.x, it++) {
    const uint32_t s = it & 1, ph = (it >> 1) & 1, tb = it & 1;
    const uint32_t nxt = seg + gridDim.x;
    Rag2 next{};
    if (nxt < nseg) next = issue(nxt, s ^ 1);
    if (push_async && tid == 0) mbar_arrive_expect_tx(&xbar[tb], cs * NW * (uint32_t)sizeof(T));
    if (!mbar_wait_bounded(&bar[s], ph) && tid == 0) note_wait_timeout();
    const T* yp = y + (uint64_t)seg * D + a0;
    T* xp = dx + (uint64_t)seg * D + a0;
    const SliceGeom<T> gy = cur.gy, gg = cur.gg;
    T* ystage = base + 2 * s * stage_elems;
    const T* ybuf = ystage + gy.sh;
    const T* gbuf = ystage + stage_elems + gg.sh;
    // all three arrays on the same offset inside a 16-byte line: paired 128-bit accesses
    const bool aligned = gy.sh == gg.sh && ((((uintptr_t)xp ^ (uintptr_t)yp) & 15u) == 0);
    const Pack<T, VEC>* yv = reinterpret_cast<const Pack<T, VEC>*>(ybuf + gy.head);
    const Pack<T, VEC>* gv = reinterpret_cast<const Pack<T, VEC>*>(gbuf + gy.head);
    const uint32_t tail0 = gy.head + gy.body;
    const WarpPart wp = warp_part<NT>(gy.body / VEC);
    const bool has_h = tid < gy.head, has_t = tid < len - tail0;
    Pack<T, VEC> a[PPT], b[PPT];          // y and dy packs of this thread (aligned case)
    T ah = (T)0, at = (T)0, bh = (T)0, bt = (T)0;
    T acc = (T)0;
    if (aligned) {
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const uint32_t v = wp.v0 + lane + 32u * k;
        if (v < wp.v1) {
          a[k] = yv[v];
          b[k] = gv[v];
        } else {
#pragma unroll
          for (uint32_t e = 0; e < VEC; e++) { a[k].v[e] = (T)0; b[k].v[e] = (T)0; }   // adds nothing to either sum
        }
      }
      if (has_h) { ah = cur.y.h; bh = cur.g.h; }
      if (has_t) { at = cur.y.t; bt = cur.g.t; }
      Two<T> acc2[VEC / 2];
#pragma unroll
      for (uint32_t e = 0; e < VEC / 2; e++) acc2[e] = two((T)0);
#pragma unroll
      for (int k = 0; k < PPT; k++)
#pragma unroll
        for (uint32_t e = 0; e < VEC; e += 2) {
          const Two<T> a2{a[k].v[e], a[k].v[e + 1]}, b2{b[k].v[e], b[k].v[e + 1]};
          acc2[e / 2] = add2(acc2[e / 2], MODE == BWD_SOFTMAX ? mul2(a2, b2) : b2);
        }
      acc = MODE == BWD_SOFTMAX ? ah * bh + at * bt : bh + bt;
#pragma unroll
      for (uint32_t e = 0; e < VEC / 2; e++) acc += acc2[e].a + acc2[e].b;
    } else {
      ragged_commit(cur.y, len, gy, ystage);
      ragged_commit(cur.g, len, gg, ystage + stage_elems);
      __syncthreads();
      for (uint32_t i = tid; i < len; i += NT) acc += MODE == BWD_SOFTMAX ? ybuf[i] * gbuf[i] : gbuf[i];
    }
    acc = warp_reduce(acc, [](T p, T q) { return p + q; });
    if (push_async) {
      if (lane < cs) {
        const uint32_t dst = mapa_u32(&table[tb][rank * NW + w], lane), dbar = mapa_u32(&xbar[tb], lane);
        if constexpr (sizeof(T) == 4) st_async_b32(dst, __float_as_uint((float)acc), dbar);
        else st_async_b64(dst, (uint64_t)__double_as_longlong((double)acc), dbar);
      }
      if (!mbar_wait_cluster_bounded(&xbar[tb], ph) && lane == 0) note_wait_timeout();
    } else if (cs > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (lane < cs) *cluster.map_shared_rank(&table[tb][rank * NW + w], lane) = acc;
      cluster.sync();
    } else {
      if (lane == 0) table[tb][w] = acc;
      __syncthreads();
    }
    T tot = (T)0;                        // every warp adds the table up for itself, in a fixed order
    for (uint32_t i = lane; i < cs * NW; i += 32) tot += table[tb][i];
    tot = warp_reduce(tot, [](T p, T q) { return p + q; });
    auto value = [&](T av, T bv) -> T {
      return MODE == BWD_SOFTMAX ? av * bv - av * tot : bv - Math<T>::exp_neg(av) * tot;
    };
    if (aligned) {
      const Two<T> neg_tot = two(-tot);
#pragma unroll
      for (int k = 0; k < PPT; k++) {
        const uint32_t v = wp.v0 + lane + 32u * k;
        if (v < wp.v1) {
          Pack<T, VEC> o;
#pragma unroll
          for (uint32_t e = 0; e < VEC; e += 2) {
            const Two<T> a2{a[k].v[e], a[k].v[e + 1]}, b2{b[k].v[e], b[k].v[e + 1]};
            const Two<T> r2 = MODE == BWD_SOFTMAX ? add2(mul2(a2, b2), mul2(a2, neg_tot))
                                                  : add2(b2, mul2(exp_neg2(a2), neg_tot));
            o.v[e] = r2.a;
            o.v[e + 1] = r2.b;
          }
          st_stream<T, VEC>(xp + gy.head + v * VEC, o);
        }
      }
      if (has_h) xp[tid] = value(ah, bh);
      if (has_t) xp[tail0 + tid] = value(at, bt);
    } else {
      segment_store<T>(xp, len, tid, NT, [&](uint32_t i) { return value(ybuf[i], gbuf[i]); });
      __syncthreads();   // the stage is read until here: hand it back before the next copy is issued
    }
    cur = next;
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
inline TmaPlan plan_tma(uint64_t D, uint32_t nseg, int arrays, int threads, int stages, int sms,
                        size_t max_slice_bytes = 0) {
  TmaPlan p{};
  // preferred bytes per stage buffer: measured best on B200 for forward and backward alike
  // (larger slices amortise the per-instance barriers; the copies keep HBM busy meanwhile)
  size_t target = 52 * 1024;
  if (const char* e = getenv("KNET_SM100_TMA_TARGET_KB")) target = (size_t)atoi(e) * 1024;   // tuning runs
  if (max_slice_bytes && target > max_slice_bytes) target = max_slice_bytes;   // what the registers of a CTA hold
  const size_t limit = 220 * 1024;                        // dynamic shared memory we are willing to ask for
  uint32_t cs = 1;
  while (cs < 8 && ((D + cs - 1) / cs) * sizeof(T) > target) cs *= 2;
  // few instances: split further so that every SM gets work
  while (cs < 8 && (uint64_t)nseg * cs < (uint64_t)2 * sms && D / (cs * 2) >= 2048) cs *= 2;
  if (const char* e = getenv("KNET_SM100_TMA_CS")) {       // tuning runs: any cluster size 1..8
    const int v = atoi(e);
    if (v >= 1 && v <= 8) cs = (uint32_t)v;
  }
  const uint64_t slice = (D + cs - 1) / cs;
  const uint64_t stage_elems = (slice + 2 * VecN<T>::value + 31) / 32 * 32;   // room for the shift, 128-byte multiple
  const size_t smem = (size_t)stage_elems * sizeof(T) * stages * arrays;
  if (smem > limit) return p;
  if (max_slice_bytes && slice * sizeof(T) > max_slice_bytes) return p;
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
