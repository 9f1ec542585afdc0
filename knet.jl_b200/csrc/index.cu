// Index kernels: whole columns / rows picked by 1-based Int32 indices (embedding lookup and
// its scatter-add backward), pitched 2-d copy and fill behind range indexing, and icat.
//
// A column of a column-major matrix is one contiguous run, so the column kernels move
// 16-byte vectors whenever the column length and both base pointers allow it, several
// independent vectors per thread; the scatter-add uses the 16-byte vector reduction
// (red.global.v4.f32.add) for Float32.  The row kernels gather single elements, which is
// what the operation is; they keep the dense side (y) coalesced.
#include "common.cuh"
#include "tma.cuh"

namespace kn {

enum { IX_GET = 0, IX_SET = 1, IX_ADD = 2, IX_SET1 = 3 };

template <typename T, int VEC> __device__ __forceinline__ void red_add(T* p, const Pack<T, VEC>& v) {
  if constexpr (sizeof(T) == 4 && VEC == 4) {
    asm volatile("red.global.v4.f32.add [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.v[0]), "f"(v.v[1]),
                 "f"(v.v[2]), "f"(v.v[3])
                 : "memory");
  } else {
#pragma unroll
    for (int e = 0; e < VEC; e++) atomicAdd(p + e, v.v[e]);
  }
}

// The matrix side x is read with an L2 evict-last policy (an index may repeat, and a
// vocabulary-sized x has hot columns) while the dense side y streams with evict-first
// accesses, so that the stream does not push the table out of L2.
__device__ __forceinline__ uint64_t l2_keep_policy() {
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> ld_keep(const T* p, uint64_t pol) {
  Pack<T, VEC> r;
  if constexpr (sizeof(T) * VEC == 16) {
    uint4 t;
    asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(t.x), "=r"(t.y), "=r"(t.z), "=r"(t.w) : "l"(p), "l"(pol));
    *reinterpret_cast<uint4*>(&r) = t;
  } else if constexpr (sizeof(T) * VEC == 8) {
    uint2 t;
    asm volatile("ld.global.nc.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;" : "=r"(t.x), "=r"(t.y) : "l"(p), "l"(pol));
    *reinterpret_cast<uint2*>(&r) = t;
  } else {
    uint32_t t;
    asm volatile("ld.global.nc.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(t) : "l"(p), "l"(pol));
    *reinterpret_cast<uint32_t*>(&r) = t;
  }
  return r;
}
template <typename T, int VEC> __device__ __forceinline__ void st_plain(T* p, const Pack<T, VEC>& v) {
  if constexpr (sizeof(T) * VEC == 16) {
    *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(&v);
  } else if constexpr (sizeof(T) * VEC == 8) {
    *reinterpret_cast<float2*>(p) = *reinterpret_cast<const float2*>(&v);
  } else {
    *p = v.v[0];
  }
}

// ---- columns ------------------------------------------------------------------------------
// rv = vectors per column, total = rv * ncols vectors of y.  I is the flat index type.
template <typename T, int MODE, int VEC, typename I>
__global__ void __launch_bounds__(256)
cols_kernel(I rv, I total, const int* __restrict__ cols, T* x, T* y, T y1) {
  constexpr int U = 4;
  const I step = (I)gridDim.x * (256 * U);
  const uint64_t keep = l2_keep_policy();
  for (I base = (I)blockIdx.x * (256 * U) + threadIdx.x; base < total; base += step) {
    Pack<T, VEC> v[U];
    int64_t xo[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const I iv = base + (I)u * 256;
      if (iv < total) {
        const I col = iv / rv, r = iv - col * rv;
        xo[u] = (((int64_t)__ldg(cols + col) - 1) * (int64_t)rv + (int64_t)r) * VEC;
        if (MODE == IX_GET) v[u] = ld_keep<T, VEC>(x + xo[u], keep);
        else if (MODE != IX_SET1) v[u] = ld_stream<T, VEC>(y + (int64_t)iv * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const I iv = base + (I)u * 256;
      if (iv < total) {
        if (MODE == IX_GET) st_stream<T, VEC>(y + (int64_t)iv * VEC, v[u]);
        else if (MODE == IX_SET) st_plain<T, VEC>(x + xo[u], v[u]);
        else if (MODE == IX_ADD) red_add<T, VEC>(x + xo[u], v[u]);
        else {
          Pack<T, VEC> c;
#pragma unroll
          for (int e = 0; e < VEC; e++) c.v[e] = y1;
          st_plain<T, VEC>(x + xo[u], c);
        }
      }
    }
  }
}

// ctas_per_sm == 0: one block per `per_block` items (each block runs its loop once and
// leaves, so blocks sweep memory in address order like the elementwise engine's); the
// kernels still loop, which covers grids clipped at the 2^31-1 limit.
inline unsigned grid_for(uint64_t items, int per_block, int ctas_per_sm) {
  uint64_t blocks = (items + per_block - 1) / per_block;
  const uint64_t cap = ctas_per_sm > 0 ? (uint64_t)sm_count() * ctas_per_sm : 0x7fffffffull;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks ? blocks : 1);
}

template <typename T, int MODE, int VEC>
void launch_cols(int xrows, int ncols, const int* cols, T* x, T* y, T y1, cudaStream_t s) {
  const uint64_t rv = (uint64_t)xrows / VEC, total = rv * (uint64_t)ncols;
  const unsigned g = grid_for(total, 256 * 4, 0);
  if (total < ((uint64_t)1 << 31))
    cols_kernel<T, MODE, VEC, uint32_t><<<g, 256, 0, s>>>((uint32_t)rv, (uint32_t)total, cols, x, y, y1);
  else
    cols_kernel<T, MODE, VEC, uint64_t><<<g, 256, 0, s>>>(rv, total, cols, x, y, y1);
}

template <typename T, int MODE>
void run_cols(int xrows, int xcols, int ncols, const int* cols, T* x, T* y, T y1, cudaStream_t s) {
  if (!(ncols > 0 && xrows > 0 && xcols > 0)) return;
  constexpr int VEC = VecN<T>::value;
  const uintptr_t bits = (uintptr_t)x | (MODE == IX_SET1 ? 0 : (uintptr_t)y);
  if (xrows % VEC == 0 && (bits & 15) == 0) launch_cols<T, MODE, VEC>(xrows, ncols, cols, x, y, y1, s);
  else if (VEC == 4 && xrows % 2 == 0 && (bits & 7) == 0) launch_cols<T, MODE, 2>(xrows, ncols, cols, x, y, y1, s);
  else launch_cols<T, MODE, 1>(xrows, ncols, cols, x, y, y1, s);
}

// ---- rows ---------------------------------------------------------------------------------
// y is (nrows, xcols); flat index over y; element (i, c) pairs with x[rows[i]-1 + c*xrows].
template <typename T, int MODE, typename I>
__global__ void __launch_bounds__(256)
rows_kernel(I nrows, I total, int64_t xrows, const int* __restrict__ rows, T* x, T* y, T y1, FastDiv fd) {
  constexpr int U = 4;
  const I step = (I)gridDim.x * (256 * U);
  for (I base = (I)blockIdx.x * (256 * U) + threadIdx.x; base < total; base += step) {
    T v[U];
    int64_t xo[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const I iy = base + (I)u * 256;
      if (iy < total) {
        // one division per element: by multiply-high when the indices fit 31 bits
        const I c = sizeof(I) == 4 ? (I)div_fast((uint32_t)iy, fd) : iy / nrows, i = iy - c * nrows;
        xo[u] = (int64_t)__ldg(rows + i) - 1 + (int64_t)c * xrows;
        if (MODE == IX_GET) v[u] = __ldg(x + xo[u]);
        else if (MODE != IX_SET1) v[u] = __ldcs(y + iy);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const I iy = base + (I)u * 256;
      if (iy < total) {
        if (MODE == IX_GET) __stcs(y + iy, v[u]);
        else if (MODE == IX_SET) x[xo[u]] = v[u];
        else if (MODE == IX_ADD) atomicAdd(x + xo[u], v[u]);
        else x[xo[u]] = y1;
      }
    }
  }
}

// getrows when the picked rows are dense in the column (nrows >= xrows / 8): single-element
// gathers then touch nearly every 32-byte sector of x, and each sector crosses from L2 to the SM
// once per element read from it.  Here a CTA copies a whole column into shared memory with
// 16-byte loads (x is read exactly once), picks from there and writes y in 16-byte groups; several
// CTAs per SM overlap one another's load and pick phases.  Indices are clamped into the column,
// so a stray index reads a neighbouring row instead of leaving the buffer.
constexpr int kRowsStageThreads = 256;
constexpr int kRowsBulkThreads = 512;    // the double-buffered forms: shared memory, not threads, limits their CTAs per SM
constexpr int kRowsStageBytes = 48 * 1024;

template <typename T, int XV, bool YVEC>
__global__ void __launch_bounds__(kRowsStageThreads)
rows_get_staged_kernel(int nrows, int xrows, int xcols, const int* __restrict__ rows, const T* __restrict__ x,
                       T* __restrict__ y) {
  extern __shared__ __align__(128) unsigned char stage_raw[];
  T* col = reinterpret_cast<T*>(stage_raw);
  const int last = xrows - 1;
  for (int c = blockIdx.x; c < xcols; c += gridDim.x) {
    const T* xc = x + (int64_t)c * xrows;
    if (XV > 1) {
#pragma unroll 4
      for (int r = threadIdx.x * XV; r < xrows; r += kRowsStageThreads * XV)
        *reinterpret_cast<Pack<T, XV>*>(col + r) = ld_stream<T, XV>(xc + r);
    } else {
      for (int r = threadIdx.x; r < xrows; r += kRowsStageThreads) col[r] = __ldcs(xc + r);
    }
    __syncthreads();
    T* yc = y + (int64_t)c * nrows;
    if (YVEC) {   // four picks per thread and step: one int4 of indices, 16-byte stores
      constexpr int PER = 16 / (int)sizeof(T);
      for (int i = threadIdx.x * 4; i < nrows; i += kRowsStageThreads * 4) {
        const int4 ix = __ldg(reinterpret_cast<const int4*>(rows + i));
        const int id[4] = {ix.x, ix.y, ix.z, ix.w};
#pragma unroll
        for (int g = 0; g < 4 / PER; g++) {
          Pack<T, PER> v;
#pragma unroll
          for (int e = 0; e < PER; e++) v.v[e] = col[min(max(id[g * PER + e] - 1, 0), last)];
          st_stream<T, PER>(yc + i + g * PER, v);
        }
      }
    } else {
      for (int i = threadIdx.x; i < nrows; i += kRowsStageThreads)
        __stcs(yc + i, col[min(max(__ldg(rows + i) - 1, 0), last)]);
    }
    __syncthreads();   // the next column overwrites the buffer
  }
}

// After a wait gave up in iteration *broken - 1 the CTA issued no further copy; the copies of that
// iteration and of the next one (if issued) may still be in flight into this CTA's shared memory,
// so thread 0 waits for them once more, bounded, before the CTA exits.
__device__ __forceinline__ void drain_after_timeout(uint64_t* bar, const int* broken, int last_issued) {
  if (threadIdx.x != 0 || *broken == 0) return;
  for (int j = *broken - 1; j <= last_issued; j++) mbar_wait_bounded(&bar[j & 1], (uint32_t)(j >> 1) & 1u);
}

// The same with the columns brought in by bulk asynchronous copies into two buffers: while the CTA
// picks from one column the next one is already in flight, so each CTA keeps a whole column of
// reads outstanding all the time.  Needs 16-byte aligned columns.  The wait on a copy is bounded;
// if one ever gave up the CTA raises the library's wait flag (knet_device_status), stops issuing
// copies, picks straight from global memory and, before it exits, waits once more (bounded) for the
// copies it still has in flight.
template <typename T, bool YVEC>
__global__ void __launch_bounds__(kRowsBulkThreads)
rows_get_bulk_kernel(int nrows, int xrows, int xcols, const int* __restrict__ rows, const T* __restrict__ x,
                     T* __restrict__ y) {
  extern __shared__ __align__(128) unsigned char stage_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(stage_raw);          // two barriers, then the broken flag
  int* broken = reinterpret_cast<int*>(stage_raw + 16);
  const uint32_t colbytes = (uint32_t)xrows * (uint32_t)sizeof(T);
  T* buf0 = reinterpret_cast<T*>(stage_raw + 32);
  const int tid = threadIdx.x, last = xrows - 1;
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *broken = 0;
    mbar_init_fence();
  }
  __syncthreads();
  auto issue = [&](int c, int s) {
    mbar_arrive_expect_tx(&bar[s], colbytes);
    bulk_copy_g2s(buf0 + (size_t)s * xrows, x + (int64_t)c * xrows, colbytes, &bar[s]);
  };
  int c = blockIdx.x;
  int last_issued = -1;                     // thread 0: the last iteration whose copy was issued
  if (tid == 0 && c < xcols) {
    issue(c, 0);
    last_issued = 0;
  }
  for (int it = 0; c < xcols; c += gridDim.x, it++) {
    const int s = it & 1;
    const uint32_t ph = (uint32_t)(it >> 1) & 1u;
    bool direct = *broken != 0;
    // the other buffer was last read before the barrier that ended the previous iteration
    if (tid == 0 && !direct && c + (int)gridDim.x < xcols) {
      issue(c + (int)gridDim.x, s ^ 1);
      last_issued = it + 1;
    }
    if (!direct && !mbar_wait_bounded(&bar[s], ph)) {
      *broken = it + 1; // any thread may say so (same value); every thread of this iteration that timed out goes direct
      note_wait_timeout();
      direct = true;
    }
    const T* col = buf0 + (size_t)s * xrows;
    const T* xc = x + (int64_t)c * xrows;
    T* yc = y + (int64_t)c * nrows;
    if (YVEC) {
      constexpr int PER = 16 / (int)sizeof(T);
      for (int i = tid * 4; i < nrows; i += kRowsBulkThreads * 4) {
        const int4 ix = __ldg(reinterpret_cast<const int4*>(rows + i));
        const int id[4] = {ix.x, ix.y, ix.z, ix.w};
#pragma unroll
        for (int g = 0; g < 4 / PER; g++) {
          Pack<T, PER> v;
#pragma unroll
          for (int e = 0; e < PER; e++) {
            const int r = min(max(id[g * PER + e] - 1, 0), last);
            v.v[e] = direct ? __ldg(xc + r) : col[r];
          }
          st_stream<T, PER>(yc + i + g * PER, v);
        }
      }
    } else {
      for (int i = tid; i < nrows; i += kRowsBulkThreads) {
        const int r = min(max(__ldg(rows + i) - 1, 0), last);
        __stcs(yc + i, direct ? __ldg(xc + r) : col[r]);
      }
    }
    __syncthreads();   // this buffer may be refilled from the next iteration on
  }
  drain_after_timeout(bar, broken, last_issued);
}

// setrows / addrows with dense picks, the mirror image: the column comes into shared memory by a
// bulk copy (two buffers, the next column in flight), the y values are stored or added there
// (shared-memory atomics for addrows: repeated indices accumulate, as the global atomics of the
// flat kernel do), and the whole column goes back with 16-byte stores.  x is read and written
// once; the flat kernel pays a read-modify-write of a 32-byte sector for every 4-byte element.
// With repeated indices setrows keeps one of the candidates, which one is not defined (nor is it
// in the reference).
template <typename T, int MODE, bool YVEC>
__global__ void __launch_bounds__(kRowsBulkThreads)
rows_put_bulk_kernel(int nrows, int xrows, int xcols, const int* __restrict__ rows, T* __restrict__ x,
                     const T* __restrict__ y) {
  constexpr int XV = VecN<T>::value;
  extern __shared__ __align__(128) unsigned char stage_raw[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(stage_raw);
  int* broken = reinterpret_cast<int*>(stage_raw + 16);
  const uint32_t colbytes = (uint32_t)xrows * (uint32_t)sizeof(T);
  T* buf0 = reinterpret_cast<T*>(stage_raw + 32);
  const int tid = threadIdx.x, last = xrows - 1;
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *broken = 0;
    mbar_init_fence();
  }
  __syncthreads();
  auto issue = [&](int c, int s) {
    mbar_arrive_expect_tx(&bar[s], colbytes);
    bulk_copy_g2s(buf0 + (size_t)s * xrows, x + (int64_t)c * xrows, colbytes, &bar[s]);
  };
  int c = blockIdx.x;
  int last_issued = -1;
  if (tid == 0 && c < xcols) {
    issue(c, 0);
    last_issued = 0;
  }
  for (int it = 0; c < xcols; c += gridDim.x, it++) {
    const int s = it & 1;
    const uint32_t ph = (uint32_t)(it >> 1) & 1u;
    T* col = buf0 + (size_t)s * xrows;
    T* xc = x + (int64_t)c * xrows;
    const T* yc = y + (int64_t)c * nrows;
    bool direct = *broken != 0;
    if (tid == 0 && !direct && c + (int)gridDim.x < xcols) {
      issue(c + (int)gridDim.x, s ^ 1);
      last_issued = it + 1;
    }
    if (!direct && !mbar_wait_bounded(&bar[s], ph)) {
      *broken = it + 1;
      note_wait_timeout();
    }
    __syncthreads();
    direct = *broken != 0;          // one answer for the whole CTA: the column is in the buffer, or nobody uses it
    T* dst = direct ? xc : col;
    auto put = [&](int r, T v) {
      r = min(max(r - 1, 0), last);
      if (MODE == IX_ADD) atomicAdd(dst + r, v);
      else dst[r] = v;
    };
    if (YVEC) {
      constexpr int PER = 16 / (int)sizeof(T);
      for (int i = tid * 4; i < nrows; i += kRowsBulkThreads * 4) {
        const int4 ix = __ldg(reinterpret_cast<const int4*>(rows + i));
        const int id[4] = {ix.x, ix.y, ix.z, ix.w};
#pragma unroll
        for (int g = 0; g < 4 / PER; g++) {
          const Pack<T, PER> v = ld_stream<T, PER>(yc + i + g * PER);
#pragma unroll
          for (int e = 0; e < PER; e++) put(id[g * PER + e], v.v[e]);
        }
      }
    } else {
      for (int i = tid; i < nrows; i += kRowsBulkThreads) put(__ldg(rows + i), __ldcs(yc + i));
    }
    __syncthreads();
    if (!direct) {
#pragma unroll 4
      for (int r = tid * XV; r < xrows; r += kRowsBulkThreads * XV)
        st_plain<T, XV>(xc + r, *reinterpret_cast<const Pack<T, XV>*>(col + r));
      // order this CTA's own accesses to the buffer before the bulk copy that will overwrite it
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
  }
  drain_after_timeout(bar, broken, last_issued);
}

template <typename T, int MODE>
bool run_rows_put_bulk(int xrows, int xcols, int nrows, const int* rows, T* x, const T* y, cudaStream_t s) {
  constexpr int VEC = VecN<T>::value;
  if ((int64_t)xrows * (int64_t)sizeof(T) > kRowsStageBytes || (int64_t)nrows * 8 < xrows) return false;
  if (!(xrows % VEC == 0 && ((uintptr_t)x & 15) == 0) || (int64_t)xcols < 2 * (int64_t)sm_count()) return false;
  const bool yv = nrows % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)rows & 15) == 0;
  const size_t smem = 32 + 2 * (size_t)xrows * sizeof(T);
  int per = (int)((size_t)200 * 1024 / (smem + 1024));
  per = per < 1 ? 1 : per > 4 ? 4 : per;      // 512 threads: four CTAs fill an SM
  const int cap = sm_count() * per;
  const unsigned g = (unsigned)(xcols / 2 < cap ? xcols / 2 : cap);
  if (yv) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rows_put_bulk_kernel<T, MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rows_put_bulk_kernel<T, MODE, true><<<g, kRowsBulkThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(rows_put_bulk_kernel<T, MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rows_put_bulk_kernel<T, MODE, false><<<g, kRowsBulkThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  }
  return true;
}

template <typename T>
bool run_rows_get_staged(int xrows, int xcols, int nrows, const int* rows, const T* x, T* y, cudaStream_t s) {
  constexpr int VEC = VecN<T>::value;
  if ((int64_t)xrows * (int64_t)sizeof(T) > kRowsStageBytes || (int64_t)nrows * 8 < xrows || xcols < 16) return false;
  const bool xv = xrows % VEC == 0 && ((uintptr_t)x & 15) == 0;
  // y in 16-byte groups: four indices per int4 load, so nrows must be a multiple of four
  const bool yv = nrows % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)rows & 15) == 0;
  if (xv && (int64_t)xcols >= 2 * (int64_t)sm_count()) {      // enough columns for every CTA to pipeline
    const size_t smem2 = 32 + 2 * (size_t)xrows * sizeof(T);
    int per = (int)((size_t)200 * 1024 / (smem2 + 1024));
    per = per < 1 ? 1 : per > 4 ? 4 : per;      // 512 threads: four CTAs fill an SM
    const int cap2 = sm_count() * per;
    const unsigned g2 = (unsigned)(xcols / 2 < cap2 ? xcols / 2 : cap2);   // at least two columns per CTA
    if (yv) {
      if (smem2 > 48 * 1024) cudaFuncSetAttribute(rows_get_bulk_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
      rows_get_bulk_kernel<T, true><<<g2, kRowsBulkThreads, smem2, s>>>(nrows, xrows, xcols, rows, x, y);
    } else {
      if (smem2 > 48 * 1024) cudaFuncSetAttribute(rows_get_bulk_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
      rows_get_bulk_kernel<T, false><<<g2, kRowsBulkThreads, smem2, s>>>(nrows, xrows, xcols, rows, x, y);
    }
    return true;
  }
  const size_t smem = (size_t)xrows * sizeof(T);
  int per_sm = (int)((size_t)200 * 1024 / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : per_sm > 8 ? 8 : per_sm;
  const int cap = sm_count() * per_sm;
  const unsigned g = (unsigned)(xcols < cap ? xcols : cap);
  if (xv && yv) rows_get_staged_kernel<T, VEC, true><<<g, kRowsStageThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  else if (xv) rows_get_staged_kernel<T, VEC, false><<<g, kRowsStageThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  else if (yv) rows_get_staged_kernel<T, 1, true><<<g, kRowsStageThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  else rows_get_staged_kernel<T, 1, false><<<g, kRowsStageThreads, smem, s>>>(nrows, xrows, xcols, rows, x, y);
  return true;
}

template <typename T, int MODE>
void run_rows(int xrows, int xcols, int nrows, const int* rows, T* x, T* y, T y1, cudaStream_t s) {
  if (!(nrows > 0 && xrows > 0 && xcols > 0)) return;
  if (MODE == IX_GET && run_rows_get_staged<T>(xrows, xcols, nrows, rows, x, y, s)) return;
  if (MODE == IX_SET && run_rows_put_bulk<T, IX_SET>(xrows, xcols, nrows, rows, x, y, s)) return;
  if (MODE == IX_ADD && run_rows_put_bulk<T, IX_ADD>(xrows, xcols, nrows, rows, x, y, s)) return;
  const uint64_t total = (uint64_t)nrows * (uint64_t)xcols;
  const unsigned g = grid_for(total, 256 * 4, 0);
  if (total < ((uint64_t)1 << 31))
    rows_kernel<T, MODE, uint32_t><<<g, 256, 0, s>>>((uint32_t)nrows, (uint32_t)total, xrows, rows, x, y, y1, fast_div((uint32_t)nrows));
  else
    rows_kernel<T, MODE, uint64_t><<<g, 256, 0, s>>>((uint64_t)nrows, total, xrows, rows, x, y, y1, fast_div(1u));
}

// ---- pitched copy / fill --------------------------------------------------------------------
// W = bytes per unit (1, 2, 4, 8 or 16); rw = units per run.
template <int W> struct Unit;
template <> struct Unit<1> { typedef unsigned char type; };
template <> struct Unit<2> { typedef unsigned short type; };
template <> struct Unit<4> { typedef unsigned int type; };
template <> struct Unit<8> { typedef uint2 type; };
template <> struct Unit<16> { typedef uint4 type; };

template <int W, typename I>
__global__ void __launch_bounds__(256)
xcopy_kernel(I rw, I total, const char* __restrict__ x, int64_t incx, char* __restrict__ y, int64_t incy) {
  typedef typename Unit<W>::type V;
  constexpr int U = 4;
  const I step = (I)gridDim.x * (256 * U);
  for (I base = (I)blockIdx.x * (256 * U) + threadIdx.x; base < total; base += step) {
    V v[U];
    int64_t yo[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const I i = base + (I)u * 256;
      if (i < total) {
        const I c = i / rw, r = i - c * rw;
        v[u] = __ldcs(reinterpret_cast<const V*>(x + (int64_t)c * incx + (int64_t)r * W));
        yo[u] = (int64_t)c * incy + (int64_t)r * W;
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++)
      if (base + (I)u * 256 < total) __stcs(reinterpret_cast<V*>(y + yo[u]), v[u]);
  }
}

template <int W>
void launch_xcopy(int nrows, int ncols, const char* x, int incx, char* y, int incy, cudaStream_t s) {
  const uint64_t rw = (uint64_t)nrows / W, total = rw * (uint64_t)ncols;
  const unsigned g = grid_for(total, 256 * 4, 0);
  if (total < ((uint64_t)1 << 31))
    xcopy_kernel<W, uint32_t><<<g, 256, 0, s>>>((uint32_t)rw, (uint32_t)total, x, incx, y, incy);
  else
    xcopy_kernel<W, uint64_t><<<g, 256, 0, s>>>(rw, total, x, incx, y, incy);
}

void run_xcopy(int nrows, int ncols, const void* x, int incx, void* y, int incy, cudaStream_t s) {
  if (!(nrows > 0 && ncols > 0)) return;
  // the widest unit that divides the run length, both pitches and both base addresses
  const uintptr_t bits = (uintptr_t)x | (uintptr_t)y | (uintptr_t)(unsigned)nrows |
                         (ncols > 1 ? ((uintptr_t)(unsigned)incx | (uintptr_t)(unsigned)incy) : 0);
  const char* xs = (const char*)x;
  char* ys = (char*)y;
  if ((bits & 15) == 0) launch_xcopy<16>(nrows, ncols, xs, incx, ys, incy, s);
  else if ((bits & 7) == 0) launch_xcopy<8>(nrows, ncols, xs, incx, ys, incy, s);
  else if ((bits & 3) == 0) launch_xcopy<4>(nrows, ncols, xs, incx, ys, incy, s);
  else if ((bits & 1) == 0) launch_xcopy<2>(nrows, ncols, xs, incx, ys, incy, s);
  else launch_xcopy<1>(nrows, ncols, xs, incx, ys, incy, s);
}

template <typename T, int VEC, typename I>
__global__ void __launch_bounds__(256) xfill_kernel(I rv, I total, T x, T* __restrict__ y, int64_t incy) {
  const I step = (I)gridDim.x * 256;
  Pack<T, VEC> c;
#pragma unroll
  for (int e = 0; e < VEC; e++) c.v[e] = x;
  for (I i = (I)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
    const I col = i / rv, r = i - col * rv;
    st_plain<T, VEC>(y + (int64_t)col * incy + (int64_t)r * VEC, c);
  }
}

template <typename T, int VEC> void launch_xfill(int nrows, int ncols, T x, T* y, int incy, cudaStream_t s) {
  const uint64_t rv = (uint64_t)nrows / VEC, total = rv * (uint64_t)ncols;
  const unsigned g = grid_for(total, 256, 16);
  if (total < ((uint64_t)1 << 31))
    xfill_kernel<T, VEC, uint32_t><<<g, 256, 0, s>>>((uint32_t)rv, (uint32_t)total, x, y, incy);
  else
    xfill_kernel<T, VEC, uint64_t><<<g, 256, 0, s>>>(rv, total, x, y, incy);
}

template <typename T> void run_xfill(int nrows, int ncols, T x, T* y, int incy, cudaStream_t s) {
  if (!(nrows > 0 && ncols > 0)) return;
  constexpr int VEC = VecN<T>::value;
  const bool wide = nrows % VEC == 0 && ((uintptr_t)y & 15) == 0 && (ncols == 1 || incy % VEC == 0);
  if (wide) launch_xfill<T, VEC>(nrows, ncols, x, y, incy, s);
  else launch_xfill<T, 1>(nrows, ncols, x, y, incy, s);
}

// ---- icat -------------------------------------------------------------------------------------
constexpr int kIcatGroup = 64;
template <typename T> struct IcatPtrs { const T* p[kIcatGroup]; };

template <typename T>
__global__ void __launch_bounds__(256) icat_kernel(int nrows, int ncols, IcatPtrs<T> src, T* __restrict__ y) {
  const int64_t total = (int64_t)nrows * ncols, step = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += step) {
    const int col = (int)(i / nrows), row = (int)(i - (int64_t)col * nrows);
    y[i] = src.p[col][row];
  }
}

template <typename T> void run_icat(int nrows, int ncols, T** x, T* y, cudaStream_t s) {
  if (!(nrows > 0 && ncols > 0) || !x) return;
  for (int c0 = 0; c0 < ncols; c0 += kIcatGroup) {
    const int nc = ncols - c0 < kIcatGroup ? ncols - c0 : kIcatGroup;
    IcatPtrs<T> src;
    for (int c = 0; c < kIcatGroup; c++) src.p[c] = c < nc ? x[c0 + c] : nullptr;
    const unsigned g = grid_for((uint64_t)nrows * nc, 256, 16);
    icat_kernel<T><<<g, 256, 0, s>>>(nrows, nc, src, y + (int64_t)c0 * nrows);
  }
}

int index_wait_flag_read_clear() { return wait_flag_read_clear(); }

// ---- the bounded wait, exercised --------------------------------------------------------------------
// One CTA announces 32 bytes on an mbarrier but copies only 16, so the phase cannot complete: the
// wait gives up after `spins` polls, the kernel raises the wait flag, then accounts for the missing
// 16 bytes itself (mbarrier.complete_tx), waits for the phase again - which now completes as soon as
// the real copy has landed - and returns.  Nothing is left in flight and nothing hangs.
// out[0] = 1 if the first wait gave up, out[1] = 1 if the second wait completed, out[2..5] = the
// four copied words.
static __device__ __align__(16) uint32_t g_probe_src[4] = {11u, 22u, 33u, 44u};

__global__ void __launch_bounds__(32) wait_probe_kernel(uint32_t spins, uint32_t* __restrict__ out) {
  __shared__ __align__(16) uint32_t dst[4];
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&bar, 32);
    bulk_copy_g2s(dst, g_probe_src, 16, &bar);
    const bool first = mbar_wait_bounded(&bar, 0, spins);
    if (!first) note_wait_timeout();
    mbar_complete_tx(&bar, 16);
    const bool second = mbar_wait_bounded(&bar, 0);
    out[0] = first ? 0u : 1u;
    out[1] = second ? 1u : 0u;
    for (int i = 0; i < 4; i++) out[2 + i] = second ? dst[i] : 0u;
  }
}

}  // namespace kn

using namespace kn;

KN_EXPORT int knet_debug_wait_probe(uint32_t spins, uint32_t* out6, cudaStream_t s) {
  if (!out6 || spins == 0 || spins > kWaitSpins) return KN_EINVAL;
  wait_probe_kernel<<<1, 32, 0, s>>>(spins, out6);
  return launch_status();
}

#define KN_DEF_COLSROWS(f, S, T)                                                                     \
  KN_EXPORT void getcols_##S##_stream(int xr, int xc, int n, const int* ix, const T* x, T* y,        \
                                      cudaStream_t s) {                                              \
    run_cols<T, IX_GET>(xr, xc, n, ix, const_cast<T*>(x), y, (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void setcols_##S##_stream(int xr, int xc, int n, const int* ix, T* x, const T* y,        \
                                      cudaStream_t s) {                                              \
    run_cols<T, IX_SET>(xr, xc, n, ix, x, const_cast<T*>(y), (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void addcols_##S##_stream(int xr, int xc, int n, const int* ix, T* x, const T* y,        \
                                      cudaStream_t s) {                                              \
    run_cols<T, IX_ADD>(xr, xc, n, ix, x, const_cast<T*>(y), (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void setcol1_##S##_stream(int xr, int xc, int n, const int* ix, T* x, T y,               \
                                      cudaStream_t s) {                                              \
    run_cols<T, IX_SET1>(xr, xc, n, ix, x, nullptr, y, s);                                           \
  }                                                                                                  \
  KN_EXPORT void getrows_##S##_stream(int xr, int xc, int n, const int* ix, const T* x, T* y,        \
                                      cudaStream_t s) {                                              \
    run_rows<T, IX_GET>(xr, xc, n, ix, const_cast<T*>(x), y, (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void setrows_##S##_stream(int xr, int xc, int n, const int* ix, T* x, const T* y,        \
                                      cudaStream_t s) {                                              \
    run_rows<T, IX_SET>(xr, xc, n, ix, x, const_cast<T*>(y), (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void addrows_##S##_stream(int xr, int xc, int n, const int* ix, T* x, const T* y,        \
                                      cudaStream_t s) {                                              \
    run_rows<T, IX_ADD>(xr, xc, n, ix, x, const_cast<T*>(y), (T)0, s);                               \
  }                                                                                                  \
  KN_EXPORT void setrow1_##S##_stream(int xr, int xc, int n, const int* ix, T* x, T y,               \
                                      cudaStream_t s) {                                              \
    run_rows<T, IX_SET1>(xr, xc, n, ix, x, nullptr, y, s);                                           \
  }                                                                                                  \
  KN_EXPORT void getcols_##S(int xr, int xc, int n, const int* ix, const T* x, T* y) {               \
    getcols_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void setcols_##S(int xr, int xc, int n, const int* ix, T* x, const T* y) {               \
    setcols_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void addcols_##S(int xr, int xc, int n, const int* ix, T* x, const T* y) {               \
    addcols_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void setcol1_##S(int xr, int xc, int n, const int* ix, T* x, T y) {                      \
    setcol1_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void getrows_##S(int xr, int xc, int n, const int* ix, const T* x, T* y) {               \
    getrows_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void setrows_##S(int xr, int xc, int n, const int* ix, T* x, const T* y) {               \
    setrows_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void addrows_##S(int xr, int xc, int n, const int* ix, T* x, const T* y) {               \
    addrows_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }                                                                                                  \
  KN_EXPORT void setrow1_##S(int xr, int xc, int n, const int* ix, T* x, T y) {                      \
    setrow1_##S##_stream(xr, xc, n, ix, x, y, cudaStreamPerThread);                                  \
  }
KNET_BOTH_TYPES(KN_DEF_COLSROWS, colsrows)

KN_EXPORT void xcopy_stream(int nrows, int ncols, const void* x, int incx, void* y, int incy, cudaStream_t s) {
  run_xcopy(nrows, ncols, x, incx, y, incy, s);
}
KN_EXPORT void xcopy(int nrows, int ncols, const void* x, int incx, void* y, int incy) {
  run_xcopy(nrows, ncols, x, incx, y, incy, cudaStreamPerThread);
}

#define KN_DEF_XFILL_ICAT(f, S, T)                                                              \
  KN_EXPORT void xfill_##S##_stream(int nrows, int ncols, T x, T* y, int incy, cudaStream_t s) { \
    run_xfill<T>(nrows, ncols, x, y, incy, s);                                                  \
  }                                                                                             \
  KN_EXPORT void xfill_##S(int nrows, int ncols, T x, T* y, int incy) {                         \
    run_xfill<T>(nrows, ncols, x, y, incy, cudaStreamPerThread);                                \
  }                                                                                             \
  KN_EXPORT void icat_##S##_stream(int nrows, int ncols, T** x, T* y, cudaStream_t s) {         \
    run_icat<T>(nrows, ncols, x, y, s);                                                         \
  }                                                                                             \
  KN_EXPORT void icat_##S(int nrows, int ncols, T** x, T* y) {                                  \
    run_icat<T>(nrows, ncols, x, y, cudaStreamPerThread);                                       \
  }
KNET_BOTH_TYPES(KN_DEF_XFILL_ICAT, xfill_icat)
