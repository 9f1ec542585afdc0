// Reductions behind the _20 (whole array), _21 (to a vector) and _22 (one middle dim)
// entry points.
//
// Two memory layouts matter.  "Rows": the kept index is contiguous and the reduced index
// has a stride (sum(x,dims=2) of a column-major matrix) - a warp reads 32 adjacent rows of
// one column per load, so every access is coalesced, columns are split over threadIdx.y
// and, when there are few rows, over the CTAs of a thread-block cluster whose partial
// results meet in distributed shared memory.  "Segments": each output reduces a
// contiguous run (sum(x,dims=1)) - a thread, a warp or a CTA (again with a cluster split
// for long runs and few outputs) walks the run with 128-bit loads.
// All merge orders are fixed by the launch geometry: results are deterministic.
#include <cstdlib>
#include <mutex>

#include "reduce.cuh"

namespace kn {

// ---- rows layout -------------------------------------------------------------------------------
// y[c*ybatch + r] = reduce over col of x[c*xbatch + col*col_stride + r]
// WY = column groups per CTA (blockDim.y), UN = columns a thread has in flight.
template <typename T, typename R, int RV, int WY, int UN>
__global__ void __launch_bounds__(32 * WY, 1024 / (32 * WY))
reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t rows, uint32_t cols,
                   uint64_t col_stride, uint64_t xbatch, uint64_t ybatch, uint32_t cs, uint32_t cols_total) {
  // cols_total != 0: the batches are chunks of `cols` columns of one matrix of cols_total columns
  // (first stage of a split reduction); the last chunk is shorter
  if (cols_total) cols = min(cols, cols_total - min(cols_total, blockIdx.z * cols));
  __shared__ T part[WY][32 * RV];
  __shared__ T total[32 * RV];
  const uint32_t lx = threadIdx.x, ly = threadIdx.y;
  const uint32_t row0 = (blockIdx.x * 32 + lx) * RV;
  const bool valid = row0 < rows;
  const T* xb = x + (uint64_t)blockIdx.z * xbatch + row0;
  // The CTAs of a cluster take blocks of UN*WY consecutive columns in turn (block b belongs to CTA
  // b % cs): at any time the cluster reads one contiguous region that moves through the array.
  constexpr uint32_t BLK = UN * WY;
  T acc[4][RV];
#pragma unroll
  for (int k = 0; k < 4; k++)
#pragma unroll
    for (int e = 0; e < RV; e++) acc[k][e] = R::init();
  if (valid) {
    for (uint32_t b0 = blockIdx.y * BLK; b0 < cols; b0 += cs * BLK) {
      const uint32_t c = b0 + ly;
      if (b0 + BLK <= cols) {
        Pack<T, RV> v[UN];
#pragma unroll
        for (int k = 0; k < UN; k++) v[k] = ld_stream<T, RV>(xb + (uint64_t)(c + k * WY) * col_stride);
#pragma unroll
        for (int k = 0; k < UN; k++)
#pragma unroll
          for (int e = 0; e < RV; e++) acc[k & 3][e] = R::merge(acc[k & 3][e], R::item(v[k].v[e]));
      } else {
#pragma unroll 4
        for (uint32_t cc = c; cc < cols; cc += WY) {
          Pack<T, RV> v = ld_stream<T, RV>(xb + (uint64_t)cc * col_stride);
#pragma unroll
          for (int e = 0; e < RV; e++) acc[0][e] = R::merge(acc[0][e], R::item(v.v[e]));
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < RV; e++) {
    T a = R::merge(R::merge(acc[0][e], acc[1][e]), R::merge(acc[2][e], acc[3][e]));
    part[ly][lx * RV + e] = a;
  }
  __syncthreads();
  if (ly == 0) {
#pragma unroll
    for (int e = 0; e < RV; e++) {
      T a = part[0][lx * RV + e];
#pragma unroll
      for (int k = 1; k < WY; k++) a = R::merge(a, part[k][lx * RV + e]);
      total[lx * RV + e] = a;
    }
  }
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (blockIdx.y == 0 && ly == 0 && valid) {
#pragma unroll
      for (int e = 0; e < RV; e++) {
        T a = total[lx * RV + e];
        for (uint32_t r = 1; r < cs; r++) a = R::merge(a, cluster.map_shared_rank(total, r)[lx * RV + e]);
        y[(uint64_t)blockIdx.z * ybatch + row0 + e] = a;
      }
    }
    cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
  } else if (ly == 0 && valid) {
#pragma unroll
    for (int e = 0; e < RV; e++) y[(uint64_t)blockIdx.z * ybatch + row0 + e] = total[lx * RV + e];
  }
}

// The same reduction with the items already applied: second stage of a split reduction.
template <typename R, typename T> struct MergeOnly : R {
  static __device__ __forceinline__ T item(T x) { return x; }
};

// Scratch for split reductions: stream-ordered allocations from a pool of this library's own (one per
// device, made on first use, never trimmed), so that a call neither synchronises nor shares scratch with
// a call on another stream, and can be captured into a graph.  nullptr: no pool (then nothing is split).
static cudaMemPool_t scratch_pool(cudaStream_t st) {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {};
  static bool tried[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!tried[dev]) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;   // not while capturing
    tried[dev] = true;
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    if (cudaMemPoolCreate(&pools[dev], &props) == cudaSuccess) {
      uint64_t keep = UINT64_MAX;
      cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep);
    } else {
      pools[dev] = nullptr;
      cudaGetLastError();
    }
  }
  return pools[dev];
}

template <typename T, typename R>
void launch_rows(const T* x, T* y, uint32_t rows, uint32_t cols, uint64_t col_stride, uint32_t nbatch,
                 uint64_t xbatch, uint64_t ybatch, uint32_t cols_total, const RowsGeom& g, cudaStream_t st) {
  // UN: every thread keeps 128 bytes in flight whatever the row vector (8 columns of 16 bytes,
  // up to 32 columns of 4 bytes).  With 8 columns a narrow row vector left the kernel short of bytes
  // in flight: sum over dims=2 of 1000 x 32768 Float32 ran at 0.41 of the copy rate.
  constexpr int VEC = VecN<T>::value;
  constexpr int WY = 8;
  constexpr int UN_V = 8, UN_2 = 8 * VEC / (VEC >= 2 ? 2 : 1), UN_1 = 8 * VEC;
  dim3 block(32, WY), grid(g.tiles, g.cs, nbatch);
  auto k = reduce_rows_kernel<T, R, 1, WY, UN_1>;
  if (g.rv == VEC) k = reduce_rows_kernel<T, R, VEC, WY, UN_V>;
  else if (g.rv == 2) k = reduce_rows_kernel<T, R, (VEC >= 2 ? 2 : 1), WY, (VEC >= 2 ? UN_2 : UN_1)>;
  launch_cluster(k, grid, block, 0, st, g.cs, x, y, rows, cols, col_stride, xbatch, ybatch, g.cs, cols_total);
}

template <typename T, typename R>
void run_rows(const T* x, T* y, uint32_t rows, uint32_t cols, uint64_t col_stride, uint32_t nbatch,
              uint64_t xbatch, uint64_t ybatch, cudaStream_t st) {
  if (rows == 0 || nbatch == 0) return;
  constexpr int VEC = VecN<T>::value;
  constexpr int WY = 8;
  static const int forced_cs = [] {
    const char* e = getenv("KNET_SM100_ROWS_CS");   // tuning knob
    return e ? atoi(e) : 0;
  }();
  static const int split_off = [] {
    const char* e = getenv("KNET_SM100_ROWS_NOSPLIT");   // tuning knob: never split a reduction in two stages
    return e ? atoi(e) : 0;
  }();
  auto ok = [&](uint32_t rv) {
    return rv == 1 || (((uintptr_t)x % (rv * sizeof(T))) == 0 && rows % rv == 0 && col_stride % rv == 0 && xbatch % rv == 0);
  };
  const RowsGeom g = rows_geometry(rows, cols, nbatch, VEC, WY, ok, forced_cs, true);
  // Few rows: even a cluster of 8 per tile of rows leaves most SMs idle (64 rows: 16 CTAs), or fills them
  // only with a narrow row vector (128-byte loads per warp: 0.7 of the copy rate at best).  Then the columns
  // are cut into chunks that run as the batches of a first stage writing one partial row vector per chunk,
  // with the widest row vector that wastes at most a quarter of a tile's lanes, and the same kernel merges
  // the partials.  Fixed chunking: repeatable bit for bit.
  const uint64_t target = (uint64_t)sm_count() * 17 / 10;
  uint32_t rvw = 1;
  for (uint32_t rv = VEC; rv > 1; rv /= 2) {
    const uint64_t covered = (uint64_t)((rows + 32 * rv - 1) / (32 * rv)) * 32 * rv;
    if (ok(rv) && covered * 4 <= (uint64_t)rows * 5) { rvw = rv; break; }
  }
  const uint32_t tiles_w = (rows + 32 * rvw - 1) / (32 * rvw);
  const uint32_t blk = 8u * VEC / rvw * WY;                         // columns a CTA takes per turn
  // starved of CTAs: split from 8 MiB on; only a narrower row vector than possible: from 64 MiB on
  // (a 33 MB matrix of 1000 rows measured the same either way, and one launch is one launch fewer)
  const bool starved = (uint64_t)g.tiles * 8 < target;
  const uint64_t nbytes = (uint64_t)rows * cols * sizeof(T);
  if (!split_off && nbatch == 1 && cols >= 16 * blk &&
      ((starved && nbytes >= ((uint64_t)8 << 20)) || (rvw > g.rv && nbytes >= ((uint64_t)64 << 20)))) {
    uint32_t nchunk = (uint32_t)((2 * target + tiles_w - 1) / tiles_w);
    if (nchunk > cols / (4 * blk)) nchunk = cols / (4 * blk);       // at least four turns per chunk
    uint32_t chunk = (cols + nchunk - 1) / nchunk;
    chunk = (chunk + blk - 1) / blk * blk;                          // whole turns, except in the last chunk
    nchunk = (cols + chunk - 1) / chunk;
    cudaMemPool_t pool = nchunk > 1 ? scratch_pool(st) : nullptr;
    T* partial = nullptr;
    if (pool && cudaMallocFromPoolAsync((void**)&partial, (size_t)nchunk * rows * sizeof(T), pool, st) == cudaSuccess) {
      const RowsGeom g1{rvw, tiles_w, 1u};
      launch_rows<T, R>(x, partial, rows, chunk, col_stride, nchunk, (uint64_t)chunk * col_stride, rows, cols, g1, st);
      // second stage: a few hundred columns at most, so 8 columns in flight per thread (turns of 64
      // columns; with turns of 256 the whole merge fell into the kernel's element-wise tail: 9 us)
      const RowsGeom g2 = rows_geometry(rows, nchunk, 1, VEC, WY, [&](uint32_t rv) { return rows % rv == 0; }, 1, false);
      auto k2 = reduce_rows_kernel<T, MergeOnly<R, T>, 1, WY, 8>;
      if (g2.rv == VEC) k2 = reduce_rows_kernel<T, MergeOnly<R, T>, VEC, WY, 8>;
      else if (g2.rv == 2) k2 = reduce_rows_kernel<T, MergeOnly<R, T>, (VEC >= 2 ? 2 : 1), WY, 8>;
      launch_cluster(k2, dim3(g2.tiles, 1, 1), dim3(32, WY), 0, st, 1u, (const T*)partial, y, rows, nchunk, (uint64_t)rows,
                     (uint64_t)0, (uint64_t)0, 1u, 0u);
      cudaFreeAsync(partial, st);
      return;
    }
    cudaGetLastError();   // no scratch: the single launch below
  }
  launch_rows<T, R>(x, y, rows, cols, col_stride, nbatch, xbatch, ybatch, 0, g, st);
}

// ---- segments layout ---------------------------------------------------------------------------
// y[b] = reduce over c in [0,outer), a in [0,len) of x[a + len*(b + ny*c)]

// one thread per output: short runs
template <typename T, typename R>
__global__ void __launch_bounds__(256)
reduce_seg_thread_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t len, uint32_t ny, uint32_t outer) {
  const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= ny) return;
  T acc = R::init();
  for (uint32_t c = 0; c < outer; c++) {
    const T* p = x + (uint64_t)len * (b + (uint64_t)ny * c);
    for (uint32_t a = 0; a < len; a++) acc = R::merge(acc, R::item(__ldg(p + a)));
  }
  y[b] = acc;
}

// one warp per output
template <typename T, typename R>
__global__ void __launch_bounds__(256)
reduce_seg_warp_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t len, uint32_t ny, uint32_t outer) {
  const uint32_t b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= ny) return;
  const uint32_t lane = threadIdx.x & 31;
  T acc = R::init();
  for (uint32_t c = 0; c < outer; c++) {
    const T* p = x + (uint64_t)len * (b + (uint64_t)ny * c);
    segment_visit<T>(p, len, lane, 32, [&](T v, uint32_t) { acc = R::merge(acc, R::item(v)); });
  }
  acc = warp_reduce(acc, [](T a, T b2) { return R::merge(a, b2); });
  if (lane == 0) y[b] = acc;
}

// a group of G lanes per output: the whole run loaded at once in NP packs of 16 bytes per lane
// (packs straddling an end of the run element by element).  Groups past the last output keep
// running with an empty run, so that every lane of the warp takes part in the shuffles.
template <typename T, typename R, int NP, int G>
__global__ void __launch_bounds__(256)
reduce_seg_group_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t len, uint32_t ny) {
  constexpr uint32_t VEC = VecN<T>::value;
  uint32_t b = (uint32_t)(((uint64_t)blockIdx.x * 256 + threadIdx.x) / G);
  const bool live = b < ny;
  if (!live) b = 0;
  const uint32_t lane = threadIdx.x % G;
  const T* p = x + (uint64_t)len * b;
  const uint32_t mis = (uint32_t)(((uintptr_t)p & 15u) / sizeof(T));
  const uint32_t total = mis + (live ? len : 0);
  const T* base = p - mis;
  Pack<T, VEC> v[NP];
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
    if (e0 >= mis && e0 + VEC <= total) v[j] = ld_stream<T, VEC>(base + e0);
  }
  T acc = R::init();
#pragma unroll
  for (int j = 0; j < NP; j++) {
    const uint32_t e0 = ((uint32_t)j * G + lane) * VEC;
    if (e0 >= mis && e0 + VEC <= total) {
#pragma unroll
      for (uint32_t e = 0; e < VEC; e++) acc = R::merge(acc, R::item(v[j].v[e]));
    } else {
#pragma unroll
      for (uint32_t e = 0; e < VEC; e++) {
        const uint32_t i = e0 + e;
        if (i >= mis && i < total) acc = R::merge(acc, R::item(__ldg(base + i)));
      }
    }
  }
#pragma unroll
  for (int o = G / 2; o > 0; o >>= 1) acc = R::merge(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  if (live && lane == 0) y[b] = acc;
}

// one CTA per output, or a cluster of `cs` CTAs that each take a slice of every run
constexpr int kSegThreads = 512;
template <typename T, typename R>
__global__ void __launch_bounds__(kSegThreads)
reduce_seg_block_kernel(const T* __restrict__ x, T* __restrict__ y, uint32_t len, uint32_t ny,
                        uint32_t outer, uint32_t cs) {
  __shared__ T red[32];
  __shared__ T total;
  const uint32_t b = blockIdx.x;
  const uint32_t slice = (len + cs - 1) / cs;
  const uint32_t a0 = min(len, blockIdx.y * slice), a1 = min(len, a0 + slice);
  T acc = R::init();
  for (uint32_t c = 0; c < outer; c++) {
    const T* p = x + (uint64_t)len * (b + (uint64_t)ny * c) + a0;
    segment_visit<T>(p, a1 - a0, threadIdx.x, kSegThreads, [&](T v, uint32_t) { acc = R::merge(acc, R::item(v)); });
  }
  acc = block_reduce(acc, [](T a, T b2) { return R::merge(a, b2); }, R::init(), red);
  if (cs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) total = acc;
    cluster.sync();
    if (blockIdx.y == 0 && threadIdx.x == 0) {
      T a = acc;
      for (uint32_t r = 1; r < cs; r++) a = R::merge(a, *cluster.map_shared_rank(&total, r));
      y[b] = a;
    }
    cluster.sync();
  } else if (threadIdx.x == 0) {
    y[b] = acc;
  }
}

template <typename T, typename R>
void run_segments(const T* x, T* y, uint32_t len, uint32_t ny, uint32_t outer, cudaStream_t st) {
  if (ny == 0) return;
  const int sms = sm_count();
  if (len <= 32) {
    reduce_seg_thread_kernel<T, R><<<(ny + 255) / 256, 256, 0, st>>>(x, y, len, ny, outer);
  } else if ((uint64_t)len * outer <= 8192 && ny >= (uint32_t)(2 * sms)) {
    // Float64: groups of 8 or 16 lanes only (runs of up to 128 elements); with a whole warp per run the
    // streaming warp kernel below measured faster (1000-element runs: 0.94 against 0.62 of the copy rate)
    GroupGeom gg = outer == 1 ? group_geometry<T>(x, len, 16) : GroupGeom{0, 0};
    if (sizeof(T) == 8 && gg.g == 32) gg = GroupGeom{0, 0};
    bool done = false;
#define KN_GROUP_RED(G_, NP_)                                                                               \
  if (gg.g == G_ && gg.np == NP_) {                                                                         \
    reduce_seg_group_kernel<T, R, NP_, G_><<<(unsigned)(((uint64_t)ny * G_ + 255) / 256), 256, 0, st>>>(x, y, len, ny); \
    done = true;                                                                                            \
  }
    KN_GROUP_RED(8, 2) KN_GROUP_RED(8, 4) KN_GROUP_RED(16, 4) KN_GROUP_RED(32, 4) KN_GROUP_RED(32, 8) KN_GROUP_RED(32, 16)
#undef KN_GROUP_RED
    if (!done) reduce_seg_warp_kernel<T, R><<<(ny + 7) / 8, 256, 0, st>>>(x, y, len, ny, outer);
  } else {
    const uint32_t cs = seg_cluster_size(ny, len);
    launch_cluster(reduce_seg_block_kernel<T, R>, dim3(ny, cs, 1), dim3(kSegThreads), 0, st, cs, x, y, len, ny, outer, cs);
  }
}

// _21: x[i] accumulates into y[(i/sy)%ny]
template <typename T, typename R>
void run_21(int nx, const T* x, int sy, int ny, T* y, cudaStream_t st) {
  if (nx <= 0 || ny <= 0 || sy <= 0) return;
  if (sy == 1) {
    run_rows<T, R>(x, y, (uint32_t)ny, (uint32_t)(nx / ny), (uint64_t)ny, 1, 0, 0, st);
  } else {
    run_segments<T, R>(x, y, (uint32_t)sy, (uint32_t)ny, (uint32_t)(nx / ((int64_t)sy * ny)), st);
  }
}

// _22: output bi starts at (bi%s1) + (bi/s1)*s2 and steps s1, xd1+1 times
template <typename T, typename R>
void run_22(int nx, int xd1, const T* x, int s1, int s2, int ny, T* y, cudaStream_t st) {
  if (nx <= 0 || ny <= 0 || s1 <= 0) return;
  const uint32_t nbatch = (uint32_t)(ny / s1);
  // blockIdx.z carries the batch; very long trailing dims go through in slabs of 65535
  for (uint32_t b0 = 0; b0 < nbatch; b0 += 65535) {
    const uint32_t nb = min(65535u, nbatch - b0);
    run_rows<T, R>(x + (uint64_t)b0 * s2, y + (uint64_t)b0 * s1, (uint32_t)s1, (uint32_t)(xd1 + 1),
                   (uint64_t)s1, nb, (uint64_t)s2, (uint64_t)s1, st);
  }
}

// ---- whole array -> scalar ---------------------------------------------------------------------
constexpr int kAllThreads = 512;
constexpr int kAllMaxBlocks = 1024;

template <typename T, typename R>
__global__ void __launch_bounds__(kAllThreads)
reduce_all_stage1(const T* __restrict__ x, uint64_t n, T* __restrict__ partial) {
  __shared__ T red[32];
  // each CTA owns one contiguous slice, so that the slices are walked with aligned loads
  const uint64_t per = (n + gridDim.x - 1) / gridDim.x;
  const uint64_t per_al = (per + 63) & ~(uint64_t)63;
  const uint64_t lo = min(n, (uint64_t)blockIdx.x * per_al), hi = min(n, lo + per_al);
  T acc = R::init();
  // slices longer than 2^31 elements are walked in pieces
  for (uint64_t s = lo; s < hi; s += (1u << 30)) {
    const uint32_t len = (uint32_t)min((uint64_t)(1u << 30), hi - s);
    segment_visit<T>(x + s, len, threadIdx.x, kAllThreads, [&](T v, uint32_t) { acc = R::merge(acc, R::item(v)); });
  }
  acc = block_reduce(acc, [](T a, T b) { return R::merge(a, b); }, R::init(), red);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

template <typename T, typename R>
__global__ void __launch_bounds__(kAllMaxBlocks)
reduce_all_stage2(const T* __restrict__ partial, uint32_t np, T* __restrict__ result) {
  __shared__ T red[32];
  T acc = threadIdx.x < np ? partial[threadIdx.x] : R::init();
  acc = block_reduce(acc, [](T a, T b) { return R::merge(a, b); }, R::init(), red);
  if (threadIdx.x == 0) *result = acc;
}

constexpr size_t kReduceWorkspaceBytes = kAllMaxBlocks * sizeof(double);

template <typename T, typename R>
int run_all(int64_t n, const T* x, T* result, void* ws, cudaStream_t st) {
  if (n < 0) return KN_EINVAL;
  uint64_t blocks = ((uint64_t)n + (uint64_t)kAllThreads * 16 - 1) / ((uint64_t)kAllThreads * 16);
  const uint64_t cap = (uint64_t)min(kAllMaxBlocks, sm_count() * 4);
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  T* partial = reinterpret_cast<T*>(ws);
  reduce_all_stage1<T, R><<<(unsigned)blocks, kAllThreads, 0, st>>>(x, (uint64_t)n, partial);
  reduce_all_stage2<T, R><<<1, kAllMaxBlocks, 0, st>>>(partial, (uint32_t)blocks, result);
  return launch_status();
}

template <typename T>
int run_all_op(int op, int64_t n, const T* x, T* result, void* ws, cudaStream_t st) {
  switch (op) {
    case 0: return run_all<T, R_sum<T>>(n, x, result, ws, st);
    case 1: return run_all<T, R_prod<T>>(n, x, result, ws, st);
    case 2: return run_all<T, R_maximum<T>>(n, x, result, ws, st);
    case 3: return run_all<T, R_minimum<T>>(n, x, result, ws, st);
    case 4: return run_all<T, R_sumabs<T>>(n, x, result, ws, st);
    case 5: return run_all<T, R_sumabs2<T>>(n, x, result, ws, st);
    case 6: return run_all<T, R_maxabs<T>>(n, x, result, ws, st);
    case 7: return run_all<T, R_minabs<T>>(n, x, result, ws, st);
    case 8: return run_all<T, R_countnz<T>>(n, x, result, ws, st);
    default: return KN_EINVAL;
  }
}

// Scratch for the value-returning _20 entry points: a few slots per device, each a device
// workspace plus a pinned host word, created on first use and handed out under a lock so
// that host threads on different streams never share one.  A slot is busy only between
// launch and the stream synchronisation inside the same call.
struct ScalarSlot {
  void* dev = nullptr;
  void* host = nullptr;
  bool busy = false;
};
constexpr int kSlotsPerDevice = 16;
static std::mutex g_slot_mutex;
static ScalarSlot g_slots[64][kSlotsPerDevice];

static ScalarSlot* acquire_slot() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_slot_mutex);
  for (int i = 0; i < kSlotsPerDevice; i++) {
    ScalarSlot& s = g_slots[dev][i];
    if (s.busy) continue;
    if (!s.dev) {
      if (cudaMalloc(&s.dev, kReduceWorkspaceBytes + 256) != cudaSuccess) {
        s.dev = nullptr;
        return nullptr;
      }
      if (cudaHostAlloc(&s.host, 16, cudaHostAllocDefault) != cudaSuccess) {   // leave no half-made slot behind
        cudaFree(s.dev);
        s.dev = s.host = nullptr;
        return nullptr;
      }
    }
    s.busy = true;
    return &s;
  }
  return nullptr;
}
static void release_slot(ScalarSlot* s) {
  std::lock_guard<std::mutex> lock(g_slot_mutex);
  s->busy = false;
}

template <typename T, typename R>
T run_20(int n, const T* x, cudaStream_t st) {
  // Julia's reduction of an empty array is an error upstream; the identity is returned here
  T r = (T)0;
  if (n <= 0) return r;
  ScalarSlot* slot = acquire_slot();
  if (!slot) return (T)NAN;
  T* result = reinterpret_cast<T*>(reinterpret_cast<char*>(slot->dev) + kReduceWorkspaceBytes);
  run_all<T, R>(n, x, result, slot->dev, st);
  cudaMemcpyAsync(slot->host, result, sizeof(T), cudaMemcpyDeviceToHost, st);
  cudaStreamSynchronize(st);
  r = *reinterpret_cast<T*>(slot->host);
  release_slot(slot);
  return r;
}

}  // namespace kn

using namespace kn;

KN_EXPORT size_t knet_reduce_workspace_bytes(void) { return kReduceWorkspaceBytes; }

#define KN_DEF_REDUCE_DEV(f, S, T)                                                              \
  KN_EXPORT int knet_reduce_##S(int op, int64_t n, const T* x, T* result, void* ws,             \
                                size_t ws_bytes, cudaStream_t s) {                              \
    if (!result || (n > 0 && !x)) return KN_EINVAL;                                             \
    if (!ws || ws_bytes < kReduceWorkspaceBytes) return KN_EWORKSPACE;                          \
    if ((uintptr_t)ws & 255) return KN_EALIGN;                                                  \
    return run_all_op<T>(op, n, x, result, ws, s);                                              \
  }
KNET_BOTH_TYPES(KN_DEF_REDUCE_DEV, reduce)

#define KN_DEF_RED(f, S, T)                                                                     \
  KN_EXPORT T f##_##S##_20_stream(int n, const T* x, cudaStream_t s) {                          \
    return run_20<T, R_##f<T>>(n, x, s);                                                        \
  }                                                                                             \
  KN_EXPORT T f##_##S##_20(int n, const T* x) { return f##_##S##_20_stream(n, x, cudaStreamPerThread); } \
  KN_EXPORT void f##_##S##_21_stream(int nx, const T* x, int sy, int ny, T* y, cudaStream_t s) { \
    run_21<T, R_##f<T>>(nx, x, sy, ny, y, s);                                                   \
  }                                                                                             \
  KN_EXPORT void f##_##S##_21(int nx, const T* x, int sy, int ny, T* y) {                       \
    f##_##S##_21_stream(nx, x, sy, ny, y, cudaStreamPerThread);                                 \
  }                                                                                             \
  KN_EXPORT void f##_##S##_22_stream(int nx, int xd1, const T* x, int s1, int s2, int ny, T* y, \
                                     cudaStream_t s) {                                          \
    run_22<T, R_##f<T>>(nx, xd1, x, s1, s2, ny, y, s);                                          \
  }                                                                                             \
  KN_EXPORT void f##_##S##_22(int nx, int xd1, const T* x, int s1, int s2, int ny, T* y) {      \
    f##_##S##_22_stream(nx, xd1, x, s1, s2, ny, y, cudaStreamPerThread);                        \
  }
#define KN_X(f) KNET_BOTH_TYPES(KN_DEF_RED, f)
KNET_REDUCTION_OPS(KN_X)
#undef KN_X

// ---- whole-array reduction for callers that must not allocate -------------------------------------
// Some hosts of this library cannot give it device memory at call time and cannot let it ask
// the driver for any: a language runtime whose own pool already owns the whole GPU, a loop
// that has promised not to allocate after start-up, a caller that has no buffer of its own to
// lend as workspace.  For them the per-block partial results live in the array below, which
// is part of the library image: every GPU that loads the library sets aside these 4 KiB
// until the process exits.  All calls on a device share it, so two calls whose kernels
// overlap on the GPU (different streams) would overwrite each other's partials: keep such
// calls on one stream or order them with events.  Nothing in the array has to start at
// zero; every launch writes each partial before it reads it, so stale contents are harmless.
constexpr int kNoAllocPartials = kAllMaxBlocks;   // 1024 partial results of 4 bytes
static __device__ __align__(256) float g_noalloc_partials[kNoAllocPartials];

// The name above is only a handle on the host side; kernels need the device address, which
// the runtime reports per device.  It is looked up once per device, with that device current.
static float* g_noalloc_ptr[64] = {nullptr};
static std::mutex g_noalloc_mutex;

static int noalloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return KN_ESIZE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return KN_OK;
}

KN_EXPORT int knet_reduce_noalloc_32(int op, int64_t n, const float* x, float* result, cudaStream_t s) {
  if (!result || (n > 0 && !x) || n < 0) return KN_EINVAL;
  if (n > KNET_REDUCE_NOALLOC_MAX_N) return KN_ESIZE;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != KN_OK) return rc;
  return run_all_op<float>(op, n, x, result, scratch, s);
}
