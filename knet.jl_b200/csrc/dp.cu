// Data-parallel collectives behind the knet_dp_* entry points: a thin, bounded-wait layer over
// NCCL for the batch-sharded training step (gradient all-reduce, or reduce-scatter ->
// update of the own shard -> all-gather).
//
// NCCL is not a link-time dependency: it is opened with dlopen the first time a knet_dp_*
// function runs (KNET_SM100_NCCL_LIB, else libnccl.so.2 - which is the copy a host such as
// PyTorch has already loaded, if any).  The communicator is non-blocking: every NCCL call
// that answers "in progress" is followed by a poll of the communicator's state with a host
// deadline, and a deadline that passes aborts the communicator and returns KN_ETIMEOUT, so
// a rank that never joins cannot hang its peers' hosts.  Only host code here: the
// reductions themselves are NCCL's kernels over NVLink / NVSwitch.
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "common.cuh"

#if __has_include(<nccl.h>)
#include <nccl.h>
#define KN_HAVE_NCCL_HEADER 1
#else
#define KN_HAVE_NCCL_HEADER 0
#endif

namespace kn {

enum : int { KN_ENCCL = -5, KN_ETIMEOUT = -6 };

#if KN_HAVE_NCCL_HEADER

struct NcclApi {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRankConfig) CommInitRankConfig = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  decltype(&ncclCommAbort) CommAbort = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclReduceScatter) ReduceScatter = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclBroadcast) Broadcast = nullptr;
  bool ok = false;
};

template <typename F> bool sym(void* h, const char* name, F& out) {
  out = reinterpret_cast<F>(dlsym(h, name));
  return out != nullptr;
}

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[3] = {getenv("KNET_SM100_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (!n || !*n) continue;
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
    void* h = api.handle;
    api.ok = sym(h, "ncclGetUniqueId", api.GetUniqueId) && sym(h, "ncclCommInitRankConfig", api.CommInitRankConfig) &&
             sym(h, "ncclCommGetAsyncError", api.CommGetAsyncError) && sym(h, "ncclCommAbort", api.CommAbort) &&
             sym(h, "ncclCommDestroy", api.CommDestroy) && sym(h, "ncclAllReduce", api.AllReduce) &&
             sym(h, "ncclReduceScatter", api.ReduceScatter) && sym(h, "ncclAllGather", api.AllGather) &&
             sym(h, "ncclBroadcast", api.Broadcast);
  });
  return api;
}

struct DpComm {
  ncclComm_t comm;
  int rank, world, timeout_ms;
  bool dead;
};

inline int nccl_status(ncclResult_t r) { return r == ncclSuccess ? KN_OK : 1000 + (int)r; }

// After a call that may have answered ncclInProgress: poll until the communicator settles.
int settle(DpComm* c, ncclResult_t r) {
  if (r != ncclSuccess && r != ncclInProgress) return nccl_status(r);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(c->timeout_ms);
  ncclResult_t state = r;
  while (true) {
    const ncclResult_t q = nccl().CommGetAsyncError(c->comm, &state);
    if (q != ncclSuccess) return nccl_status(q);
    if (state == ncclSuccess) return KN_OK;
    if (state != ncclInProgress) return nccl_status(state);
    if (std::chrono::steady_clock::now() > deadline) {
      nccl().CommAbort(c->comm);
      c->dead = true;
      return KN_ETIMEOUT;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

template <typename T> constexpr ncclDataType_t nccl_type();
template <> constexpr ncclDataType_t nccl_type<float>() { return ncclFloat32; }
template <> constexpr ncclDataType_t nccl_type<double>() { return ncclFloat64; }

inline DpComm* live(void* comm) {
  DpComm* c = static_cast<DpComm*>(comm);
  return (c && !c->dead && nccl().ok) ? c : nullptr;
}

template <typename T> int dp_allreduce(void* comm, T* buf, int64_t n, cudaStream_t s) {
  DpComm* c = live(comm);
  if (!c || n < 0 || (n > 0 && !buf)) return KN_EINVAL;
  if (n == 0) return KN_OK;
  return settle(c, nccl().AllReduce(buf, buf, (size_t)n, nccl_type<T>(), ncclSum, c->comm, s));
}
template <typename T> int dp_reduce_scatter(void* comm, const T* send, T* recv, int64_t n, cudaStream_t s) {
  DpComm* c = live(comm);
  if (!c || n < 0 || (n > 0 && (!send || !recv))) return KN_EINVAL;
  if (n == 0) return KN_OK;
  return settle(c, nccl().ReduceScatter(send, recv, (size_t)n, nccl_type<T>(), ncclSum, c->comm, s));
}
template <typename T> int dp_allgather(void* comm, const T* send, T* recv, int64_t n, cudaStream_t s) {
  DpComm* c = live(comm);
  if (!c || n < 0 || (n > 0 && (!send || !recv))) return KN_EINVAL;
  if (n == 0) return KN_OK;
  return settle(c, nccl().AllGather(send, recv, (size_t)n, nccl_type<T>(), c->comm, s));
}
template <typename T> int dp_broadcast(void* comm, T* buf, int64_t n, int root, cudaStream_t s) {
  DpComm* c = live(comm);
  if (!c || n < 0 || (n > 0 && !buf) || root < 0 || root >= c->world) return KN_EINVAL;
  if (n == 0) return KN_OK;
  return settle(c, nccl().Broadcast(buf, buf, (size_t)n, nccl_type<T>(), root, c->comm, s));
}

#endif  // KN_HAVE_NCCL_HEADER

}  // namespace kn

using namespace kn;

#if KN_HAVE_NCCL_HEADER

static_assert(sizeof(ncclUniqueId) == KNET_DP_ID_BYTES, "the unique id is 128 bytes in every NCCL 2 release");

KN_EXPORT int knet_dp_unique_id(void* id128) {
  if (!id128) return KN_EINVAL;
  if (!nccl().ok) return KN_ENCCL;
  ncclUniqueId id;
  const ncclResult_t r = nccl().GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_status(r);
  std::memcpy(id128, &id, sizeof(id));
  return KN_OK;
}

KN_EXPORT int knet_dp_init(const void* id128, int rank, int world, int timeout_ms, void** comm) {
  if (!id128 || !comm || world < 1 || rank < 0 || rank >= world || timeout_ms <= 0) return KN_EINVAL;
  if (!nccl().ok) return KN_ENCCL;
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  DpComm* c = new DpComm{nullptr, rank, world, timeout_ms, false};
  const ncclResult_t r = nccl().CommInitRankConfig(&c->comm, world, id, rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) {
    delete c;
    return nccl_status(r);
  }
  const int st = settle(c, r);
  if (st != KN_OK) {
    if (!c->dead && c->comm) nccl().CommAbort(c->comm);
    delete c;
    return st;
  }
  *comm = c;
  return KN_OK;
}

KN_EXPORT int knet_dp_rank(void* comm) { return comm ? static_cast<DpComm*>(comm)->rank : KN_EINVAL; }
KN_EXPORT int knet_dp_world(void* comm) { return comm ? static_cast<DpComm*>(comm)->world : KN_EINVAL; }

KN_EXPORT int knet_dp_destroy(void* comm) {
  DpComm* c = static_cast<DpComm*>(comm);
  if (!c) return KN_EINVAL;
  int st = KN_OK;
  if (!c->dead && nccl().ok) {
    const ncclResult_t r = nccl().CommDestroy(c->comm);
    st = (r == ncclSuccess || r == ncclInProgress) ? KN_OK : nccl_status(r);
  }
  delete c;
  return st;
}

#define KN_DEF_DP(f, S, T)                                                                                 \
  KN_EXPORT int knet_dp_allreduce_sum_##S(void* comm, T* buf, int64_t n, cudaStream_t s) {                 \
    return dp_allreduce<T>(comm, buf, n, s);                                                               \
  }                                                                                                        \
  KN_EXPORT int knet_dp_reduce_scatter_sum_##S(void* comm, const T* send, T* recv, int64_t n,              \
                                               cudaStream_t s) {                                           \
    return dp_reduce_scatter<T>(comm, send, recv, n, s);                                                   \
  }                                                                                                        \
  KN_EXPORT int knet_dp_allgather_##S(void* comm, const T* send, T* recv, int64_t n, cudaStream_t s) {     \
    return dp_allgather<T>(comm, send, recv, n, s);                                                        \
  }                                                                                                        \
  KN_EXPORT int knet_dp_broadcast_##S(void* comm, T* buf, int64_t n, int root, cudaStream_t s) {           \
    return dp_broadcast<T>(comm, buf, n, root, s);                                                         \
  }
KNET_BOTH_TYPES(KN_DEF_DP, dp)

#else  // built without nccl.h: the entry points exist and say so

KN_EXPORT int knet_dp_unique_id(void*) { return KN_ENCCL; }
KN_EXPORT int knet_dp_init(const void*, int, int, int, void**) { return KN_ENCCL; }
KN_EXPORT int knet_dp_rank(void*) { return KN_ENCCL; }
KN_EXPORT int knet_dp_world(void*) { return KN_ENCCL; }
KN_EXPORT int knet_dp_destroy(void*) { return KN_ENCCL; }
#define KN_DEF_DP(f, S, T)                                                                              \
  KN_EXPORT int knet_dp_allreduce_sum_##S(void*, T*, int64_t, cudaStream_t) { return KN_ENCCL; }        \
  KN_EXPORT int knet_dp_reduce_scatter_sum_##S(void*, const T*, T*, int64_t, cudaStream_t) { return KN_ENCCL; } \
  KN_EXPORT int knet_dp_allgather_##S(void*, const T*, T*, int64_t, cudaStream_t) { return KN_ENCCL; }  \
  KN_EXPORT int knet_dp_broadcast_##S(void*, T*, int64_t, int, cudaStream_t) { return KN_ENCCL; }
KNET_BOTH_TYPES(KN_DEF_DP, dp)

#endif
