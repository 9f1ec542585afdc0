// Bulk asynchronous copies (the 1-D form of the Tensor Memory Accelerator) and the mbarrier
// objects that signal their completion, as inline PTX for sm_100a.
//
// Rules these helpers rely on: source, destination and size of a bulk copy are multiples of
// 16 bytes; a thread arms the barrier with the byte count before issuing the copy; every
// wait is bounded, so a copy that never lands turns into an error flag, not a hang.
// No multicast form is used anywhere: every copy reads this GPU's own memory into the
// issuing CTA's own shared memory.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace kn {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}

// makes the initialised barrier visible to the asynchronous proxy that completes the copy
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// one arrival that also announces `bytes` of copy traffic for the current phase
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// global -> this CTA's shared memory; completion is counted in bytes on `bar`
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Set when a bounded wait gives up.  The library is built without relocatable device code, so
// every translation unit that includes this header has its own copy of the flag;
// knet_device_status() reads and clears all of them through wait_flag_read_clear().
static __device__ int g_wait_timeout_flag = 0;
__device__ __forceinline__ void note_wait_timeout() { atomicExch(&g_wait_timeout_flag, 1); }
// host side: this unit's flag (1 = some wait gave up since the last call), cleared; -1 on a CUDA error
static inline int wait_flag_read_clear() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_wait_timeout_flag, sizeof(int)) != cudaSuccess) return -1;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_wait_timeout_flag, &zero, sizeof(int));
  }
  return v ? 1 : 0;
}

constexpr uint32_t kWaitSpins = 1u << 20;

// mbarrier.complete_tx: counts `bytes` as delivered without a copy (used to balance a barrier
// whose announced byte count will not arrive)
__device__ __forceinline__ void mbar_complete_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// Wait for the phase with the given parity, at most `spins` polls (the default is about a
// second); false = gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t spins = kWaitSpins) {
  for (uint32_t i = 0; i < spins; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 32) __nanosleep(256);
  }
  return false;
}

}  // namespace kn

// ---- remote stores that signal an mbarrier of the receiving CTA (st.async) ------------------------
// A CTA of a cluster writes 8 or 16 bytes into a peer's shared memory and the peer's mbarrier
// counts the bytes, so the peer needs no cluster-wide barrier to know that the data is there.
namespace kn {

// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA `rank`
__device__ __forceinline__ uint32_t mapa_u32(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_async_b64(uint32_t remote_addr, uint64_t v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b64 [%0], %1, [%2];" ::"r"(remote_addr),
               "l"(v), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_v2b64(uint32_t remote_addr, uint64_t v0, uint64_t v1, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b64 [%0], {%1, %2}, [%3];" ::"r"(
                   remote_addr),
               "l"(v0), "l"(v1), "r"(remote_bar)
               : "memory");
}
// the wait of a barrier completed by other CTAs of the cluster: acquire at cluster scope
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Latency matters here (a few hundred cycles are expected): poll back to back for a while before
// backing off; bounded like every wait of this library.  false = gave up.
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 20); i++) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (i > 4096) __nanosleep(256);
  }
  return false;
}

}  // namespace kn

namespace kn {
__device__ __forceinline__ void st_async_b32(uint32_t remote_addr, uint32_t v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(remote_addr),
               "r"(v), "r"(remote_bar)
               : "memory");
}
}  // namespace kn
