// sm_100a asynchronous-copy primitives used by the pipelined kernels: mbarrier
// (init / expect-tx / arrive / bounded parity wait) and the 1-D bulk copy
// global -> shared that completes on an mbarrier (the TMA engine moves the
// bytes; no thread holds them in registers while they are in flight).
//
// Every wait is bounded by wall-clock time (%globaltimer): after kWaitLimitNs it
// gives up, raises a flag that the host can read (dlb_pipeline_timeouts) and
// lets the kernel run to its end with garbage results instead of hanging the
// GPU.  The layer classes read the counter where they synchronise anyway
// (gradient clipping, checkpoint writing) and fail loudly when it is non-zero.
#pragma once

#include "common.cuh"

namespace dlb {

// Device address of the counter of waits that gave up (one per device, owned
// by core.cu); kernels get it as a parameter.  Host side.
unsigned int *wait_timeouts_counter();

constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // one second per wait

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes the initialised barriers visible to the async proxy (the copy engine).
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Waits until the phase with the given parity has completed.  Returns false if
// it gave up; *dead (a shared flag of the CTA) then makes every later wait of
// the CTA return at once, and *timeouts (global) counts the event for the host.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, volatile int *dead,
                                          unsigned int *timeouts) {
  const uint32_t addr = smem_u32(bar);
  unsigned long long start = 0;
  for (unsigned i = 0;; i++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (*dead) return false;
    // The clock is read every 32nd poll only: a poll already suspends the thread for a while.
    if ((i & 31u) == 31u) {
      const unsigned long long now = global_ns();
      if (start == 0) start = now;
      else if (now - start > kWaitLimitNs) break;
    }
  }
  *dead = 1;
  atomicAdd(timeouts, 1u);
  return false;
}

// 1-D bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned)
// from global to this CTA's shared memory; completion is signalled on `bar` as
// `bytes` transaction bytes.  No multicast.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void *smem) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(smem_u32(smem)));
  return v;
}

}  // namespace dlb
