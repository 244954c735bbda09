// pipeline.cuh -- shared-memory pipeline primitives used by the streaming
// kernels: mbarrier helpers with time-bounded waits and the 1-D bulk async copy
// (global -> shared, completion counted on an mbarrier, no multicast).
//
// A wait that runs out of time raises the CTA-local abort flag and the
// device-wide status word (`status`, from kernel_status_ptr()), and returns false; callers stop consuming and the
// host reports the launch as failed (kernel_take_status).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace smith {

constexpr long long kWaitLimitCycles = 400ll * 1000ll * 1000ll;  // ~0.2 s at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint (nanoseconds): the thread may stay suspended that long, and is
// resumed as soon as the phase completes.  Without the hint a waiting thread comes back after a short
// system-chosen time and polls again, and the polls of a CTA's waiting warps take issue slots (and
// power) from the warps that work: a quarter of all instructions of the list kernel were such polls.
__device__ __forceinline__ bool mbar_try_suspended(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
constexpr uint32_t kSuspendNs = 20000;   // per try; the limit below is checked after each

// Bounded wait.  Returns false if the limit ran out or another thread of the
// CTA gave up.  The limit is counted on the SM's cycle counter, consulted after
// every suspended try.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  // short waits (a stage that is about to land) keep the plain poll and its wake-up latency ...
#pragma unroll 1
  for (int spin = 0; spin < 64; spin++)
    if (mbar_try(bar, parity)) return true;
  // ... long ones (an epilogue warp during the main loop, a producer behind a full ring) go to sleep
  const long long t0 = clock64();
#pragma unroll 1
  for (;;) {
    if (mbar_try_suspended(bar, parity, kSuspendNs)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicExch(status, 1);
      return false;
    }
  }
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                          uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

// Same copy without a cache hint (for data that other CTAs read too and that should stay in L2).
__device__ __forceinline__ void bulk_load_default(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

}  // namespace smith
