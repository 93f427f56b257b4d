// mbarrier / bulk-copy (TMA) primitives as inline PTX, with bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the warp is descheduled until the phase completes or the
// hint (nanoseconds) runs out, instead of burning issue slots that the working warps need.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity, but never forever: the first probe costs one
// instruction; after that the clock is read between probes (each probe suspends the warp for up
// to 20 us) and the wait gives up after 2^31 cycles, about one second.  The caller records the
// failure in the status word and leaves.
constexpr long long kWaitCycleLimit = 1ll << 31;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    if (clock64() - t0 > kWaitCycleLimit) return false;
  }
}
// A short, bounded wait (about 1 ms) used on an abort path to let copies that are already in
// flight land before the warp gives its shared memory up.
__device__ __forceinline__ bool mbar_wait_brief(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    if (clock64() - t0 > (1ll << 21)) return false;
  }
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}

}  // namespace b200moe
