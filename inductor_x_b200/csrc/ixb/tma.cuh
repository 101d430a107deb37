// mbarrier and bulk-copy (TMA) primitives with bounded waits.  Every spin has an
// iteration limit; a wait that runs out bumps a device-side counter the host can read
// (ixb_pipeline_timeouts) and the caller leaves its loop instead of hanging the SM.
#pragma once
#include "common.cuh"

namespace ixb {

// Number of mbarrier waits that gave up since the library was loaded on this device.
// One copy per translation unit (the library is built without relocatable device code);
// each unit that includes this header exposes its copy through IXB_DEFINE_TIMEOUT_READER.
static __device__ unsigned int g_wait_timeouts = 0;
#define IXB_DEFINE_TIMEOUT_READER(fn_name)                                              \
  cudaError_t fn_name(unsigned int* out) {                                              \
    return cudaMemcpyFromSymbol(out, ixb::g_wait_timeouts, sizeof(unsigned int));       \
  }

constexpr long long kWaitCycles = 2000000000LL;  // about one second of SM clock

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals)
               : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// One attempt: the thread may be suspended by the hardware for up to `suspend_ns`
// nanoseconds waiting for the phase, so a waiting warp does not burn issue slots.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity,
                                              uint32_t suspend_ns = 1000000u) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_ns)
      : "memory");
  return ok != 0;
}
// Non-blocking probe of a phase.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about a second of SM clock (counter bumped), or as soon as
// `abort` (a flag another role of the CTA raises when its own wait gave up) is non-zero.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          const volatile int* abort = nullptr) {
  if (mbar_test_wait(bar, parity)) return true;  // already complete: the common case on a hot path
#pragma unroll 1
  for (int quick = 0; quick < 64; ++quick)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (abort != nullptr && *abort != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      atomicAdd(&g_wait_timeouts, 1u);
      return false;
    }
  }
}
// Bulk asynchronous copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

}  // namespace ixb
