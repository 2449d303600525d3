/*
 * Thin wrappers over the Blackwell/Hopper bulk asynchronous copy (the linear form of the
 * Tensor Memory Accelerator) and the shared-memory transaction barrier that tracks it.
 * Used to stage whole image planes into shared memory with one instruction issued by one
 * thread, leaving the other threads' registers and issue slots free.
 *
 * Rules the callers must keep (the hardware faults otherwise): source and destination
 * addresses 16-byte aligned, byte count a multiple of 16.  Copies never leave the issuing
 * CTA's own shared memory and always read this GPU's own global memory.
 *
 * Every wait is bounded: after one second (or kWaitSpins unsuccessful polls, whichever comes
 * first) WaitBounded() gives up and reports false, and the caller records
 * kStatusBulkCopyTimeout in the device status word instead of computing on missing data.
 */
#ifndef MSHADOW_GPU_TMA_CUH_
#define MSHADOW_GPU_TMA_CUH_

#include <cstdint>

namespace mshadow {
namespace cuda {
namespace tma {

const int kStatusBulkCopyTimeout = 1;
const uint32_t kWaitSpins = 1u << 20;
const uint64_t kWaitNanos = 1000000000ull;  // one second: a staged copy completes in microseconds

__device__ __forceinline__ uint32_t SharedAddr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void BarrierInit(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SharedAddr(bar)), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

/*! \brief one arrival that also announces `bytes` of asynchronous data to come */
__device__ __forceinline__ void BarrierExpect(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SharedAddr(bar)), "r"(bytes)
               : "memory");
}

/*! \brief one plain arrival (no data announced) */
__device__ __forceinline__ void BarrierArrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SharedAddr(bar)) : "memory");
}

/*! \brief start copying `bytes` from global to this CTA's shared memory; completion lands on `bar` */
__device__ __forceinline__ void BulkLoad(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   SharedAddr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(SharedAddr(bar))
               : "memory");
}

/*! \brief order earlier generic-proxy accesses to shared memory before later asynchronous ones */
__device__ __forceinline__ void FenceAsyncShared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

/*!
 * \brief one potentially blocking test of the phase.  (With an explicit suspend-time hint of 20 us
 *  the ring kernels were no faster -- LRN forward 0.349 -> 0.359 ms, softmax 1.305 -> 1.317 ms --
 *  so the instruction's own time limit stays.)
 */
__device__ __forceinline__ bool BarrierTest(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(SharedAddr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

/*! \brief nanoseconds of the device-wide timer */
__device__ __forceinline__ uint64_t GlobalNanos() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

/*!
 * \brief wait for the phase with the given parity; false if it did not complete within
 *  `limit_ns` (looked at every 64 polls, a poll may itself block for a while) or kWaitSpins polls
 */
__device__ __forceinline__ bool WaitBounded(uint64_t *bar, uint32_t parity, uint64_t limit_ns = kWaitNanos) {
  uint64_t start = 0;  // the clock is first read after 64 polls: a wait that succeeds quickly never reads it
  for (uint32_t spin = 1; spin <= kWaitSpins; ++spin) {
    if (BarrierTest(bar, parity)) return true;
    if ((spin & 63u) == 0) {
      const uint64_t now = GlobalNanos();
      if (start == 0) start = now;
      else if (now - start > limit_ns) return false;
    }
  }
  return false;
}

}  // namespace tma
}  // namespace cuda
}  // namespace mshadow
#endif  // MSHADOW_GPU_TMA_CUH_
