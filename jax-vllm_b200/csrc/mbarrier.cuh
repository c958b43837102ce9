// Shared-memory barriers (mbarrier) as the TMA and tcgen05 kernels of this engine use them, with the one rule
// that all of them keep: no wait spins forever.
//
// `mbar_wait` tries once, which is the usual case and reads no clock, and then polls until a clock deadline
// (about a second by default).  A wait that runs out returns false; the role that called it records
// JV_STATUS_WAIT_EXPIRED in the status word, stops taking work and goes to the block's tear-down, where
// `drain_after_failure` lets what is still in flight (tensor-core products, bulk copies) finish, again with a
// deadline, before tensor memory is freed and the block leaves.  The host sees the bit after the step and raises.
#pragma once

#include "common.cuh"

constexpr long long JV_WAIT_CYCLES = 2000000000LL;   // about a second at the clocks of a B200

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
// Makes freshly initialised barriers visible to the asynchronous units (TMA, tensor cores).
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival that also announces `bytes` of bulk copies which will complete on the barrier.
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, int parity) {
  uint32_t done;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
// Waits until the phase of parity `parity` has completed, at most `cycles` clocks; false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, int parity, long long cycles = JV_WAIT_CYCLES) {
  if (mbar_try(bar, parity)) return true;          // the usual case costs no reading of the clock
  const long long deadline = clock64() + cycles;
  while (!mbar_try(bar, parity))
    if (clock64() > deadline) return false;
  return true;
}

// Arrives on `bar` once every tcgen05.mma that this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// After a wait ran out somewhere in the block: called by the thread that issues the block's tcgen05.mma, with a
// barrier of count 1 that nothing else uses (phase 0 not yet completed).  Products issued before the failure may
// still be running and may still write tensor memory; the commit arrives when they are done, and the wait for it is
// bounded like every other.  Only then may tensor memory be freed.
__device__ __forceinline__ void drain_products_after_failure(uint64_t* drain_bar) {
  umma_commit(drain_bar);
  mbar_wait(drain_bar, 0);
}

// After a wait ran out: called by the thread that issued bulk copies onto `bar` whose last armed phase has parity
// `parity`; the copies land whether or not anybody still wants them, and the block must not leave (its shared
// memory would be given to another block) before they have.  Bounded.
__device__ __forceinline__ void drain_copies_after_failure(uint64_t* bar, int parity) { mbar_wait(bar, parity); }
