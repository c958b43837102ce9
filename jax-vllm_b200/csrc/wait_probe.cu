// A probe of the bounded wait that every TMA and tcgen05 kernel of this engine is built on (mbarrier.cuh): one
// block, one barrier.  With `arrive` = 0 nothing ever arrives on the barrier, so the wait runs into its
// deadline of `cycles` clocks, the kernel records JV_STATUS_WAIT_EXPIRED in the status word exactly as the
// product kernels do, and returns: the context stays usable and the host raises when it reads the word.  With
// `arrive` = 1 another thread arrives and the wait succeeds.  It is used by the tests and by nothing else.
//
//   outcome[0] = 1 the wait succeeded, 2 it ran out;  outcome[1] = clocks spent in the wait (saturated to int).
#include "common.cuh"
#include "mbarrier.cuh"

namespace {

__global__ void wait_probe_kernel(long long cycles, int arrive, int* status, int* outcome) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 1 && arrive) mbar_arrive(&bar);
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0, cycles);
    const long long spent = clock64() - t0;
    if (!ok) atomicOr(status, JV_STATUS_WAIT_EXPIRED);
    outcome[0] = ok ? 1 : 2;
    outcome[1] = spent > 0x7fffffffLL ? 0x7fffffff : (int)spent;
  }
}

}  // namespace

JV_EXPORT int jv_wait_probe(long long cycles, int arrive, int* status, int* outcome, cudaStream_t stream) {
  if (cycles < 1 || cycles > JV_WAIT_CYCLES) return JV_ERR_UNSUPPORTED;    // never longer than the product's own bound
  wait_probe_kernel<<<1, 32, 0, stream>>>(cycles, arrive, status, outcome);
  return jv_check_launch();
}
