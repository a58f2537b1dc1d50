// Self-test of the error path that every bounded wait of the tensor-core kernels takes.
//
// One CTA initialises an mbarrier that NOTHING will ever arrive on (no copy, no MMA, no other
// thread targets it), waits for it with the kernels' own wait helper and a small limit, and, when
// the limit runs out, records a code in the same status word the real kernels use and returns in
// the ordinary way.  Nothing is in flight when it gives up, so the context stays usable; the host
// must then see the code and raise.
#include "tc_common.cuh"

__global__ void selftest_wait_kernel(int* __restrict__ status, unsigned tries, int code) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait_limited(&bar, 0, tries)) atomicExch(status, code);
  }
}

CO_EXPORT int coheryn_selftest_bounded_wait(int* status, unsigned tries, int code, cudaStream_t stream) {
  if (!status) CO_FAIL("selftest_bounded_wait: no status word");
  if (tries > 100000u) CO_FAIL("selftest_bounded_wait: at most 100000 tries (a self-test, not a delay)");
  selftest_wait_kernel<<<1, 32, 0, stream>>>(status, tries, code);
  CO_CHECK_LAUNCH("selftest_bounded_wait");
  return 0;
}
