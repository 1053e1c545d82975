// Test-only kernel: one thread waits, with the engine's own bounded wait (mbar_wait of
// csrc/tc_common.cuh), on an mbarrier at which nothing ever arrives.  No copy is in flight and no
// tensor memory is held, so when the limit passes (this file is built with a limit of a few
// milliseconds) the wait returns false, the kernel leaves its code in the status word, as the
// engine's kernels do, and ends normally: the context stays usable.
#include "tc_common.cuh"

TLLM_DEFINE_LAST_ERROR

namespace tllm {
__global__ void wait_probe_kernel(int* status, int code, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait(&bar, 0, &abort_flag);
    *waited_ns = global_timer_ns() - t0;
    if (!ok) atomicCAS(status, 0, code);
  }
}
}  // namespace tllm

extern "C" int tllm_wait_probe(int* status, int code, unsigned long long* waited_ns, void* stream) {
  tllm::wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, code, waited_ns);
  TLLM_CHECK_LAUNCH("wait_probe");
  return TLLM_OK;
}
