// Self-check of the bounded device-side wait the tensor-core kernels are built on (tc::mbar_wait_limited): one
// thread waits on an mbarrier that nothing ever arrives on, with a short time limit.  The wait gives up, records
// where in the status words, and the kernel returns normally -- the path a stalled pipeline takes, exercised without
// stalling anything.  The dispatch layer exposes it as MCA_FN_WAIT_PROBE so that the chain status words ->
// ERROR_ATTN_KERNEL_TIMEOUT -> message -> reset can be tested end to end.
#include "common.cuh"
#include "kernels.h"

#include "tc_common.cuh"

namespace {

__global__ void wait_probe_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = tc::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    tc::mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // phase 0 never completes: nobody arrives.  Stage 99 marks the probe in the status words.
    tc::mbar_wait_limited(bar, 0, status, 99, 0, limit_ns);
  }
}

}  // namespace

int mca_wait_probe(int* status, int limit_us, void* stream) {
  if (!status) return ERROR_PARAM_NULL;
  if (limit_us <= 0 || limit_us > 100000) return ERROR_PARAM_OUT_OF_RANGE;   // at most 0.1 s
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_us * 1000ull);
  return mca_launch_status();
}
