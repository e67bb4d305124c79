// A one-CTA kernel that waits on an mbarrier nothing ever arrives at, with the same bounded wait the
// TMA-fed kernels use (`mbar_wait` in tma.cuh): it shows that such a wait ends after its limit,
// reports it through the status word and leaves the context usable.  The limit is the caller's,
// a few milliseconds in the test.  Nothing in the engine calls it.
// (The reference has no device-side waits: its kernels are one-shot launches, kernels/cuda/kernels.cu.)
#include <stdio.h>

#include "tma.cuh"

namespace sllm {

__global__ void wait_probe_kernel(int* status, unsigned long long limit_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint64_t t0 = global_ns();
    const bool ok = mbar_wait(&bar, 0, limit_ns);      // phase 0 never completes
    *waited_ns = global_ns() - t0;
    if (!ok) atomicExch(status, 99);
  }
}

}  // namespace sllm

using namespace sllm;

// status: one int of device memory, zero before the launch, 99 after it (the wait ran out);
// waited_ns: one 64-bit word of device memory, the time the wait took.
SLLM_EXPORT int sllm_wait_probe(int* status, unsigned long long limit_ns, unsigned long long* waited_ns, cudaStream_t stream) {
  SLLM_REQUIRE(status != nullptr && waited_ns != nullptr, "wait_probe: status and waited_ns are required");
  SLLM_REQUIRE(limit_ns <= 100000000ull, "wait_probe: the limit is at most 100 ms (%llu ns asked)", limit_ns);
  launch_kernel(wait_probe_kernel, 1, 32, 0, stream, status, limit_ns, waited_ns);
  return launch_status("wait_probe");
}
