// Self-test of the bounded waits: a kernel whose wait can never complete.
//
// One CTA initialises an mbarrier that expects one arrival and nobody arrives.  Every thread waits on it through
// the same mbar_wait the tensor-core kernels use; the wait gives up after the configured limit, records its code,
// and the kernel returns through the same teardown helper.  Nothing faults and the context stays usable: the host
// reads the flag with px_device_error_flags.  A second launch while the flag is still set returns at once
// (cta_skip_after_error), which the out word shows.
#include "px_tcgen05.cuh"

namespace px {

__global__ void selftest_wait_kernel(unsigned int* out) {
  __shared__ uint64_t bar;
  if (cta_skip_after_error()) {
    if (threadIdx.x == 0) out[0] = 2u;   // skipped: an earlier failure is still recorded
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  const bool ok = mbar_wait(&bar, 0, 1u);          // phase 0 never completes
  const bool all_ok = __all_sync(0xffffffffu, ok);
  cta_teardown_sync();
  if (threadIdx.x == 0) out[0] = all_ok ? 0u : 1u;  // 1: the wait gave up and the kernel still got here
}

PX_DEFINE_FAMILY_HOOKS(selftest)

}  // namespace px

extern "C" int32_t px_selftest_wait_timeout(uint32_t* out_word, void* stream) {
  if (!out_word) return PX_ERR_BAD_ARG;
  px::selftest_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(out_word);
  return cudaGetLastError() == cudaSuccess ? PX_OK : PX_ERR_LAUNCH;
}
