// Diagnostics that exercise the library's own safety nets without faulting or hanging anything.
#include "saf_internal.h"
#include "sm100_prims.cuh"

namespace saf {
namespace {

// One CTA waits on an mbarrier that nobody will ever arrive on.  The bounded wait runs out after `limit_ns`,
// the CTA records (SAF_DEV_TIMEOUT_SELFTEST | 99 << 8) in *status exactly as the production kernels record
// their own give-ups, and returns normally: the context stays usable.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_limit(&bar, 0, limit_ns);
  // group-uniform decision, the way the kernels take it before a named barrier
  const bool gave_up = named_bar_or(1, blockDim.x, !ok);
  if (gave_up && threadIdx.x == 0) dev_set_error(status, SAF_DEV_TIMEOUT_SELFTEST, 99);
}

}  // namespace
}  // namespace saf

using namespace saf;

extern "C" int saf_selftest_wait_timeout(int* status, int64_t limit_ns, void* stream) {
  if (!status) return fail(SAF_ERR_INVALID, "status must be a device pointer to an int32 word");
  if (limit_ns <= 0 || limit_ns > 100000000) return fail(SAF_ERR_INVALID, "limit_ns must lie in (0, 1e8]");
  wait_timeout_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ns);
  count_launch();
  return check_launch("wait_timeout_selftest_kernel");
}
