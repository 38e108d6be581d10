// Self-test of the bounded device-side wait every kernel of this library is built on: one thread waits on an
// mbarrier that nothing ever completes, gives up after `limit_ns`, raises FMOE_STATUS_WAIT_TIMEOUT and the kernel
// returns normally - the context stays usable, which is the point of bounding the waits.  The limit is clamped to
// 10 ms; nothing here can spin for long.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fmoe {
namespace {

__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns, int32_t* status, int32_t* result) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    const uint32_t b = ptx::smem_u32(&bar);
    ptx::mbar_init(b, 1);
    abort_flag = 0;
    ptx::mbar_fence_init();
    const bool completed = ptx::mbar_wait_bounded(b, 0u, &abort_flag, limit_ns);
    if (!completed && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
    if (result != nullptr) *result = completed ? 1 : 2;  // 2: the wait ran out, as it must
  }
}

}  // namespace
}  // namespace fmoe

extern "C" int fmoe_selftest_wait_timeout(uint64_t limit_ns, int32_t* status, int32_t* result, fmoe_stream_t stream) {
  if (limit_ns == 0 || limit_ns > 10000000ull) limit_ns = 10000000ull;
  fmoe::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status, result);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}
