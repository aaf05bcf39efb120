// Self-test of the failure path every tcgen05 kernel shares: a bounded mbarrier wait that runs out,
// the abort flag, the status word.  Nothing here traps or spins without a limit.
#include "sm100_common.cuh"
#include "sm100_kernels.cuh"

namespace vafa {
namespace {

using namespace ptx;

__global__ void __launch_bounds__(32, 1) bounded_wait_selftest_kernel(int32_t* status, int wait_limit) {
  __shared__ alignas(8) uint64_t never;  // initialised for one arrival that does not come
  __shared__ int ctl[2];                 // [0] abort flag, [1] the limit, as in the kernels' shared state
  if (threadIdx.x == 0) {
    ctl[0] = 0;
    ctl[1] = wait_limit;
    mbar_init(smem_u32(&never), 1);
    fence_barrier_init();
  }
  __syncthreads();
  bool completed = true;
  if (threadIdx.x == 0) completed = mbar_wait(smem_u32(&never), 0, ctl);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!completed && ctl[0] != 0) report_error(status, 1, 900, wait_limit);
    else report_error(status, 3, 901, 0);  // the wait came back as complete: the self-test itself is broken
  }
}

}  // namespace

int sm100_selftest_bounded_wait(int32_t* status, cudaStream_t s) {
  bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(status, wait_limit_units());
  VAFA_LAUNCH_CHECK("bounded_wait_selftest_kernel");
  return 0;
}

}  // namespace vafa
