// Single-CTA scheduler kernel: see sm100_sched.cuh and sm100_sched_body.cuh.
#include "sm100_sched_body.cuh"
#include "profile.cuh"

namespace vafa {
namespace {

// One CTA per tile list: blockIdx.x picks the parameter set.
__global__ void __launch_bounds__(sched_impl::kSchedThreads) sched_kernel(const SchedParams p0, const SchedParams p1) {
  sched_impl::sched_build(blockIdx.x == 0 ? p0 : p1);
}

}  // namespace

int launch_scheduler(const SchedParams& p, cudaStream_t s) {
  LaunchScope scope(kKSched, s);
  sched_kernel<<<1, sched_impl::kSchedThreads, 0, s>>>(p, p);
  VAFA_LAUNCH_CHECK("sched_kernel");
  return 0;
}

int launch_scheduler_pair(const SchedParams& a, const SchedParams& b, cudaStream_t s) {
  LaunchScope scope(kKSched, s);
  sched_kernel<<<2, sched_impl::kSchedThreads, 0, s>>>(a, b);
  VAFA_LAUNCH_CHECK("sched_kernel");
  return 0;
}

}  // namespace vafa
