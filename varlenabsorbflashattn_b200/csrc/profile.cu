#include "profile.cuh"

#include <atomic>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

namespace vafa {
namespace {

const char* kNames[kKCount] = {
    "sched_kernel", "varlen_fwd_kernel", "varlen_combine_kernel", "bwd_preprocess_kernel", "varlen_bwd_kernel<dQ>",
    "varlen_bwd_kernel<dKV>", "simt_fwd_kernel", "simt_delta_kernel", "simt_dq_kernel", "simt_dkv_kernel",
    "simt_gemm_kernel", "cast_kernel", "varlen_fwd_kernel<absorb>", "varlen_bwd_kernel<absorb dU>", "gemm_nn_k256_kernel", "varlen_bwd_kernel<absorb dX>", "gemm_tn_kernel",
    "varlen_bwd_kernel<fused>", "dq_finalize_kernel"};

std::atomic<long long> g_launches[kKCount];
std::atomic<int> g_enabled{0};
std::mutex g_mu;
std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_events[kKCount];
double g_ms[kKCount];
long long g_timed[kKCount];

}  // namespace

LaunchScope::LaunchScope(int id, cudaStream_t s) : id_(id), s_(s), stop_(nullptr) {
  g_launches[id].fetch_add(1, std::memory_order_relaxed);
  if (g_enabled.load(std::memory_order_relaxed)) {
    cudaEvent_t a = nullptr, b = nullptr;
    if (cudaEventCreate(&a) == cudaSuccess && cudaEventCreate(&b) == cudaSuccess) {
      cudaEventRecord(a, s);
      stop_ = b;
      std::lock_guard<std::mutex> lk(g_mu);
      g_events[id].emplace_back(a, b);
    }
  }
}

LaunchScope::~LaunchScope() {
  if (stop_) cudaEventRecord(stop_, s_);
}

}  // namespace vafa

using namespace vafa;

extern "C" {
#pragma GCC visibility push(default)

int vafa_profile_enable(int on) {
  g_enabled.store(on ? 1 : 0);
  return 0;
}

int vafa_profile_kernel_count(void) { return kKCount; }

const char* vafa_profile_kernel_name(int id) { return (id >= 0 && id < kKCount) ? kNames[id] : ""; }

// Fold finished events into the totals (synchronises on each pending stop event), then report.
int vafa_profile_read(int id, double* total_ms, long long* timed_launches, long long* all_launches) {
  if (id < 0 || id >= kKCount) return VAFA_ERR_INVALID;
  std::lock_guard<std::mutex> lk(g_mu);
  for (auto& ev : g_events[id]) {
    float ms = 0.f;
    if (cudaEventSynchronize(ev.second) == cudaSuccess && cudaEventElapsedTime(&ms, ev.first, ev.second) == cudaSuccess) {
      g_ms[id] += ms;
      g_timed[id] += 1;
    }
    cudaEventDestroy(ev.first);
    cudaEventDestroy(ev.second);
  }
  g_events[id].clear();
  if (total_ms) *total_ms = g_ms[id];
  if (timed_launches) *timed_launches = g_timed[id];
  if (all_launches) *all_launches = g_launches[id].load();
  return 0;
}

int vafa_profile_reset(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (int id = 0; id < kKCount; ++id) {
    for (auto& ev : g_events[id]) {
      cudaEventDestroy(ev.first);
      cudaEventDestroy(ev.second);
    }
    g_events[id].clear();
    g_ms[id] = 0.0;
    g_timed[id] = 0;
    g_launches[id].store(0);
  }
  return 0;
}

#pragma GCC visibility pop
}
