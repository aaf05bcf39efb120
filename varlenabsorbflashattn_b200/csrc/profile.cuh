// Optional per-kernel timing with CUDA events, and launch counters.
// Off by default; when on, every kernel launch is bracketed by two events on its stream.
#pragma once
#include <cuda_runtime.h>

namespace vafa {

enum KernelId {
  kKSched = 0,
  kKFwd,
  kKCombine,
  kKBwdPre,
  kKBwdDq,
  kKBwdDkv,
  kKSimtFwd,
  kKSimtDelta,
  kKSimtDq,
  kKSimtDkv,
  kKSimtGemm,
  kKCast,
  kKAbsorbFwd,
  kKAbsorbBwd,
  kKAbsorbGemm,
  kKAbsorbBwdDx,
  kKAbsorbGemmTn,
  kKBwdFused,
  kKBwdDqFin,
  kKCount
};

struct LaunchScope {
  LaunchScope(int id, cudaStream_t s);
  ~LaunchScope();
  int id_;
  cudaStream_t s_;
  cudaEvent_t stop_;
};

}  // namespace vafa
