// Pieces shared by the tcgen05 kernels: tensor-map encoding on the host, work-item order.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "sm100_sched.cuh"

namespace vafa {

// Encode a tiled, 128-byte-swizzled tensor map over a row-major [rows, heads, dim] tensor of
// 16-bit elements (heads = 1, dim = row width for a plain matrix).  Box = 64 columns x box_heads heads x
// box_rows rows, so one copy fills one [(box_rows * box_heads) x 128 B] swizzled sub-tile (row-major
// over (row, head)).
int encode_tmap_rows(CUtensorMap* m, const void* base, int dtype, long long rows, int heads, int dim, int box_rows,
                     int box_heads = 1);

// Tensor map over the fold array [rows, heads, 32] of 16-bit elements (see sm100_varlen_bwd128.cu):
// box = 16 elements x 1 head x 128 rows with the 32-byte swizzle, so one copy fills one K = 16 operand
// tile of 128 rows x 32 B.
int encode_tmap_fold(CUtensorMap* m, const void* base, int dtype, long long rows, int heads);

// Dynamic work distribution inside a persistent CTA.  The TMA-producer thread draws the next item
// index from a global counter and publishes it through a small shared-memory ring; the other roles
// (MMA issuer, element-wise warps) read the same sequence.  Items are handed out in list order, so
// the CTAs that run at the same time work on neighbouring items (same segment and head: shared
// K/V blocks in L2) and a CTA that finishes early simply takes the next one.
constexpr int kWqSlots = 4;
struct WorkQueue {
  uint64_t full[kWqSlots], empty[kWqSlots];
  int idx[kWqSlots];
};

// consumers = number of arrivals per slot: one per consuming warp (or single consuming thread)
__device__ __forceinline__ void wq_init(WorkQueue& q, int consumers) {
  for (int i = 0; i < kWqSlots; ++i) {
    ptx::mbar_init(ptx::smem_u32(&q.full[i]), 1);
    ptx::mbar_init(ptx::smem_u32(&q.empty[i]), consumers);
  }
}

// Producer (one thread): returns the n-th item index of this CTA, or -1 when the list is exhausted
// (published to the consumers as well) or a wait was abandoned.
__device__ __forceinline__ int wq_produce(WorkQueue& q, uint32_t n, int* counter, int total, volatile int* abort_flag) {
  const int slot = n % kWqSlots;
  if (!ptx::mbar_wait(ptx::smem_u32(&q.empty[slot]), ((n / kWqSlots) & 1) ^ 1, abort_flag)) return -1;
  int idx = atomicAdd(counter, 1);
  if (idx >= total) idx = -1;
  q.idx[slot] = idx;
  ptx::mbar_arrive(ptx::smem_u32(&q.full[slot]));
  return idx;
}

// Consumer, whole warp: every lane gets the index, lane 0 releases the slot.
__device__ __forceinline__ int wq_consume_warp(WorkQueue& q, uint32_t n, volatile int* abort_flag) {
  const int slot = n % kWqSlots;
  if (!ptx::mbar_wait(ptx::smem_u32(&q.full[slot]), (n / kWqSlots) & 1, abort_flag)) return -1;
  const int idx = q.idx[slot];
  __syncwarp();
  if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(ptx::smem_u32(&q.empty[slot]));
  return idx;
}

// Consumer, single thread of a warp.
__device__ __forceinline__ int wq_consume_thread(WorkQueue& q, uint32_t n, volatile int* abort_flag) {
  const int slot = n % kWqSlots;
  if (!ptx::mbar_wait(ptx::smem_u32(&q.full[slot]), (n / kWqSlots) & 1, abort_flag)) return -1;
  const int idx = q.idx[slot];
  ptx::mbar_arrive(ptx::smem_u32(&q.empty[slot]));
  return idx;
}

}  // namespace vafa
