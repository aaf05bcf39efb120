// Device-side tile scheduler: turns cu_seqlens into a cost-sorted list of work items.
//
// A work item is one 128-row "outer" tile of one segment (query rows for the forward and dQ
// kernels, key rows for the dK/dV kernel) together with the range of "inner" rows it has to
// walk (keys, or query rows), already trimmed by the causal mask.  The forward pass may cut the
// inner range of a tile into several items (split-K); each such item writes a partial result
// that the combine kernel merges.  Items are bucket-sorted by cost, largest first, and
// persistent CTAs take them in that order, so the ragged tail is filled with small items.
//
// It replaces the reference's host-side index builders
// (triton_fa_varlen_v2/triton_fa_varlen_v2/chunk_indices.py:25-75 and :144-287), which copy
// cu_seqlens to the CPU and loop in Python on every call.
#pragma once
#include "common.cuh"

namespace vafa {

constexpr int kTile = 128;

struct alignas(16) WorkItem {
  int32_t o_start;  // global row of the tile's first outer row
  int32_t o_rows;   // valid outer rows (1..128)
  int32_t i_start;  // global row of the first inner row
  int32_t i_len;    // inner rows to walk; 0: the tile sees nothing and its outputs are zero-filled
  int32_t diag;     // causal mask offset (meaning depends on the kernel, see there)
  int32_t masked;   // 1: causal mask applies inside this item
  int32_t partial;  // forward split-K: first row of this item's partial block, else -1
  int32_t head;     // head index of this item
};

struct alignas(16) CombineUnit {
  int32_t q_start;  // global row
  int32_t q_rows;
  int32_t base;     // partial row of split 0; split s starts at base + s * q_rows
  int32_t n_splits;
};

struct alignas(256) SchedHeader {
  int32_t n_items;
  int32_t n_combine;
  int32_t n_partial_rows;
  int32_t block_len;   // inner blocks per split that was finally used (0 = no split)
  int32_t reserved0;
  int32_t next_item;   // dynamic scheduling counter
  int32_t pad[2];
};

enum SchedMode { kSchedFwd = 0, kSchedDq = 1, kSchedDkv = 2 };

struct SchedParams {
  const int32_t* cu_q;
  const int32_t* cu_k;
  int32_t n_seg;
  int32_t mode;
  int32_t causal;
  int32_t H;
  int32_t sm_count;
  int32_t split_len;    // forced inner slice length (multiple of 128), 0 = automatic
  int32_t tile_rows = kTile;  // outer rows per tile in the forward / dQ modes (absorb: 128 / H)
  int32_t cap_items;
  int32_t cap_combine;
  int32_t cap_rows;
  SchedHeader* header;
  WorkItem* items;
  CombineUnit* combine;
};

struct SchedCaps {
  int32_t cap_items, cap_combine, cap_rows;
};

// Host-side capacity bounds (no knowledge of the lengths needed).
static inline SchedCaps sched_caps(int mode, int total_outer, int total_inner, int n_seg, int H, int sm_count, int split_len) {
  SchedCaps c;
  const long long units = (long long)total_outer / kTile + n_seg + 1;
  long long extra = 0;
  if (mode == kSchedFwd) {
    extra = 2LL * sm_count + 64;
    if (split_len > 0) extra += (long long)total_inner / split_len;
  }
  long long items = (units + extra) * (H > 0 ? H : 1);
  if (items > (1LL << 26)) items = 1LL << 26;
  c.cap_items = (int32_t)items;
  c.cap_combine = (int32_t)units;
  long long rows = 0;
  if (mode == kSchedFwd) {
    rows = 512LL * sm_count / (H > 0 ? H : 1) + 256;
    if (split_len > 0) rows += 4LL * total_outer;
    if (rows > (1LL << 22)) rows = 1LL << 22;
  }
  c.cap_rows = (int32_t)rows;
  return c;
}

int launch_scheduler(const SchedParams& p, cudaStream_t s);
// two independent tile lists in one launch (one CTA each)
int launch_scheduler_pair(const SchedParams& a, const SchedParams& b, cudaStream_t s);

}  // namespace vafa
