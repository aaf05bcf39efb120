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

// Persistent CTAs walk the cost-sorted item list in "snake" order: pass n covers items
// [n*G, (n+1)*G), forwards on even passes and backwards on odd ones, so that the CTA that drew
// the largest item of one pass draws the smallest of the next.
__device__ __forceinline__ long long snake_index(int pass, int cta, int n_ctas) {
  return (long long)pass * n_ctas + ((pass & 1) ? (n_ctas - 1 - cta) : cta);
}

}  // namespace vafa
