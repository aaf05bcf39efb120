// Shared helpers for libvafa_b200: dtype conversion, status word, error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/vafa.h"

namespace vafa {

// ---- host-side error text (thread local) --------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

// Bound of every device-side wait (mbarrier spins), in units of 65536 clock cycles, as the kernels take
// it in their launch parameters.  Set through vafa_set_wait_limit_cycles(); default about two seconds.
int wait_limit_units();

// Which backward packed_varlen_attn runs on the tcgen05 path: 0 = the dQ + dK/dV kernel pair (bit-reproducible
// gradients, the default), 1 = the one-pass kernel where it applies (head dim 128).  vafa_set_varlen_bwd_mode().
int varlen_bwd_mode();

#define VAFA_CUDA_CHECK(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return ::vafa::fail(VAFA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                          __FILE__, __LINE__);                                             \
  } while (0)

#define VAFA_LAUNCH_CHECK(name)                                                            \
  do {                                                                                     \
    cudaError_t _e = cudaGetLastError();                                                   \
    if (_e != cudaSuccess)                                                                 \
      return ::vafa::fail(VAFA_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
  } while (0)

// ---- device-side status word ----------------------------------------------------------
// Kernels report failures (a wait that ran out, a bad work item) by writing a non-zero code
// once; they never trap.  Codes: 1 = mbarrier wait ran out, 2 = bad work item, 3 = TMEM.
__device__ __forceinline__ void report_error(int32_t* status, int code, int site, int detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0, code) == 0) {
      status[1] = site;
      status[2] = detail;
    }
  }
}

// ---- dtype helpers -------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

// Pack two floats into one 32-bit word of 16-bit values (low half = first argument).
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
// bf16 is the upper half of the fp32 pattern, so rounding is an integer add and the packing one
// byte permute.  This keeps the conversion off the XU pipe (16 lanes/clk/SM), which the kernels
// need for exp2; cvt.rn.bf16x2 shares that pipe and, where every exponential runs there (the backward
// kernels), costs as much as it saves.
// Ties round away from zero instead of to even: they differ on exact ties only (1 in 2^16 values).
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const uint32_t a = __float_as_uint(lo) + 0x8000u;
  const uint32_t b = __float_as_uint(hi) + 0x8000u;
  return __byte_perm(a, b, 0x7632);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// The same packing for values that leave the kernel (O, dQ, dK, dV, the combine's result): IEEE
// round-to-nearest-even and NaN stays NaN.  pack2 above is for the P / dS operands inside the block
// loops only: its integer rounding turns a NaN whose mantissa is all ones (what the arithmetic units
// produce) into -0, which is harmless in an operand whose row is marked NaN through its row sum, but would
// hide a diverged run in an output.  Epilogues run once per tile, so the XU-pipe conversion costs nothing.
// (The forward kernels also use it for P, see pack_p there.)
template <typename T> __device__ __forceinline__ uint32_t pack2_out(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_out<__nv_bfloat16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack2_out<__half>(float lo, float hi) { return pack2<__half>(lo, hi); }

// Coalesced store of a 32-column, 16-bit chunk (64 bytes) of each lane's row.
// In the epilogues a thread owns one row of the tile (TMEM lane = row), so a plain store of its chunk
// sends 32 lanes to 32 different rows: 32 memory requests of 16 bytes per instruction, which made the
// store pipe, not the tensor pipe, the limit of short items.  Here the four lanes of a group first
// transpose their 4 x 4 block of 16-byte pieces by shuffle, so that each store instruction writes 64
// contiguous bytes of one row per group: 8 requests of 64 bytes.
//   w          the lane's chunk as 16 packed words (16-byte pieces w[0..3], w[4..7], ...)
//   my_chunk   address of the chunk in the lane's own row (the rows of a warp are `row_stride`
//              elements apart, in lane order), 16-byte aligned
//   my_row     index of the lane's row in the tile; rows >= n_rows are not written
//   n_pieces   leading 16-byte pieces of the chunk that exist in the output (0..4)
template <typename T>
__device__ __forceinline__ void store_chunk_coalesced(uint32_t (&w)[16], T* my_chunk, long long row_stride, int my_row,
                                                      int n_rows, int n_pieces) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 1; m <= 2; m <<= 1) {
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j & m) continue;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // low lane gives its piece j|m and takes the high lane's piece j
        const uint32_t send = hi ? w[4 * j + e] : w[4 * (j | m) + e];
        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, m);
        if (hi) w[4 * j + e] = recv; else w[4 * (j | m) + e] = recv;
      }
    }
  }
  // piece k now holds piece (lane & 3) of the row of lane (lane & ~3) + k
  const int i = lane & 3;
  if (i < n_pieces) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int row = my_row - i + k;
      if (row < n_rows) {
        uint4* dst = reinterpret_cast<uint4*>(my_chunk + (long long)(k - i) * row_stride) + i;
        *dst = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
      }
    }
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

constexpr float kLog2e = 1.4426950408889634f;

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static inline int elem_size(int dtype) { return dtype == VAFA_F32 ? 4 : 2; }

// Index of the segment that holds `row`: largest s with cu[s] <= row (cu non-decreasing, so
// empty segments are skipped).
__device__ __forceinline__ int find_segment(const int32_t* __restrict__ cu, int n_seg, int row) {
  int lo = 0, hi = n_seg;  // invariant: cu[lo] <= row < cu[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (cu[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

}  // namespace vafa
