// Packed variable-length attention backward in one pass over the score tiles (head dim 128):
// five matrix products per 128 x 128 tile instead of the seven of the dQ + dK/dV kernel pair, and one
// exponential per score instead of two.  Opt-in (vafa_set_varlen_bwd_mode(1)); the kernel pair of
// sm100_varlen_bwd128.cu stays the default, for two reasons given at the end of this comment.
//
// One item = one 128-row key tile of one head (outer = K, V); it walks the segment's query rows in
// 128-row blocks (inner = Q, dO).  dK and dV of the tile accumulate in tensor memory as in the dK/dV
// kernel; the tile's contribution to dQ, dS . K (128 query rows x 128), is formed per block and added
// into an fp32 dQ array in global memory (vector reductions at L2), which a small kernel scales and
// rounds afterwards.
//
// Tensor memory (512 columns):  A [0,128)  S^T, then P^T packed to 16 bit in [0,64)
//                               B [128,256) dP^T, then (after dS is formed) the block's dQ contribution
//                               dV [256,384)  dK [384,512)
// dS^T goes to shared memory only ([key][query], 128-byte swizzle): the same bytes are the K-major A
// operand of dK += dS^T Q and the MN-major A operand of dQ_blk = dS K.
//
// Issue order of the MMA thread in steady state (the pipe runs in order):
//     dV += P^T dO(g) ; S^T(g+1)   |   dQ_blk = dS K ; dK += dS^T Q(g)   |   dP^T(g+1) once B is read out
// Element-wise warps per block: P (needs S^T), dS (needs dP^T).  Four more warps drain dQ_blk out of B and
// issue its reductions.  (lse, delta) are folded into the score products as in the dK/dV kernel.
//
// Why it is not the default:
//  * The order in which the key tiles of a sequence add into a query tile is not fixed, so the last bits of
//    dQ change from run to run (dK and dV do not).  The reference's gradients are bit-reproducible.
//  * It is not faster on a B200.  An SM adds 64 KB of fp32 into global memory in 1.3 us at best (measured
//    with red.global.add.v4.f32 in every coalescing pattern and with cp.reduce.async.bulk, on 8 or on 148
//    SMs alike: about 26 B per clock and SM), and every block produces 64 KB.  Tensor memory is full
//    (S^T, dP^T, dV, dK), so the dQ contribution has to reuse B and the next dP^T waits until B has been
//    read out; shared memory is full too (K, V, two Q slots, dO, dS^T), so there is no room to stage the
//    tile for an asynchronous bulk reduction.  Measured on a 62 k-token slice of the 1 M-token batch:
//    6.0-6.9 ms against 5.7-6.0 ms for the kernel pair (3.9-4.1 ms with the reductions switched off); on
//    the full batch 134.7 ms against 122.7 ms.
//
// Reference: the authors' own sketch of a fused backward, never launched there:
// triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:923-1099 (K-block-major, fp32 dQ partials).
#include <cuda.h>
#include <type_traits>

#include "profile.cuh"
#include "sm100_common.cuh"
#include "sm100_kernels.cuh"

namespace vafa {
namespace {

using namespace ptx;

// 14 warps: 0-7 element-wise, 8 TMA, 9 MMA, 10-13 drain the per-block dQ contribution out of tensor memory
// and add it into global memory (issued by the element-wise warps the reductions stalled those for the 1.3-1.6 us
// they take per block).  Registers are allotted per four warps, so 14 warps count as 16: 128 per thread.
constexpr int kThreads = 448;
constexpr int kIn = 128;        // query rows per inner block
constexpr int kD = 128;         // head dim
// Exponentials as in the kernel pair (all on the special-function unit unless VAFA_BWD_POLY_PERIOD says
// otherwise), so that dK and dV of the two modes stay bit-identical.
#ifndef VAFA_BWD_POLY_PERIOD
#define VAFA_BWD_POLY_PERIOD 0
#endif
constexpr int kPolyPeriod = VAFA_BWD_POLY_PERIOD;
constexpr bool use_poly(int i) { return kPolyPeriod > 0 && (i % (kPolyPeriod > 0 ? kPolyPeriod : 1)) == kPolyPeriod - 1; }
constexpr int kAugBytes = 128 * 32;
constexpr int kSubBytes = 128 * 128;      // one 64-column sub tile: 128 rows x 128 B
constexpr int kTileBytes = 2 * kSubBytes; // 128 rows x 128 columns of 16 bit
constexpr int kSA = 2;                    // Q ring (live from S^T to dK of its block); dO has one slot
constexpr uint32_t kColX = 0, kColY = 128, kColDv = 256, kColDk = 384;

struct SmemF {
  alignas(1024) uint8_t k[kTileBytes];
  alignas(1024) uint8_t v[kTileBytes];
  alignas(1024) uint8_t q[kSA][kTileBytes];
  alignas(1024) uint8_t d_o[kTileBytes];
  alignas(1024) uint8_t ds[kTileBytes];           // dS^T [key][query]: sub tile = 64 queries
  alignas(1024) uint8_t aug[kSA][2][kAugBytes];   // fold rows of the Q slot: [lse pieces, delta pieces]
  alignas(1024) uint8_t ones[kAugBytes];
  alignas(8) uint64_t outer_full, outer_free;
  uint64_t a_full[kSA], a_empty[kSA], b_full, b_empty;
  uint64_t x_full, y_full, p_full, ds_full, ds_free, dq_full, dq_free, acc_done;
  uint64_t pair_bar[4];  // the two warps that share a TMEM lane quadrant
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};
static_assert(sizeof(SmemF) + 1024 <= 227 * 1024, "shared memory budget");

struct ParamsF {
  void* dv;
  void* dk;
  float* dq_acc;  // [T_q, H, 128] fp32, zeroed before the launch
  const SchedHeader* header;
  const WorkItem* items;
  int H;
  float scale;
  float scale_log2;
  int32_t* status;
  int wait_limit;
};

constexpr uint32_t kDescHiSw32 = (256u >> 4) | (1u << 14) | (6u << 29);  // fold tiles: SBO 256 B, SWIZZLE_32B

__device__ __forceinline__ void red_add_v4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

// Adds a 16-float chunk (64 bytes) of each lane's row into global memory.  A thread owns a tile row (TMEM
// lane = row), so a plain reduction of its chunk sends the 32 lanes of an instruction to 32 rows; the four
// lanes of a group first transpose their 4 x 4 block of 16-byte pieces by shuffle (as the epilogues'
// store_chunk_coalesced does), so that each instruction covers 64 contiguous bytes of one row per group.
__device__ __forceinline__ void red_chunk_coalesced(uint32_t (&w)[16], float* my_chunk, long long row_stride, int my_row,
                                                    int n_rows) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int m = 1; m <= 2; m <<= 1) {
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j & m) continue;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t send = hi ? w[4 * j + e] : w[4 * (j | m) + e];
        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, m);
        if (hi) w[4 * j + e] = recv; else w[4 * (j | m) + e] = recv;
      }
    }
  }
  const int i = lane & 3;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int row = my_row - i + k;
    if (row < n_rows) red_add_v4(my_chunk + (long long)(k - i) * row_stride + i * 4, w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
  }
}

template <typename T>
__global__ void __maxnreg__(128)
varlen_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                        const __grid_constant__ CUtensorMap tmap_aug, const ParamsF p) {
  extern __shared__ uint8_t smem_raw[];
  SmemF& sm = *reinterpret_cast<SmemF*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    wq_init(sm.wq, 13);  // 8 element-wise warps, the MMA thread, 4 drain warps
    mbar_init(smem_u32(&sm.outer_full), 1);
    mbar_init(smem_u32(&sm.outer_free), 1);
    for (int i = 0; i < kSA; ++i) {
      mbar_init(smem_u32(&sm.a_full[i]), 1);
      mbar_init(smem_u32(&sm.a_empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.b_full), 1);
    mbar_init(smem_u32(&sm.b_empty), 1);
    mbar_init(smem_u32(&sm.x_full), 1);
    mbar_init(smem_u32(&sm.y_full), 1);
    mbar_init(smem_u32(&sm.p_full), 8);    // one arrival per element-wise warp
    mbar_init(smem_u32(&sm.ds_full), 8);
    mbar_init(smem_u32(&sm.ds_free), 1);
    mbar_init(smem_u32(&sm.dq_full), 1);
    mbar_init(smem_u32(&sm.dq_free), 4);   // one arrival per drain warp
    mbar_init(smem_u32(&sm.acc_done), 1);
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&sm.pair_bar[i]), 64);
    fence_barrier_init();
  }
  if (warp < 8) {
    // constant operand of the fold step: every element 1 (bf16) or 64 (fp16, whose pieces are stored / 64)
    const uint32_t one2 = std::is_same<T, __nv_bfloat16>::value ? 0x3F803F80u : 0x54005400u;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(sm.ones);
    for (int i = threadIdx.x; i < kAugBytes / 4; i += 256) o32[i] = one2;
    fence_proxy_async();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_do);
    prefetch_tensormap(&tmap_aug);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sm.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;

  const int n_items = p.header->n_items;
  const int total = max(n_items, 0);
  int* const next_item = const_cast<int*>(&p.header->next_item);
  if (n_items < 0 && threadIdx.x == 0) report_error(p.status, 2, 150, n_items);

  if (warp >= 10) {
    // ---------------- drain warps: dQ contribution of every block -> global fp32 dQ ----------------
    // thread -> query row r of the block (TMEM lane), 128 columns in two halves of 64 registers: B is free
    // for the next dP^T once the second half has been read, i.e. after the first half's reductions are issued
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    uint32_t gk = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int h = w.head;
      const int nb = (w.i_len + kIn - 1) / kIn;
      for (int b = 0; b < nb; ++b) {
        const uint32_t g = gk + b;
        if (!mbar_wait(smem_u32(&sm.dq_full), g & 1, abort_flag)) { alive = false; break; }
        tc_fence_after();
        const int n_rows = min(kIn, w.i_len - b * kIn);
        float* my = p.dq_acc + (((long long)w.i_start + b * kIn + r) * p.H + h) * kD;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t t[64];
          tmem_ld64(lane_base + kColY + hf * 64, t);
          tmem_wait_ld();
          if (hf == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm.dq_free));
          }
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t piece[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) piece[i] = t[c4 * 16 + i];
            red_chunk_coalesced(piece, my + hf * 64 + c4 * 16, (long long)p.H * kD, r, n_rows);
          }
        }
      }
      gk += nb;
    }
  } else if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t gk = 0, qi = 0;
      bool alive = true;
      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_produce(sm.wq, n, next_item, total, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const int h = w.head;
        const int nb = (w.i_len + kIn - 1) / kIn;
        if (nb == 0) continue;
        if (!mbar_wait(smem_u32(&sm.outer_free), (qi & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(smem_u32(&sm.outer_full), 2 * kTileBytes);
        for (int c = 0; c < 2; ++c) {
          tma_load_3d(smem_u32(sm.k) + c * kSubBytes, &tmap_k, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
          tma_load_3d(smem_u32(sm.v) + c * kSubBytes, &tmap_v, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
        }
        for (int b = 0; b < nb; ++b, ++gk) {
          const int sa = gk % kSA;
          const int row = w.i_start + b * kIn;
          if (!mbar_wait(smem_u32(&sm.a_empty[sa]), ((gk / kSA) & 1) ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.a_full[sa]), kTileBytes + 2 * kAugBytes);
          for (int c = 0; c < 2; ++c)
            tma_load_3d(smem_u32(sm.q[sa]) + c * kSubBytes, &tmap_q, smem_u32(&sm.a_full[sa]), c * 64, h, row);
          tma_load_3d(smem_u32(sm.aug[sa][0]), &tmap_aug, smem_u32(&sm.a_full[sa]), 0, h, row);
          tma_load_3d(smem_u32(sm.aug[sa][1]), &tmap_aug, smem_u32(&sm.a_full[sa]), 16, h, row);
          // the single dO slot is free once dV of the previous block is complete; its next tile is pulled into
          // L2 meanwhile, so that the load that follows the release is short
          if (b + 1 < nb)
            for (int c = 0; c < 2; ++c) tma_prefetch_3d(&tmap_do, c * 64, h, row + kIn);
          if (!mbar_wait(smem_u32(&sm.b_empty), (gk & 1) ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.b_full), kTileBytes);
          for (int c = 0; c < 2; ++c)
            tma_load_3d(smem_u32(sm.d_o) + c * kSubBytes, &tmap_do, smem_u32(&sm.b_full), c * 64, h, row);
        }
        ++qi;
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_xy = make_idesc(kFmt, 0, 0, 128, kIn);   // both operands K-major
      constexpr uint32_t idesc_acc = make_idesc(kFmt, 0, 1, 128, kD);   // A K-major (TMEM or shared), B MN-major
      constexpr uint32_t idesc_dq = make_idesc(kFmt, 1, 1, 128, kD);    // A MN-major (dS: queries along M), B MN-major
      uint32_t gk = 0, qi = 0;
      bool alive = true;
      const uint32_t k_lo = desc_lo_sw128(smem_u32(sm.k), 16), v_lo = desc_lo_sw128(smem_u32(sm.v), 16);
      const uint32_t k_mn_lo = desc_lo_sw128(smem_u32(sm.k), kSubBytes);    // K tile as an MN-major B operand
      const uint32_t ds_k_lo = desc_lo_sw128(smem_u32(sm.ds), 16);          // dS^T, K-major A (rows = keys)
      const uint32_t ds_mn_lo = desc_lo_sw128(smem_u32(sm.ds), kSubBytes);  // dS, MN-major A (M = queries)
      const uint32_t do_mn_lo = desc_lo_sw128(smem_u32(sm.d_o), kSubBytes);
      const uint32_t do_lo = desc_lo_sw128(smem_u32(sm.d_o), 16);
      const uint32_t ones_lo = desc_lo_sw128(smem_u32(sm.ones), 16);

      // S^T'(g) = K . Q(g)^T + 1 . L^T
      auto issue_x = [&](uint32_t g) -> bool {
        const int sa = g % kSA;
        if (!mbar_wait(smem_u32(&sm.a_full[sa]), (g / kSA) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_lo = desc_lo_sw128(smem_u32(sm.q[sa]), 16);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (kSubBytes >> 4) + (kk & 3) * 2;  // 16-byte units
          mma_ss2(tbase + kColX, k_lo + off, q_lo + off, idesc_xy, kk > 0);
        }
        mma_ss2h(tbase + kColX, ones_lo, desc_lo_sw128(smem_u32(sm.aug[sa][0]), 16), idesc_xy, 1u, kDescHiSw32);
        mma_commit(smem_u32(&sm.x_full));
        return true;
      };
      // dP^T'(g) = V . dO(g)^T - delta
      auto issue_y = [&](uint32_t g) -> bool {
        const int sa = g % kSA;
        if (!mbar_wait(smem_u32(&sm.b_full), g & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (kSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(tbase + kColY, v_lo + off, do_lo + off, idesc_xy, kk > 0);
        }
        mma_ss2h(tbase + kColY, ones_lo, desc_lo_sw128(smem_u32(sm.aug[sa][1]), 16), idesc_xy, 1u, kDescHiSw32);
        mma_commit(smem_u32(&sm.y_full));
        return true;
      };

      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_consume_thread(sm.wq, n, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const int nb = (w.i_len + kIn - 1) / kIn;
        if (nb == 0) continue;
        if (!mbar_wait(smem_u32(&sm.outer_full), qi & 1, abort_flag)) break;
        tc_fence_after();
        if (!issue_x(gk)) break;
        // B still holds the dQ contribution of the previous item's last block until it is read out
        if (gk > 0 && !mbar_wait(smem_u32(&sm.dq_free), (gk - 1) & 1, abort_flag)) break;
        tc_fence_after();
        if (!issue_y(gk)) break;
        for (int b = 0; b < nb; ++b) {
          const uint32_t g = gk + b;
          const int sa = g % kSA;
          // dV += P^T dO(g): P^T packed in A[0,64), K-step kk (16 queries) = 8 columns
          if (!mbar_wait(smem_u32(&sm.p_full), g & 1, abort_flag)) { alive = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kIn / 16; ++kk)
            mma_ts2(tbase + kColDv, tbase + kColX + kk * 8, do_mn_lo + kk * (2048 >> 4), idesc_acc, (b > 0 || kk > 0) ? 1u : 0u);
          mma_commit(smem_u32(&sm.b_empty));
          if (b + 1 < nb && !issue_x(g + 1)) { alive = false; break; }
          // dQ_blk = dS K into B (dP^T has been consumed), then dK += dS^T Q(g), both from the shared-memory dS^T
          if (!mbar_wait(smem_u32(&sm.ds_full), g & 1, abort_flag)) { alive = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kIn / 16; ++kk)
            mma_ss2(tbase + kColY, ds_mn_lo + kk * (2048 >> 4), k_mn_lo + kk * (2048 >> 4), idesc_dq, kk > 0);
          mma_commit(smem_u32(&sm.dq_full));
          {
            const uint32_t q_mn_lo = desc_lo_sw128(smem_u32(sm.q[sa]), kSubBytes);
#pragma unroll
            for (int kk = 0; kk < kIn / 16; ++kk) {
              const uint32_t off = (kk >> 2) * (kSubBytes >> 4) + (kk & 3) * 2;
              mma_ss2(tbase + kColDk, ds_k_lo + off, q_mn_lo + kk * (2048 >> 4), idesc_acc, (b > 0 || kk > 0) ? 1u : 0u);
            }
          }
          mma_commit(smem_u32(&sm.a_empty[sa]));
          mma_commit(smem_u32(&sm.ds_free));
          if (b + 1 < nb) {
            if (!mbar_wait(smem_u32(&sm.dq_free), g & 1, abort_flag)) { alive = false; break; }
            tc_fence_after();
            if (!issue_y(g + 1)) { alive = false; break; }
          } else {
            mma_commit(smem_u32(&sm.acc_done));
            mma_commit(smem_u32(&sm.outer_free));
          }
        }
        gk += nb;
        ++qi;
      }
    }
  } else if (warp < 8) {
    // ---------------- element-wise warps + epilogue (warps 0-7) ----------------
    // thread -> key row r = tid % 128 (TMEM lane; warp w may only touch lane quadrant w % 4);
    // warps 0-3 take query columns [0,64) of every block, warps 4-7 columns [64,128)
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t pair_bar = smem_u32(&sm.pair_bar[warp & 3]);
    uint32_t pair_cnt = 0;
    const float c = p.scale_log2;
    uint32_t gk = 0, qi = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int h = w.head;
      const int nb = (w.i_len + kIn - 1) / kIn;

      for (int b = 0; b < nb; ++b) {
        const uint32_t g = gk + b;
        // visibility of query jj = b*128 + col for key row r: jj < i_len and (causal) jj >= r + diag
        int lo = 0;
        const int hi = w.i_len - 1 - b * kIn;
        if (w.masked) lo = r + w.diag - b * kIn;
        // key rows past the tile's last valid row hold the next segment's keys (or zero fill): their dK / dV rows
        // are simply not stored, but here they would add into dQ, so their P is forced to zero
        if (r >= w.o_rows) lo = kIn;
        const bool need_mask = (hi < kIn - 1) || (lo > 0);

        // ---- phase 1: P^T = 2^(c S^T') ----
        if (!mbar_wait(smem_u32(&sm.x_full), g & 1, abort_flag)) { alive = false; break; }
        tc_fence_after();
        float pf[64];
        auto phase1 = [&](auto mask_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
          uint32_t xs[64];
          tmem_ld64(lane_base + kColX + half * 64, xs);
          tmem_wait_ld();
          mbar_arrive(pair_bar);  // my columns are in registers: the other half may overwrite them
          const uint64_t c2 = pack_f2(c, c);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint64_t t2 = mul_f2(pack_f2(__uint_as_float(xs[2 * i]), __uint_as_float(xs[2 * i + 1])), c2);
            float p0, p1;
            if (use_poly(i)) {
              ex2_poly2(t2, p0, p1);
            } else {
              float t0, t1;
              unpack_f2(t2, t0, t1);
              p0 = ex2(t0);
              p1 = ex2(t1);
            }
            if (kMask) {
              const int col = half * 64 + 2 * i;
              p0 = ((col >= lo) && (col <= hi)) ? p0 : 0.f;
              p1 = ((col + 1 >= lo) && (col + 1 <= hi)) ? p1 : 0.f;
            }
            pf[2 * i] = p0;
            pf[2 * i + 1] = p1;
          }
        };
        if (__any_sync(0xffffffffu, need_mask)) phase1(std::true_type{}); else phase1(std::false_type{});
        {
          // P^T packed over A[0,64): my 64 queries become 32 columns at [32 * half, 32 * half + 32)
          uint32_t pp[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pp[i] = pack2_out<T>(pf[2 * i], pf[2 * i + 1]);  // as the dK/dV kernel of the pair
          if (!mbar_wait(pair_bar, pair_cnt & 1, abort_flag)) { alive = false; break; }
          ++pair_cnt;
          tmem_st32(lane_base + kColX + half * 32, pp);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.p_full));

        // ---- phase 2: dS^T = P^T dP^T' -> shared memory ----
        if (!mbar_wait(smem_u32(&sm.y_full), g & 1, abort_flag)) { alive = false; break; }
        tc_fence_after();
        {
          uint32_t ys[64];
          tmem_ld64(lane_base + kColY + half * 64, ys);
          tmem_wait_ld();
          uint32_t dd[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // the product already holds dP - delta; masked columns have P = 0 exactly and a finite factor
            float d0, d1;
            unpack_f2(mul_f2(pack_f2(pf[2 * i], pf[2 * i + 1]),
                             pack_f2(__uint_as_float(ys[2 * i]), __uint_as_float(ys[2 * i + 1]))), d0, d1);
            dd[i] = pack2_out<T>(d0, d1);
          }
          // the MMAs that read dS^T of the previous block are complete
          if (g > 0 && !mbar_wait(smem_u32(&sm.ds_free), (g - 1) & 1, abort_flag)) { alive = false; break; }
          // row r of sub tile `half`: eight 16-byte pieces, piece j stored at position j ^ (r & 7)
          uint8_t* rowp = sm.ds + half * kSubBytes + r * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(rowp + ((j ^ (r & 7)) << 4)) = make_uint4(dd[4 * j], dd[4 * j + 1], dd[4 * j + 2], dd[4 * j + 3]);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.ds_full));

      }
      if (!alive) break;
      gk += nb;

      // ---- epilogue: dV (unscaled) and dK (scaled), each half of the warps half of the columns ----
      if (nb > 0) {
        if (!mbar_wait(smem_u32(&sm.acc_done), qi & 1, abort_flag)) break;
        tc_fence_after();
        ++qi;
      }
      const long long out_row = ((long long)w.o_start + r) * p.H + h;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        T* optr = reinterpret_cast<T*>(which == 0 ? p.dv : p.dk) + out_row * kD;
        const float mul = which == 0 ? 1.f : p.scale;
        const uint32_t acc_col = which == 0 ? kColDv : kColDk;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          const int cc = half * 2 + c2;
          uint32_t t[32];
          if (nb > 0) {
            tmem_ld32(lane_base + acc_col + cc * 32, t);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = 0u;
          }
          uint32_t pw[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pw[i] = pack2_out<T>(__uint_as_float(t[2 * i]) * mul, __uint_as_float(t[2 * i + 1]) * mul);
          store_chunk_coalesced<T>(pw, optr + cc * 32, (long long)p.H * kD, r, w.o_rows, 4);
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    if (threadIdx.x == 0) report_error(p.status, 1, 151, blockIdx.x);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 9) tmem_dealloc(tbase, 512);
}

// dq = (I/O dtype)(scale * acc): eight elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) dq_finalize_kernel(const float* __restrict__ acc, T* __restrict__ dq, long long n8, float scale) {
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    const float4 a = reinterpret_cast<const float4*>(acc)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    uint4 o;
    o.x = pack2_out<T>(a.x * scale, a.y * scale);
    o.y = pack2_out<T>(a.z * scale, a.w * scale);
    o.z = pack2_out<T>(b.x * scale, b.y * scale);
    o.w = pack2_out<T>(b.z * scale, b.w * scale);
    reinterpret_cast<uint4*>(dq)[i] = o;
  }
}

template <typename T>
int launch_fused(const Bwd128Launch& L, cudaStream_t s) {
  const size_t n = (size_t)L.total_q * L.H * kD;
  VAFA_CUDA_CHECK(cudaMemsetAsync(L.dq_acc, 0, n * sizeof(float), s));
  ParamsF p;
  p.dv = L.dv; p.dk = L.dk; p.dq_acc = L.dq_acc;
  p.header = (const SchedHeader*)L.hdr_dkv; p.items = (const WorkItem*)L.items_dkv;
  p.H = L.H; p.scale = L.scale; p.scale_log2 = L.scale * kLog2e; p.status = L.status;
  p.wait_limit = wait_limit_units();
  CUtensorMap q128, do128, k128, v128, aug;
  int rc;
  if ((rc = encode_tmap_rows(&q128, L.q, L.dtype, L.total_q, L.H, kD, 128))) return rc;
  if ((rc = encode_tmap_rows(&do128, L.d_o, L.dtype, L.total_q, L.H, kD, 128))) return rc;
  if ((rc = encode_tmap_rows(&k128, L.k, L.dtype, L.total_k, L.H, kD, 128))) return rc;
  if ((rc = encode_tmap_rows(&v128, L.v, L.dtype, L.total_k, L.H, kD, 128))) return rc;
  if ((rc = encode_tmap_fold(&aug, L.aug, L.dtype, L.total_q, L.H))) return rc;
  const size_t smem = sizeof(SmemF) + 1024;
  VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    LaunchScope scope(kKBwdFused, s);
    varlen_bwd_fused_kernel<T><<<L.sms, kThreads, smem, s>>>(k128, v128, q128, do128, aug, p);
  }
  VAFA_LAUNCH_CHECK("varlen_bwd_fused_kernel");
  {
    const long long n8 = (long long)(n / 8);
    const unsigned grid = (unsigned)((n8 + 255) / 256 < (long long)L.sms * 16 ? (n8 + 255) / 256 : (long long)L.sms * 16);
    LaunchScope scope(kKBwdDqFin, s);
    dq_finalize_kernel<T><<<grid ? grid : 1, 256, 0, s>>>(L.dq_acc, (T*)L.dq, n8, L.scale);
  }
  VAFA_LAUNCH_CHECK("dq_finalize_kernel");
  return 0;
}

}  // namespace

int sm100_varlen_bwd_fused_launch(const Bwd128Launch& L, cudaStream_t s) {
  if (L.D != kD || L.dq_acc == nullptr) return fail(VAFA_ERR_UNSUPPORTED, "the fused backward takes head_dim 128 and an fp32 dQ array");
  return L.dtype == VAFA_BF16 ? launch_fused<__nv_bfloat16>(L, s) : launch_fused<__half>(L, s);
}

}  // namespace vafa
