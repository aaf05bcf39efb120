// Packed variable-length attention backward, 128 x 128 tiles (tcgen05 + TMA + TMEM).
//
// Two kernels from one template, no atomics (gradients are run-to-run identical):
//   dQ    : one 128-row query tile per item (outer = Q, dO), walks the segment's keys (inner = K, V)
//   dK/dV : one 128-row key tile per item (outer = K, V), walks the segment's query rows (inner = Q, dO)
// All score products are M128 x N128 MMAs (N = 64 measured 56 % of the tensor rate).
//
// The element-wise work of a block is split in two phases, so that with single score buffers the
// tensor pipe always has the other phase's product to run:
//   phase 1:  P  = 2^(c X - lse)          needs X = outerA . innerA^T
//   phase 2:  dS = P (Y - delta)          needs Y = outerB . innerB^T
// dK/dV (TMEM: X [0,128) Y [128,256) dV [256,384) dK [384,512)), issue order in steady state
//     dV += P^T dO(g) ; X(g+1)   |   dK += dS^T Q(g) ; Y(g+1)
//   P^T overwrites X and dS^T overwrites Y in place (16-bit, packed); the next X is issued behind
//   the product that reads P^T, the next Y behind the product that reads dS^T (the pipe runs in order).
// dQ (TMEM: X0 [0,128) X1 [128,256) Y [256,384) dQ [384,512)), steady state
//     dQ += dS K(g) ; Y(g+1) ; X(g+2)
//   dS overwrites X[g&1] in place; the scores of block g+1 are already there when phase 1 of g+1 starts.
//
// In the dK/dV kernel a thread owns a key row, so lse and delta vary along its columns.  Instead of
// reading them per element from shared memory (measured: about 1000 cycles per block), they are
// folded into the score products as one extra K = 16 step:  X' = K Q^T + 1 . L^T with
// L[q] = split3(-lse[q] / c) in the I/O dtype (three 16-bit pieces carry a 24-bit value, the products
// with 1 are exact and the sum is accumulated in fp32), likewise Y' = V dO^T - delta.  The pieces are
// written once per (token, head) by the preprocess kernel and arrive by TMA with the Q block.
// Then P = 2^(c X') and dS = P Y' need no per-column operand at all.
//
// Reference: triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:233-350 (dQ), :367-494 (dK/dV).
#include <cuda.h>
#include <type_traits>

#include "profile.cuh"
#include "sm100_common.cuh"
#include "sm100_kernels.cuh"

namespace vafa {
namespace {

using namespace ptx;

#ifdef VAFA_TRACE
#define TRACE_T0() const long long _t0 = clock64()
#define TRACE_ADD(slot) tr[slot] += clock64() - _t0
#else
#define TRACE_T0()
#define TRACE_ADD(slot)
#endif

// Element-wise warps: 8 (two per TMEM lane quadrant, 64 score columns per thread) or 16 (four per quadrant, 32
// columns per thread).  The backward needs no row statistics, so the columns of a row split freely.
#ifndef VAFA_BWD_EW_WARPS
#define VAFA_BWD_EW_WARPS 8
#endif
constexpr int kEw = VAFA_BWD_EW_WARPS;
// Rounding of P and dS to the I/O type: pack2 (two adds and a byte permute on the integer pipe) or pack2_out (one
// conversion on the special-function pipe, which also runs the exponentials).  Measured: the dK/dV kernel, with two
// roundings per score, is 0.5-1.7 % faster with the conversion; the dQ kernel is level to 1.5 % slower with it.
template <typename T, bool kDKV>
__device__ __forceinline__ uint32_t pack_bwd(float lo, float hi) {
  if constexpr (kDKV) return pack2_out<T>(lo, hi);
  else return pack2<T>(lo, hi);
}
static_assert(kEw == 8 || kEw == 16, "element-wise warps");
constexpr int kGroups = kEw / 4;        // column groups of a row
constexpr int kC = 128 / kGroups;       // score columns per thread
constexpr int kTmaWarp = kEw, kMmaWarp = kEw + 1;
// Registers are granted per four warps, so ten warps leave every thread 168.  With two spare warps the
// producer / issuer warp group can hand most of its share to the element-wise warp groups (setmaxnreg), which
// then have 216 each (build with -DVAFA_BWD_SETMAXNREG=1; eight element-wise warps only).
#ifndef VAFA_BWD_SETMAXNREG
#define VAFA_BWD_SETMAXNREG 0
#endif
static_assert(!VAFA_BWD_SETMAXNREG || kEw == 8, "register hand-over is laid out for eight element-wise warps");
constexpr int kThreads = kEw * 32 + (VAFA_BWD_SETMAXNREG ? 128 : 64);  // + 1 TMA warp, 1 MMA warp (+ 2 spare)
#if VAFA_BWD_SETMAXNREG
#define VAFA_REG_DEC() asm volatile("setmaxnreg.dec.sync.aligned.u32 72;")
#define VAFA_REG_INC() asm volatile("setmaxnreg.inc.sync.aligned.u32 216;")
#else
#define VAFA_REG_DEC()
#define VAFA_REG_INC()
#endif
// one tcgen05.ld for a thread's kC columns
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[64]) { tmem_ld64(taddr, r); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
constexpr int kIn = 128;       // rows per inner block
// One pair of exponentials in kPolyPeriod can take the polynomial 2^t on the FMA pipe instead of the
// special-function unit; 0 = none.  In these kernels none is fastest (measured: period 4 costs 3-5 % on long
// non-causal batches and 2.5 % on the 1 M-token causal batch): per score they already issue five integer-pipe
// instructions (two rounding adds and a byte permute for each of P and dS), that pipe runs at half rate and is
// the busiest one, and the polynomial adds six more per pair.  The forward, with one rounding per score,
// keeps period 4.
#ifndef VAFA_BWD_POLY_PERIOD
#define VAFA_BWD_POLY_PERIOD 0
#endif
constexpr int kPolyPeriod = VAFA_BWD_POLY_PERIOD;
constexpr bool use_poly(int i) { return kPolyPeriod > 0 && (i % (kPolyPeriod > 0 ? kPolyPeriod : 1)) == kPolyPeriod - 1; }
constexpr int kAugBytes = 128 * 32;  // one fold tile: 128 rows x 16 elements, 32-byte swizzle

template <int D, bool kDKV>
struct Cfg128 {
  // ring A holds K (dQ) or Q (dK/dV): live from the score product to the accumulate product of its
  // block; ring B holds V (dQ: read once) or dO (dK/dV)
  static constexpr int kSA = kDKV ? (D == 128 ? 2 : 4) : (D == 128 ? 3 : 6);
  static constexpr int kSB = (D == 128) ? 2 : 4;
  static constexpr int kSub = D / 64;
  static constexpr int kSubBytes = 128 * 128;  // 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;
  static constexpr uint32_t kX = 0;
  static constexpr uint32_t kY = kDKV ? 128 : 256;
  static constexpr uint32_t kAcc0 = kDKV ? 256 : 384;
  static constexpr uint32_t kAcc1 = 384;  // dK (dK/dV kernel only)
};

template <int D, bool kDKV>
struct Smem128 {
  using Cfg = Cfg128<D, kDKV>;
  alignas(1024) uint8_t outer_a[Cfg::kTileBytes];
  alignas(1024) uint8_t outer_b[Cfg::kTileBytes];
  alignas(1024) uint8_t inner_a[Cfg::kSA][Cfg::kTileBytes];
  alignas(1024) uint8_t inner_b[Cfg::kSB][Cfg::kTileBytes];
  alignas(1024) uint8_t aug[kDKV ? Cfg::kSA : 1][2][kDKV ? kAugBytes : 16];  // [slot][lse, delta]
  alignas(1024) uint8_t ones[kDKV ? kAugBytes : 16];
  alignas(8) uint64_t outer_full, outer_free;
  uint64_t a_full[Cfg::kSA], a_empty[Cfg::kSA];
  uint64_t b_full[Cfg::kSB], b_empty[Cfg::kSB];
  uint64_t x_full[2], y_full, p_full, ds_full, acc_done;
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};
static_assert(sizeof(Smem128<128, false>) + 1024 <= 227 * 1024 && sizeof(Smem128<128, true>) + 1024 <= 227 * 1024 &&
                  sizeof(Smem128<64, false>) + 1024 <= 227 * 1024 && sizeof(Smem128<64, true>) + 1024 <= 227 * 1024,
              "shared memory budget");

struct Params128 {
  void* out0;        // dQ, or dV
  void* out1;        // unused, or dK
  const float2* ld;  // [H][ld_stride] (lse, or +inf for rows that saw no key; delta): dQ kernel
  long long ld_stride;
  const SchedHeader* header;
  const WorkItem* items;
  int H;      // heads of the outer tensors and of the outputs (dQ kernel: query heads; dK/dV kernel: K/V heads)
  int group;  // query heads per K/V head: the dQ kernel reads K/V head h / group, the dK/dV kernel walks the
              // query rows of its `group` query heads one head after the other, into the same accumulators
  float scale;
  float scale_log2;
  int32_t* status;
  int wait_limit;    // bound of every device-side wait, in units of 65536 cycles
  long long* trace;
};

// descriptor high word of the fold tiles: SBO = 256 B (8 rows x 32 B), version 1, SWIZZLE_32B
constexpr uint32_t kDescHiSw32 = (256u >> 4) | (1u << 14) | (6u << 29);

template <typename T, int D, bool kDKV>
__global__ void __launch_bounds__(kThreads, 1)
varlen_bwd128_kernel(const __grid_constant__ CUtensorMap tmap_outer_a, const __grid_constant__ CUtensorMap tmap_outer_b,
                     const __grid_constant__ CUtensorMap tmap_inner_a, const __grid_constant__ CUtensorMap tmap_inner_b,
                     const __grid_constant__ CUtensorMap tmap_aug, const Params128 p) {
  using Cfg = Cfg128<D, kDKV>;
  constexpr int SA = Cfg::kSA, SB = Cfg::kSB;
  extern __shared__ uint8_t smem_raw[];
  using Smem = Smem128<D, kDKV>;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    wq_init(sm.wq, kEw + 1);
    mbar_init(smem_u32(&sm.outer_full), 1);
    mbar_init(smem_u32(&sm.outer_free), 1);
    for (int i = 0; i < SA; ++i) {
      mbar_init(smem_u32(&sm.a_full[i]), 1);
      mbar_init(smem_u32(&sm.a_empty[i]), 1);
    }
    for (int i = 0; i < SB; ++i) {
      mbar_init(smem_u32(&sm.b_full[i]), 1);
      mbar_init(smem_u32(&sm.b_empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.x_full[0]), 1);
    mbar_init(smem_u32(&sm.x_full[1]), 1);
    mbar_init(smem_u32(&sm.y_full), 1);
    mbar_init(smem_u32(&sm.p_full), kEw);   // one arrival per element-wise warp
    mbar_init(smem_u32(&sm.ds_full), kEw);
    mbar_init(smem_u32(&sm.acc_done), 1);
    fence_barrier_init();
  }
  if (kDKV && warp < kEw) {
    // the constant operand of the fold step: every element 1 (bf16) or 64 (fp16, whose pieces are
    // stored divided by 64 to keep them in range); uniform, so the swizzle does not matter
    const uint32_t one2 = std::is_same<T, __nv_bfloat16>::value ? 0x3F803F80u : 0x54005400u;
    uint32_t* o32 = reinterpret_cast<uint32_t*>(sm.ones);
    for (int i = threadIdx.x; i < kAugBytes / 4; i += kEw * 32) o32[i] = one2;
    fence_proxy_async();
  }
  if (warp == kTmaWarp && lane == 0) {
    prefetch_tensormap(&tmap_outer_a);
    prefetch_tensormap(&tmap_outer_b);
    prefetch_tensormap(&tmap_inner_a);
    prefetch_tensormap(&tmap_inner_b);
    if (kDKV) prefetch_tensormap(&tmap_aug);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&sm.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;

  const int n_items = p.header->n_items;
  const int total = max(n_items, 0);  // one entry per head already
  int* const next_item = const_cast<int*>(&p.header->next_item);
  if (n_items < 0 && threadIdx.x == 0) report_error(p.status, 2, kDKV ? 140 : 130, n_items);
#ifdef VAFA_TRACE
  long long tr[16];
  for (int i = 0; i < 16; ++i) tr[i] = 0;
  const long long t_begin = clock64();
#endif

  // each setmaxnreg sits inside its own role's branch: after a join the compiler assumes the smaller budget
  if (warp > kMmaWarp) {
    VAFA_REG_DEC();  // spare warps of the third warp group
  } else if (warp == kTmaWarp) {
    VAFA_REG_DEC();
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
        mbar_expect_tx(smem_u32(&sm.outer_full), 2 * Cfg::kTileBytes);
        for (int c = 0; c < Cfg::kSub; ++c) {
          tma_load_3d(smem_u32(sm.outer_a) + c * Cfg::kSubBytes, &tmap_outer_a, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
          tma_load_3d(smem_u32(sm.outer_b) + c * Cfg::kSubBytes, &tmap_outer_b, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
        }
        const int nbt = kDKV ? nb * p.group : nb;
        for (int bb = 0; bb < nbt; ++bb, ++gk) {
          const int sa = gk % SA, sb = gk % SB;
          const int b = kDKV ? bb % nb : bb;
          const int hin = kDKV ? h * p.group + bb / nb : h / p.group;  // head of the inner tensors
          const int row = w.i_start + b * kIn;
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.a_empty[sa]), ((gk / SA) & 1) ^ 1, abort_flag)) { alive = false; break; } TRACE_ADD(0); }
          mbar_expect_tx(smem_u32(&sm.a_full[sa]), Cfg::kTileBytes + (kDKV ? 2 * kAugBytes : 0));
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.inner_a[sa]) + c * Cfg::kSubBytes, &tmap_inner_a, smem_u32(&sm.a_full[sa]), c * 64, hin, row);
          if (kDKV) {
            // fold pieces of the block's 128 query rows: elements [0,16) for lse, [16,32) for delta
            tma_load_3d(smem_u32(sm.aug[sa][0]), &tmap_aug, smem_u32(&sm.a_full[sa]), 0, hin, row);
            tma_load_3d(smem_u32(sm.aug[sa][1]), &tmap_aug, smem_u32(&sm.a_full[sa]), 16, hin, row);
          }
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.b_empty[sb]), ((gk / SB) & 1) ^ 1, abort_flag)) { alive = false; break; } TRACE_ADD(1); }
          mbar_expect_tx(smem_u32(&sm.b_full[sb]), Cfg::kTileBytes);
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.inner_b[sb]) + c * Cfg::kSubBytes, &tmap_inner_b, smem_u32(&sm.b_full[sb]), c * 64, hin, row);
        }
        ++qi;
      }
    }
  } else if (warp == kMmaWarp) {
    VAFA_REG_DEC();
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_xy = make_idesc(kFmt, 0, 0, 128, kIn);  // both operands K-major
      constexpr uint32_t idesc_acc = make_idesc(kFmt, 0, 1, 128, D);   // A from TMEM, B MN-major
      uint32_t gk = 0, qi = 0;
      bool alive = true;
      const uint32_t oa_lo = desc_lo_sw128(smem_u32(sm.outer_a), 16), ob_lo = desc_lo_sw128(smem_u32(sm.outer_b), 16);
      const uint32_t ones_lo = desc_lo_sw128(smem_u32(sm.ones), 16);

      // X(g) = outerA . innerA(g)^T  (+ fold step)
      auto issue_x = [&](uint32_t g) -> bool {
        const int sa = g % SA;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.a_full[sa]), (g / SA) & 1, abort_flag)) return false; TRACE_ADD(4); }
        tc_fence_after();
        TRACE_T0();
        const uint32_t x_tmem = tbase + Cfg::kX + (kDKV ? 0u : (g & 1) * 128u);
        const uint32_t ia_lo = desc_lo_sw128(smem_u32(sm.inner_a[sa]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (Cfg::kSubBytes >> 4) + (kk & 3) * 2;  // 16-byte units
          mma_ss2(x_tmem, oa_lo + off, ia_lo + off, idesc_xy, kk > 0);
        }
        if (kDKV) mma_ss2h(x_tmem, ones_lo, desc_lo_sw128(smem_u32(sm.aug[sa][0]), 16), idesc_xy, 1u, kDescHiSw32);
        mma_commit(smem_u32(&sm.x_full[kDKV ? 0 : (g & 1)]));
        TRACE_ADD(14);
        return true;
      };
      // Y(g) = outerB . innerB(g)^T  (+ fold step); the last one of an item releases the outer tiles
      auto issue_y = [&](uint32_t g, bool last) -> bool {
        const int sa = g % SA, sb = g % SB;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.b_full[sb]), (g / SB) & 1, abort_flag)) return false; TRACE_ADD(5); }
        tc_fence_after();
        TRACE_T0();
        const uint32_t ib_lo = desc_lo_sw128(smem_u32(sm.inner_b[sb]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (Cfg::kSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(tbase + Cfg::kY, ob_lo + off, ib_lo + off, idesc_xy, kk > 0);
        }
        if (kDKV) mma_ss2h(tbase + Cfg::kY, ones_lo, desc_lo_sw128(smem_u32(sm.aug[sa][1]), 16), idesc_xy, 1u, kDescHiSw32);
        mma_commit(smem_u32(&sm.y_full));
        if (!kDKV) mma_commit(smem_u32(&sm.b_empty[sb]));  // V is read by this product only
        if (last) mma_commit(smem_u32(&sm.outer_free));
        TRACE_ADD(14);
        return true;
      };
      // ACC (+)= A[TMEM, 16-bit packed: K-step kk at column (kk/2)*32 + (kk%2)*8] . B[shared, MN-major]
      auto issue_acc = [&](uint32_t d_tmem, uint32_t a_tmem, const uint8_t* b_tile, bool first) {
        TRACE_T0();
        const uint32_t b_lo = desc_lo_sw128(smem_u32(b_tile), Cfg::kSubBytes);
#pragma unroll
        for (int kk = 0; kk < kIn / 16; ++kk)
          mma_ts2(d_tmem, a_tmem + (kk >> 1) * 32 + (kk & 1) * 8, b_lo + kk * (2048 >> 4), idesc_acc, (!first || kk > 0) ? 1u : 0u);
        TRACE_ADD(2);
      };

      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_consume_thread(sm.wq, n, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const int nb = ((w.i_len + kIn - 1) / kIn) * (kDKV ? p.group : 1);  // blocks of the item, over all its query heads
        if (nb == 0) continue;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.outer_full), qi & 1, abort_flag)) break; TRACE_ADD(3); }
        tc_fence_after();
        if (!issue_x(gk) || !issue_y(gk, nb == 1)) break;
        if (!kDKV && nb > 1 && !issue_x(gk + 1)) break;
        for (int b = 0; b < nb; ++b) {
          const uint32_t g = gk + b;
          const int sa = g % SA, sb = g % SB;
          if (kDKV) {
            { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.p_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(6); }
            tc_fence_after();
            issue_acc(tbase + Cfg::kAcc0, tbase + Cfg::kX, sm.inner_b[sb], b == 0);  // dV += P^T dO
            mma_commit(smem_u32(&sm.b_empty[sb]));
            if (b + 1 < nb && !issue_x(g + 1)) { alive = false; break; }
            { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.ds_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(7); }
            tc_fence_after();
            issue_acc(tbase + Cfg::kAcc1, tbase + Cfg::kY, sm.inner_a[sa], b == 0);  // dK += dS^T Q
            mma_commit(smem_u32(&sm.a_empty[sa]));
            if (b + 1 < nb) {
              if (!issue_y(g + 1, b + 2 == nb)) { alive = false; break; }
            } else {
              mma_commit(smem_u32(&sm.acc_done));
            }
          } else {
            { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.ds_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(7); }
            tc_fence_after();
            issue_acc(tbase + Cfg::kAcc0, tbase + Cfg::kX + (g & 1) * 128u, sm.inner_a[sa], b == 0);  // dQ += dS K
            mma_commit(smem_u32(&sm.a_empty[sa]));
            if (b + 1 < nb) {
              if (!issue_y(g + 1, b + 2 == nb)) { alive = false; break; }
              if (b + 2 < nb && !issue_x(g + 2)) { alive = false; break; }
            } else {
              mma_commit(smem_u32(&sm.acc_done));
            }
          }
        }
        gk += nb;
        ++qi;
      }
    }
  } else {
    // ---------------- element-wise warps + epilogue (warps 0-7) ----------------
    VAFA_REG_INC();
    // thread -> outer row r = tid % 128 (TMEM lane; a warp may only touch lane quadrant warp % 4);
    // warps 0-3 take inner columns [0,64) of every block, warps 4-7 columns [64,128)
    const int r = threadIdx.x & 127;
    const int grp = threadIdx.x >> 7;  // column group of this thread
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const float c = p.scale_log2;
    uint32_t gk = 0, qi = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int h = w.head;
      const int nb1 = (w.i_len + kIn - 1) / kIn;      // blocks per query head
      const int nb = nb1 * (kDKV ? p.group : 1);
      const bool row_ok = r < w.o_rows;
      float neg_lse = -INFINITY, my_delta = 0.f;
      if (!kDKV && row_ok && nb > 0) {
        const float2 t = p.ld[(long long)h * p.ld_stride + w.o_start + r];
        neg_lse = -t.x;
        my_delta = t.y;
      }

      for (int bb = 0; bb < nb; ++bb) {
        const uint32_t g = gk + bb;
        const int b = kDKV ? bb % nb1 : bb;  // block within the query head's rows
        // visibility of inner index jj = b*128 + col for this thread's outer row r
        //   dQ : jj < i_len and (causal) jj <= r + diag
        //   dKV: jj < i_len and (causal) jj >= r + diag
        int lo = 0, hi = w.i_len - 1 - b * kIn;
        if (w.masked) {
          if (!kDKV) hi = min(hi, r + w.diag - b * kIn);
          else lo = r + w.diag - b * kIn;
        }
        const bool need_mask = (hi < kIn - 1) || (lo > 0);
        const uint32_t x_addr = lane_base + Cfg::kX + (kDKV ? 0u : (g & 1) * 128u);
        const uint32_t y_addr = lane_base + Cfg::kY;

        // ---- phase 1: P ----
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.x_full[kDKV ? 0 : (g & 1)]), kDKV ? (g & 1) : ((g >> 1) & 1), abort_flag)) { alive = false; break; } TRACE_ADD(8); }
        tc_fence_after();
#ifdef VAFA_TRACE
        const long long t_p1 = clock64();
#endif
        float pf[kC];
        // masked blocks (tails, the causal diagonal) take their own copy of the loop: folded into one
        // loop the two compares and the select per element ran in every block
        auto phase1 = [&](auto mask_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
          // this thread's columns [kC * grp, kC * grp + kC) in one load
          uint32_t xs[kC];
          tmem_ld_cols(x_addr + grp * kC, xs);
          tmem_wait_ld();
          // exponent t = c X' (dK/dV: the product already holds S - lse/c) or c S - lse, in pairs; every
          // kPolyPeriod-th pair takes the polynomial 2^t on the FMA pipe, the others the special-function unit
          const uint64_t c2 = pack_f2(c, c), nl2 = pack_f2(neg_lse, neg_lse);
#pragma unroll
          for (int i = 0; i < kC / 2; ++i) {
            const uint64_t x2 = pack_f2(__uint_as_float(xs[2 * i]), __uint_as_float(xs[2 * i + 1]));
            const uint64_t t2 = kDKV ? mul_f2(x2, c2) : fma_f2(x2, c2, nl2);
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
              const int col = grp * kC + 2 * i;
              p0 = ((col >= lo) && (col <= hi)) ? p0 : 0.f;
              p1 = ((col + 1 >= lo) && (col + 1 <= hi)) ? p1 : 0.f;
            }
            pf[2 * i] = p0;
            pf[2 * i + 1] = p1;
          }
          if (kDKV) {
            // P^T in place: each 32-column chunk becomes 16 packed columns over its own first half
#pragma unroll
            for (int q2 = 0; q2 < kC / 32; ++q2) {
              uint32_t pp[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) pp[i] = pack_bwd<T, kDKV>(pf[q2 * 32 + 2 * i], pf[q2 * 32 + 2 * i + 1]);
              tmem_st16(x_addr + (grp * (kC / 32) + q2) * 32, pp);
            }
          }
        };
        // warp-uniform choice: the TMEM loads and stores inside are .sync.aligned
        if (__any_sync(0xffffffffu, need_mask)) phase1(std::true_type{}); else phase1(std::false_type{});
        if (kDKV) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm.p_full));
        }

#ifdef VAFA_TRACE
        tr[12] += clock64() - t_p1;
#endif
        // ---- phase 2: dS ----
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.y_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(9); }
        tc_fence_after();
#ifdef VAFA_TRACE
        const long long t_p2 = clock64();
#endif
        {
          uint32_t ys[kC];
          const uint64_t nd2 = pack_f2(-my_delta, -my_delta);
          tmem_ld_cols(y_addr + grp * kC, ys);
          tmem_wait_ld();
#pragma unroll
          for (int q2 = 0; q2 < kC / 32; ++q2) {
            uint32_t dd[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              // dK/dV: the product already holds dP - delta.  Masked columns have P = 0 exactly, and the
              // other factor is finite there (rows of a neighbouring segment, or zero fill past the end)
              uint64_t y2 = pack_f2(__uint_as_float(ys[q2 * 32 + 2 * i]), __uint_as_float(ys[q2 * 32 + 2 * i + 1]));
              if (!kDKV) y2 = add_f2(y2, nd2);
              float d0, d1;
              unpack_f2(mul_f2(pack_f2(pf[q2 * 32 + 2 * i], pf[q2 * 32 + 2 * i + 1]), y2), d0, d1);
              dd[i] = pack_bwd<T, kDKV>(d0, d1);
            }
            // dQ: dS over the scores just consumed (X[g&1]); dK/dV: dS^T over dP^T (Y); in place as above
            tmem_st16((kDKV ? y_addr : x_addr) + (grp * (kC / 32) + q2) * 32, dd);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.ds_full));
#ifdef VAFA_TRACE
        tr[13] += clock64() - t_p2;
        tr[11] += 1;
#endif
      }
      if (!alive) break;
      gk += nb;

      // ---- epilogue: each half of the warps converts and stores half of the columns ----
      if (nb > 0) {
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.acc_done), qi & 1, abort_flag)) break; TRACE_ADD(10); }
        tc_fence_after();
        ++qi;
      }
      const long long out_row = ((long long)w.o_start + r) * p.H + h;
#pragma unroll
      for (int which = 0; which < (kDKV ? 2 : 1); ++which) {
        T* optr = reinterpret_cast<T*>(which == 0 ? p.out0 : p.out1) + out_row * D;
        // dV unscaled; dQ and dK scaled; dQ rows that saw no key are exact zeros (the polynomial 2^t
        // leaves about 1e-38 where the special-function unit gives 0)
        // a row whose lse or delta is NaN (the forward saw a NaN, or dO holds one) goes out as NaN: the packed
        // dS operand cannot carry it (see pack2)
        const float poison = kDKV ? 0.f : ((neg_lse == -INFINITY ? 0.f : neg_lse * 0.f) + my_delta * 0.f);
        const float mul = (kDKV && which == 0) ? 1.f : ((!kDKV && neg_lse == -INFINITY) ? 0.f : p.scale + poison);
        const uint32_t acc_col = which == 0 ? Cfg::kAcc0 : Cfg::kAcc1;
#pragma unroll
        for (int cc = grp; cc < D / 32; cc += kGroups) {  // 32-column chunks of the accumulator, dealt to the groups
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
          store_chunk_coalesced<T>(pw, optr + cc * 32, (long long)p.H * D, r, w.o_rows, 4);
        }
      }
    }
  }

#ifdef VAFA_TRACE
  if (p.trace != nullptr && (threadIdx.x == 0 || threadIdx.x == 256 || threadIdx.x == 288)) {
    tr[15] = clock64() - t_begin;
    for (int i = 0; i < 16; ++i)
      if (tr[i] != 0) p.trace[((long long)(kDKV ? 1 : 0) * 256 + blockIdx.x) * 16 + i] = tr[i];
  }
#endif
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    if (threadIdx.x == 0) report_error(p.status, 1, kDKV ? 141 : 131, blockIdx.x);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == kMmaWarp) tmem_dealloc(tbase, 512);
}

}  // namespace

#ifdef VAFA_TRACE
long long* vafa_trace_buffer_bwd = nullptr;
#endif

template <typename T, int D>
static int launch128(const Bwd128Launch& L, cudaStream_t s) {
  Params128 p;
  p.wait_limit = wait_limit_units();
  p.ld = (const float2*)L.ld; p.ld_stride = L.ld_stride; p.H = L.H;
  p.scale = L.scale; p.scale_log2 = L.scale * kLog2e; p.status = L.status;
  p.trace = nullptr;
#ifdef VAFA_TRACE
  {
    static long long* g_trace = nullptr;  // debugging aid only
    if (!g_trace) cudaMalloc(&g_trace, 512 * 16 * sizeof(long long));
    cudaMemsetAsync(g_trace, 0, 512 * 16 * sizeof(long long), s);
    p.trace = g_trace;
    vafa_trace_buffer_bwd = g_trace;
  }
#endif
  CUtensorMap q128, do128, k128, v128, aug;
  int rc;
  if ((rc = encode_tmap_rows(&q128, L.q, L.dtype, L.total_q, L.H, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&do128, L.d_o, L.dtype, L.total_q, L.H, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&k128, L.k, L.dtype, L.total_k, L.H_kv, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&v128, L.v, L.dtype, L.total_k, L.H_kv, D, 128))) return rc;
  if ((rc = encode_tmap_fold(&aug, L.aug, L.dtype, L.total_q, L.H))) return rc;
  p.group = L.H / L.H_kv;
  if (L.run_dq) {
    // dQ: outer = (Q, dO) tiles, inner = (K, V) blocks
    const size_t smem = sizeof(Smem128<D, false>) + 1024;
    p.out0 = L.dq; p.out1 = nullptr; p.header = (const SchedHeader*)L.hdr_dq; p.items = (const WorkItem*)L.items_dq;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd128_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    {
      LaunchScope scope(kKBwdDq, s);
      varlen_bwd128_kernel<T, D, false><<<L.sms, kThreads, smem, s>>>(q128, do128, k128, v128, aug, p);
    }
    VAFA_LAUNCH_CHECK("varlen_bwd128_kernel<dQ>");
  }
  if (L.run_dkv) {
    // dK/dV: outer = (K, V) tiles, inner = (Q, dO) blocks
    const size_t smem = sizeof(Smem128<D, true>) + 1024;
    p.out0 = L.dv; p.out1 = L.dk; p.header = (const SchedHeader*)L.hdr_dkv; p.items = (const WorkItem*)L.items_dkv;
    p.H = L.H_kv;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd128_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    {
      LaunchScope scope(kKBwdDkv, s);
      varlen_bwd128_kernel<T, D, true><<<L.sms, kThreads, smem, s>>>(k128, v128, q128, do128, aug, p);
    }
    VAFA_LAUNCH_CHECK("varlen_bwd128_kernel<dKV>");
  }
  return 0;
}

int sm100_varlen_bwd128_launch(const Bwd128Launch& L, cudaStream_t s) {
  if (L.dtype == VAFA_BF16) return L.D == 128 ? launch128<__nv_bfloat16, 128>(L, s) : launch128<__nv_bfloat16, 64>(L, s);
  return L.D == 128 ? launch128<__half, 128>(L, s) : launch128<__half, 64>(L, s);
}

}  // namespace vafa

#ifdef VAFA_TRACE
extern "C" __attribute__((visibility("default"))) int vafa_trace_read_bwd(long long* host, int n) {
  if (!vafa::vafa_trace_buffer_bwd) return -1;
  return (int)cudaMemcpy(host, vafa::vafa_trace_buffer_bwd, (size_t)n * 16 * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif
