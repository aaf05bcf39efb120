// Packed variable-length attention backward for sm_100a: host side (tile lists, preprocess kernel,
// launch of the 128 x 128-tile dQ and dK/dV kernels of sm100_varlen_bwd128.cu), and the 64-row-block
// kernel template that the absorb operator's backward core (D = d_kv = 256) runs on.
//
// Three kernels per backward, no atomics, so gradients are run-to-run identical:
//   1. preprocess: delta[t,h] = sum_d O*dO (fp32), written together with the LSE as float2
//      pairs in a head-major array LD[h][t] = (lse, delta)  (reference: kernels.py:186-216), and as
//      16-bit fold rows for the dK/dV kernel
//   2. dQ kernel : one 128-row query tile per item, walks the segment's keys (reference: kernels.py:233-350)
//   3. dKV kernel: one 128-row key tile per item, walks the segment's query rows (reference: kernels.py:367-494)
// (paths: triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py)
//
// The 64-row-block template.  "Outer" is the 128-row tile that stays in shared memory, "inner" the
// 64-row blocks streamed through a ring.  Per inner block g, with X/Y double buffered in TMEM so the
// next block's scores are computed while the current block's element-wise work runs:
//     X[g&1] = outerA . innerA^T        (S   = Q K^T      or  S^T  = K Q^T)
//     Y[g&1] = outerB . innerB^T        (dP  = dO V^T     or  dP^T = V dO^T)
//   compute warps (thread = outer row):  P = 2^(X c - lse),  dS = P (Y - delta)
//     dQ : dS (16-bit) overwrites X;               ACC0 += dS . K_g
//     dKV: P^T overwrites X, dS^T overwrites Y;    ACC0 += P^T . dO_g ,  ACC1 += dS^T . Q_g
// TMEM columns: X0 [0,64) X1 [64,128) Y0 [128,192) Y1 [192,256) ACC0 [256,256+D) ACC1 [384,384+D).
// The softmax scale multiplies dQ and dK once, in fp32, in the epilogue (reference:
// kernels.py:336-348, :476-491).
#include <cuda.h>
#include <type_traits>

#include "sm100_common.cuh"
#include "sm100_kernels.cuh"
#include "sm100_sched_body.cuh"
#include "profile.cuh"

namespace vafa {
namespace {

// Rounding of P and dS to the I/O type in the element-wise phases: the conversion instruction in the kernel that
// walks query chunks (absorb dU: 4-6 % faster with it, measured), the integer form (see common.cuh) in the one
// that walks key tiles (absorb dX: level to 2 % slower with the conversion).
template <typename T, bool kDKV>
__device__ __forceinline__ uint32_t pack_ew(float lo, float hi) {
  if constexpr (kDKV) return pack2<T>(lo, hi);
  else return pack2_out<T>(lo, hi);
}

using namespace ptx;

// Optional wait-time tracing (build with -DVAFA_TRACE), as in sm100_varlen_fwd.cu.
#ifdef VAFA_TRACE
#define TRACE_T0() const long long _t0 = clock64()
#define TRACE_ADD(slot) tr[slot] += clock64() - _t0
#else
#define TRACE_T0()
#define TRACE_ADD(slot)
#endif

constexpr int kBwdThreads = 320;  // 8 element-wise warps, 1 TMA warp, 1 MMA warp
constexpr int kLdRow = 68;        // float2 slots per staged (lse, delta) block: 64 + 2 of alignment slack, padded
constexpr int kInner = 64;  // rows per inner block
constexpr int kPlanarRow = 72;  // floats per staged planar block: 64 + 3 of alignment slack, padded; 68 are copied

template <int D>
struct BwdCfg {
  static constexpr int kStages = (D == 128) ? 4 : (D == 64 ? 8 : 2);
  static constexpr int kSub = D / 64;
  static constexpr int kOuterSubBytes = 128 * 128;   // 128 rows x 128 B
  static constexpr int kInnerSubBytes = kInner * 128;  // 64 rows x 128 B
  static constexpr int kOuterBytes = kSub * kOuterSubBytes;
  static constexpr int kInnerBytes = kSub * kInnerSubBytes;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kXCol = 0, kYCol = 128, kAcc0 = 256, kAcc1 = 384;
};

// kAbsorb (the absorb operator, D = d_kv = 256): keys and values are the same X rows, so the dU
// kernel has one inner operand and the dX kernel one outer operand; the unused buffer shrinks.
// Ring depth.  The absorb dU kernel streams X from HBM and releases a block only after its second use
// (dU += dS X), while the next score product is issued one block ahead: with two stages that product
// always waited a full load; its unused inner_b and (lse, delta) staging shrink to make room for three.
template <int D, bool kDKV, bool kAbsorb>
constexpr int bwd_stages() { return (D == 256 && kAbsorb && !kDKV) ? 3 : BwdCfg<D>::kStages; }

template <int D, bool kDKV = false, bool kAbsorb = false>
struct BwdSmem {
  static constexpr int kS = bwd_stages<D, kDKV, kAbsorb>();
  alignas(1024) uint8_t outer_a[BwdCfg<D>::kOuterBytes];
  alignas(1024) uint8_t outer_b[(kAbsorb && kDKV) ? 1024 : BwdCfg<D>::kOuterBytes];
  alignas(1024) uint8_t inner_a[kS][BwdCfg<D>::kInnerBytes];
  alignas(1024) uint8_t inner_b[kS][(kAbsorb && !kDKV) ? 16 : BwdCfg<D>::kInnerBytes];
  alignas(8) uint64_t outer_full, outer_free;
  uint64_t in_full[kS], in_empty[kS];
  uint64_t xy_full[2], ds_full[2], acc_done;
  alignas(16) float2 ld[kS][(kDKV && !kAbsorb) ? kLdRow : 2];  // dKV: (lse, delta) of the inner block's query rows
  // absorb dX: the same two numbers planar, as -lse and -delta * scale, so that a pair of neighbouring
  // columns is one 8-byte operand of the packed fp32 instructions
  alignas(16) float nl[kS][(kDKV && kAbsorb) ? kPlanarRow : 4];
  alignas(16) float nd[kS][(kDKV && kAbsorb) ? kPlanarRow : 4];
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};

static_assert(sizeof(BwdSmem<128>) + 1024 <= 227 * 1024 && sizeof(BwdSmem<64>) + 1024 <= 227 * 1024 &&
                  sizeof(BwdSmem<256, false, true>) + 1024 <= 227 * 1024 && sizeof(BwdSmem<256, true, true>) + 1024 <= 227 * 1024,
              "shared memory budget");

struct BwdParams {
  void* out0;            // dQ, or dV
  void* out1;            // unused, or dK
  const float2* ld;      // varlen: [H][ld_stride]; absorb: [T_q * H] token-major.  (lse, or +inf for dead rows; delta)
  long long ld_stride;
  const SchedHeader* header;
  const WorkItem* items;
  int H;
  float scale;
  float scale_log2;
  int32_t* status;
  int wait_limit;        // bound of every device-side wait, in units of 65536 cycles
  int out_width;         // absorb dX: columns written per row (= row stride of the output), <= D
  long long* trace;
};

// Only the absorb forms (kAbsorb = true, D = 256) are launched: packed_varlen_attn's dQ and dK/dV run on
// the 128 x 128-tile kernels of sm100_varlen_bwd128.cu, which replaced the kAbsorb = false form of this
// template (kept because the two forms share every line but the operand bookkeeping).
// kAbsorb = false: items x heads; outer/inner operands are per-head [rows, D] slices.
// kAbsorb = true : heads are stacked into the tile rows (row = q*H + h) exactly as in the forward;
//   dU kernel (kDKV = false): outer = (U, dAlphaX) stacked rows of 128/H queries, inner = X blocks,
//                             S = U X^T, dP = dAlphaX X^T, dU += dS X;
//   dX kernel (kDKV = true) : outer = 128 rows of X, inner = 64 stacked rows of (U, dAlphaX),
//                             S^T = X U^T, dP^T = X dAlphaX^T, dX += P^T dAlphaX + (scale dS^T) U
//                             (one accumulator; the scale is folded into dS before rounding).
template <typename T, int D, bool kDKV, bool kAbsorb>
__global__ void __launch_bounds__(kBwdThreads, 1)
varlen_bwd_kernel(const __grid_constant__ CUtensorMap tmap_outer_a, const __grid_constant__ CUtensorMap tmap_outer_b,
                  const __grid_constant__ CUtensorMap tmap_inner_a, const __grid_constant__ CUtensorMap tmap_inner_b,
                  const BwdParams p) {
  using Cfg = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  using Smem = BwdSmem<D, kDKV, kAbsorb>;
  constexpr int S = Smem::kS;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    wq_init(sm.wq, 9);
    mbar_init(smem_u32(&sm.outer_full), 1);
    mbar_init(smem_u32(&sm.outer_free), 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&sm.in_full[i]), 1);
      mbar_init(smem_u32(&sm.in_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.xy_full[i]), 1);
      mbar_init(smem_u32(&sm.ds_full[i]), 256);
    }
    mbar_init(smem_u32(&sm.acc_done), 1);
    fence_barrier_init();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tensormap(&tmap_outer_a);
    prefetch_tensormap(&tmap_outer_b);
    prefetch_tensormap(&tmap_inner_a);
    prefetch_tensormap(&tmap_inner_b);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sm.tmem_base), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;

  const int n_items = p.header->n_items;
  // inner rows (in the units of WorkItem::i_start / i_len) per 64-wide inner block
  const int ib = (kAbsorb && kDKV) ? kInner / p.H : kInner;
  const int total = max(n_items, 0);  // one entry per head already
  int* const next_item = const_cast<int*>(&p.header->next_item);
  if (n_items < 0 && threadIdx.x == 0) report_error(p.status, 2, kDKV ? 120 : 110, n_items);
#ifdef VAFA_TRACE
  long long tr[16];
  for (int i = 0; i < 16; ++i) tr[i] = 0;
  const long long t_begin = clock64();
#endif

  if (warp == 8) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t gk = 0, qi = 0;
      bool alive = true;
      constexpr int kPrefetch = 6;  // inner blocks pulled into L2 ahead of their load (dU: X streams from HBM)
      int idx = wq_produce(sm.wq, 0, next_item, total, abort_flag);
      for (uint32_t n = 0; alive && idx >= 0; ++n) {
        const WorkItem w = p.items[idx];
        const int h = w.head;
        const int nb = (w.i_len + ib - 1) / ib;
        if (nb == 0) {
          idx = wq_produce(sm.wq, n + 1, next_item, total, abort_flag);
          continue;
        }
        constexpr bool kOneOuter = kAbsorb && kDKV;   // dX: the X tile is both outer operands
        constexpr bool kOneInner = kAbsorb && !kDKV;  // dU: the X block is both inner operands
        if (kOneInner)
          for (int b = 2; b < kPrefetch && b < nb; ++b)
            for (int c = 0; c < Cfg::kSub; ++c) tma_prefetch_3d(&tmap_inner_a, c * 64, h, w.i_start + b * ib);
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.outer_free), (qi & 1) ^ 1, abort_flag)) break; TRACE_ADD(0); }
        mbar_expect_tx(smem_u32(&sm.outer_full), (kOneOuter ? 1 : 2) * Cfg::kOuterBytes);
        for (int c = 0; c < Cfg::kSub; ++c) {
          tma_load_3d(smem_u32(sm.outer_a) + c * Cfg::kOuterSubBytes, &tmap_outer_a, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
          if (!kOneOuter)
            tma_load_3d(smem_u32(sm.outer_b) + c * Cfg::kOuterSubBytes, &tmap_outer_b, smem_u32(&sm.outer_full), c * 64, h, w.o_start);
        }
        for (int b = 0; b < nb; ++b, ++gk) {
          const int st = gk % S;
          const uint32_t ph = (gk / S) & 1;
          const int row = w.i_start + b * ib;
          if (kOneInner && b + kPrefetch < nb)
            for (int c = 0; c < Cfg::kSub; ++c) tma_prefetch_3d(&tmap_inner_a, c * 64, h, row + kPrefetch * ib);
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.in_empty[st]), ph ^ 1, abort_flag)) { alive = false; break; } TRACE_ADD(1); }
          mbar_expect_tx(smem_u32(&sm.in_full[st]),
                         (kOneInner ? 1 : 2) * Cfg::kInnerBytes + (kDKV ? (kAbsorb ? 2 * 68 * 4 : 66 * 8) : 0));
          if (kDKV && kAbsorb) {
            // planar -lse and -delta*scale of the block's 64 stacked rows, from the 16-byte boundary at or
            // below the first (readers skip first & 3 slots); the arrays follow the float2 array
            const long long first = (long long)row * p.H;
            const float* nlg = reinterpret_cast<const float*>(p.ld + p.ld_stride);
            const float* ndg = nlg + p.ld_stride;
            bulk_load_1d(smem_u32(&sm.nl[st][0]), nlg + (first & ~3LL), 68 * 4, smem_u32(&sm.in_full[st]));
            bulk_load_1d(smem_u32(&sm.nd[st][0]), ndg + (first & ~3LL), 68 * 4, smem_u32(&sm.in_full[st]));
          } else if (kDKV) {
            // (lse, delta) pairs of the block's 64 inner columns: the copy starts at the even index
            // at or below the first pair (16-byte alignment) and takes 66 pairs; readers skip
            // (index & 1) slots
            const long long first = kAbsorb ? (long long)row * p.H : (long long)h * p.ld_stride + row;
            bulk_load_1d(smem_u32(&sm.ld[st][0]), p.ld + (first & ~1LL), 66 * 8, smem_u32(&sm.in_full[st]));
          }
          for (int c = 0; c < Cfg::kSub; ++c) {
            tma_load_3d(smem_u32(sm.inner_a[st]) + c * Cfg::kInnerSubBytes, &tmap_inner_a, smem_u32(&sm.in_full[st]), c * 64, h, row);
            if (!kOneInner)
              tma_load_3d(smem_u32(sm.inner_b[st]) + c * Cfg::kInnerSubBytes, &tmap_inner_b, smem_u32(&sm.in_full[st]), c * 64, h, row);
          }
        }
        ++qi;
        // The next item is drawn now, while this one is being worked on, and its outer tile pulled into
        // L2: the outer tiles are single-buffered, so their load is exposed once per item (dX has one
        // inner block per item on user batches, and its X tile comes from HBM).
        idx = alive ? wq_produce(sm.wq, n + 1, next_item, total, abort_flag) : -1;
        if (idx >= 0) {
          const WorkItem wn = p.items[idx];
          for (int c = 0; c < Cfg::kSub; ++c) {
            tma_prefetch_3d(&tmap_outer_a, c * 64, wn.head, wn.o_start);
            if (!kOneOuter) tma_prefetch_3d(&tmap_outer_b, c * 64, wn.head, wn.o_start);
          }
        }
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_xy = make_idesc(kFmt, 0, 0, 128, kInner);  // outer(128) x inner(64), both K-major
      constexpr uint32_t idesc_acc = make_idesc(kFmt, 0, 1, 128, D);      // A from TMEM, B MN-major
      uint32_t gk = 0, qi = 0;
      bool alive = true;

      auto issue_xy = [&](uint32_t g, bool last) -> bool {
        const int st = g % S;
        const uint32_t ph = (g / S) & 1;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.in_full[st]), ph, abort_flag)) return false; TRACE_ADD(4); }
        tc_fence_after();
        const uint32_t x_tmem = tbase + Cfg::kXCol + (g & 1) * kInner;
        const uint32_t y_tmem = tbase + Cfg::kYCol + (g & 1) * kInner;
        const uint32_t oa_lo = desc_lo_sw128(smem_u32(sm.outer_a), 16);
        const uint32_t ob_lo = desc_lo_sw128(smem_u32((kAbsorb && kDKV) ? sm.outer_a : sm.outer_b), 16);
        const uint32_t ia_lo = desc_lo_sw128(smem_u32(sm.inner_a[st]), 16);
        const uint32_t ib_lo = desc_lo_sw128(smem_u32((kAbsorb && !kDKV) ? sm.inner_a[st] : sm.inner_b[st]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offo = (kk >> 2) * (Cfg::kOuterSubBytes >> 4) + (kk & 3) * 2;  // 16-byte units
          const uint32_t offi = (kk >> 2) * (Cfg::kInnerSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(x_tmem, oa_lo + offo, ia_lo + offi, idesc_xy, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offo = (kk >> 2) * (Cfg::kOuterSubBytes >> 4) + (kk & 3) * 2;
          const uint32_t offi = (kk >> 2) * (Cfg::kInnerSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(y_tmem, ob_lo + offo, ib_lo + offi, idesc_xy, kk > 0);
        }
        mma_commit(smem_u32(&sm.xy_full[g & 1]));
        if (last) mma_commit(smem_u32(&sm.outer_free));
        return true;
      };

      // Items are walked with a lookahead of one block across item boundaries: the score products of the
      // next item's first block are issued before the last accumulate products of this item, which wait
      // for the element-wise warps (absorb dX has one block per item: without the lookahead its score
      // products, element-wise phase, accumulate products and epilogue ran back to back).
      uint32_t n_next = 0;
      int nb_next = 0;
      // draws items until one has inner blocks; waits for its outer tile and issues its first score products
      auto start_next_item = [&]() -> bool {
        while (true) {
          const int idx = wq_consume_thread(sm.wq, n_next++, abort_flag);
          if (idx < 0) return false;
          const WorkItem w = p.items[idx];
          nb_next = (w.i_len + ib - 1) / ib;
          if (nb_next > 0) break;
        }
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.outer_full), qi & 1, abort_flag)) return false; TRACE_ADD(3); }
        tc_fence_after();
        ++qi;
        return issue_xy(gk, nb_next == 1);
      };
      bool have = start_next_item();
      while (have && alive) {
        const int nb = nb_next;
        const uint32_t g0 = gk;
        gk += nb;  // start_next_item() issues block gk
        have = false;
        for (int b = 0; b < nb; ++b) {
          const uint32_t g = g0 + b;
          if (b + 1 < nb) {
            if (!issue_xy(g + 1, b + 2 == nb)) { alive = false; break; }
          } else {
            have = start_next_item();
          }
          const int st = g % S;
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.ds_full[g & 1]), (g >> 1) & 1, abort_flag)) { alive = false; break; } TRACE_ADD(7); }
          tc_fence_after();
          const uint32_t x_tmem = tbase + Cfg::kXCol + (g & 1) * kInner;
          const uint32_t y_tmem = tbase + Cfg::kYCol + (g & 1) * kInner;
          const uint32_t acc = (b > 0) ? 1u : 0u;
          const uint32_t ma_lo = desc_lo_sw128(smem_u32(sm.inner_a[st]), Cfg::kInnerSubBytes);
          const uint32_t mb_lo = desc_lo_sw128(smem_u32((kAbsorb && !kDKV) ? sm.inner_a[st] : sm.inner_b[st]), Cfg::kInnerSubBytes);
          if (!kDKV) {
            // dQ += dS . K_g     (dS in X, 16-bit packed; K block MN-major)
#pragma unroll
            for (int kk = 0; kk < kInner / 16; ++kk)
              mma_ts2(tbase + Cfg::kAcc0, x_tmem + (kk >> 1) * 32 + (kk & 1) * 8, ma_lo + kk * (2048 >> 4), idesc_acc,
                      (acc | (kk > 0)) ? 1u : 0u);
          } else {
            // dV += P^T . dO_g ;  dK += dS^T . Q_g
#pragma unroll
            for (int kk = 0; kk < kInner / 16; ++kk)
              mma_ts2(tbase + Cfg::kAcc0, x_tmem + (kk >> 1) * 32 + (kk & 1) * 8, mb_lo + kk * (2048 >> 4), idesc_acc,
                      (acc | (kk > 0)) ? 1u : 0u);
#pragma unroll
            for (int kk = 0; kk < kInner / 16; ++kk)
              mma_ts2(tbase + (kAbsorb ? Cfg::kAcc0 : Cfg::kAcc1), y_tmem + (kk >> 1) * 32 + (kk & 1) * 8, ma_lo + kk * (2048 >> 4),
                      idesc_acc, (kAbsorb || acc || kk > 0) ? 1u : 0u);
          }
          mma_commit(smem_u32(&sm.in_empty[st]));
          if (b + 1 == nb) mma_commit(smem_u32(&sm.acc_done));
        }
      }
    }
  } else {
    // ---------------- element-wise warps + epilogue (warps 0-7) ----------------
    // thread -> outer row r = tid % 128 (TMEM lane; a warp may only touch lane quadrant warp % 4);
    // warps 0-3 take inner columns [0,32) of every block, warps 4-7 columns [32,64)
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const float c = p.scale_log2;
    uint32_t gk = 0, qi = 0;
    bool alive = true;
    // ---- epilogue of one item: accumulator (nb > 0) or zeros -> global memory ----
    auto epilogue = [&](const WorkItem& w, int nb) -> bool {
      const int h = w.head;
      if (nb > 0) {
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.acc_done), qi & 1, abort_flag)) return false; TRACE_ADD(10); }
        tc_fence_after();
        ++qi;
      }
#ifdef VAFA_TRACE
      const long long t_e0 = clock64();
      tr[14] += 1;
#endif
      // output row: varlen (token, head); absorb dU stacked row (token*H + head); absorb dX key row
      const long long out_row = kAbsorb ? (kDKV ? (long long)w.o_start + r : (long long)w.o_start * p.H + r)
                                        : ((long long)w.o_start + r) * p.H + h;
      // absorb dX rows are out_width wide (the caller's X may be narrower than the 256-column tile)
      const int out_w = (kAbsorb && kDKV) ? p.out_width : D;
#pragma unroll
      for (int which = 0; which < ((kDKV && !kAbsorb) ? 2 : 1); ++which) {
        T* optr = reinterpret_cast<T*>(which == 0 ? p.out0 : p.out1) + out_row * out_w;
        // dV unscaled; dQ, dK and dU scaled here; absorb dX carries the scale inside dS
        const float mul = (kDKV && (which == 0)) ? 1.f : p.scale;
        const uint32_t acc_col = which == 0 ? Cfg::kAcc0 : Cfg::kAcc1;
#pragma unroll
        for (int c2 = 0; c2 < D / 64; ++c2) {
          const int cc = half * (D / 64) + c2;  // each half of the compute warps writes half of the columns
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
          // consecutive tile rows are consecutive output rows in every mode of this template
          const long long row_stride = kAbsorb ? (long long)out_w : (long long)p.H * D;
          const int n_valid_rows = (kAbsorb && !kDKV) ? w.o_rows * p.H : w.o_rows;
          store_chunk_coalesced<T>(pw, optr + cc * 32, row_stride, r, n_valid_rows, min(4, max(0, (out_w - cc * 32) / 8)));
        }
      }
#ifdef VAFA_TRACE
      tr[13] += clock64() - t_e0;
#endif
      return true;
    };
    bool pend = false;
    WorkItem pend_w;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int h = w.head;
      const int nb = (w.i_len + ib - 1) / ib;
      // valid outer rows of the tile: absorb dU stacks H heads per query row
      const bool row_ok = r < ((kAbsorb && !kDKV) ? w.o_rows * p.H : w.o_rows);
      float my_lse = INFINITY, my_delta = 0.f;
      if (!kDKV) {
        if (row_ok && nb > 0) {
          const float2 t = kAbsorb ? p.ld[(long long)w.o_start * p.H + r] : p.ld[(long long)h * p.ld_stride + w.o_start + r];
          my_lse = t.x;
          my_delta = t.y;
        }
      }
      const float ds_mul = (kAbsorb && kDKV) ? p.scale : 1.f;

      for (int b = 0; b < nb; ++b) {
        const uint32_t g = gk + b;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.xy_full[g & 1]), (g >> 1) & 1, abort_flag)) { alive = false; break; } TRACE_ADD(8); }
        tc_fence_after();
#ifdef VAFA_TRACE
        const long long t_c0 = clock64();
#endif
        const uint32_t x_addr = lane_base + Cfg::kXCol + (g & 1) * kInner;
        const uint32_t y_addr = lane_base + Cfg::kYCol + (g & 1) * kInner;
        // visibility of inner index jj = b*64 + i for this thread's outer row r
        //   dQ : jj < i_len and (causal) jj <= r + diag
        //   dKV: jj < i_len and (causal) jj >= r + diag
        const int lim_tail = (w.i_len - b * ib) * (kInner / ib) - 1;
        int lo = 0, hi = lim_tail;
        if (w.masked) {
          if (!kDKV) hi = min(hi, r + w.diag - b * kInner);
          else lo = r + w.diag - b * kInner;
        }
        const bool need_mask = (hi < kInner - 1) || (lo > 0);
        const int st = g % S;
        const int ld_skip = kAbsorb ? (int)(((long long)(w.i_start + b * ib) * p.H) & 1) : ((w.i_start + b * kInner) & 1);
        if (kDKV) {
          // the staged (lse, delta) block arrived with this stage's tiles (already complete here;
          // this wait only orders the reads below after the copy)
          if (!mbar_wait(smem_u32(&sm.in_full[st]), (g / S) & 1, abort_flag)) { alive = false; break; }
        }
        // masked blocks (tails, the causal diagonal) take their own copy of the loop; the choice is
        // warp-uniform because the TMEM loads and stores inside are .sync.aligned
        auto block_body = [&](auto mask_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
          uint32_t xs[32], ys[32];
          tmem_ld32(x_addr + half * 32, xs);
          tmem_ld32(y_addr + half * 32, ys);
          tmem_wait_ld();
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float pv[2], dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = half * 32 + i + e;
              float lse_v, delta_v;
              if (kDKV && !kAbsorb) {
                const float2 t = sm.ld[st][ld_skip + col];
                lse_v = t.x;
                delta_v = t.y;
              } else {
                lse_v = my_lse;
                delta_v = my_delta;
              }
              float pr = ex2(fmaf(__uint_as_float(xs[i + e]), c, -lse_v));
              float ds = pr * (__uint_as_float(ys[i + e]) - delta_v) * ds_mul;
              if (kMask) {
                const bool vis = (col >= lo) && (col <= hi);
                pr = vis ? pr : 0.f;
                ds = vis ? ds : 0.f;
              }
              pv[e] = pr;
              dv[e] = ds;
            }
            pp[i >> 1] = pack_ew<T, kDKV>(pv[0], pv[1]);
            dd[i >> 1] = pack_ew<T, kDKV>(dv[0], dv[1]);
          }
          // 32 fp32 columns become 16 packed columns, written over the first 16 of the columns this
          // thread has just read, so the two halves never touch each other's source columns; the MMA
          // issuer addresses K-step kk at column (kk/2)*32 + (kk%2)*8
          if (!kDKV) {
            tmem_st16(x_addr + half * 32, dd);
          } else {
            tmem_st16(x_addr + half * 32, pp);
            tmem_st16(y_addr + half * 32, dd);
          }
        };
        if constexpr (kDKV && kAbsorb) {
          // absorb dX: the staged -lse / -delta*scale rows of columns past the user's last stacked row (they
          // belong to the next user, or to the padding) become -inf / 0, which makes P and dS exact zeros
          // there without a compare per element; then packed fp32 pairs all the way:
          //   P = 2^(S c - lse),  dS = P (dP scale - delta scale)
          const int skip = (int)(((long long)(w.i_start + b * ib) * p.H) & 3);
          if (hi < kInner - 1) {  // same for every thread: the absorb operator has no causal mask
            const int t = threadIdx.x;
            if (t < kInner && t > hi) {
              sm.nl[st][skip + t] = -INFINITY;
              sm.nd[st][skip + t] = 0.f;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
          }
          uint32_t xs[32], ys[32];
          tmem_ld32(x_addr + half * 32, xs);
          tmem_ld32(y_addr + half * 32, ys);
          tmem_wait_ld();
          uint32_t pp[16], dd[16];
          const uint64_t c2 = pack_f2(c, c), s2 = pack_f2(p.scale, p.scale);
          const float* nlp = &sm.nl[st][skip + half * 32];
          const float* ndp = &sm.nd[st][skip + half * 32];
          auto pairs = [&](auto even_tag) {
            constexpr bool kEven = decltype(even_tag)::value;  // 8-byte aligned pairs
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float2 n2, d2;
              if (kEven) {
                n2 = *reinterpret_cast<const float2*>(nlp + 2 * i);
                d2 = *reinterpret_cast<const float2*>(ndp + 2 * i);
              } else {
                n2 = make_float2(nlp[2 * i], nlp[2 * i + 1]);
                d2 = make_float2(ndp[2 * i], ndp[2 * i + 1]);
              }
              const uint64_t t2 = fma_f2(pack_f2(__uint_as_float(xs[2 * i]), __uint_as_float(xs[2 * i + 1])), c2, pack_f2(n2.x, n2.y));
              float t0, t1;
              unpack_f2(t2, t0, t1);
              const float p0 = ex2(t0), p1 = ex2(t1);
              const uint64_t u2 = fma_f2(pack_f2(__uint_as_float(ys[2 * i]), __uint_as_float(ys[2 * i + 1])), s2, pack_f2(d2.x, d2.y));
              float e0, e1;
              unpack_f2(mul_f2(pack_f2(p0, p1), u2), e0, e1);
              pp[i] = pack_ew<T, kDKV>(p0, p1);
              dd[i] = pack_ew<T, kDKV>(e0, e1);
            }
          };
          if ((skip & 1) == 0) pairs(std::true_type{}); else pairs(std::false_type{});
          tmem_st16(x_addr + half * 32, pp);
          tmem_st16(y_addr + half * 32, dd);
        } else {
          if (__any_sync(0xffffffffu, need_mask)) block_body(std::true_type{}); else block_body(std::false_type{});
        }
        tmem_wait_st();
        // The previous item's accumulator is read back here, after this item's first block has been
        // through the element-wise phase and before its products are released (they overwrite the
        // accumulator): the wait for the last accumulate products of an item then runs under the next
        // item's element-wise work instead of stalling these warps (absorb dX: one block per item).
        if (pend) {
          pend = false;
          if (!epilogue(pend_w, 1)) { alive = false; break; }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&sm.ds_full[g & 1]));
#ifdef VAFA_TRACE
        tr[12] += clock64() - t_c0;
        tr[11] += 1;
#endif
      }
      if (!alive) break;
      gk += nb;

      // The accumulator is read back only after the first block of the next item has been through the
      // element-wise phase (see there); an item without inner rows writes its zeros at once.
      if (nb > 0) {
        pend = true;
        pend_w = w;
      } else {
        epilogue(w, 0);
      }
    }
    if (alive && pend) epilogue(pend_w, 1);
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
    if (threadIdx.x == 0) report_error(p.status, 1, kDKV ? 121 : 111, blockIdx.x);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 5) tmem_dealloc(tbase, Cfg::kTmemCols);
}

// A value as three 16-bit pieces (hi, mid, lo) whose exact sum, times 1 (bf16) or 64 (fp16), gives it
// back to about 24 bits: the operand rows of the fold step of the dK/dV kernel.  Non-finite values keep
// only the first piece (-inf stays -inf under the sum).  fp16 pieces are stored divided by 64 so that
// values up to 4.2e6 stay in range; larger ones saturate.
template <typename T>
__device__ __forceinline__ uint2 fold_pieces(float a) {
  constexpr bool kBf = std::is_same<T, __nv_bfloat16>::value;
  if (!kBf) a = isfinite(a) ? fminf(fmaxf(a * (1.f / 64.f), -65504.f), 65504.f) : a;
  const T hi = from_float<T>(a);
  T mid = from_float<T>(0.f), lo = mid;
  if (isfinite(a)) {
    const float r1 = a - to_float(hi);
    mid = from_float<T>(r1);
    lo = from_float<T>(r1 - to_float(mid));
  }
  auto bits = [](T x) -> uint32_t { return (uint32_t)(*reinterpret_cast<const unsigned short*>(&x)); };
  return make_uint2(bits(hi) | (bits(mid) << 16), bits(lo));
}

// delta = rowsum(O * dO); LD[h][t] = (lse or +inf for rows that saw no key, delta); and the same two
// numbers as fold rows fold[t][h][0:16] = pieces(-lse / c), fold[t][h][16:32] = pieces(-delta).
// The first two CTAs of the grid build the tile lists of the dQ and dK/dV kernels instead (they depend
// on cu_seqlens only): the list builder is latency-bound on one SM and hides under the row pass.
template <typename T, int D>
__global__ void __launch_bounds__(sched_impl::kSchedThreads) bwd_prepare_kernel(
    const SchedParams sched_dq, const SchedParams sched_dkv, const T* __restrict__ o, const T* __restrict__ d_o,
    const float* __restrict__ lse, float2* __restrict__ ld, uint4* __restrict__ fold, float inv_c, long long ld_stride,
    int total_q, int H) {
  if (blockIdx.x < 2) {
    sched_impl::sched_build(blockIdx.x == 0 ? sched_dq : sched_dkv);
    return;
  }
  // D/8 lanes per (token, head) row, 16 bytes each; a warp takes 32/(D/8) rows per step and kSteps steps
  // per group.  The data CTAs stay resident (one per SM) and stride over the groups with the next group's
  // loads in flight while the current one is reduced and written: with one short-lived CTA per 256 rows
  // the loads, the arithmetic and the stores of an SM ran one after the other, wave by wave.
  constexpr int kLanes = D / 8, kRowsPerStep = 32 / kLanes, kSteps = 2;
  const int lane = threadIdx.x & 31, sub = lane / kLanes, li = lane % kLanes;
  const long long n_rows = (long long)total_q * H;
  constexpr int kWarpsPerCta = sched_impl::kSchedThreads / 32;
  constexpr int kRowsPerGroup = kRowsPerStep * kSteps;
  const long long n_groups = (n_rows + kRowsPerGroup - 1) / kRowsPerGroup;
  const long long n_warps = (long long)(gridDim.x - 2) * kWarpsPerCta;
  auto load = [&](long long grp, uint4 (&a)[kSteps], uint4 (&b)[kSteps]) {
#pragma unroll
    for (int st = 0; st < kSteps; ++st) {
      const long long row = grp * kRowsPerGroup + st * kRowsPerStep + sub;
      a[st] = b[st] = make_uint4(0u, 0u, 0u, 0u);
      if (row < n_rows) {
        a[st] = reinterpret_cast<const uint4*>(o + row * D)[li];
        b[st] = reinterpret_cast<const uint4*>(d_o + row * D)[li];
      }
    }
  };
  auto reduce_and_store = [&](long long grp, const uint4 (&a)[kSteps], const uint4 (&b)[kSteps]) {
#pragma unroll
    for (int st = 0; st < kSteps; ++st) {
      const long long row = grp * kRowsPerGroup + st * kRowsPerStep + sub;
      const T* pa = reinterpret_cast<const T*>(&a[st]);
      const T* pb = reinterpret_cast<const T*>(&b[st]);
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) part += to_float(pa[i]) * to_float(pb[i]);
#pragma unroll
      for (int off = kLanes / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
      if (row < n_rows && li < 4) {
        const int t = (int)(row / H), h = (int)(row % H);
        const float l = lse[row];
        if (li == 0) ld[(long long)h * ld_stride + t] = make_float2(l == -INFINITY ? INFINITY : l, part);
        // fold row: 32 elements = 64 B = four 16-byte pieces, one per lane
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (li == 0) {
          const uint2 fl = fold_pieces<T>(l == -INFINITY ? -INFINITY : -l * inv_c);
          v.x = fl.x; v.y = fl.y;
        } else if (li == 2) {
          const uint2 fd = fold_pieces<T>(-part);
          v.x = fd.x; v.y = fd.y;
        }
        fold[row * 4 + li] = v;
      }
    }
  };
  uint4 a0[kSteps], b0[kSteps], a1[kSteps], b1[kSteps];
  long long grp = (long long)(blockIdx.x - 2) * kWarpsPerCta + (threadIdx.x >> 5);
  if (grp < n_groups) load(grp, a0, b0);
  // two groups per trip so that the register sets swap roles without copies
  while (grp < n_groups) {
    const long long g1 = grp + n_warps, g2 = g1 + n_warps;
    if (g1 < n_groups) load(g1, a1, b1);
    reduce_and_store(grp, a0, b0);
    if (g1 >= n_groups) break;
    if (g2 < n_groups) load(g2, a0, b0);
    reduce_and_store(g1, a1, b1);
    grp = g2;
  }
}

struct BwdWorkspace {
  size_t hdr_dq, hdr_dkv, items_dq, items_dkv, ld, fold, dq_acc, total;
  SchedCaps caps_dq, caps_dkv;
  long long ld_stride;
};

int resolve_sm_count_bwd(int given) {
  if (given > 0) return given;
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

BwdWorkspace bwd_workspace(const vafa_varlen_args* a, int sms) {
  BwdWorkspace w;
  w.caps_dq = sched_caps(kSchedDq, a->total_q, a->total_k, a->n_seg, a->num_heads, sms, 0);
  w.caps_dkv = sched_caps(kSchedDkv, a->total_k, a->total_q, a->n_seg, a->num_heads, sms, 0);
  w.ld_stride = ((long long)a->total_q + 136 + 3) & ~3LL;  // padding: inner blocks read past the last row
  w.hdr_dq = 0;
  w.hdr_dkv = 256;
  w.items_dq = 512;
  w.items_dkv = w.items_dq + align_up((size_t)w.caps_dq.cap_items * sizeof(WorkItem), 256);
  w.ld = w.items_dkv + align_up((size_t)w.caps_dkv.cap_items * sizeof(WorkItem), 256);
  w.fold = w.ld + align_up((size_t)a->num_heads * w.ld_stride * sizeof(float2), 256);
  w.dq_acc = w.fold + align_up((size_t)a->total_q * a->num_heads * 64, 256);
  // the one-pass backward sums dQ in fp32 here
  const bool fused = varlen_bwd_mode() == 1 && a->head_dim == 128 && (a->num_kv_heads == 0 || a->num_kv_heads == a->num_heads);
  w.total = w.dq_acc + (fused ? align_up((size_t)a->total_q * a->num_heads * a->head_dim * sizeof(float), 256) : 0);
  return w;
}

template <typename T, int D>
int launch_bwd(const vafa_varlen_args* a, cudaStream_t s) {
  const int sms = resolve_sm_count_bwd(a->sm_count);
  const BwdWorkspace ws = bwd_workspace(a, sms);
  char* base = (char*)a->workspace;

  SchedParams sq;
  sq.cu_q = a->cu_seqlens_q; sq.cu_k = a->cu_seqlens_k; sq.n_seg = a->n_seg; sq.mode = kSchedDq;
  sq.causal = a->causal; sq.H = a->num_heads; sq.sm_count = sms; sq.split_len = 0;
  sq.cap_items = ws.caps_dq.cap_items; sq.cap_combine = 0; sq.cap_rows = 0;
  sq.header = (SchedHeader*)(base + ws.hdr_dq);
  sq.items = (WorkItem*)(base + ws.items_dq);
  sq.combine = nullptr;
  const int h_kv = a->num_kv_heads > 0 ? a->num_kv_heads : a->num_heads;
  SchedParams sk = sq;
  sk.mode = kSchedDkv;
  sk.H = h_kv;  // one dK/dV item per key tile and K/V head; it walks the query rows of all heads of its group
  sk.cap_items = ws.caps_dkv.cap_items;
  sk.header = (SchedHeader*)(base + ws.hdr_dkv);
  sk.items = (WorkItem*)(base + ws.items_dkv);

  float2* ld = (float2*)(base + ws.ld);
  {
    const long long n = (long long)a->total_q * a->num_heads;
    // two list-building CTAs plus resident data CTAs: one per remaining SM, fewer for small batches
    constexpr int kRowsPerCtaTrip = (32 / (D / 8)) * 2 * (sched_impl::kSchedThreads / 32);
    const long long want = (n + kRowsPerCtaTrip - 1) / kRowsPerCtaTrip;
    const long long room = sms > 3 ? sms - 2 : 1;
    const unsigned grid = 2u + (unsigned)(want < room ? (want > 0 ? want : 1) : room);
    LaunchScope scope(kKBwdPre, s);
    bwd_prepare_kernel<T, D><<<grid, sched_impl::kSchedThreads, 0, s>>>(
        sq, sk, (const T*)a->o, (const T*)a->d_o, a->lse, ld, (uint4*)(base + ws.fold), 1.f / (a->scale * kLog2e),
        ws.ld_stride, a->total_q, a->num_heads);
    VAFA_LAUNCH_CHECK("bwd_prepare_kernel");
  }

  // both kernels on 128 x 128 tiles (sm100_varlen_bwd128.cu); the 64-row-block template below serves
  // the absorb operator (D = 256), whose tiles leave no room for 128-row inner blocks
  Bwd128Launch L;
  L.q = a->q; L.k = a->k; L.v = a->v; L.d_o = a->d_o; L.dq = a->dq; L.dk = a->dk; L.dv = a->dv;
  L.ld = ld; L.ld_stride = ws.ld_stride; L.aug = base + ws.fold;
  L.hdr_dq = sq.header; L.items_dq = sq.items; L.hdr_dkv = sk.header; L.items_dkv = sk.items;
  L.total_q = a->total_q; L.total_k = a->total_k; L.H = a->num_heads; L.H_kv = h_kv; L.D = D; L.dtype = a->dtype; L.sms = sms;
  L.scale = a->scale; L.status = a->status;
  L.run_dq = 1; L.run_dkv = 1;
  L.dq_acc = nullptr;
  if (varlen_bwd_mode() == 1 && D == 128 && h_kv == a->num_heads) {
    L.dq_acc = (float*)(base + ws.dq_acc);
    return sm100_varlen_bwd_fused_launch(L, s);
  }
  return sm100_varlen_bwd128_launch(L, s);
}


// ---------------- absorb operator: backward core ---------------------------------------------
// LD[t*H + h] = (lse, or +inf where the row saw no key; delta = sum_d O*dO), token-major, followed by
// the same numbers planar for the dX kernel: NL[row] = -LD.x and ND[row] = -delta * scale, each n_pad
// long (n_pad = n_rows + padding, a multiple of 4; the padding rows hold -inf / 0).
template <typename T>
__global__ void __launch_bounds__(256) absorb_ld_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                        const float* __restrict__ lse, float2* __restrict__ ld,
                                                        long long n_rows, long long n_pad, float scale, int D_H) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n_pad) return;
  float* nl = reinterpret_cast<float*>(ld + n_pad);
  float* nd = nl + n_pad;
  if (i >= n_rows) {
    nl[i] = -INFINITY;
    nd[i] = 0.f;
    return;
  }
  const T* a = o + i * D_H;
  const T* b = d_o + i * D_H;
  float acc = 0.f;
  for (int d = 0; d < D_H; ++d) acc += to_float(a[d]) * to_float(b[d]);
  const float l = lse[i];
  ld[i] = make_float2(l == -INFINITY ? INFINITY : l, acc);
  nl[i] = (l == -INFINITY) ? -INFINITY : -l;
  nd[i] = -acc * scale;
}

// The same with D_H/8 lanes per row and 16-byte loads (D_H = 8, 16, ..., 256): a warp reads whole lines.
template <typename T>
__global__ void __launch_bounds__(256) absorb_ld_vec_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                            const float* __restrict__ lse, float2* __restrict__ ld,
                                                            long long n_rows, long long n_pad, float scale, int lanes_log2) {
  const int lanes = 1 << lanes_log2;  // lanes per row, <= 32
  const long long gi = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long row = gi >> lanes_log2;
  const int li = (int)(gi & (lanes - 1));
  float part = 0.f;
  if (row < n_rows) {
    const uint4 a = reinterpret_cast<const uint4*>(o + (row << (lanes_log2 + 3)))[li];
    const uint4 b = reinterpret_cast<const uint4*>(d_o + (row << (lanes_log2 + 3)))[li];
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) part += to_float(pa[i]) * to_float(pb[i]);
  }
  for (int off = lanes >> 1; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if (li == 0 && row < n_pad) {
    float* nl = reinterpret_cast<float*>(ld + n_pad);
    float* nd = nl + n_pad;
    if (row < n_rows) {
      const float l = lse[row];
      ld[row] = make_float2(l == -INFINITY ? INFINITY : l, part);
      nl[row] = (l == -INFINITY) ? -INFINITY : -l;
      nd[row] = -part * scale;
    } else {
      nl[row] = -INFINITY;
      nd[row] = 0.f;
    }
  }
}

// Bexp[(h',dd), (h,kv)] = W_V[kv,h,dd] if h == h' else 0: with it dAlphaX = dO . Bexp is one dense
// product over all heads (dAlphaX[t,h,kv] = sum_dd dO[t,h,dd] W_V[kv,h,dd]).
template <typename T>
__global__ void __launch_bounds__(256) absorb_expand_wv_kernel(const T* __restrict__ w_v, T* __restrict__ bexp, int H, int D_H,
                                                               int d_kv) {
  const int n = H * d_kv;                       // columns of Bexp
  const long long total = (long long)H * D_H * n;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int col = (int)(i % n), row = (int)(i / n);
    const int h = col / d_kv, kv = col % d_kv, hp = row / D_H, dd = row % D_H;
    bexp[i] = (h == hp) ? w_v[((long long)kv * H + h) * D_H + dd] : from_float<T>(0.f);
  }
}

#ifdef VAFA_TRACE
}  // namespace
long long* vafa_trace_buffer_abs = nullptr;
namespace {
#endif

struct AbsorbBwdWs {
  size_t hdr_du, hdr_dx, items_du, items_dx, total;
  int cap_du, cap_dx;
};

AbsorbBwdWs absorb_bwd_ws(int total_q, int total_k, int n_seg, int H) {
  AbsorbBwdWs w;
  w.cap_du = total_q / (kTile / H) + n_seg + 1;
  w.cap_dx = total_k / kTile + n_seg + 1;
  w.hdr_du = 0;
  w.hdr_dx = 256;
  w.items_du = 512;
  w.items_dx = w.items_du + align_up((size_t)w.cap_du * sizeof(WorkItem), 256);
  w.total = w.items_dx + align_up((size_t)w.cap_dx * sizeof(WorkItem), 256);
  return w;
}

struct AbsorbBwdSched {
  SchedParams du, dx;
};

AbsorbBwdSched absorb_bwd_sched_params(const AbsorbCoreBwdArgs& a, int sms) {
  const AbsorbBwdWs ws = absorb_bwd_ws(a.total_q, a.total_k, a.n_seg, a.H);
  char* base = (char*)a.workspace;
  AbsorbBwdSched r;
  SchedParams& sq = r.du;
  sq.cu_q = a.cu_q; sq.cu_k = a.cu_k; sq.n_seg = a.n_seg; sq.mode = kSchedDq; sq.causal = 0; sq.H = 1;
  sq.sm_count = sms; sq.split_len = 0; sq.tile_rows = kTile / a.H;
  sq.cap_items = ws.cap_du; sq.cap_combine = 0; sq.cap_rows = 0;
  sq.header = (SchedHeader*)(base + ws.hdr_du); sq.items = (WorkItem*)(base + ws.items_du); sq.combine = nullptr;
  r.dx = sq;
  SchedParams& sk = r.dx;
  sk.mode = kSchedDkv; sk.tile_rows = kTile; sk.cap_items = ws.cap_dx;
  sk.header = (SchedHeader*)(base + ws.hdr_dx); sk.items = (WorkItem*)(base + ws.items_dx);
  return r;
}

template <typename T>
int launch_absorb_core_bwd(const AbsorbCoreBwdArgs& a, cudaStream_t s) {
  constexpr int D = 256;
  const int sms = resolve_sm_count_bwd(a.sm_count);
  const AbsorbBwdSched sch = absorb_bwd_sched_params(a, sms);
  const SchedParams& sq = sch.du;
  const SchedParams& sk = sch.dx;
  int rc;
  if (!a.lists_built && (rc = launch_scheduler_pair(sq, sk, s))) return rc;

  CUtensorMap u128, g128, x64, x128, u64, g64;
  if ((rc = encode_tmap_rows(&u128, a.u, a.dtype, a.total_q, a.H, D, kTile / a.H, a.H))) return rc;
  if ((rc = encode_tmap_rows(&g128, a.dax, a.dtype, a.total_q, a.H, D, kTile / a.H, a.H))) return rc;
  if ((rc = encode_tmap_rows(&x64, a.x, a.dtype, a.total_k, 1, a.x_width, kInner))) return rc;
  if ((rc = encode_tmap_rows(&x128, a.x, a.dtype, a.total_k, 1, a.x_width, kTile))) return rc;
  if ((rc = encode_tmap_rows(&u64, a.u, a.dtype, a.total_q, a.H, D, kInner / a.H, a.H))) return rc;
  if ((rc = encode_tmap_rows(&g64, a.dax, a.dtype, a.total_q, a.H, D, kInner / a.H, a.H))) return rc;

  BwdParams p;
  p.wait_limit = wait_limit_units();
  p.ld = (const float2*)a.ld; p.ld_stride = sm100_absorb_ld_pad((long long)a.total_q * a.H); p.H = a.H; p.scale = a.scale; p.scale_log2 = a.scale * kLog2e; p.status = a.status;
  p.out_width = a.x_width;
  p.trace = nullptr;
#ifdef VAFA_TRACE
  {
    static long long* g_trace = nullptr;  // debugging aid only
    if (!g_trace) cudaMalloc(&g_trace, 512 * 16 * sizeof(long long));
    cudaMemsetAsync(g_trace, 0, 512 * 16 * sizeof(long long), s);
    p.trace = g_trace;
    vafa_trace_buffer_abs = g_trace;
  }
#endif
  p.out1 = nullptr;
  if (a.which != 2) {
    p.out0 = a.du; p.header = sq.header; p.items = sq.items;
    const size_t smem = sizeof(BwdSmem<D, false, true>) + 1024;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd_kernel<T, D, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(kKAbsorbBwd, s);
    varlen_bwd_kernel<T, D, false, true><<<sms, kBwdThreads, smem, s>>>(u128, g128, x64, x64, p);
  }
  VAFA_LAUNCH_CHECK("varlen_bwd_kernel<absorb dU>");
  if (a.which != 1) {
    p.out0 = a.dx; p.header = sk.header; p.items = sk.items;
    const size_t smem = sizeof(BwdSmem<D, true, true>) + 1024;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd_kernel<T, D, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(kKAbsorbBwdDx, s);
    varlen_bwd_kernel<T, D, true, true><<<sms, kBwdThreads, smem, s>>>(x128, x128, u64, g64, p);
  }
  VAFA_LAUNCH_CHECK("varlen_bwd_kernel<absorb dX>");
  return 0;
}

}  // namespace

size_t sm100_absorb_core_bwd_workspace_bytes(int total_q, int total_k, int n_seg, int H) {
  return absorb_bwd_ws(total_q, total_k, n_seg, H).total;
}

int sm100_absorb_core_bwd_lists(const AbsorbCoreBwdArgs& a, cudaStream_t s) {
  const AbsorbBwdSched sch = absorb_bwd_sched_params(a, resolve_sm_count_bwd(a.sm_count));
  return launch_scheduler_pair(sch.du, sch.dx, s);
}

int sm100_absorb_core_bwd(const AbsorbCoreBwdArgs& a, cudaStream_t s) {
  return a.dtype == VAFA_BF16 ? launch_absorb_core_bwd<__nv_bfloat16>(a, s) : launch_absorb_core_bwd<__half>(a, s);
}

size_t sm100_absorb_ld_bytes(long long n_rows) { return (size_t)sm100_absorb_ld_pad(n_rows) * 16; }

int sm100_absorb_ld(const void* o, const void* d_o, const float* lse, void* ld, long long n_rows, int D_H, float scale, int dtype,
                    cudaStream_t s) {
  if (n_rows <= 0) return 0;
  const long long n_pad = sm100_absorb_ld_pad(n_rows);
  LaunchScope scope(kKBwdPre, s);
  const bool aligned = ((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o)) & 15) == 0;
  if (aligned && D_H >= 8 && D_H <= 256 && (D_H & (D_H - 1)) == 0) {
    int lanes_log2 = 0;
    while ((8 << lanes_log2) < D_H) ++lanes_log2;
    const unsigned vgrid = (unsigned)(((n_pad << lanes_log2) + 255) / 256);
    if (dtype == VAFA_BF16)
      absorb_ld_vec_kernel<__nv_bfloat16><<<vgrid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, lse, (float2*)ld, n_rows, n_pad, scale, lanes_log2);
    else
      absorb_ld_vec_kernel<__half><<<vgrid, 256, 0, s>>>((const __half*)o, (const __half*)d_o, lse, (float2*)ld, n_rows, n_pad, scale, lanes_log2);
    VAFA_LAUNCH_CHECK("absorb_ld_vec_kernel");
    return 0;
  }
  const unsigned grid = (unsigned)((n_pad + 255) / 256);
  if (dtype == VAFA_BF16)
    absorb_ld_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, lse, (float2*)ld, n_rows, n_pad, scale, D_H);
  else
    absorb_ld_kernel<__half><<<grid, 256, 0, s>>>((const __half*)o, (const __half*)d_o, lse, (float2*)ld, n_rows, n_pad, scale, D_H);
  VAFA_LAUNCH_CHECK("absorb_ld_kernel");
  return 0;
}

int sm100_absorb_expand_wv(const void* w_v, void* bexp, int H, int D_H, int d_kv, int dtype, cudaStream_t s) {
  LaunchScope scope(kKCast, s);
  if (dtype == VAFA_BF16)
    absorb_expand_wv_kernel<__nv_bfloat16><<<512, 256, 0, s>>>((const __nv_bfloat16*)w_v, (__nv_bfloat16*)bexp, H, D_H, d_kv);
  else
    absorb_expand_wv_kernel<__half><<<512, 256, 0, s>>>((const __half*)w_v, (__half*)bexp, H, D_H, d_kv);
  VAFA_LAUNCH_CHECK("absorb_expand_wv_kernel");
  return 0;
}

namespace {
}  // namespace

bool sm100_varlen_bwd_supported(const vafa_varlen_args* a) {
  if (!sm100_varlen_fwd_supported(a)) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(a->d_o) && al(a->dq) && al(a->dk) && al(a->dv);
}

size_t sm100_varlen_bwd_workspace_bytes(const vafa_varlen_args* a) {
  return bwd_workspace(a, resolve_sm_count_bwd(a->sm_count)).total;
}

int sm100_varlen_bwd(const vafa_varlen_args* a, cudaStream_t s) {
  if (a->dtype == VAFA_BF16) {
    return a->head_dim == 128 ? launch_bwd<__nv_bfloat16, 128>(a, s) : launch_bwd<__nv_bfloat16, 64>(a, s);
  }
  return a->head_dim == 128 ? launch_bwd<__half, 128>(a, s) : launch_bwd<__half, 64>(a, s);
}

}  // namespace vafa

#ifdef VAFA_TRACE
extern "C" __attribute__((visibility("default"))) int vafa_trace_read_abs(long long* host, int n) {
  if (!vafa::vafa_trace_buffer_abs) return -1;
  return (int)cudaMemcpy(host, vafa::vafa_trace_buffer_abs, (size_t)n * 16 * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif
