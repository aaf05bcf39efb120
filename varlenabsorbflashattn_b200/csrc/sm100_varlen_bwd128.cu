// Packed variable-length attention backward, 128 x 128 tiles (tcgen05 + TMA + TMEM).
//
// Same mathematics and the same two-kernel split as sm100_varlen_bwd.cu (dQ kernel per query tile,
// dK/dV kernel per key tile, no atomics), but the inner blocks are 128 rows: the score products
// run as M128 x N128 MMAs, which reach the full tensor rate (N = 64 MMAs measured 56 % of it), and
// every outer tile is read from shared memory half as often per inner row.
//
// TMEM (512 columns): X [0,128) and Y [128,256) fp32 scores (single buffered), ACC0 [256,384),
// ACC1 [384,512).
//   dQ : S = Q K^T -> X, dP = dO V^T -> Y; the element-wise warps write the 16-bit dS into one of
//        two 64-column buffers inside the ACC1 range (unused by dQ), so the next block's S/dP
//        MMAs are issued as soon as X/Y have been read, and dQ += dS K (from the dS buffer) runs
//        while the next block's element-wise work does.
//   dKV: S^T -> X, dP^T -> Y; P^T and dS^T overwrite the first halves of their own source chunks;
//        dV += P^T dO, dK += dS^T Q use all four regions, so the phases of a block run in sequence.
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

constexpr int kThreads = 320;  // 8 element-wise warps, 1 TMA warp, 1 MMA warp
constexpr int kIn = 128;       // rows per inner block
constexpr int kLdSlots = 132;  // staged (lse, delta) pairs per block: 128 + alignment slack, padded

template <int D>
struct Cfg128 {
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kSub = D / 64;
  static constexpr int kSubBytes = 128 * 128;  // 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;
  static constexpr uint32_t kX = 0, kY = 128, kAcc0 = 256, kAcc1 = 384;
};

template <int D>
struct Smem128 {
  alignas(1024) uint8_t outer_a[Cfg128<D>::kTileBytes];
  alignas(1024) uint8_t outer_b[Cfg128<D>::kTileBytes];
  alignas(1024) uint8_t inner_a[Cfg128<D>::kStages][Cfg128<D>::kTileBytes];
  alignas(1024) uint8_t inner_b[Cfg128<D>::kStages][Cfg128<D>::kTileBytes];
  alignas(8) uint64_t outer_full, outer_free;
  uint64_t in_full[Cfg128<D>::kStages], in_empty[Cfg128<D>::kStages];
  uint64_t xy_full, ds_full, acc_done;
  alignas(16) float2 ld[Cfg128<D>::kStages][kLdSlots];
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Smem128<128>) + 1024 <= 227 * 1024 && sizeof(Smem128<64>) + 1024 <= 227 * 1024, "shared memory budget");

struct Params128 {
  void* out0;        // dQ, or dV
  void* out1;        // unused, or dK
  const float2* ld;  // [H][ld_stride] (lse, or +inf for rows that saw no key; delta)
  long long ld_stride;
  const SchedHeader* header;
  const WorkItem* items;
  int H;
  float scale;
  float scale_log2;
  int32_t* status;
  long long* trace;
};

template <typename T, int D, bool kDKV>
__global__ void __launch_bounds__(kThreads, 1)
varlen_bwd128_kernel(const __grid_constant__ CUtensorMap tmap_outer_a, const __grid_constant__ CUtensorMap tmap_outer_b,
                     const __grid_constant__ CUtensorMap tmap_inner_a, const __grid_constant__ CUtensorMap tmap_inner_b,
                     const Params128 p) {
  using Cfg = Cfg128<D>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  Smem128<D>& sm = *reinterpret_cast<Smem128<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    wq_init(sm.wq, 9);
    mbar_init(smem_u32(&sm.outer_full), 1);
    mbar_init(smem_u32(&sm.outer_free), 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&sm.in_full[i]), 1);
      mbar_init(smem_u32(&sm.in_empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.xy_full), 1);
    mbar_init(smem_u32(&sm.ds_full), 256);
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

  if (warp == 8) {
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
        for (int b = 0; b < nb; ++b, ++gk) {
          const int st = gk % S;
          const uint32_t ph = (gk / S) & 1;
          const int row = w.i_start + b * kIn;
          if (!mbar_wait(smem_u32(&sm.in_empty[st]), ph ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.in_full[st]), 2 * Cfg::kTileBytes + (kDKV ? 130 * 8 : 0));
          if (kDKV) {
            // (lse, delta) of rows [row, row+128): start at the even index at or below `row` (16-byte
            // alignment), 130 pairs; readers skip (row & 1) slots
            const float2* src = p.ld + (long long)h * p.ld_stride + (row & ~1);
            bulk_load_1d(smem_u32(&sm.ld[st][0]), src, 130 * 8, smem_u32(&sm.in_full[st]));
          }
          for (int c = 0; c < Cfg::kSub; ++c) {
            tma_load_3d(smem_u32(sm.inner_a[st]) + c * Cfg::kSubBytes, &tmap_inner_a, smem_u32(&sm.in_full[st]), c * 64, h, row);
            tma_load_3d(smem_u32(sm.inner_b[st]) + c * Cfg::kSubBytes, &tmap_inner_b, smem_u32(&sm.in_full[st]), c * 64, h, row);
          }
        }
        ++qi;
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_xy = make_idesc(kFmt, 0, 0, 128, kIn);  // both operands K-major
      constexpr uint32_t idesc_acc = make_idesc(kFmt, 0, 1, 128, D);   // A from TMEM, B MN-major
      uint32_t gk = 0, qi = 0;
      bool alive = true;

      auto issue_xy = [&](uint32_t g, bool last) -> bool {
        const int st = g % S;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.in_full[st]), (g / S) & 1, abort_flag)) return false; TRACE_ADD(4); }
        tc_fence_after();
        TRACE_T0();
        const uint32_t oa_lo = desc_lo_sw128(smem_u32(sm.outer_a), 16), ob_lo = desc_lo_sw128(smem_u32(sm.outer_b), 16);
        const uint32_t ia_lo = desc_lo_sw128(smem_u32(sm.inner_a[st]), 16), ib_lo = desc_lo_sw128(smem_u32(sm.inner_b[st]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (Cfg::kSubBytes >> 4) + (kk & 3) * 2;  // 16-byte units
          mma_ss2(tbase + Cfg::kX, oa_lo + off, ia_lo + off, idesc_xy, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (Cfg::kSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(tbase + Cfg::kY, ob_lo + off, ib_lo + off, idesc_xy, kk > 0);
        }
        mma_commit(smem_u32(&sm.xy_full));
        if (last) mma_commit(smem_u32(&sm.outer_free));
        TRACE_ADD(6);
        return true;
      };
      auto issue_acc = [&](uint32_t g, bool first, bool last) {
        const int st = g % S;
        const uint32_t acc = first ? 0u : 1u;
        TRACE_T0();
        const uint32_t ma_lo = desc_lo_sw128(smem_u32(sm.inner_a[st]), Cfg::kSubBytes);
        const uint32_t mb_lo = desc_lo_sw128(smem_u32(sm.inner_b[st]), Cfg::kSubBytes);
        if (!kDKV) {
          // dQ += dS . K_g   (dS: 16-bit, contiguous in its buffer; K block MN-major)
          const uint32_t ds_tmem = tbase + Cfg::kAcc1 + (g & 1) * 64;
#pragma unroll
          for (int kk = 0; kk < kIn / 16; ++kk)
            mma_ts2(tbase + Cfg::kAcc0, ds_tmem + kk * 8, ma_lo + kk * (2048 >> 4), idesc_acc, (acc | (kk > 0)) ? 1u : 0u);
        } else {
          // dV += P^T . dO_g ;  dK += dS^T . Q_g   (K-step kk sits at column (kk/2)*32 + (kk%2)*8)
#pragma unroll
          for (int kk = 0; kk < kIn / 16; ++kk)
            mma_ts2(tbase + Cfg::kAcc0, tbase + Cfg::kX + (kk >> 1) * 32 + (kk & 1) * 8, mb_lo + kk * (2048 >> 4), idesc_acc,
                    (acc | (kk > 0)) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < kIn / 16; ++kk)
            mma_ts2(tbase + Cfg::kAcc1, tbase + Cfg::kY + (kk >> 1) * 32 + (kk & 1) * 8, ma_lo + kk * (2048 >> 4), idesc_acc,
                    (acc | (kk > 0)) ? 1u : 0u);
        }
        mma_commit(smem_u32(&sm.in_empty[st]));
        if (last) mma_commit(smem_u32(&sm.acc_done));
        TRACE_ADD(7);
      };

      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_consume_thread(sm.wq, n, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const int nb = (w.i_len + kIn - 1) / kIn;
        if (nb == 0) continue;
        if (!mbar_wait(smem_u32(&sm.outer_full), qi & 1, abort_flag)) break;
        tc_fence_after();
        if (!issue_xy(gk, nb == 1)) break;
        for (int b = 0; b < nb; ++b) {
          const uint32_t g = gk + b;
          // the element-wise warps have read X/Y of block g and written dS (or P^T, dS^T)
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.ds_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(5); }
          tc_fence_after();
          if (!kDKV) {
            // X/Y are free again: next scores first, then this block's dQ product overlaps the
            // element-wise work on those scores
            if (b + 1 < nb && !issue_xy(g + 1, b + 2 == nb)) { alive = false; break; }
            issue_acc(g, b == 0, b + 1 == nb);
          } else {
            issue_acc(g, b == 0, b + 1 == nb);
            if (b + 1 < nb && !issue_xy(g + 1, b + 2 == nb)) { alive = false; break; }
          }
        }
        gk += nb;
        ++qi;
      }
    }
  } else {
    // ---------------- element-wise warps + epilogue (warps 0-7) ----------------
    // thread -> outer row r = tid % 128 (TMEM lane; a warp may only touch lane quadrant warp % 4);
    // warps 0-3 take inner columns [0,64) of every block, warps 4-7 columns [64,128)
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const float c = p.scale_log2;
    uint32_t gk = 0, qi = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int h = w.head;
      const int nb = (w.i_len + kIn - 1) / kIn;
      const bool row_ok = r < w.o_rows;
      float my_lse = INFINITY, my_delta = 0.f;
      if (!kDKV && row_ok && nb > 0) {
        const float2 t = p.ld[(long long)h * p.ld_stride + w.o_start + r];
        my_lse = t.x;
        my_delta = t.y;
      }

      for (int b = 0; b < nb; ++b) {
        const uint32_t g = gk + b;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.xy_full), g & 1, abort_flag)) { alive = false; break; } TRACE_ADD(8); }
        tc_fence_after();
#ifdef VAFA_TRACE
        const long long t_c0 = clock64();
#endif
        // visibility of inner index jj = b*128 + col for this thread's outer row r
        //   dQ : jj < i_len and (causal) jj <= r + diag
        //   dKV: jj < i_len and (causal) jj >= r + diag
        int lo = 0, hi = w.i_len - 1 - b * kIn;
        if (w.masked) {
          if (!kDKV) hi = min(hi, r + w.diag - b * kIn);
          else lo = r + w.diag - b * kIn;
        }
        const bool need_mask = (hi < kIn - 1) || (lo > 0);
        const int st = g % S;
        const int ld_skip = (w.i_start + b * kIn) & 1;
        if (kDKV) {
          // the staged (lse, delta) block arrived with this stage's tiles (complete by now; the wait
          // orders the reads below after the copy)
          if (!mbar_wait(smem_u32(&sm.in_full[st]), (g / S) & 1, abort_flag)) { alive = false; break; }
        }
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int chunk = half * 2 + q2;  // 32-column chunk of the block
          uint32_t xs[32], ys[32];
          tmem_ld32(lane_base + Cfg::kX + chunk * 32, xs);
          tmem_ld32(lane_base + Cfg::kY + chunk * 32, ys);
          tmem_wait_ld();
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float pv[2], dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = chunk * 32 + i + e;
              float lse_v, delta_v;
#ifdef VAFA_EXP_NOLDS
              if (false) {
#else
              if (kDKV) {
#endif
                const float2 t = sm.ld[st][ld_skip + col];
                lse_v = t.x;
                delta_v = t.y;
              } else {
                lse_v = my_lse;
                delta_v = my_delta;
              }
              float pr = ex2(fmaf(__uint_as_float(xs[i + e]), c, -lse_v));
              float ds = pr * (__uint_as_float(ys[i + e]) - delta_v);
              if (need_mask) {
                const bool vis = (col >= lo) && (col <= hi);
                pr = vis ? pr : 0.f;
                ds = vis ? ds : 0.f;
              }
              pv[e] = pr;
              dv[e] = ds;
            }
            pp[i >> 1] = pack2<T>(pv[0], pv[1]);
            dd[i >> 1] = pack2<T>(dv[0], dv[1]);
          }
          if (!kDKV) {
            // dS buffer (g & 1) inside the ACC1 range, packed contiguously: chunk -> 16 columns
            tmem_st16(lane_base + Cfg::kAcc1 + (g & 1) * 64 + chunk * 16, dd);
          } else {
            // in place: 16 packed columns over the first half of the chunk just read
            tmem_st16(lane_base + Cfg::kX + chunk * 32, pp);
            tmem_st16(lane_base + Cfg::kY + chunk * 32, dd);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sm.ds_full));
#ifdef VAFA_TRACE
        tr[10] += clock64() - t_c0;
        tr[11] += 1;
#endif
      }
      if (!alive) break;
      gk += nb;

      // ---- epilogue: each half of the warps converts and stores half of the columns ----
      if (nb > 0) {
        if (!mbar_wait(smem_u32(&sm.acc_done), qi & 1, abort_flag)) break;
        tc_fence_after();
        ++qi;
      }
      const long long out_row = ((long long)w.o_start + r) * p.H + h;
#pragma unroll
      for (int which = 0; which < (kDKV ? 2 : 1); ++which) {
        T* optr = reinterpret_cast<T*>(which == 0 ? p.out0 : p.out1) + out_row * D;
        const float mul = (kDKV && which == 0) ? 1.f : p.scale;  // dV unscaled; dQ and dK scaled
        const uint32_t acc_col = which == 0 ? Cfg::kAcc0 : Cfg::kAcc1;
#pragma unroll
        for (int c2 = 0; c2 < D / 64; ++c2) {
          const int cc = half * (D / 64) + c2;
          uint32_t t[32];
          if (nb > 0) {
            tmem_ld32(lane_base + acc_col + cc * 32, t);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = 0u;
          }
          if (row_ok) {
            uint4* dst = reinterpret_cast<uint4*>(optr + cc * 32);
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              uint4 u;
              u.x = pack2<T>(__uint_as_float(t[8 * v4 + 0]) * mul, __uint_as_float(t[8 * v4 + 1]) * mul);
              u.y = pack2<T>(__uint_as_float(t[8 * v4 + 2]) * mul, __uint_as_float(t[8 * v4 + 3]) * mul);
              u.z = pack2<T>(__uint_as_float(t[8 * v4 + 4]) * mul, __uint_as_float(t[8 * v4 + 5]) * mul);
              u.w = pack2<T>(__uint_as_float(t[8 * v4 + 6]) * mul, __uint_as_float(t[8 * v4 + 7]) * mul);
              dst[v4] = u;
            }
          }
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
  if (warp == 9) tmem_dealloc(tbase, 512);
}

}  // namespace

#ifdef VAFA_TRACE
long long* vafa_trace_buffer_bwd = nullptr;
#endif

template <typename T, int D>
static int launch128(const Bwd128Launch& L, cudaStream_t s) {
  Params128 p;
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
  const size_t smem = sizeof(Smem128<D>) + 1024;
  CUtensorMap q128, do128, k128, v128;
  int rc;
  if ((rc = encode_tmap_rows(&q128, L.q, L.dtype, L.total_q, L.H, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&do128, L.d_o, L.dtype, L.total_q, L.H, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&k128, L.k, L.dtype, L.total_k, L.H, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&v128, L.v, L.dtype, L.total_k, L.H, D, 128))) return rc;
  if (L.run_dq) {
  // dQ: outer = (Q, dO) tiles, inner = (K, V) blocks
  p.out0 = L.dq; p.out1 = nullptr; p.header = (const SchedHeader*)L.hdr_dq; p.items = (const WorkItem*)L.items_dq;
  VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd128_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    LaunchScope scope(kKBwdDq, s);
    varlen_bwd128_kernel<T, D, false><<<L.sms, kThreads, smem, s>>>(q128, do128, k128, v128, p);
  }
  VAFA_LAUNCH_CHECK("varlen_bwd128_kernel<dQ>");
  }
  if (!L.run_dkv) return 0;
  // dK/dV: outer = (K, V) tiles, inner = (Q, dO) blocks
  p.out0 = L.dv; p.out1 = L.dk; p.header = (const SchedHeader*)L.hdr_dkv; p.items = (const WorkItem*)L.items_dkv;
  VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_bwd128_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    LaunchScope scope(kKBwdDkv, s);
    varlen_bwd128_kernel<T, D, true><<<L.sms, kThreads, smem, s>>>(k128, v128, q128, do128, p);
  }
  VAFA_LAUNCH_CHECK("varlen_bwd128_kernel<dKV>");
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
