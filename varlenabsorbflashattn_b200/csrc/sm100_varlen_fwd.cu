// Packed variable-length attention forward for sm_100a: TMA -> shared memory -> tcgen05.mma
// with TMEM accumulators, online softmax in registers, split-K partials + LSE combine.
//
// One persistent CTA per SM, 10 warps:
//   warps 0-7  softmax + epilogue: two threads per query row of the 128-row tile (TMEM lane = row),
//              each owning half of the score and output columns
//   warp 8     TMA producer (one lane): Q tile once per item, K and V tiles through a ring
//   warp 9     tcgen05.mma issuer (one lane) and TMEM owner
// TMEM (512 columns): S0 [0,128), S1 [128,256) fp32 scores, double buffered; the 16-bit
// probabilities P overwrite the first 64 columns of their S buffer; O accumulator at [256,256+D).
//
// Per KV block g:  S[g&1] = Q K_g^T  ->  softmax warps read S, write P, rescale O when the
// running maximum moved by more than 2^8  ->  O += P V_g.  S for block g+1 is issued before
// block g's P is ready, so the tensor pipe works on the next scores while the softmax runs.
//
// Numerics follow the reference kernels (triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:
// 127-166): scores scaled by scale*log2(e) in fp32 after the dot, exp2-domain online softmax,
// P rounded to the I/O dtype before P.V, fp32 row sums from the unrounded P, O = acc / l,
// LSE = m + log2(l).
#include <cuda.h>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "sm100_common.cuh"
#include "sm100_kernels.cuh"
#include "profile.cuh"

namespace vafa {
namespace {

using namespace ptx;

// Optional wait-time tracing (build with -DVAFA_TRACE): per CTA, cycles each role spent waiting on
// each barrier, written to FwdParams::trace[cta][16].
#ifdef VAFA_TRACE
#define TRACE_T0() const long long _t0 = clock64()
#define TRACE_ADD(slot) tr[slot] += clock64() - _t0
#else
#define TRACE_T0()
#define TRACE_ADD(slot)
#endif

constexpr int kFwdThreads = 320;  // 8 softmax warps, 1 TMA warp, 1 MMA warp
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef VAFA_FWD_POLY_PERIOD
#define VAFA_FWD_POLY_PERIOD 4
#endif
constexpr int kPolyPeriod = VAFA_FWD_POLY_PERIOD;  // one pair of exponentials in this many runs as a polynomial on the FMA pipe

// Rounding of P to the I/O type.  The forward takes a quarter of its exponentials off the special-function pipe
// (polynomial), so the conversion instruction has room there and relieves the integer pipe of two adds and a
// byte permute per pair of scores: 2-3 % faster than pack2 (measured; in the backward kernels, whose
// exponentials all run on that pipe, the two are level and pack2 stays).  -DVAFA_FWD_INT_PACK restores pack2.
template <typename T>
__device__ __forceinline__ uint32_t pack_p(float lo, float hi) {
#ifdef VAFA_FWD_INT_PACK
  return pack2<T>(lo, hi);
#else
  return pack2_out<T>(lo, hi);
#endif
}

template <int D>
struct FwdCfg {
  // two stages: K slot g&1 is free again when S(g) is complete and V slot g&1 when P.V(g) is, so
  // the producer waits on the very barriers the softmax warps use and the MMA issuer needs only two
  // tcgen05.commit per block (each commit costs the tensor pipe 40-130 cycles)
  static constexpr int kStages = 2;
  static constexpr int kSub = D / 64;                 // 64-column (128-byte) sub tiles per row
  static constexpr int kSubBytes = 128 * 128;         // one sub tile: 128 rows x 128 B
  static constexpr int kTileBytes = kSub * kSubBytes;
  static constexpr uint32_t kTmemCols = 512;
  static constexpr uint32_t kOCol = 256;
};

// Keys per block and ring depth of the key tiles.  The absorb operator's X tile serves both products of
// its block, so its slot is held from the load to the end of P.X; with 128-key blocks (64 KB) only two
// slots fit beside the 64 KB query tile and a load could start only when the block two back had finished.
// Blocks of 96 keys (48 KB) leave room for three slots.
template <bool kAbsorb> constexpr int fwd_block_keys() { return kAbsorb ? 96 : kTile; }
template <bool kAbsorb> constexpr int fwd_key_stages() { return kAbsorb ? 3 : 2; }

// kAbsorb: keys and values are the same rows (the absorb operator attends over raw X), so there
// is one ring and no V tiles.
template <int D, bool kAbsorb = false>
struct FwdSmem {
  alignas(1024) uint8_t q[FwdCfg<D>::kTileBytes];
  alignas(1024) uint8_t k[fwd_key_stages<kAbsorb>()][FwdCfg<D>::kSub * fwd_block_keys<kAbsorb>() * 128];
  alignas(1024) uint8_t v[kAbsorb ? 1 : FwdCfg<D>::kStages][kAbsorb ? 1024 : FwdCfg<D>::kTileBytes];
  alignas(8) uint64_t q_full, q_free;
  uint64_t k_full[3], v_full[2];
  uint64_t s_full[2], p_full[2];  // indexed by block parity; phase = (block / 2) & 1
  uint64_t o_done[3];             // P.V of block g complete: index g % stages, phase (g / stages) & 1; it also
                                  // frees the V slot (absorb: the X slot) of the block
  uint64_t pair_bar[4];       // the two softmax warps of one TMEM lane quadrant
  float xmax[2][2][128];      // [block parity][half][row] partial row maxima
  float xsum[2][128];         // [half][row] partial row sums at the end of an item
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};

static_assert(sizeof(FwdSmem<128>) + 1024 <= 227 * 1024 && sizeof(FwdSmem<64>) + 1024 <= 227 * 1024 &&
                  sizeof(FwdSmem<256, true>) + 1024 <= 227 * 1024,
              "shared memory budget");

struct FwdParams {
  void* o;
  float* lse;
  float* partial_o;
  float* partial_lse;
  const SchedHeader* header;
  const WorkItem* items;
  int H;
  int group;  // query heads per K/V head (1 = one K/V head per query head)
  float scale_log2;
  int32_t* status;
  int wait_limit;  // bound of every device-side wait, in units of 65536 cycles
  long long* trace;
};

// kAbsorb = false: one item = one 128-row query tile of one head (grid of items x heads).
// kAbsorb = true : one item = 128/H query rows of one user with all H heads stacked into the 128
//   tile rows (row = q*H + h, the order the 64 x H x (128/H) TMA box delivers), K = V = the user's X
//   rows (one tile serves Q.X^T as a K-major operand and P.X as an MN-major operand), D = d_kv.
template <typename T, int D, bool kAbsorb>
__global__ void __launch_bounds__(kFwdThreads, 1)
varlen_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int S = fwd_key_stages<kAbsorb>();
  constexpr int kBlk = fwd_block_keys<kAbsorb>();   // keys per block
  constexpr int kHalf = kBlk / 2;                   // score columns per softmax thread
  constexpr int kKSubBytes = kBlk * 128;            // one 64-column sub tile of a key tile
  constexpr int kKTileBytes = Cfg::kSub * kKSubBytes;
  extern __shared__ uint8_t smem_raw[];
  using Smem = FwdSmem<D, kAbsorb>;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    wq_init(sm.wq, 9);
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&sm.pair_bar[i]), 64);
    mbar_init(smem_u32(&sm.q_full), 1);
    mbar_init(smem_u32(&sm.q_free), 1);
    for (int i = 0; i < S; ++i) {
      mbar_init(smem_u32(&sm.k_full[i]), 1);
      mbar_init(smem_u32(&sm.o_done[i]), 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&sm.v_full[i]), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.s_full[i]), 1);
      mbar_init(smem_u32(&sm.p_full[i]), 8);  // lane 0 of each softmax warp
    }
    fence_barrier_init();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
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
  const int total = max(n_items, 0);  // the item list already holds one entry per head
  int* const next_item = const_cast<int*>(&p.header->next_item);
  if (n_items < 0 && threadIdx.x == 0) report_error(p.status, 2, 100, n_items);
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
        const int hk = kAbsorb ? h : h / p.group;  // K/V head of this query head
        const int nb = (w.i_len + kBlk - 1) / kBlk;
        if (nb == 0) continue;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.q_free), (qi & 1) ^ 1, abort_flag)) break; TRACE_ADD(0); }
        mbar_expect_tx(smem_u32(&sm.q_full), Cfg::kTileBytes);
        for (int c = 0; c < Cfg::kSub; ++c)
          tma_load_3d(smem_u32(sm.q) + c * Cfg::kSubBytes, &tmap_q, smem_u32(&sm.q_full), c * 64, h, w.o_start);
        // absorb: X is streamed once from HBM (no other CTA reads this user's keys), and a K slot is only
        // released after P.X of its block, so the two-slot ring alone leaves the HBM latency exposed
        // (measured: the MMA issuer waited for tiles half of the time).  Tiles a few blocks ahead are
        // therefore pulled into L2 first.
        constexpr int kPrefetch = 4;
        if (kAbsorb)
          for (int b = 2; b < kPrefetch && b < nb; ++b)
            for (int c = 0; c < Cfg::kSub; ++c) tma_prefetch_3d(&tmap_k, c * 64, hk, w.i_start + b * kBlk);
        for (int b = 0; b < nb; ++b, ++gk) {
          const int st = gk % S;
          const uint32_t ph = (gk / S) & 1;
          const int row = w.i_start + b * kBlk;
          if (kAbsorb && b + kPrefetch < nb)
            for (int c = 0; c < Cfg::kSub; ++c) tma_prefetch_3d(&tmap_k, c * 64, hk, row + kPrefetch * kBlk);
          // slot free: S(gk-2) complete (absorb: P.X(gk-3) complete, the tile doubles as V)
          { TRACE_T0(); if (!mbar_wait(smem_u32(kAbsorb ? &sm.o_done[st] : &sm.s_full[st]), ph ^ 1, abort_flag)) { alive = false; break; } TRACE_ADD(1); }
          mbar_expect_tx(smem_u32(&sm.k_full[st]), kKTileBytes);
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.k[st]) + c * kKSubBytes, &tmap_k, smem_u32(&sm.k_full[st]), c * 64, hk, row);
          if (!kAbsorb) {
            { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.o_done[st]), ph ^ 1, abort_flag)) { alive = false; break; } TRACE_ADD(2); }
            mbar_expect_tx(smem_u32(&sm.v_full[st]), Cfg::kTileBytes);
            for (int c = 0; c < Cfg::kSub; ++c)
              tma_load_3d(smem_u32(sm.v[st]) + c * Cfg::kSubBytes, &tmap_v, smem_u32(&sm.v_full[st]), c * 64, hk, row);
          }
        }
        ++qi;
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_qk = make_idesc(kFmt, 0, 0, 128, kBlk);
      constexpr uint32_t idesc_pv = make_idesc(kFmt, 0, 1, 128, D);
      uint32_t gk = 0, qi = 0;
      bool alive = true;

      auto issue_qk = [&](uint32_t g, bool last) -> bool {
        const int st = g % S;
        const uint32_t ph = (g / S) & 1;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.k_full[st]), ph, abort_flag)) return false; TRACE_ADD(4); }
        tc_fence_after();
        const uint32_t d_tmem = tbase + (g & 1) * 128;
        const uint32_t q_lo = desc_lo_sw128(smem_u32(sm.q), 16), k_lo = desc_lo_sw128(smem_u32(sm.k[st]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          // in 16-byte units: 64-column sub tiles are a whole sub tile apart, 16 columns are 32 bytes
          const uint32_t off_q = (kk >> 2) * (Cfg::kSubBytes >> 4) + (kk & 3) * 2;
          const uint32_t off_k = (kk >> 2) * (kKSubBytes >> 4) + (kk & 3) * 2;
          mma_ss2(d_tmem, q_lo + off_q, k_lo + off_k, idesc_qk, kk > 0);
        }
        mma_commit(smem_u32(&sm.s_full[g & 1]));
        if (last) mma_commit(smem_u32(&sm.q_free));
        return true;
      };

      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_consume_thread(sm.wq, n, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const int nb = (w.i_len + kBlk - 1) / kBlk;
        if (nb == 0) continue;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.q_full), qi & 1, abort_flag)) break; TRACE_ADD(3); }
        tc_fence_after();
        if (!issue_qk(gk, nb == 1)) break;
        for (int b = 0; b < nb; ++b) {
          const uint32_t g = gk + b;
          const int st = g % S;
          const uint32_t ph = (g / S) & 1;
          bool qk_pending = b + 1 < nb, qk_first = true;
          if (kAbsorb && qk_pending) {
            // The X tile of block g+1 is only requested once P.X of block g-1 has released its slot, so it
            // can still be on its way when P of block g is ready.  Waiting for it here would put the load
            // latency in series with both products of every block (measured: half of this thread's time):
            // the product whose operands are there first is issued first.
            TRACE_T0();
            const int first = mbar_wait_either(smem_u32(&sm.k_full[(g + 1) % S]), ((g + 1) / S) & 1,
                                               smem_u32(&sm.p_full[g & 1]), (g >> 1) & 1, abort_flag);
            TRACE_ADD(7);
            if (first == 0) { alive = false; break; }
            qk_first = first == 1;
          }
          if (qk_pending && qk_first) {
            if (!issue_qk(g + 1, b + 2 == nb)) { alive = false; break; }
            qk_pending = false;
          }
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.p_full[g & 1]), (g >> 1) & 1, abort_flag)) { alive = false; break; } TRACE_ADD(5); }
          if (!kAbsorb) { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.v_full[st]), ph, abort_flag)) { alive = false; break; } TRACE_ADD(6); }
          tc_fence_after();
          const uint32_t a_tmem = tbase + (g & 1) * 128;
          // V tile: [keys][D] as D/64 sub tiles; 16 keys = 2 KB; sub tiles one sub tile apart (the LBO)
          const uint32_t v_lo = desc_lo_sw128(smem_u32(kAbsorb ? sm.k[st] : sm.v[st]), kKSubBytes);
          // P: each softmax thread packed its kHalf columns into the first kHalf/2 of them, so K-step kk
          // (16 keys = 8 packed columns) sits at column (kk / steps_per_half) * kHalf + (kk % steps_per_half) * 8
          constexpr int kStepsPerHalf = kHalf / 16;
#pragma unroll
          for (int kk = 0; kk < kBlk / 16; ++kk)
            mma_ts2(tbase + Cfg::kOCol, a_tmem + (kk / kStepsPerHalf) * kHalf + (kk % kStepsPerHalf) * 8, v_lo + kk * (2048 >> 4),
                    idesc_pv, (b > 0 || kk > 0) ? 1u : 0u);
          mma_commit(smem_u32(&sm.o_done[st]));
          if (qk_pending && !issue_qk(g + 1, b + 2 == nb)) { alive = false; break; }
        }
        gk += nb;
        ++qi;
      }
    }
  } else {
    // ---------------- softmax + epilogue (warps 0-7) ----------------
    // Two threads per tile row: thread (r, half) owns score columns [64*half, 64*half+64) of every
    // block and output columns [D/2*half, D/2*(half+1)).  The two halves of a row sit in warps w and
    // w+4 (same TMEM lane quadrant) and exchange their partial row maximum through shared memory;
    // two warps per scheduler also give the exp2-heavy loop a second instruction stream to overlap.
    const int r = threadIdx.x & 127;
    const int half = threadIdx.x >> 7;
    const uint32_t pair_bar = smem_u32(&sm.pair_bar[warp & 3]);
    uint32_t pair_cnt = 0;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const float c = p.scale_log2;
    uint32_t gk = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const int nb = (w.i_len + kBlk - 1) / kBlk;
      // tile row r -> (query row of the tile, head)
      const int rq = kAbsorb ? r / p.H : r;
      const int h = kAbsorb ? r % p.H : w.head;
      const bool row_ok = rq < w.o_rows;
      float m_ref = -INFINITY, l = 0.f;  // l: sum over this thread's columns only

      for (int b = 0; b < nb; ++b) {
        const uint32_t g = gk + b;
        { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.s_full[g & 1]), (g >> 1) & 1, abort_flag)) { alive = false; break; } TRACE_ADD(8); }
        tc_fence_after();
#ifdef VAFA_TRACE
        const long long t_sm0 = clock64();
#endif
        const uint32_t s_addr = lane_base + (g & 1) * 128 + half * kHalf;
        float s[kHalf];
        if constexpr (kHalf == 64) {
          uint32_t t0[64];
          tmem_ld64(s_addr, t0);
          { TRACE_T0(); tmem_wait_ld(); TRACE_ADD(13); }
#pragma unroll
          for (int i = 0; i < 64; ++i) s[i] = __uint_as_float(t0[i]);
        } else {
          static_assert(kHalf == 64 || kHalf == 48, "score columns per thread");
          uint32_t t0[32], t1[16];
          tmem_ld32(s_addr, t0);
          tmem_ld16(s_addr + 32, t1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(t0[i]);
#pragma unroll
          for (int i = 0; i < 16; ++i) s[32 + i] = __uint_as_float(t1[i]);
        }
        // mask: inner index jj = b*kBlk + col is visible iff jj < i_len and (causal) jj <= r + diag
        const int lim_tail = w.i_len - 1 - b * kBlk;
        const int lim_diag = w.masked ? (w.diag - b * kBlk) : 0x3fffffff;  // for row 0
        const bool masked_block = lim_tail < kBlk - 1 || lim_diag < kBlk - 1;  // same for the whole CTA
        if (masked_block) {
          const int lim = min(lim_tail, w.masked ? lim_diag + r : 0x3fffffff) - half * kHalf;
#pragma unroll
          for (int i = 0; i < kHalf; ++i) s[i] = (i <= lim) ? s[i] : -INFINITY;
        }
        // row maximum of this half: eight independent chains of 3-input max
        float m8[8];
#pragma unroll
        for (int j2 = 0; j2 < 8; ++j2) m8[j2] = max3(s[j2], s[8 + j2], s[16 + j2]);
#pragma unroll
        for (int i = 24; i + 16 <= kHalf; i += 16) {
#pragma unroll
          for (int j2 = 0; j2 < 8; ++j2) m8[j2] = max3(m8[j2], s[i + j2], s[i + 8 + j2]);
        }
        // 24 + 16k columns done; one more group of eight is left for both 64 and 48 columns
#pragma unroll
        for (int j2 = 0; j2 < 8; ++j2) m8[j2] = fmaxf(m8[j2], s[kHalf - 8 + j2]);
        float mx = max3(max3(m8[0], m8[1], m8[2]), max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
        // combine with the other half of the row
        sm.xmax[g & 1][half][r] = mx;
        mbar_arrive(pair_bar);
        { TRACE_T0(); if (!mbar_wait(pair_bar, pair_cnt & 1, abort_flag)) { alive = false; break; } TRACE_ADD(12); }
        ++pair_cnt;
        mx = fmaxf(mx, sm.xmax[g & 1][half ^ 1][r]);
        const float m_blk = mx * c;  // c > 0
        float m_new = fmaxf(m_ref, m_blk);
        const bool resc = m_new > m_ref + kRescaleThreshold;
        if (!resc) m_new = m_ref;
        const float alpha = resc ? ex2(m_ref - m_new) : 1.f;
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        // exponents and row sums in packed pairs (one FMA-pipe instruction for two values); in unmasked
        // blocks every kPolyPeriod-th pair takes the polynomial 2^t instead of the special-function unit
        // (16 results/clk/SM).  Masked blocks keep the unit for all: it returns exactly 0 for -inf, which
        // the dead-row test (row sum == 0) relies on.
        const uint64_t cs2 = pack_f2(c, c), nm2 = pack_f2(-m_use, -m_use);
        uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
        uint32_t pk[kHalf / 2];
        auto exps = [&](auto poly_tag) {
          constexpr bool kPoly = decltype(poly_tag)::value;
#pragma unroll
          for (int i = 0; i < kHalf / 2; ++i) {
            const uint64_t t2 = fma_f2(pack_f2(s[2 * i], s[2 * i + 1]), cs2, nm2);
            float p0, p1;
            if (kPoly && (i % kPolyPeriod == kPolyPeriod - 1)) {
              ex2_poly2(t2, p0, p1);
            } else {
              float t0, t1;
              unpack_f2(t2, t0, t1);
              p0 = ex2(t0);
              p1 = ex2(t1);
            }
            sum2[i & 3] = add_f2(sum2[i & 3], pack_f2(p0, p1));
            pk[i] = pack_p<T>(p0, p1);
          }
        };
        if (masked_block) exps(std::false_type{}); else exps(std::true_type{});
        {
          float a0, a1, b0, b1;
          unpack_f2(add_f2(sum2[0], sum2[1]), a0, a1);
          unpack_f2(add_f2(sum2[2], sum2[3]), b0, b1);
          l = l * alpha + ((a0 + a1) + (b0 + b1));
        }
        m_ref = m_new;
        // kHalf probabilities -> kHalf/2 packed columns over the first half of the columns just read
        // (the MMA issuer's addressing of the K-steps is next to its P.V loop)
        if constexpr (kHalf == 64) {
          tmem_st32(s_addr, pk);
        } else {
          uint32_t pa[16], pb[8];
#pragma unroll
          for (int i = 0; i < 16; ++i) pa[i] = pk[i];
#pragma unroll
          for (int i = 0; i < 8; ++i) pb[i] = pk[16 + i];
          tmem_st16(s_addr, pa);
          tmem_st8(s_addr + 16, pb);
        }
        if (b > 0 && __any_sync(0xffffffffu, resc)) {
#ifdef VAFA_TRACE
          tr[10] += clock64() - t_sm0;
#endif
          // O may be rescaled once P.V of the previous block is complete (the next one waits for this
          // warp's arrival below).  No alias in the parity wait: S(g) complete implies P.V(g-2) complete.
          { TRACE_T0(); if (!mbar_wait(smem_u32(&sm.o_done[(g - 1) % S]), ((g - 1) / S) & 1, abort_flag)) { alive = false; break; } TRACE_ADD(9); }
          tc_fence_after();
          {
#pragma unroll
            for (int c2 = 0; c2 < D / 64; ++c2) {
              const int cc = half * (D / 64) + c2;
              uint32_t t[32];
              tmem_ld32(lane_base + Cfg::kOCol + cc * 32, t);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
              tmem_st32(lane_base + Cfg::kOCol + cc * 32, t);
            }
          }
        }
        { TRACE_T0(); tmem_wait_st(); TRACE_ADD(14); }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.p_full[g & 1]));
#ifdef VAFA_TRACE
        tr[11] += 1;
#endif
      }
      if (!alive) break;
      gk += nb;

      // ---- epilogue ----
      float l_tot = 0.f;
      if (nb > 0) {
        if (!mbar_wait(smem_u32(&sm.o_done[(gk - 1) % S]), ((gk - 1) / S) & 1, abort_flag)) break;
        tc_fence_after();
        sm.xsum[half][r] = l;
        mbar_arrive(pair_bar);
        if (!mbar_wait(pair_bar, pair_cnt & 1, abort_flag)) break;
        ++pair_cnt;
        l_tot = l + sm.xsum[half ^ 1][r];
      }
      const bool dead = (nb == 0) || (l_tot == 0.f);  // a NaN row sum is not a dead row: it goes out as NaN
      const float inv_l = dead ? 0.f : 1.f / l_tot;
      const float lse_val = dead ? -INFINITY : m_ref + log2f(l_tot);
      if (w.partial < 0) {
        const long long row = (long long)w.o_start + rq;
        T* optr = reinterpret_cast<T*>(p.o) + (row * p.H + h) * D;
#pragma unroll
        for (int c2 = 0; c2 < D / 64; ++c2) {
          const int cc = half * (D / 64) + c2;
          uint32_t t[32];
          if (nb > 0) {
            tmem_ld32(lane_base + Cfg::kOCol + cc * 32, t);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = 0u;
          }
          uint32_t pw[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pw[i] = pack2_out<T>(__uint_as_float(t[2 * i]) * inv_l, __uint_as_float(t[2 * i + 1]) * inv_l);
          // rows of the tile are consecutive (token, head) rows of O: H*D apart (absorb: D apart)
          store_chunk_coalesced<T>(pw, optr + cc * 32, kAbsorb ? (long long)D : (long long)p.H * D, r,
                                   kAbsorb ? w.o_rows * p.H : w.o_rows, 4);
        }
        if (row_ok && half == 0) p.lse[row * p.H + h] = lse_val;
      } else {
        const long long prow = (long long)w.partial + rq;
        float* optr = p.partial_o + (prow * p.H + h) * D;
#pragma unroll
        for (int c2 = 0; c2 < D / 64; ++c2) {
          const int cc = half * (D / 64) + c2;
          uint32_t t[32];
          if (nb > 0) {
            tmem_ld32(lane_base + Cfg::kOCol + cc * 32, t);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = 0u;
          }
          if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(optr + cc * 32);
#pragma unroll
            for (int v4 = 0; v4 < 8; ++v4) {
              float4 f;
              f.x = __uint_as_float(t[4 * v4 + 0]) * inv_l;
              f.y = __uint_as_float(t[4 * v4 + 1]) * inv_l;
              f.z = __uint_as_float(t[4 * v4 + 2]) * inv_l;
              f.w = __uint_as_float(t[4 * v4 + 3]) * inv_l;
              dst[v4] = f;
            }
          }
        }
        if (row_ok && half == 0) p.partial_lse[prow * p.H + h] = lse_val;
      }
      // the TMEM reads of O above finish (tcgen05.wait::ld) before this thread's next p_full arrival,
      // and the next item's first P.V, which overwrites O, is issued only after that arrival
    }
  }

#ifdef VAFA_TRACE
  if (p.trace != nullptr && (threadIdx.x == 0 || threadIdx.x == 256 || threadIdx.x == 288)) {
    tr[15] = clock64() - t_begin;
    for (int i = 0; i < 16; ++i)
      if (tr[i] != 0) p.trace[(long long)blockIdx.x * 16 + i] = tr[i];
  }
#endif
  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    if (threadIdx.x == 0) report_error(p.status, 1, 101, blockIdx.x);
    // let copies that are still in flight land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 9) tmem_dealloc(tbase, Cfg::kTmemCols);
}

// ---------------- two query tiles per CTA --------------------------------------------------------
// The same operator for batches of long query segments (head dim 64 / 128): an item is a tile of up to 256
// query rows of one head, worked on as two 128-row tiles A and B against one K/V ring.
//   warps 0-3  softmax + epilogue of tile A, warps 4-7 of tile B: one thread per query row (TMEM lane = row)
//              with all 128 score columns of a block, so a row's maximum and sum need no exchange
//   warp 8     TMA producer, warp 9 tcgen05.mma issuer, as above
// TMEM: S_A [0,128), S_B [128,256) (one score buffer per tile; P overwrites its first 64 columns),
// O_A [256,256+D), O_B [256+D,256+2D).  Per block the issuer runs  P_A.V, S_A(next), P_B.V, S_B(next):  while
// the tensor pipe works for one tile the other tile's threads run their exponentials, and the fixed cost of a
// block (TMEM round trips, barriers) is paid once per 128 scores of a thread instead of once per 64.
// Under the causal mask tile A ends one block before tile B; barriers of a tile are indexed by the tile's own
// block count.
// Opt-in (environment variable VAFA_FWD_PAIR=1, read once per process): measured on a B200 it is 4 % faster than
// the one-tile kernel above on long non-causal segments (8 x 8192: 4.40 against 4.60 ms), 6-14 % slower on
// causal batches (tile A idles through tile B's last block of every item) and on batches of short segments
// (half as many items, so the scheduler splits keys more often), and level on the 500-query production shapes.
template <int D>
struct PairSmem {
  alignas(1024) uint8_t q[2][FwdCfg<D>::kTileBytes];
  alignas(1024) uint8_t k[2][FwdCfg<D>::kTileBytes];
  alignas(1024) uint8_t v[2][FwdCfg<D>::kTileBytes];
  alignas(8) uint64_t q_full, q_free;
  uint64_t k_full[2], v_full[2];
  uint64_t s_full[2][2], p_full[2][2];  // [tile][the tile's block count & 1], phase (count / 2) & 1
  uint64_t o_done[2];                   // P.V of both tiles for block g complete: index g & 1 of the K/V ring
  uint64_t o_ready[2];                  // [tile] the tile's last P.V of an item complete
  WorkQueue wq;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};
static_assert(sizeof(PairSmem<128>) + 1024 <= 227 * 1024, "shared memory budget");

// Blocks of an item per tile.  Row r of tile t (row 128 t + r of the item) sees inner index jj iff
// jj < i_len and (masked) jj <= 128 t + r + diag.
struct PairShape {
  int nb, nb_t[2], rows_t[2];
};
__device__ __forceinline__ PairShape pair_shape(const WorkItem& w) {
  PairShape z;
  z.nb = (w.i_len + kTile - 1) / kTile;
  z.rows_t[0] = min(kTile, w.o_rows);
  z.rows_t[1] = max(0, w.o_rows - kTile);
  const int seen_a = w.masked ? min(w.i_len, z.rows_t[0] + w.diag) : w.i_len;  // keys the last row of A sees
  z.nb_t[0] = max(0, (seen_a + kTile - 1) / kTile);
  z.nb_t[1] = z.rows_t[1] > 0 ? z.nb : 0;
  return z;
}

// Registers: a softmax thread holds the 128 scores of its row.  The launch gives every thread 168 registers
// (twelve warps; registers are granted per four warps); the producer / issuer warp group hands most of its
// share to the two softmax warp groups (setmaxnreg), which then have 216 each.
#ifndef VAFA_FWD_PAIR_SETMAXNREG
#define VAFA_FWD_PAIR_SETMAXNREG 1
#endif
constexpr int kPairThreads = VAFA_FWD_PAIR_SETMAXNREG ? 384 : kFwdThreads;

template <typename T, int D>
__global__ void __launch_bounds__(kPairThreads, 1)
varlen_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int kSubB = Cfg::kSubBytes;
  extern __shared__ uint8_t smem_raw[];
  using Smem = PairSmem<D>;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    wq_init(sm.wq, 9);
    mbar_init(smem_u32(&sm.q_full), 1);
    mbar_init(smem_u32(&sm.q_free), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.k_full[i]), 1);
      mbar_init(smem_u32(&sm.v_full[i]), 1);
      mbar_init(smem_u32(&sm.o_done[i]), 1);
      mbar_init(smem_u32(&sm.o_ready[i]), 1);
      for (int j = 0; j < 2; ++j) {
        mbar_init(smem_u32(&sm.s_full[i][j]), 1);
        mbar_init(smem_u32(&sm.p_full[i][j]), 4);  // lane 0 of each of the tile's four warps
      }
    }
    fence_barrier_init();
  }
  if (warp == 8 && lane == 0) {
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
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
  const int total = max(n_items, 0);
  int* const next_item = const_cast<int*>(&p.header->next_item);
  if (n_items < 0 && threadIdx.x == 0) report_error(p.status, 2, 110, n_items);

  // (each setmaxnreg sits inside its own role's branch: after a join of the two the compiler would have to
  // assume the smaller budget for everything that follows)
  if (warp >= 10) {
    // the two spare warps of the third warp group
#if VAFA_FWD_PAIR_SETMAXNREG
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
#endif
  } else if (warp == 8) {
#if VAFA_FWD_PAIR_SETMAXNREG
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
#endif
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t gk = 0, qi = 0, cnt[2] = {0, 0};
      // what frees a K slot: the last score product issued for the block that used it
      uint32_t rel_bar[2] = {0, 0}, rel_par[2] = {0, 0};
      bool alive = true;
      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_produce(sm.wq, n, next_item, total, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const PairShape z = pair_shape(w);
        if (z.nb == 0) continue;
        const int hk = w.head / p.group;
        const bool has_b = z.rows_t[1] > 0;
        if (!mbar_wait(smem_u32(&sm.q_free), (qi & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(smem_u32(&sm.q_full), (has_b ? 2 : 1) * Cfg::kTileBytes);
        for (int t = 0; t < (has_b ? 2 : 1); ++t)
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.q[t]) + c * kSubB, &tmap_q, smem_u32(&sm.q_full), c * 64, w.head, w.o_start + t * kTile);
        for (int b = 0; b < z.nb; ++b, ++gk) {
          const int st = gk & 1;
          const uint32_t ph = (gk >> 1) & 1;
          const int row = w.i_start + b * kTile;
          if (rel_bar[st] != 0 && !mbar_wait(rel_bar[st], rel_par[st], abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.k_full[st]), Cfg::kTileBytes);
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.k[st]) + c * kSubB, &tmap_k, smem_u32(&sm.k_full[st]), c * 64, hk, row);
          const int t_last = has_b ? 1 : 0;  // tile B runs every block of the item when it exists
          rel_bar[st] = smem_u32(&sm.s_full[t_last][cnt[t_last] & 1]);
          rel_par[st] = (cnt[t_last] >> 1) & 1;
          if (b < z.nb_t[0]) ++cnt[0];
          if (has_b) ++cnt[1];
          if (!mbar_wait(smem_u32(&sm.o_done[st]), ph ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.v_full[st]), Cfg::kTileBytes);
          for (int c = 0; c < Cfg::kSub; ++c)
            tma_load_3d(smem_u32(sm.v[st]) + c * kSubB, &tmap_v, smem_u32(&sm.v_full[st]), c * 64, hk, row);
        }
        ++qi;
      }
    }
  } else if (warp == 9) {
#if VAFA_FWD_PAIR_SETMAXNREG
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
#endif
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_qk = make_idesc(kFmt, 0, 0, 128, kTile);
      constexpr uint32_t idesc_pv = make_idesc(kFmt, 0, 1, 128, D);
      uint32_t gk = 0, qi = 0, cnt[2] = {0, 0};
      bool alive = true;

      // S_t = Q_t K(g)^T, announced on the tile's barrier for its block count c
      auto issue_s = [&](int t, uint32_t g, uint32_t c) {
        const uint32_t q_lo = desc_lo_sw128(smem_u32(sm.q[t]), 16), k_lo = desc_lo_sw128(smem_u32(sm.k[g & 1]), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (kSubB >> 4) + (kk & 3) * 2;
          mma_ss2(tbase + t * kTile, q_lo + off, k_lo + off, idesc_qk, kk > 0);
        }
        mma_commit(smem_u32(&sm.s_full[t][c & 1]));
      };
      // O_t (+)= P_t V(g); P sits in the first 64 columns of the tile's score buffer, two keys per column
      auto issue_pv = [&](int t, uint32_t g, bool first) {
        const uint32_t v_lo = desc_lo_sw128(smem_u32(sm.v[g & 1]), kSubB);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)
          mma_ts2(tbase + Cfg::kOCol + t * D, tbase + t * kTile + kk * 8, v_lo + kk * (2048 >> 4), idesc_pv,
                  (!first || kk > 0) ? 1u : 0u);
      };

      for (uint32_t n = 0; alive; ++n) {
        const int idx = wq_consume_thread(sm.wq, n, abort_flag);
        if (idx < 0) break;
        const WorkItem w = p.items[idx];
        const PairShape z = pair_shape(w);
        if (z.nb == 0) continue;
        const bool has_b = z.rows_t[1] > 0;
        const int t_last = has_b ? 1 : 0;
        if (!mbar_wait(smem_u32(&sm.q_full), qi & 1, abort_flag)) break;
        if (!mbar_wait(smem_u32(&sm.k_full[gk & 1]), (gk >> 1) & 1, abort_flag)) break;
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (z.nb_t[t] > 0) issue_s(t, gk, cnt[t]);
        if (z.nb == 1) mma_commit(smem_u32(&sm.q_free));
        for (int b = 0; b < z.nb && alive; ++b) {
          const uint32_t g = gk + b;
          bool v_ready = false, k_ready = false;
          for (int t = 0; t < 2; ++t) {
            if (b >= z.nb_t[t]) continue;
            const uint32_t c = cnt[t];
            if (!mbar_wait(smem_u32(&sm.p_full[t][c & 1]), (c >> 1) & 1, abort_flag)) { alive = false; break; }
            if (!v_ready) {
              if (!mbar_wait(smem_u32(&sm.v_full[g & 1]), (g >> 1) & 1, abort_flag)) { alive = false; break; }
              v_ready = true;
            }
            tc_fence_after();
            issue_pv(t, g, b == 0);
            if (t == t_last) mma_commit(smem_u32(&sm.o_done[g & 1]));
            if (b + 1 == z.nb_t[t]) mma_commit(smem_u32(&sm.o_ready[t]));
            ++cnt[t];
            if (b + 1 < z.nb_t[t]) {
              if (!k_ready) {
                if (!mbar_wait(smem_u32(&sm.k_full[(g + 1) & 1]), ((g + 1) >> 1) & 1, abort_flag)) { alive = false; break; }
                tc_fence_after();
                k_ready = true;
              }
              issue_s(t, g + 1, cnt[t]);
              if (t == t_last && b + 2 == z.nb) mma_commit(smem_u32(&sm.q_free));
            }
          }
        }
        gk += z.nb;
        ++qi;
      }
    }
  } else {
    // ---------------- softmax + epilogue: warps 0-3 tile A, warps 4-7 tile B ----------------
#if VAFA_FWD_PAIR_SETMAXNREG
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
#endif
    const int t = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_base + t * kTile;
    const uint32_t o_addr = lane_base + Cfg::kOCol + t * D;
    const float c = p.scale_log2;
    uint32_t gk = 0, cnt = 0, n_ready = 0;
    bool alive = true;
    for (uint32_t n = 0; alive; ++n) {
      const int idx = wq_consume_warp(sm.wq, n, abort_flag);
      if (idx < 0) break;
      const WorkItem w = p.items[idx];
      const PairShape z = pair_shape(w);
      const int my_nb = z.nb_t[t], my_rows = z.rows_t[t];
      const int h = w.head;
      float m_ref = -INFINITY, l = 0.f;

      for (int b = 0; b < my_nb; ++b, ++cnt) {
        const uint32_t g = gk + b;
        if (!mbar_wait(smem_u32(&sm.s_full[t][cnt & 1]), (cnt >> 1) & 1, abort_flag)) { alive = false; break; }
        tc_fence_after();
        float s[kTile];
        {
          uint32_t u0[64], u1[64];
          tmem_ld64(s_addr, u0);
          tmem_ld64(s_addr + 64, u1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            s[i] = __uint_as_float(u0[i]);
            s[64 + i] = __uint_as_float(u1[i]);
          }
        }
        const int lim_tail = w.i_len - 1 - b * kTile;
        const int lim_diag = w.masked ? (w.diag + t * kTile - b * kTile) : 0x3fffffff;  // for row 0 of the tile
        const bool masked_block = lim_tail < kTile - 1 || lim_diag < kTile - 1;          // same for the whole tile
        if (masked_block) {
          const int lim = min(lim_tail, w.masked ? lim_diag + r : 0x3fffffff);
#pragma unroll
          for (int i = 0; i < kTile; ++i) s[i] = (i <= lim) ? s[i] : -INFINITY;
        }
        float m8[8];
#pragma unroll
        for (int j2 = 0; j2 < 8; ++j2) m8[j2] = max3(s[j2], s[8 + j2], s[16 + j2]);
#pragma unroll
        for (int i = 24; i + 16 <= kTile; i += 16) {
#pragma unroll
          for (int j2 = 0; j2 < 8; ++j2) m8[j2] = max3(m8[j2], s[i + j2], s[i + 8 + j2]);
        }
#pragma unroll
        for (int j2 = 0; j2 < 8; ++j2) m8[j2] = fmaxf(m8[j2], s[kTile - 8 + j2]);
        const float mx = max3(max3(m8[0], m8[1], m8[2]), max3(m8[3], m8[4], m8[5]), fmaxf(m8[6], m8[7]));
        const float m_blk = mx * c;  // c > 0
        float m_new = fmaxf(m_ref, m_blk);
        const bool resc = m_new > m_ref + kRescaleThreshold;
        if (!resc) m_new = m_ref;
        const float alpha = resc ? ex2(m_ref - m_new) : 1.f;
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        // exponents, row sum and P in two halves of 64 columns (the first half of P is on its way to TMEM while
        // the second is computed); unmasked blocks take every kPolyPeriod-th pair as a polynomial on the FMA pipe
        const uint64_t cs2 = pack_f2(c, c), nm2 = pack_f2(-m_use, -m_use);
        uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
        auto exps = [&](auto poly_tag) {
          constexpr bool kPoly = decltype(poly_tag)::value;
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int e = 64 * hf + 2 * i;
              const uint64_t t2 = fma_f2(pack_f2(s[e], s[e + 1]), cs2, nm2);
              float p0, p1;
              if (kPoly && (i % kPolyPeriod == kPolyPeriod - 1)) {
                ex2_poly2(t2, p0, p1);
              } else {
                float t0, t1;
                unpack_f2(t2, t0, t1);
                p0 = ex2(t0);
                p1 = ex2(t1);
              }
              sum2[i & 3] = add_f2(sum2[i & 3], pack_f2(p0, p1));
              pk[i] = pack_p<T>(p0, p1);
            }
            tmem_st32(s_addr + 32 * hf, pk);
          }
        };
        if (masked_block) exps(std::false_type{}); else exps(std::true_type{});
        {
          float a0, a1, b0, b1;
          unpack_f2(add_f2(sum2[0], sum2[1]), a0, a1);
          unpack_f2(add_f2(sum2[2], sum2[3]), b0, b1);
          l = l * alpha + ((a0 + a1) + (b0 + b1));
        }
        m_ref = m_new;
        if (b > 0 && __any_sync(0xffffffffu, resc)) {
          // O may be rescaled once P.V of the previous block is complete; the next one waits for this warp's
          // arrival below.  No alias in the parity wait: the block after next cannot be issued before it.
          if (!mbar_wait(smem_u32(&sm.o_done[(g - 1) & 1]), ((g - 1) >> 1) & 1, abort_flag)) { alive = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c2 = 0; c2 < D / 32; ++c2) {
            uint32_t tt[32];
            tmem_ld32(o_addr + c2 * 32, tt);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) tt[i] = __float_as_uint(__uint_as_float(tt[i]) * alpha);
            tmem_st32(o_addr + c2 * 32, tt);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.p_full[t][cnt & 1]));
      }
      if (!alive) break;
      gk += z.nb;
      if (my_rows <= 0) continue;  // no tile B in this item

      // ---- epilogue ----
      if (my_nb > 0) {
        if (!mbar_wait(smem_u32(&sm.o_ready[t]), n_ready & 1, abort_flag)) break;
        ++n_ready;
        tc_fence_after();
      }
      const bool row_ok = r < my_rows;
      const bool dead = (my_nb == 0) || (l == 0.f);  // a NaN row sum is not a dead row: it goes out as NaN
      const float inv_l = dead ? 0.f : 1.f / l;
      const float lse_val = dead ? -INFINITY : m_ref + log2f(l);
      if (w.partial < 0) {
        const long long row = (long long)w.o_start + t * kTile + r;
        T* optr = reinterpret_cast<T*>(p.o) + (row * p.H + h) * D;
#pragma unroll
        for (int c2 = 0; c2 < D / 32; ++c2) {
          uint32_t tt[32];
          if (my_nb > 0) {
            tmem_ld32(o_addr + c2 * 32, tt);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) tt[i] = 0u;
          }
          uint32_t pw[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pw[i] = pack2_out<T>(__uint_as_float(tt[2 * i]) * inv_l, __uint_as_float(tt[2 * i + 1]) * inv_l);
          store_chunk_coalesced<T>(pw, optr + c2 * 32, (long long)p.H * D, r, my_rows, 4);
        }
        if (row_ok) p.lse[row * p.H + h] = lse_val;
      } else {
        const long long prow = (long long)w.partial + t * kTile + r;
        float* optr = p.partial_o + (prow * p.H + h) * D;
#pragma unroll
        for (int c2 = 0; c2 < D / 32; ++c2) {
          uint32_t tt[32];
          if (my_nb > 0) {
            tmem_ld32(o_addr + c2 * 32, tt);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) tt[i] = 0u;
          }
          if (row_ok) {
            float4* dst = reinterpret_cast<float4*>(optr + c2 * 32);
#pragma unroll
            for (int v4 = 0; v4 < 8; ++v4) {
              float4 f;
              f.x = __uint_as_float(tt[4 * v4 + 0]) * inv_l;
              f.y = __uint_as_float(tt[4 * v4 + 1]) * inv_l;
              f.z = __uint_as_float(tt[4 * v4 + 2]) * inv_l;
              f.w = __uint_as_float(tt[4 * v4 + 3]) * inv_l;
              dst[v4] = f;
            }
          }
        }
        if (row_ok) p.partial_lse[prow * p.H + h] = lse_val;
      }
      // the TMEM reads of O above finish (tcgen05.wait::ld) before this thread's next p_full arrival, and the
      // next item's first P.V of this tile, which overwrites O, is issued only after that arrival
    }
  }

  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    if (threadIdx.x == 0) report_error(p.status, 1, 111, blockIdx.x);
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 9) tmem_dealloc(tbase, Cfg::kTmemCols);
}

// ---------------- split-K combine -------------------------------------------------------------
// Merge the per-split partial outputs (already normalised, fp32) with their log2-domain LSE:
//   m = max_s lse_s;  w_s = 2^(lse_s - m);  o = sum_s w_s o_s / sum_s w_s;  lse = m + log2 sum_s w_s
// (reference: triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:652-734).  One warp per
// (row, head); each lane owns D/32 consecutive columns and reads them with one vector load.
template <typename T, int D>
__global__ void __launch_bounds__(256) varlen_combine_kernel(const SchedHeader* __restrict__ header,
                                                             const CombineUnit* __restrict__ units,
                                                             const float* __restrict__ partial_o,
                                                             const float* __restrict__ partial_lse, T* __restrict__ o,
                                                             float* __restrict__ lse, int H) {
  constexpr int V = D / 32;  // floats per lane: 4 (D=128) or 2 (D=64)
  const int n_units = header->n_combine;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    const CombineUnit cu = units[u];
    const int n_rh = cu.q_rows * H;
    for (int rh = wib; rh < n_rh; rh += 8) {
      const int r = rh / H, h = rh % H;
      float m = -INFINITY;
      for (int s = lane; s < cu.n_splits; s += 32)
        m = fmaxf(m, partial_lse[((long long)cu.base + (long long)s * cu.q_rows + r) * H + h]);
#pragma unroll
      for (int o_ = 16; o_ > 0; o_ >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o_));
      const float m_use = (m == -INFINITY) ? 0.f : m;
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      float den = 0.f;
      for (int s = 0; s < cu.n_splits; ++s) {
        const long long prow = (long long)cu.base + (long long)s * cu.q_rows + r;
        const float wgt = exp2f(partial_lse[prow * H + h] - m_use);
        den += wgt;
        const float* src = partial_o + (prow * H + h) * D + lane * V;
        if (V == 4) {
          const float4 f = *reinterpret_cast<const float4*>(src);
          acc[0] += wgt * f.x; acc[1] += wgt * f.y; acc[V - 2] += wgt * f.z; acc[V - 1] += wgt * f.w;
        } else {
          const float2 f = *reinterpret_cast<const float2*>(src);
          acc[0] += wgt * f.x; acc[1] += wgt * f.y;
        }
      }
      const float inv = den == 0.f ? 0.f : 1.f / den;  // a NaN weight sum goes out as NaN
      const long long row = (long long)cu.q_start + r;
      T* dst = o + (row * H + h) * D + lane * V;
      if (V == 4) {
        uint2 pk;
        pk.x = pack2_out<T>(acc[0] * inv, acc[1] * inv);
        pk.y = pack2_out<T>(acc[V - 2] * inv, acc[V - 1] * inv);
        *reinterpret_cast<uint2*>(dst) = pk;
      } else {
        *reinterpret_cast<uint32_t*>(dst) = pack2_out<T>(acc[0] * inv, acc[1] * inv);
      }
      if (lane == 0) lse[row * H + h] = den == 0.f ? -INFINITY : m_use + log2f(den);
    }
  }
}

#ifdef VAFA_TRACE
}  // namespace
long long* vafa_trace_buffer = nullptr;
namespace {
#endif

// Switch of the two-tile forward kernel (environment variable VAFA_FWD_PAIR=1; off by default, see the kernel).
bool fwd_pair_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("VAFA_FWD_PAIR");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

struct FwdWorkspace {
  size_t header, items, combine, plse, po, total;
  SchedCaps caps;
};

// `limit` > 0 shrinks the split-K partial area so that the whole layout fits in `limit` bytes
// (the scheduler then splits less, or not at all); total > limit afterwards means it cannot fit.
FwdWorkspace fwd_workspace(const vafa_varlen_args* a, int sm_count, size_t limit = 0) {
  FwdWorkspace w;
  w.caps = sched_caps(kSchedFwd, a->total_q, a->total_k, a->n_seg, a->num_heads, sm_count, a->split_k_block);
  w.header = 0;
  w.items = 256;
  w.combine = w.items + align_up((size_t)w.caps.cap_items * sizeof(WorkItem), 256);
  w.plse = w.combine + align_up((size_t)w.caps.cap_combine * sizeof(CombineUnit), 256);
  if (limit > 0) {
    const size_t per_row = (size_t)a->num_heads * (a->head_dim + 1) * 4;
    const size_t room = limit > w.plse + 1024 ? limit - w.plse - 1024 : 0;
    const size_t rows = room / per_row;
    if (rows < (size_t)w.caps.cap_rows) w.caps.cap_rows = (int32_t)rows;
  }
  w.po = w.plse + align_up((size_t)w.caps.cap_rows * a->num_heads * 4, 256);
  w.total = w.po + align_up((size_t)w.caps.cap_rows * a->num_heads * a->head_dim * 4, 256);
  return w;
}

int resolve_sm_count(int given) {
  if (given > 0) return given;
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
  return n;
}

// `scratch` == nullptr: the caller's workspace with the default layout; otherwise the given
// buffer of `scratch_bytes` with a layout shrunk to fit it.
template <typename T, int D>
int launch_fwd(const vafa_varlen_args* a, cudaStream_t s, void* scratch = nullptr, size_t scratch_bytes = 0) {
  const int sms = resolve_sm_count(a->sm_count);
  const FwdWorkspace ws = fwd_workspace(a, sms, scratch ? scratch_bytes : 0);
  char* base = scratch ? (char*)scratch : (char*)a->workspace;
  SchedParams sp;
  sp.cu_q = a->cu_seqlens_q; sp.cu_k = a->cu_seqlens_k; sp.n_seg = a->n_seg; sp.mode = kSchedFwd;
  sp.causal = a->causal; sp.H = a->num_heads; sp.sm_count = sms; sp.split_len = a->split_k_block;
  sp.cap_items = ws.caps.cap_items; sp.cap_combine = ws.caps.cap_combine; sp.cap_rows = ws.caps.cap_rows;
  sp.header = (SchedHeader*)(base + ws.header);
  sp.items = (WorkItem*)(base + ws.items);
  sp.combine = (CombineUnit*)(base + ws.combine);
  // long query segments: tiles of 256 rows, worked on as two 128-row tiles per CTA
  const bool pair = fwd_pair_enabled() && (long long)a->total_q > 160LL * a->n_seg;
  if (pair) sp.tile_rows = 2 * kTile;
  int rc = launch_scheduler(sp, s);
  if (rc) return rc;

  CUtensorMap tq, tk, tv;
  if ((rc = encode_tmap_rows(&tq, a->q, a->dtype, a->total_q, a->num_heads, D, 128))) return rc;
  const int h_kv = a->num_kv_heads > 0 ? a->num_kv_heads : a->num_heads;
  if ((rc = encode_tmap_rows(&tk, a->k, a->dtype, a->total_k, h_kv, D, 128))) return rc;
  if ((rc = encode_tmap_rows(&tv, a->v, a->dtype, a->total_k, h_kv, D, 128))) return rc;

  FwdParams p;
  p.wait_limit = wait_limit_units();
  p.o = a->o; p.lse = a->lse;
  p.partial_lse = (float*)(base + ws.plse);
  p.partial_o = (float*)(base + ws.po);
  p.header = sp.header; p.items = sp.items; p.H = a->num_heads;
  p.group = a->num_heads / h_kv;
  p.scale_log2 = a->scale * kLog2e;
  p.status = a->status;
  p.trace = nullptr;
#ifdef VAFA_TRACE
  {
    static long long* g_trace = nullptr;  // debugging aid only: leaked on purpose
    if (!g_trace) cudaMalloc(&g_trace, 1024 * 16 * sizeof(long long));
    cudaMemsetAsync(g_trace, 0, 1024 * 16 * sizeof(long long), s);
    p.trace = g_trace;
    vafa_trace_buffer = g_trace;
  }
#endif

  if (pair) {
    const size_t smem = sizeof(PairSmem<D>) + 1024;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_fwd_pair_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(kKFwd, s);
    varlen_fwd_pair_kernel<T, D><<<sms, kPairThreads, smem, s>>>(tq, tk, tv, p);
  } else {
    const size_t smem = sizeof(FwdSmem<D, false>) + 1024;
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_fwd_kernel<T, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    LaunchScope scope(kKFwd, s);
    varlen_fwd_kernel<T, D, false><<<sms, kFwdThreads, smem, s>>>(tq, tk, tv, p);
  }
  VAFA_LAUNCH_CHECK("varlen_fwd_kernel");
  LaunchScope scope(kKCombine, s);
  varlen_combine_kernel<T, D><<<2 * sms, 256, 0, s>>>(sp.header, sp.combine, p.partial_o, p.partial_lse,
                                                      (T*)a->o, a->lse, a->num_heads);
  VAFA_LAUNCH_CHECK("varlen_combine_kernel");
  return 0;
}

struct AbsorbCoreWs {
  size_t header, items, total;
  SchedCaps caps;
};

AbsorbCoreWs absorb_core_ws(int total_q, int n_seg, int H) {
  AbsorbCoreWs w;
  const int tile_rows = kTile / H;
  w.caps.cap_items = total_q / tile_rows + n_seg + 1;
  w.caps.cap_combine = 0;
  w.caps.cap_rows = 0;
  w.header = 0;
  w.items = 256;
  w.total = w.items + align_up((size_t)w.caps.cap_items * sizeof(WorkItem), 256);
  return w;
}

SchedParams absorb_fwd_sched_params(const AbsorbCoreArgs& a, int sms) {
  const AbsorbCoreWs ws = absorb_core_ws(a.total_q, a.n_seg, a.H);
  char* base = (char*)a.workspace;
  SchedParams sp;
  sp.cu_q = a.cu_q; sp.cu_k = a.cu_k; sp.n_seg = a.n_seg; sp.mode = kSchedDq;  // no split-K
  sp.causal = 0; sp.H = 1; sp.sm_count = sms; sp.split_len = 0; sp.tile_rows = kTile / a.H;
  sp.cap_items = ws.caps.cap_items; sp.cap_combine = 0; sp.cap_rows = 0;
  sp.header = (SchedHeader*)(base + ws.header);
  sp.items = (WorkItem*)(base + ws.items);
  sp.combine = nullptr;
  return sp;
}

template <typename T>
int launch_absorb_core_fwd(const AbsorbCoreArgs& a, cudaStream_t s) {
  constexpr int D = 256;
  const int sms = resolve_sm_count(a.sm_count);
  const SchedParams sp = absorb_fwd_sched_params(a, sms);
  int rc = a.lists_built ? 0 : launch_scheduler(sp, s);
  if (rc) return rc;
  CUtensorMap tu, tx;
  if ((rc = encode_tmap_rows(&tu, a.u, a.dtype, a.total_q, a.H, D, kTile / a.H, a.H))) return rc;
  if ((rc = encode_tmap_rows(&tx, a.x, a.dtype, a.total_k, 1, a.x_width, fwd_block_keys<true>()))) return rc;
  FwdParams p;
  p.wait_limit = wait_limit_units();
  p.o = a.axn; p.lse = a.lse; p.partial_o = nullptr; p.partial_lse = nullptr;
  p.header = sp.header; p.items = sp.items; p.H = a.H;
  p.group = 1;
  p.scale_log2 = a.scale * kLog2e;
  p.status = a.status;
  p.trace = nullptr;
#ifdef VAFA_TRACE
  {
    static long long* g_trace_a = nullptr;  // debugging aid only: leaked on purpose
    if (!g_trace_a) cudaMalloc(&g_trace_a, 1024 * 16 * sizeof(long long));
    cudaMemsetAsync(g_trace_a, 0, 1024 * 16 * sizeof(long long), s);
    p.trace = g_trace_a;
    vafa_trace_buffer = g_trace_a;
  }
#endif
  const size_t smem = sizeof(FwdSmem<D, true>) + 1024;
  VAFA_CUDA_CHECK(cudaFuncSetAttribute(varlen_fwd_kernel<T, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  LaunchScope scope(kKAbsorbFwd, s);
  varlen_fwd_kernel<T, D, true><<<sms, kFwdThreads, smem, s>>>(tu, tx, tx, p);
  VAFA_LAUNCH_CHECK("varlen_fwd_kernel<absorb>");
  return 0;
}

}  // namespace

size_t sm100_absorb_core_fwd_workspace_bytes(int total_q, int n_seg, int H) { return absorb_core_ws(total_q, n_seg, H).total; }

int sm100_absorb_core_fwd_lists(const AbsorbCoreArgs& a, cudaStream_t s) {
  return launch_scheduler(absorb_fwd_sched_params(a, resolve_sm_count(a.sm_count)), s);
}

int sm100_absorb_core_fwd(const AbsorbCoreArgs& a, cudaStream_t s) {
  return a.dtype == VAFA_BF16 ? launch_absorb_core_fwd<__nv_bfloat16>(a, s) : launch_absorb_core_fwd<__half>(a, s);
}

bool sm100_varlen_fwd_supported(const vafa_varlen_args* a) {
  if (!(a->dtype == VAFA_BF16 || a->dtype == VAFA_F16)) return false;
  if (!(a->head_dim == 64 || a->head_dim == 128)) return false;
  if (!(a->scale > 0.f)) return false;  // the row maximum is taken before scaling
  if (a->total_q <= 0 || a->total_k <= 0) return false;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(a->q) && al(a->k) && al(a->v) && al(a->o);
}

size_t sm100_varlen_fwd_workspace_bytes(const vafa_varlen_args* a) {
  return fwd_workspace(a, resolve_sm_count(a->sm_count)).total;
}

int sm100_varlen_fwd(const vafa_varlen_args* a, cudaStream_t s) {
  if (a->dtype == VAFA_BF16) {
    return a->head_dim == 128 ? launch_fwd<__nv_bfloat16, 128>(a, s) : launch_fwd<__nv_bfloat16, 64>(a, s);
  }
  return a->head_dim == 128 ? launch_fwd<__half, 128>(a, s) : launch_fwd<__half, 64>(a, s);
}

// ---------------- forward without any allocation by anyone ------------------------------------
// Scratch for vafa_varlen_fwd_noalloc(): a fixed array in the library's own device image.  Every
// GPU that loads the library carries these bytes until the process exits.
constexpr size_t kNoAllocScratchBytes = VAFA_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kMaxDevices] = {};

// Device address of g_noalloc_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel can use, so the address is asked for
// once per device (with that device current) and cached.
int noalloc_scratch(void** out) {
  int dev = -1;
  VAFA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(VAFA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(VAFA_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
    g_noalloc_ptr[dev] = ptr;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace

int sm100_varlen_fwd_noalloc(const vafa_varlen_args* a, cudaStream_t s) {
  const int sms = resolve_sm_count(a->sm_count);
  const FwdWorkspace ws = fwd_workspace(a, sms, kNoAllocScratchBytes);
  if (ws.total > kNoAllocScratchBytes)
    return fail(VAFA_ERR_WORKSPACE,
                "vafa_varlen_fwd_noalloc: the tile lists of this batch need %zu bytes, more than the built-in "
                "%zu-byte scratch (they grow with total_q/128 + n_seg); use vafa_varlen_fwd with a caller-owned "
                "workspace",
                ws.total, kNoAllocScratchBytes);
  void* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  if (a->dtype == VAFA_BF16) {
    return a->head_dim == 128 ? launch_fwd<__nv_bfloat16, 128>(a, s, scratch, kNoAllocScratchBytes)
                              : launch_fwd<__nv_bfloat16, 64>(a, s, scratch, kNoAllocScratchBytes);
  }
  return a->head_dim == 128 ? launch_fwd<__half, 128>(a, s, scratch, kNoAllocScratchBytes)
                            : launch_fwd<__half, 64>(a, s, scratch, kNoAllocScratchBytes);
}

}  // namespace vafa

#ifdef VAFA_TRACE
extern "C" __attribute__((visibility("default"))) int vafa_trace_read(long long* host, int n_ctas) {
  if (!vafa::vafa_trace_buffer) return -1;
  return (int)cudaMemcpy(host, vafa::vafa_trace_buffer, (size_t)n_ctas * 16 * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif
