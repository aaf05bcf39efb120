// Dense product for the absorb operator's prologue and epilogue:
//   C[M, N] = A[M, K] . B[K, N]        (16-bit operands, fp32 accumulation, 16-bit result; K = 256 k)
// K = 256: one persistent CTA per SM keeps its 256 x 256 slice of B in shared memory (128 KB,
// MN-major) and streams 128-row tiles of A through a second buffer.  K = 512, 768, ...: the B slice of
// each 256-deep chunk is streamed with the A chunk instead and the chunks accumulate in TMEM.  The
// accumulator (256 TMEM columns) is double buffered so the epilogue of tile i overlaps the load and
// MMAs of tile i+1.
// It stands in for the two torch matmuls of the reference's prologue
// (triton_target_attn_absorb/triton_target_attn_absorb/interface.py:434-435, here as one product
// with the pre-multiplied W_Q W_K^T) and for the per-head W_V projection the reference does at the
// end of its forward kernel (triton_target_attn_absorb/triton_target_attn_absorb/kernels.py:273-279).
#include <cuda.h>
#include <type_traits>

#include "profile.cuh"
#include "sm100_common.cuh"
#include "sm100_kernels.cuh"

namespace vafa {
namespace {

using namespace ptx;

constexpr int kGemmThreads = 192;
constexpr int kK = 256;
constexpr int kNTile = 256;

struct GemmSmem {
  alignas(1024) uint8_t b[4][kK * 128];    // 4 column chunks of 64: [256 k-rows x 128 B] each
  alignas(1024) uint8_t a[4][128 * 128];   // 4 k chunks of 64: [128 rows x 128 B] each
  alignas(8) uint64_t b_full, a_full, a_empty, acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};
static_assert(sizeof(GemmSmem) + 1024 <= 227 * 1024, "shared memory budget");

struct GemmParams {
  void* C;
  long long M;
  int ldc;
  int n_tiles;     // N / 256
  int m_tiles;     // ceil(M / 128)
  int k_chunks;    // K / 256
  int diag_heads;  // 0: full rows
  int wait_limit;  // bound of every device-side wait, in units of 65536 cycles
};

template <typename T>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_nn_k256_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmem& sm = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;
  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    mbar_init(smem_u32(&sm.b_full), 1);
    mbar_init(smem_u32(&sm.a_full), 1);
    mbar_init(smem_u32(&sm.a_empty), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.acc_full[i]), 1);
      mbar_init(smem_u32(&sm.acc_empty[i]), 128);
    }
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sm.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;

  // CTA -> (column tile, first row tile, row tile stride)
  const int groups = gridDim.x / p.n_tiles;  // CTAs per column tile (grid is a multiple of n_tiles)
  const int n_tile = blockIdx.x % p.n_tiles;
  const int m_first = blockIdx.x / p.n_tiles;

  if (warp == 4) {
    if (lane == 0) {
      const bool resident = p.k_chunks == 1;
      if (resident) {
        mbar_expect_tx(smem_u32(&sm.b_full), 4 * kK * 128);
        for (int c = 0; c < 4; ++c) tma_load_3d(smem_u32(sm.b[c]), &tmap_b, smem_u32(&sm.b_full), n_tile * kNTile + c * 64, 0, 0);
      }
      uint32_t it = 0;
      bool alive = true;
      for (int m = m_first; alive && m < p.m_tiles; m += groups) {
        for (int kc = 0; kc < p.k_chunks; ++kc, ++it) {
          if (!mbar_wait(smem_u32(&sm.a_empty), (it & 1) ^ 1, abort_flag)) { alive = false; break; }
          mbar_expect_tx(smem_u32(&sm.a_full), 4 * 128 * 128 + (resident ? 0 : 4 * kK * 128));
          for (int c = 0; c < 4; ++c)
            tma_load_3d(smem_u32(sm.a[c]), &tmap_a, smem_u32(&sm.a_full), kc * kK + c * 64, 0, m * 128);
          if (!resident)
            for (int c = 0; c < 4; ++c)
              tma_load_3d(smem_u32(sm.b[c]), &tmap_b, smem_u32(&sm.a_full), n_tile * kNTile + c * 64, 0, kc * kK);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc = make_idesc(kFmt, 0, 1, 128, kNTile);
      bool ok = p.k_chunks > 1 || mbar_wait(smem_u32(&sm.b_full), 0, abort_flag);
      uint32_t it = 0, tile = 0;
      for (int m = m_first; ok && m < p.m_tiles; m += groups, ++tile) {
        const uint32_t buf = tile & 1;
        if (!mbar_wait(smem_u32(&sm.acc_empty[buf]), ((tile >> 1) & 1) ^ 1, abort_flag)) break;
        for (int kc = 0; kc < p.k_chunks; ++kc, ++it) {
          if (!mbar_wait(smem_u32(&sm.a_full), it & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kK / 16; ++kk) {
            const uint64_t da = make_desc_sw128(smem_u32(sm.a[kk >> 2]) + (kk & 3) * 32, 16, 1024);
            const uint64_t db = make_desc_sw128(smem_u32(sm.b[0]) + kk * 2048, kK * 128, 1024);
            mma_ss(tbase + buf * kNTile, da, db, idesc, (kc > 0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(smem_u32(&sm.a_empty));
        }
        if (ok) mma_commit(smem_u32(&sm.acc_full[buf]));
      }
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = tbase + ((uint32_t)(warp * 32) << 16);
    T* C = reinterpret_cast<T*>(p.C);
    uint32_t it = 0;
    for (int m = m_first; m < p.m_tiles; m += groups, ++it) {
      const uint32_t buf = it & 1;
      if (!mbar_wait(smem_u32(&sm.acc_full[buf]), (it >> 1) & 1, abort_flag)) break;
      tc_fence_after();
      const long long row = (long long)m * 128 + r;
      const bool row_ok = row < p.M;
      int c_begin = 0, c_end = kNTile / 32;
      long long col0 = (long long)n_tile * kNTile;  // first output column of chunk c_begin
      if (p.diag_heads > 0) {
        const int per = (kNTile / p.diag_heads) / 32;  // 32-column chunks per head block
        c_begin = (int)(row % p.diag_heads) * per;
        c_end = c_begin + per;
        col0 = 0;
      }
      // c_begin/c_end differ per thread in diag mode, but tcgen05.ld is warp-collective: walk all
      // chunks uniformly and keep only this thread's range
      for (int cc = 0; cc < kNTile / 32; ++cc) {
        if (p.diag_heads > 0) {
          const bool any = __any_sync(0xffffffffu, cc >= c_begin && cc < c_end);
          if (!any) continue;
        }
        uint32_t t[32];
        tmem_ld32(lane_base + buf * kNTile + cc * 32, t);
        tmem_wait_ld();
        if (row_ok && cc >= c_begin && cc < c_end) {
          uint4* dst = reinterpret_cast<uint4*>(C + row * p.ldc + col0 + (cc - c_begin) * 32);
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 u;
            u.x = pack2_out<T>(__uint_as_float(t[8 * v4 + 0]), __uint_as_float(t[8 * v4 + 1]));
            u.y = pack2_out<T>(__uint_as_float(t[8 * v4 + 2]), __uint_as_float(t[8 * v4 + 3]));
            u.z = pack2_out<T>(__uint_as_float(t[8 * v4 + 4]), __uint_as_float(t[8 * v4 + 5]));
            u.w = pack2_out<T>(__uint_as_float(t[8 * v4 + 6]), __uint_as_float(t[8 * v4 + 7]));
            dst[v4] = u;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sm.acc_empty[buf]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 5) tmem_dealloc(tbase, 512);
}

}  // namespace

int sm100_gemm_nn_k256(const GemmNNArgs& g, cudaStream_t s) {
  if (g.M <= 0) return 0;
  if (g.N % kNTile != 0 || (g.diag_heads > 0 && (g.N != kNTile || (kNTile / g.diag_heads) % 32 != 0)))
    return fail(VAFA_ERR_UNSUPPORTED, "gemm_nn_k256: N=%d diag_heads=%d not supported", g.N, g.diag_heads);
  int sms = g.sm_count;
  if (sms <= 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  GemmParams p;
  p.wait_limit = wait_limit_units();
  p.C = g.C; p.M = g.M; p.ldc = g.ldc; p.n_tiles = g.N / kNTile; p.m_tiles = (int)((g.M + 127) / 128);
  p.diag_heads = g.diag_heads;
  p.k_chunks = g.lda / kK;
  int groups = sms / p.n_tiles;
  if (groups < 1) groups = 1;
  if (groups > p.m_tiles) groups = p.m_tiles;
  const int grid = groups * p.n_tiles;
  CUtensorMap ta, tb;
  int rc;
  // K = lda (A rows densely packed), a multiple of 256; B is [K, N] densely packed
  if (g.lda < kK || g.lda % kK != 0 || g.ldb != g.N) return fail(VAFA_ERR_UNSUPPORTED, "gemm_nn_k256: K=%d ldb=%d not supported", g.lda, g.ldb);
  if ((rc = encode_tmap_rows(&ta, g.A, g.dtype, g.M, 1, g.lda, 128))) return rc;
  if ((rc = encode_tmap_rows(&tb, g.B, g.dtype, g.lda, 1, g.N, 256))) return rc;
  const size_t smem = sizeof(GemmSmem) + 1024;
  LaunchScope scope(kKAbsorbGemm, s);
  if (g.dtype == VAFA_BF16) {
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(gemm_nn_k256_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_nn_k256_kernel<__nv_bfloat16><<<grid, kGemmThreads, smem, s>>>(ta, tb, p);
  } else {
    VAFA_CUDA_CHECK(cudaFuncSetAttribute(gemm_nn_k256_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_nn_k256_kernel<__half><<<grid, kGemmThreads, smem, s>>>(ta, tb, p);
  }
  VAFA_LAUNCH_CHECK("gemm_nn_k256_kernel");
  return 0;
}

}  // namespace vafa
