// Token-reduction products for the absorb operator's weight gradients:
//   C_b[m, n] = sum_t A_b[t, m] * B_b[t, n]      m in [0,256), n in [0, n_keep)
// A and B are row-major over tokens, so both operands reach tcgen05.mma MN-major straight from the
// TMA tiles (no transposes in memory).  The token range is split across CTAs; every CTA writes an
// fp32 partial and a second kernel adds the partials in a fixed order, so the weight gradients are
// run-to-run identical (the reference accumulates dW_V with fp32 atomics,
// triton_target_attn_absorb/triton_target_attn_absorb/kernels.py:482-493, and leaves dW_Q / dW_K to
// torch autograd, triton_target_attn_absorb/triton_target_attn_absorb/interface.py:430-435).
#include <cuda.h>
#include <type_traits>

#include "profile.cuh"
#include "sm100_common.cuh"
#include "sm100_kernels.cuh"

namespace vafa {
namespace {

using namespace ptx;

constexpr int kTnThreads = 192;
constexpr int kChunk = 64;     // tokens per pipeline stage
constexpr int kTnStages = 4;

struct TnSmem {
  alignas(1024) uint8_t a[kTnStages][2 * kChunk * 128];  // 2 chunks of 64 m: [64 tokens x 128 B] each
  alignas(1024) uint8_t b[kTnStages][4 * kChunk * 128];  // up to 4 chunks of 64 n
  alignas(8) uint64_t full[kTnStages], empty[kTnStages], done;
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;  // read by the bounded waits as abort_flag[1]: keep it right behind abort_flag
};
static_assert(sizeof(TnSmem) + 1024 <= 227 * 1024, "shared memory budget");

struct TnParams {
  float* partial;        // [splits][batch][256][n_keep]
  int n_chunks;          // ceil(T / 64)
  int chunks_per_split;
  int splits, batch;
  int n_box;             // columns of B per MMA: 256 or 64
  int n_keep;            // leading columns of the box that are kept
  int a_head_step;       // head coordinate of A for batch b: b * a_head_step
  int b_col_step;        // first B column for batch b: b * b_col_step
  int wait_limit;        // bound of every device-side wait, in units of 65536 cycles
};

template <typename T>
__global__ void __launch_bounds__(kTnThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const TnParams p) {
  extern __shared__ uint8_t smem_raw[];
  TnSmem& sm = *reinterpret_cast<TnSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sm.abort_flag;
  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.wait_limit = p.wait_limit;
    for (int i = 0; i < kTnStages; ++i) {
      mbar_init(smem_u32(&sm.full[i]), 1);
      mbar_init(smem_u32(&sm.empty[i]), 1);
    }
    mbar_init(smem_u32(&sm.done), 1);
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sm.tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = sm.tmem_base;

  // CTA -> (m half, batch, split)
  const int m_half = blockIdx.x & 1;
  const int bidx = (blockIdx.x >> 1) % p.batch;
  const int split = (blockIdx.x >> 1) / p.batch;
  const int c_begin = split * p.chunks_per_split;
  const int c_end = min(p.n_chunks, c_begin + p.chunks_per_split);
  const int n_sub = p.n_box / 64;
  const uint32_t stage_bytes = (uint32_t)(2 + n_sub) * kChunk * 128;

  if (warp == 4) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int c = c_begin; c < c_end; ++c, ++it) {
        const int st = it % kTnStages;
        if (!mbar_wait(smem_u32(&sm.empty[st]), ((it / kTnStages) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(smem_u32(&sm.full[st]), stage_bytes);
        for (int j = 0; j < 2; ++j)
          tma_load_3d(smem_u32(sm.a[st]) + j * kChunk * 128, &tmap_a, smem_u32(&sm.full[st]), m_half * 128 + j * 64,
                      bidx * p.a_head_step, c * kChunk);
        for (int j = 0; j < n_sub; ++j)
          tma_load_3d(smem_u32(sm.b[st]) + j * kChunk * 128, &tmap_b, smem_u32(&sm.full[st]), bidx * p.b_col_step + j * 64, 0,
                      c * kChunk);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const uint32_t idesc = make_idesc(kFmt, 1, 1, 128, p.n_box);
      uint32_t it = 0;
      bool ok = true;
      for (int c = c_begin; ok && c < c_end; ++c, ++it) {
        const int st = it % kTnStages;
        if (!mbar_wait(smem_u32(&sm.full[st]), (it / kTnStages) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk) {
          const uint64_t da = make_desc_sw128(smem_u32(sm.a[st]) + kk * 2048, kChunk * 128, 1024);
          const uint64_t db = make_desc_sw128(smem_u32(sm.b[st]) + kk * 2048, kChunk * 128, 1024);
          mma_ss(tbase, da, db, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(smem_u32(&sm.empty[st]));
      }
      if (ok) mma_commit(smem_u32(&sm.done));
    }
  } else {
    const int r = threadIdx.x;
    const uint32_t lane_base = tbase + ((uint32_t)(warp * 32) << 16);
    const bool have = c_end > c_begin;
    bool ok = true;
    if (have) {
      ok = mbar_wait(smem_u32(&sm.done), 0, abort_flag);
      tc_fence_after();
    }
    if (ok) {
      float* dst = p.partial + (((long long)split * p.batch + bidx) * 256 + m_half * 128 + r) * p.n_keep;
      for (int cc = 0; cc < p.n_keep / 32; ++cc) {
        uint32_t t[32];
        if (have) {
          tmem_ld32(lane_base + cc * 32, t);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        float4* d4 = reinterpret_cast<float4*>(dst + cc * 32);
#pragma unroll
        for (int v = 0; v < 8; ++v)
          d4[v] = make_float4(__uint_as_float(t[4 * v]), __uint_as_float(t[4 * v + 1]), __uint_as_float(t[4 * v + 2]),
                              __uint_as_float(t[4 * v + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (sm.abort_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { }
    __syncthreads();
  }
  if (warp == 5) tmem_dealloc(tbase, 256);
}

// out[b*out_b + m*out_m + n] = sum_s partial[s][b][m][n], splits added in order.
__global__ void __launch_bounds__(256) tn_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, int splits,
                                                        int batch, int n_keep, long long out_b, long long out_m) {
  const long long total = (long long)batch * 256 * n_keep;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += partial[(long long)s * total + i];
    const int n = (int)(i % n_keep);
    const int m = (int)((i / n_keep) % 256);
    const int b = (int)(i / ((long long)n_keep * 256));
    out[b * out_b + m * out_m + n] = acc;
  }
}

int tn_splits(long long T, int batch, int sms) {
  const int n_chunks = (int)((T + kChunk - 1) / kChunk);
  int splits = sms / (2 * batch);
  if (splits < 1) splits = 1;
  if (splits > 32) splits = 32;
  if (splits > n_chunks) splits = n_chunks > 0 ? n_chunks : 1;
  return splits;
}

}  // namespace

size_t sm100_gemm_tn_workspace_bytes(long long T, int batch, int n_keep, int sm_count) {
  return align_up((size_t)tn_splits(T, batch, sm_count > 0 ? sm_count : 148) * batch * 256 * n_keep * 4, 256);
}

int sm100_gemm_tn(const GemmTNArgs& g, cudaStream_t s) {
  if (g.T <= 0) {  // no tokens: the gradient is zero
    LaunchScope scope(kKCast, s);
    tn_reduce_kernel<<<256, 256, 0, s>>>(nullptr, g.out, 0, g.batch, g.n_keep, g.out_b, g.out_m);
    VAFA_LAUNCH_CHECK("tn_reduce_kernel");
    return 0;
  }
  if (!((g.n_box == 256 && g.n_keep == 256) || (g.n_box == 64 && g.n_keep == 32)))
    return fail(VAFA_ERR_UNSUPPORTED, "gemm_tn: n_box=%d n_keep=%d not supported", g.n_box, g.n_keep);
  const int sms = g.sm_count > 0 ? g.sm_count : 148;
  TnParams p;
  p.wait_limit = wait_limit_units();
  p.partial = (float*)g.workspace;
  p.n_chunks = (int)((g.T + kChunk - 1) / kChunk);
  p.splits = tn_splits(g.T, g.batch, sms);
  p.chunks_per_split = (p.n_chunks + p.splits - 1) / p.splits;
  p.batch = g.batch; p.n_box = g.n_box; p.n_keep = g.n_keep;
  p.a_head_step = g.a_heads > 1 ? 1 : 0;
  p.b_col_step = g.b_col_step;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = encode_tmap_rows(&ta, g.A, g.dtype, g.T, g.a_heads, 256, kChunk))) return rc;
  if ((rc = encode_tmap_rows(&tb, g.B, g.dtype, g.T, 1, g.b_width, kChunk))) return rc;
  const size_t smem = sizeof(TnSmem) + 1024;
  const int grid = 2 * g.batch * p.splits;
  {
    LaunchScope scope(kKAbsorbGemmTn, s);
    if (g.dtype == VAFA_BF16) {
      VAFA_CUDA_CHECK(cudaFuncSetAttribute(gemm_tn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      gemm_tn_kernel<__nv_bfloat16><<<grid, kTnThreads, smem, s>>>(ta, tb, p);
    } else {
      VAFA_CUDA_CHECK(cudaFuncSetAttribute(gemm_tn_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      gemm_tn_kernel<__half><<<grid, kTnThreads, smem, s>>>(ta, tb, p);
    }
  }
  VAFA_LAUNCH_CHECK("gemm_tn_kernel");
  LaunchScope scope(kKCast, s);
  tn_reduce_kernel<<<256, 256, 0, s>>>(p.partial, g.out, p.splits, g.batch, g.n_keep, g.out_b, g.out_m);
  VAFA_LAUNCH_CHECK("tn_reduce_kernel");
  return 0;
}

}  // namespace vafa

namespace vafa {
namespace {
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols) {
  __shared__ T tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;    // bx over columns, by over rows of `in`
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int j = ty; j < 32; j += 8)
    if (by + j < rows && bx + tx < cols) tile[j][tx] = in[(long long)(by + j) * cols + bx + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (bx + j < cols && by + tx < rows) out[(long long)(bx + j) * rows + by + tx] = tile[tx][j];
}
}  // namespace

// out[j][i] = in[i][j] for a rows x cols 16-bit matrix (out is cols x rows).
int sm100_transpose(const void* in, void* out, int rows, int cols, int dtype, cudaStream_t s) {
  LaunchScope scope(kKCast, s);
  dim3 grid((cols + 31) / 32, (rows + 31) / 32);
  if (dtype == VAFA_BF16)
    transpose_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, cols);
  else
    transpose_kernel<__half><<<grid, 256, 0, s>>>((const __half*)in, (__half*)out, rows, cols);
  VAFA_LAUNCH_CHECK("transpose_kernel");
  return 0;
}
}  // namespace vafa
