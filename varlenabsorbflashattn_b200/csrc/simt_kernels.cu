// Scalar (SIMT) kernels: one warp per output row, lanes across the head dimension.
// fp32 arithmetic throughout, no shared memory, no atomics: results are run-to-run identical.
#include "simt_kernels.cuh"
#include "profile.cuh"

namespace vafa {

namespace {

constexpr int kMaxT = 16;  // head dim <= 32 * kMaxT = 512
constexpr int kWarpsPerBlock = 4;

struct SegInfo {
  int q0, Lq, k0, Lk;
};

__device__ __forceinline__ SegInfo load_seg(const int32_t* cu_q, const int32_t* cu_k, int seg) {
  SegInfo s;
  s.q0 = cu_q[seg];
  s.Lq = cu_q[seg + 1] - s.q0;
  s.k0 = cu_k[seg];
  s.Lk = cu_k[seg + 1] - s.k0;
  return s;
}

// ---- forward ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_fwd_kernel(SimtAttnParams p) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (w >= (long long)p.total_q * p.H) return;
  const int row = (int)(w / p.H), h = (int)(w % p.H);
  const int seg = find_segment(p.cu_q, p.n_seg, row);
  const SegInfo s = load_seg(p.cu_q, p.cu_k, seg);
  const int i = row - s.q0;
  int kend = p.causal ? min(s.Lk, i + s.Lk - s.Lq + 1) : s.Lk;
  const int nd = (p.D + 31) >> 5;
  const float c = p.scale * kLog2e;

  const T* q = (const T*)p.q + (int64_t)row * p.q_row + (int64_t)h * p.q_head;
  const T* kb = (const T*)p.k + (int64_t)s.k0 * p.k_row + (int64_t)h * p.k_head;
  const T* vb = (const T*)p.v + (int64_t)s.k0 * p.v_row + (int64_t)h * p.v_head;

  float qr[kMaxT], acc[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    const int d = lane + 32 * t;
    qr[t] = (t < nd && d < p.D) ? to_float(q[d]) : 0.f;
    acc[t] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j < kend; ++j) {
    const T* kr = kb + (int64_t)j * p.k_row;
    const T* vr = vb + (int64_t)j * p.v_row;
    float part = 0.f;
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) {
      const int d = lane + 32 * t;
      if (t < nd && d < p.D) part += qr[t] * to_float(kr[d]);
    }
    const float sc = warp_sum(part) * c;
    const float m_new = fmaxf(m, sc);
    const float corr = exp2f(m - m_new);
    const float pr = exp2f(sc - m_new);
    l = l * corr + pr;
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) {
      const int d = lane + 32 * t;
      if (t < nd && d < p.D) acc[t] = acc[t] * corr + pr * to_float(vr[d]);
    }
    m = m_new;
  }
  T* o = (T*)p.o + (int64_t)row * p.q_row + (int64_t)h * p.q_head;
  const bool dead = (kend <= 0) || !(l > 0.f);
  const float inv = dead ? 0.f : 1.f / l;
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    const int d = lane + 32 * t;
    if (t < nd && d < p.D) o[d] = from_float<T>(acc[t] * inv);
  }
  if (lane == 0) p.lse[(int64_t)row * p.H + h] = dead ? -INFINITY : m + log2f(l);
}

// ---- delta = rowsum(O * dO) --------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
simt_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, long long n_rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (w >= n_rows) return;
  const T* a = o + w * D;
  const T* b = d_o + w * D;
  float part = 0.f;
  for (int d = lane; d < D; d += 32) part += to_float(a[d]) * to_float(b[d]);
  part = warp_sum(part);
  if (lane == 0) delta[w] = part;
}

// ---- dQ ------------------------------------------------------------------------------------
template <typename T, typename TDO>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_dq_kernel(SimtAttnParams p) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (w >= (long long)p.total_q * p.H) return;
  const int row = (int)(w / p.H), h = (int)(w % p.H);
  const int seg = find_segment(p.cu_q, p.n_seg, row);
  const SegInfo s = load_seg(p.cu_q, p.cu_k, seg);
  const int i = row - s.q0;
  int kend = p.causal ? min(s.Lk, i + s.Lk - s.Lq + 1) : s.Lk;
  const int nd = (p.D + 31) >> 5;
  const float c = p.scale * kLog2e;

  const T* q = (const T*)p.q + (int64_t)row * p.q_row + (int64_t)h * p.q_head;
  const TDO* dor = (const TDO*)p.d_o + (int64_t)row * p.do_row + (int64_t)h * p.do_head;
  const T* kb = (const T*)p.k + (int64_t)s.k0 * p.k_row + (int64_t)h * p.k_head;
  const T* vb = (const T*)p.v + (int64_t)s.k0 * p.v_row + (int64_t)h * p.v_head;
  const float lse = p.lse[(int64_t)row * p.H + h];
  const float dl = p.delta[(int64_t)row * p.H + h];
  if (lse == -INFINITY) kend = 0;

  float qr[kMaxT], dr[kMaxT], acc[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    const int d = lane + 32 * t;
    const bool ok = (t < nd && d < p.D);
    qr[t] = ok ? to_float(q[d]) : 0.f;
    dr[t] = ok ? to_float(dor[d]) : 0.f;
    acc[t] = 0.f;
  }
  for (int j = 0; j < kend; ++j) {
    const T* kr = kb + (int64_t)j * p.k_row;
    const T* vr = vb + (int64_t)j * p.v_row;
    float kv[kMaxT];
    float ps = 0.f, pd = 0.f;
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) {
      const int d = lane + 32 * t;
      if (t < nd && d < p.D) {
        kv[t] = to_float(kr[d]);
        ps += qr[t] * kv[t];
        pd += dr[t] * to_float(vr[d]);
      } else {
        kv[t] = 0.f;
      }
    }
    const float sc = warp_sum(ps) * c;
    const float dp = warp_sum(pd);
    const float pr = exp2f(sc - lse);
    const float ds = pr * (dp - dl);
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) acc[t] += ds * kv[t];
  }
  T* dq = (T*)p.dq + (int64_t)row * p.q_row + (int64_t)h * p.q_head;
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) {
    const int d = lane + 32 * t;
    if (t < nd && d < p.D) dq[d] = from_float<T>(acc[t] * p.scale);
  }
}

// ---- dK, dV (or their head-summed combination when K/V rows are shared by all heads) --------
template <typename T, typename TDO>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_dkv_kernel(SimtAttnParams p) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_units = p.shared_kv ? (long long)p.total_k : (long long)p.total_k * p.H;
  if (w >= n_units) return;
  const int krow = p.shared_kv ? (int)w : (int)(w / p.H);
  const int h_first = p.shared_kv ? 0 : (int)(w % p.H);
  const int h_last = p.shared_kv ? p.H : h_first + 1;
  const int seg = find_segment(p.cu_k, p.n_seg, krow);
  const SegInfo s = load_seg(p.cu_q, p.cu_k, seg);
  const int j = krow - s.k0;
  const int i_start = p.causal ? max(0, j - (s.Lk - s.Lq)) : 0;
  const int nd = (p.D + 31) >> 5;
  const float c = p.scale * kLog2e;

  float tot[kMaxT];
#pragma unroll
  for (int t = 0; t < kMaxT; ++t) tot[t] = 0.f;

  for (int h = h_first; h < h_last; ++h) {
    const T* kr = (const T*)p.k + (int64_t)krow * p.k_row + (int64_t)h * p.k_head;
    const T* vr = (const T*)p.v + (int64_t)krow * p.v_row + (int64_t)h * p.v_head;
    float kreg[kMaxT], vreg[kMaxT], dka[kMaxT], dva[kMaxT];
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) {
      const int d = lane + 32 * t;
      const bool ok = (t < nd && d < p.D);
      kreg[t] = ok ? to_float(kr[d]) : 0.f;
      vreg[t] = ok ? to_float(vr[d]) : 0.f;
      dka[t] = 0.f;
      dva[t] = 0.f;
    }
    for (int i = i_start; i < s.Lq; ++i) {
      const int row = s.q0 + i;
      const float lse = p.lse[(int64_t)row * p.H + h];
      if (lse == -INFINITY) continue;
      const float dl = p.delta[(int64_t)row * p.H + h];
      const T* q = (const T*)p.q + (int64_t)row * p.q_row + (int64_t)h * p.q_head;
      const TDO* dor = (const TDO*)p.d_o + (int64_t)row * p.do_row + (int64_t)h * p.do_head;
      float qv[kMaxT], dv_[kMaxT];
      float ps = 0.f, pd = 0.f;
#pragma unroll
      for (int t = 0; t < kMaxT; ++t) {
        const int d = lane + 32 * t;
        if (t < nd && d < p.D) {
          qv[t] = to_float(q[d]);
          dv_[t] = to_float(dor[d]);
          ps += qv[t] * kreg[t];
          pd += dv_[t] * vreg[t];
        } else {
          qv[t] = 0.f;
          dv_[t] = 0.f;
        }
      }
      const float sc = warp_sum(ps) * c;
      const float dp = warp_sum(pd);
      const float pr = exp2f(sc - lse);
      const float ds = pr * (dp - dl);
#pragma unroll
      for (int t = 0; t < kMaxT; ++t) {
        dva[t] += pr * dv_[t];
        dka[t] += ds * qv[t];
      }
    }
    if (p.shared_kv) {
#pragma unroll
      for (int t = 0; t < kMaxT; ++t) tot[t] += dka[t] * p.scale + dva[t];
    } else {
      T* dk = (T*)p.dk + (int64_t)krow * p.k_row + (int64_t)h * p.k_head;
      T* dv = (T*)p.dv + (int64_t)krow * p.v_row + (int64_t)h * p.v_head;
#pragma unroll
      for (int t = 0; t < kMaxT; ++t) {
        const int d = lane + 32 * t;
        if (t < nd && d < p.D) {
          dk[d] = from_float<T>(dka[t] * p.scale);
          dv[d] = from_float<T>(dva[t]);
        }
      }
    }
  }
  if (p.shared_kv) {
    T* dk = (T*)p.dk + (int64_t)krow * p.k_row;
#pragma unroll
    for (int t = 0; t < kMaxT; ++t) {
      const int d = lane + 32 * t;
      if (t < nd && d < p.D) dk[d] = from_float<T>(tot[t]);
    }
  }
}

// ---- small dense products -------------------------------------------------------------------
template <typename TA, typename TB, typename TC>
__global__ void __launch_bounds__(256) simt_gemm_kernel(SimtGemm g) {
  __shared__ float As[16][17];
  __shared__ float Bs[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int n0 = blockIdx.x * 16, m0 = blockIdx.y * 16, b = blockIdx.z;
  const TA* A = (const TA*)g.A + (int64_t)b * g.a_b;
  const TB* B = (const TB*)g.B + (int64_t)b * g.b_b;
  float acc = 0.f;
  for (int k0 = 0; k0 < g.K; k0 += 16) {
    const int am = m0 + ty, ak = k0 + tx;
    As[ty][tx] = (am < g.M && ak < g.K) ? to_float(A[(int64_t)am * g.a_m + (int64_t)ak * g.a_k]) : 0.f;
    const int bk = k0 + ty, bn = n0 + tx;
    Bs[ty][tx] = (bk < g.K && bn < g.N) ? to_float(B[(int64_t)bk * g.b_k + (int64_t)bn * g.b_n]) : 0.f;
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) acc += As[ty][kk] * Bs[kk][tx];
    __syncthreads();
  }
  const int m = m0 + ty, n = n0 + tx;
  if (m < g.M && n < g.N) {
    TC* C = (TC*)g.C + (int64_t)b * g.c_b;
    C[(int64_t)m * g.c_m + (int64_t)n * g.c_n] = from_float<TC>(acc * g.alpha);
  }
}

// W_QK tile: 32 rows of W_Q against all of W_K for one head.  The general kernel above gives a CTA one
// 16 x 16 tile (8192 CTAs with 32 multiply-adds per thread for the production widths: 36 us for 0.13 GFLOP);
// here a thread owns output columns kv = tid, tid + 256, ... of all 32 rows, with W_K's slice of the head
// and the W_Q rows staged in shared memory 32 head-dim columns at a time.
constexpr int kWqkRows = 16;
template <typename T>
__global__ void __launch_bounds__(256) absorb_wqk_kernel(const T* __restrict__ w_q, const T* __restrict__ w_k, T* __restrict__ out,
                                                         int d_q, int d_kv, int H, int D_H) {
  __shared__ float ks[256][33];                          // [kv][dd]
  __shared__ __align__(16) float qs[32][kWqkRows];       // [dd][row]: a float4 serves four rows
  const int h = blockIdx.y, a0 = blockIdx.x * kWqkRows, tid = threadIdx.x;
  const bool vec = (D_H % 8) == 0;  // 16-byte loads (the launcher checks the bases)
  for (int kv0 = 0; kv0 < d_kv; kv0 += 256) {
    float acc[kWqkRows];
#pragma unroll
    for (int i = 0; i < kWqkRows; ++i) acc[i] = 0.f;
    for (int d0 = 0; d0 < D_H; d0 += 32) {
      __syncthreads();
      if (vec) {
        for (int i = tid; i < 256 * 4; i += 256) {
          const int kv = kv0 + (i >> 2), dd = d0 + (i & 3) * 8;
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (kv < d_kv && dd < D_H) v = *reinterpret_cast<const uint4*>(w_k + ((long long)kv * H + h) * D_H + dd);
          const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int e = 0; e < 8; ++e) ks[i >> 2][(i & 3) * 8 + e] = to_float(pv[e]);
        }
        if (tid < kWqkRows * 4) {
          const int a = a0 + (tid >> 2), dd = d0 + (tid & 3) * 8;
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (a < d_q && dd < D_H) v = *reinterpret_cast<const uint4*>(w_q + ((long long)a * H + h) * D_H + dd);
          const T* pv = reinterpret_cast<const T*>(&v);
#pragma unroll
          for (int e = 0; e < 8; ++e) qs[(tid & 3) * 8 + e][tid >> 2] = to_float(pv[e]);
        }
      } else {
        for (int i = tid; i < 256 * 32; i += 256) {
          const int kv = kv0 + (i >> 5), dd = d0 + (i & 31);
          ks[i >> 5][i & 31] = (kv < d_kv && dd < D_H) ? to_float(w_k[((long long)kv * H + h) * D_H + dd]) : 0.f;
        }
        for (int i = tid; i < kWqkRows * 32; i += 256) {
          const int a = a0 + (i >> 5), dd = d0 + (i & 31);
          qs[i & 31][i >> 5] = (a < d_q && dd < D_H) ? to_float(w_q[((long long)a * H + h) * D_H + dd]) : 0.f;
        }
      }
      __syncthreads();
#pragma unroll 8
      for (int dd = 0; dd < 32; ++dd) {
        const float kvv = ks[tid][dd];
        const float4* q4 = reinterpret_cast<const float4*>(qs[dd]);
#pragma unroll
        for (int i = 0; i < kWqkRows / 4; ++i) {
          const float4 q = q4[i];
          acc[4 * i + 0] = fmaf(q.x, kvv, acc[4 * i + 0]);
          acc[4 * i + 1] = fmaf(q.y, kvv, acc[4 * i + 1]);
          acc[4 * i + 2] = fmaf(q.z, kvv, acc[4 * i + 2]);
          acc[4 * i + 3] = fmaf(q.w, kvv, acc[4 * i + 3]);
        }
      }
    }
    const int kv = kv0 + tid;
    if (kv < d_kv) {
#pragma unroll
      for (int i = 0; i < kWqkRows; ++i)
        if (a0 + i < d_q) out[((long long)(a0 + i) * H + h) * d_kv + kv] = from_float<T>(acc[i]);
    }
  }
}

template <typename T>
__global__ void cast_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = from_float<T>(src[i]);
}

inline unsigned warp_grid(long long n_warps) {
  return (unsigned)((n_warps + kWarpsPerBlock - 1) / kWarpsPerBlock);
}

}  // namespace

#define DISPATCH_T(dtype, ...)                                          \
  switch (dtype) {                                                      \
    case VAFA_F32: { using T = float; __VA_ARGS__; break; }             \
    case VAFA_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }    \
    case VAFA_F16: { using T = __half; __VA_ARGS__; break; }            \
    default: return fail(VAFA_ERR_INVALID, "unknown dtype %d", dtype);  \
  }

int simt_attn_fwd(const SimtAttnParams& p, cudaStream_t s) {
  if (p.D > 32 * kMaxT) return fail(VAFA_ERR_UNSUPPORTED, "head dim %d > %d", p.D, 32 * kMaxT);
  const long long n = (long long)p.total_q * p.H;
  if (n == 0) return 0;
  LaunchScope scope(kKSimtFwd, s);
  DISPATCH_T(p.dtype, simt_fwd_kernel<T><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>(p));
  VAFA_LAUNCH_CHECK("simt_fwd_kernel");
  return 0;
}

int simt_attn_delta(const void* o, const void* d_o, float* delta, int rows, int H, int D, int dtype, cudaStream_t s) {
  const long long n = (long long)rows * H;
  if (n == 0) return 0;
  LaunchScope scope(kKSimtDelta, s);
  DISPATCH_T(dtype, simt_delta_kernel<T><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>((const T*)o, (const T*)d_o, delta, n, D));
  VAFA_LAUNCH_CHECK("simt_delta_kernel");
  return 0;
}

int simt_attn_dq(const SimtAttnParams& p, cudaStream_t s) {
  if (p.D > 32 * kMaxT) return fail(VAFA_ERR_UNSUPPORTED, "head dim %d > %d", p.D, 32 * kMaxT);
  const long long n = (long long)p.total_q * p.H;
  if (n == 0) return 0;
  LaunchScope scope(kKSimtDq, s);
  if (p.do_f32) {
    DISPATCH_T(p.dtype, simt_dq_kernel<T, float><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>(p));
  } else {
    DISPATCH_T(p.dtype, simt_dq_kernel<T, T><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>(p));
  }
  VAFA_LAUNCH_CHECK("simt_dq_kernel");
  return 0;
}

int simt_attn_dkv(const SimtAttnParams& p, cudaStream_t s) {
  if (p.D > 32 * kMaxT) return fail(VAFA_ERR_UNSUPPORTED, "head dim %d > %d", p.D, 32 * kMaxT);
  const long long n = p.shared_kv ? (long long)p.total_k : (long long)p.total_k * p.H;
  if (n == 0) return 0;
  LaunchScope scope(kKSimtDkv, s);
  if (p.do_f32) {
    DISPATCH_T(p.dtype, simt_dkv_kernel<T, float><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>(p));
  } else {
    DISPATCH_T(p.dtype, simt_dkv_kernel<T, T><<<warp_grid(n), kWarpsPerBlock * 32, 0, s>>>(p));
  }
  VAFA_LAUNCH_CHECK("simt_dkv_kernel");
  return 0;
}

namespace {
template <typename TA, typename TB>
int gemm_c(const SimtGemm& g, dim3 grid, cudaStream_t s) {
  switch (g.c_type) {
    case VAFA_F32: simt_gemm_kernel<TA, TB, float><<<grid, 256, 0, s>>>(g); break;
    case VAFA_BF16: simt_gemm_kernel<TA, TB, __nv_bfloat16><<<grid, 256, 0, s>>>(g); break;
    case VAFA_F16: simt_gemm_kernel<TA, TB, __half><<<grid, 256, 0, s>>>(g); break;
    default: return fail(VAFA_ERR_INVALID, "unknown dtype %d", g.c_type);
  }
  return 0;
}
template <typename TA>
int gemm_b(const SimtGemm& g, dim3 grid, cudaStream_t s) {
  switch (g.b_type) {
    case VAFA_F32: return gemm_c<TA, float>(g, grid, s);
    case VAFA_BF16: return gemm_c<TA, __nv_bfloat16>(g, grid, s);
    case VAFA_F16: return gemm_c<TA, __half>(g, grid, s);
    default: return fail(VAFA_ERR_INVALID, "unknown dtype %d", g.b_type);
  }
}
}  // namespace

int simt_gemm(const SimtGemm& g, cudaStream_t s) {
  if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return 0;
  dim3 grid((g.N + 15) / 16, (g.M + 15) / 16, g.batch);
  if (grid.y > 65535 || grid.z > 65535) return fail(VAFA_ERR_UNSUPPORTED, "simt_gemm grid too large");
  int rc;
  LaunchScope scope(kKSimtGemm, s);
  switch (g.a_type) {
    case VAFA_F32: rc = gemm_b<float>(g, grid, s); break;
    case VAFA_BF16: rc = gemm_b<__nv_bfloat16>(g, grid, s); break;
    case VAFA_F16: rc = gemm_b<__half>(g, grid, s); break;
    default: return fail(VAFA_ERR_INVALID, "unknown dtype %d", g.a_type);
  }
  if (rc) return rc;
  VAFA_LAUNCH_CHECK("simt_gemm_kernel");
  return 0;
}

int absorb_wqk(const void* w_q, const void* w_k, void* w_qk, int d_q, int d_kv, int H, int D_H, int dtype, cudaStream_t s) {
  if (d_q <= 0 || d_kv <= 0 || H <= 0) return 0;
  if (H > 65535) return fail(VAFA_ERR_UNSUPPORTED, "absorb_wqk: %d heads", H);
  if (((reinterpret_cast<uintptr_t>(w_q) | reinterpret_cast<uintptr_t>(w_k)) & 15) != 0)
    return fail(VAFA_ERR_INVALID, "absorb_wqk: weights must be 16-byte aligned");
  const dim3 grid((d_q + kWqkRows - 1) / kWqkRows, H);
  LaunchScope scope(kKSimtGemm, s);
  if (dtype == VAFA_BF16)
    absorb_wqk_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)w_q, (const __nv_bfloat16*)w_k, (__nv_bfloat16*)w_qk, d_q, d_kv, H, D_H);
  else if (dtype == VAFA_F16)
    absorb_wqk_kernel<__half><<<grid, 256, 0, s>>>((const __half*)w_q, (const __half*)w_k, (__half*)w_qk, d_q, d_kv, H, D_H);
  else
    return fail(VAFA_ERR_UNSUPPORTED, "absorb_wqk: 16-bit weights only");
  VAFA_LAUNCH_CHECK("absorb_wqk_kernel");
  return 0;
}

int cast_from_f32(const float* src, void* dst, size_t n, int dtype, cudaStream_t s) {
  if (n == 0) return 0;
  const unsigned grid = (unsigned)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
  LaunchScope scope(kKCast, s);
  DISPATCH_T(dtype, cast_kernel<T><<<grid, 256, 0, s>>>(src, (T*)dst, n));
  VAFA_LAUNCH_CHECK("cast_kernel");
  return 0;
}

}  // namespace vafa
