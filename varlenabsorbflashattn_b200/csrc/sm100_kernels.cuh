// tcgen05 / TMA kernels for sm_100a: host-side launchers.
#pragma once
#include "common.cuh"

namespace vafa {

// true when the tcgen05 kernels cover this shape and dtype
bool sm100_varlen_fwd_supported(const vafa_varlen_args* a);
bool sm100_varlen_bwd_supported(const vafa_varlen_args* a);

size_t sm100_varlen_fwd_workspace_bytes(const vafa_varlen_args* a);
size_t sm100_varlen_bwd_workspace_bytes(const vafa_varlen_args* a);
int sm100_varlen_fwd(const vafa_varlen_args* a, cudaStream_t s);
int sm100_varlen_bwd(const vafa_varlen_args* a, cudaStream_t s);
// forward with the library's built-in scratch array instead of a workspace
int sm100_varlen_fwd_noalloc(const vafa_varlen_args* a, cudaStream_t s);

// The two 128 x 128-tile backward kernels (dQ, then dK/dV) on prepared tile lists and (lse, delta).
struct Bwd128Launch {
  const void* q; const void* k; const void* v; const void* d_o;
  void* dq; void* dk; void* dv;
  const void* ld; long long ld_stride;
  const void* aug;  // fold array [total_q, H, 32] (dK/dV kernel)
  const void* hdr_dq; const void* items_dq; const void* hdr_dkv; const void* items_dkv;
  int total_q, total_k, H, D, dtype, sms;
  int H_kv;             // K/V heads (a divisor of H; H for plain multi-head attention)
  float scale;
  int32_t* status;
  int run_dq, run_dkv;  // which of the two kernels to launch
  float* dq_acc;        // fused backward only: fp32 [T_q, H, D] accumulator of dQ
};
int sm100_varlen_bwd128_launch(const Bwd128Launch& L, cudaStream_t s);
// One-pass backward (head dim 128): dK, dV and the dQ contributions of every score tile from one kernel over
// the dK/dV tile list, dQ summed in L.dq_acc by reductions in global memory and rounded by a second kernel.
int sm100_varlen_bwd_fused_launch(const Bwd128Launch& L, cudaStream_t s);

// One CTA waits, with the bounded wait every kernel uses, on an mbarrier that nobody arrives on; when the
// wait runs out it reports code 1 / site 900 through the status word and returns.
int sm100_selftest_bounded_wait(int32_t* status, cudaStream_t s);

// ---- absorb operator on the tcgen05 kernels ------------------------------------------------
// Attention core on a pre-projected u: axn[t,h,:] = softmax_h(scale * u[t,h,:] . X^T) . X, normalised,
// in the I/O dtype; lse[t,h] log2-domain.  Requires d_kv == 256, 16-bit dtype, H dividing 128.
struct AbsorbCoreArgs {
  const void* u;       // [T_q, H, 256]
  const void* x;       // [T_k, x_width], x_width <= 256 (missing columns read as zero)
  void* axn;           // [T_q, H, 256]
  float* lse;          // [T_q, H]
  const int32_t* cu_q;
  const int32_t* cu_k;
  int n_seg, total_q, total_k, H, dtype;
  float scale;
  int sm_count;
  void* workspace;
  int32_t* status;
  int x_width;
  int lists_built;     // the tile list was already built by sm100_absorb_core_fwd_lists() (ordered before this call)
};
size_t sm100_absorb_core_fwd_workspace_bytes(int total_q, int n_seg, int H);
int sm100_absorb_core_fwd(const AbsorbCoreArgs& a, cudaStream_t s);

// Backward of the attention core: dU [T_q,H,256] (scaled) and dX [T_k,256] from u, X, dAlphaX
// ([T_q,H,256], I/O dtype) and LD[t*H+h] = (lse, delta).  Needs H dividing 64.
struct AbsorbCoreBwdArgs {
  const void* u; const void* x; const void* dax; const void* ld;
  void* du; void* dx;
  const int32_t* cu_q; const int32_t* cu_k;
  int n_seg, total_q, total_k, H, dtype;
  float scale;
  int sm_count;
  void* workspace;
  int32_t* status;
  int x_width;         // row width of x and dx (<= 256)
  int lists_built;     // the tile lists were already built by sm100_absorb_core_bwd_lists()
  int which;           // 0: both kernels; 1: the dU kernel only; 2: the dX kernel only
};
size_t sm100_absorb_core_bwd_workspace_bytes(int total_q, int total_k, int n_seg, int H);
int sm100_absorb_core_bwd(const AbsorbCoreBwdArgs& a, cudaStream_t s);
// The tile lists depend on cu_seqlens only: these build them on their own (on any stream the caller
// orders before the core call), so that the single-CTA list builder runs beside the projections.
int sm100_absorb_core_fwd_lists(const AbsorbCoreArgs& a, cudaStream_t s);
int sm100_absorb_core_bwd_lists(const AbsorbCoreBwdArgs& a, cudaStream_t s);
// (lse, delta) rows of the absorb backward: a float2 array of n_pad entries followed by two planar float
// arrays of n_pad entries each (-lse and -delta * scale, for the dX kernel); n_pad = sm100_absorb_ld_pad().
inline long long sm100_absorb_ld_pad(long long n_rows) { return (n_rows + 128 + 3) & ~3LL; }
size_t sm100_absorb_ld_bytes(long long n_rows);
int sm100_absorb_ld(const void* o, const void* d_o, const float* lse, void* ld, long long n_rows, int D_H, float scale, int dtype,
                    cudaStream_t s);
int sm100_absorb_expand_wv(const void* w_v, void* bexp, int H, int D_H, int d_kv, int dtype, cudaStream_t s);

// C[M, ldc] (16-bit) = A[M, K] . B[K, N] with A rows densely packed (K = lda, a multiple of 256) and B
// row-major [K, N] (N a multiple of 256, row stride ldb = N).  diag_heads > 0: row m keeps only the
// 256/diag_heads columns of block (m % diag_heads) and writes them to C[m, 0 : 256/diag_heads]
// (per-head projection of head-stacked rows); N must then be 256.
struct GemmNNArgs {
  const void* A; const void* B; void* C;
  long long M; int N; int lda, ldb, ldc;
  int dtype; int diag_heads; int sm_count;
};
int sm100_gemm_nn_k256(const GemmNNArgs& g, cudaStream_t s);

// out[b*out_b + m*out_m + n] = sum_t A[t, (head b), m] * B[t, b*b_col_step + n], m < 256, n < n_keep
// (fp32 result, deterministic split over tokens).  A: [T, a_heads, 256] (a_heads = 1 or batch);
// B: [T, b_width].  (n_box, n_keep) is (256, 256) or (64, 32).
struct GemmTNArgs {
  const void* A; const void* B; float* out; void* workspace;
  long long T; int dtype; int a_heads; int batch; int n_box; int n_keep; int b_width; int b_col_step;
  long long out_b, out_m;
  int sm_count;
};
size_t sm100_gemm_tn_workspace_bytes(long long T, int batch, int n_keep, int sm_count);
int sm100_gemm_tn(const GemmTNArgs& g, cudaStream_t s);
int sm100_transpose(const void* in, void* out, int rows, int cols, int dtype, cudaStream_t s);

}  // namespace vafa
