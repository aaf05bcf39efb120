// Scalar (SIMT) CUDA kernels: any dtype, any head dim up to 512, fp32 arithmetic.
// They serve the shapes the tcgen05 kernels do not cover (fp32 I/O, head dims other than
// 64/128) and the small dense products of the absorb operator's prologue and epilogue.
#pragma once
#include "common.cuh"

namespace vafa {

struct SimtAttnParams {
  const void* q; const void* k; const void* v;
  void* o; float* lse;
  const void* d_o; const float* delta;
  void* dq; void* dk; void* dv;
  const int32_t* cu_q; const int32_t* cu_k;
  int n_seg, total_q, total_k, H, D;
  // strides in elements
  int64_t q_row, q_head;     // q, o, dq
  int64_t k_row, k_head;     // k, dk
  int64_t v_row, v_head;     // v, dv
  int64_t do_row, do_head;   // d_o
  int causal;
  float scale;
  int shared_kv;  // 1: one K/V row set for all heads; backward writes sum over heads of
                  // (scale*dK_h + dV_h) into dk [total_k, D]
  int dtype;      // q/k/v/o/dq/dk/dv
  int do_f32;     // 1: d_o is fp32 regardless of dtype
};

int simt_attn_fwd(const SimtAttnParams& p, cudaStream_t s);
int simt_attn_delta(const void* o, const void* d_o, float* delta, int rows, int H, int D, int dtype, cudaStream_t s);
int simt_attn_dq(const SimtAttnParams& p, cudaStream_t s);
int simt_attn_dkv(const SimtAttnParams& p, cudaStream_t s);

// C[b][m][n] = alpha * sum_k A[b][m][k] * B[b][k][n]; strides in elements; fp32 accumulate.
struct SimtGemm {
  const void* A; const void* B; void* C;
  int a_type, b_type, c_type;  // vafa_dtype
  int M, N, K, batch;
  int64_t a_m, a_k, a_b;
  int64_t b_k, b_n, b_b;
  int64_t c_m, c_n, c_b;
  float alpha;
};
int simt_gemm(const SimtGemm& g, cudaStream_t s);

int cast_from_f32(const float* src, void* dst, size_t n, int dtype, cudaStream_t s);

// W_QK[a, h, kv] = sum_dd W_Q[a, h, dd] * W_K[kv, h, dd]: the per-head product of the two absorbed
// projections, [d_q, H, d_kv] in the weights' 16-bit dtype (fp32 accumulation).
int absorb_wqk(const void* w_q, const void* w_k, void* w_qk, int d_q, int d_kv, int H, int D_H, int dtype, cudaStream_t s);

}  // namespace vafa
