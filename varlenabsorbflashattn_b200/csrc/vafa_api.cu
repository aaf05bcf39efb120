// C ABI of libvafa_b200.so: argument checks, implementation choice, workspace carving.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "simt_kernels.cuh"
#include "sm100_kernels.cuh"

namespace vafa {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<long long> g_wait_limit_cycles{4000000000LL};  // about two seconds at 2 GHz

int wait_limit_units() {
  const long long u = (g_wait_limit_cycles.load(std::memory_order_relaxed) + 65535) >> 16;
  return (int)(u < 1 ? 1 : (u > 0x7fffffffLL ? 0x7fffffffLL : u));
}

static std::atomic<int> g_varlen_bwd_mode{0};
int varlen_bwd_mode() { return g_varlen_bwd_mode.load(std::memory_order_relaxed); }

namespace {

bool valid_dtype(int d) { return d == VAFA_F32 || d == VAFA_BF16 || d == VAFA_F16; }

int check_varlen(const vafa_varlen_args* a, bool bwd) {
  if (!a) return fail(VAFA_ERR_INVALID, "null args");
  if (!valid_dtype(a->dtype)) return fail(VAFA_ERR_INVALID, "bad dtype %d", a->dtype);
  if (a->n_seg < 1 || a->total_q < 0 || a->total_k < 0 || a->num_heads < 1)
    return fail(VAFA_ERR_INVALID, "bad sizes n_seg=%d T_q=%d T_k=%d H=%d", a->n_seg, a->total_q, a->total_k, a->num_heads);
  const int D = a->head_dim;
  if (!(D == 16 || D == 32 || D == 64 || D == 128 || D == 256))
    return fail(VAFA_ERR_UNSUPPORTED, "head_dim %d not supported (16/32/64/128/256)", D);
  if (!a->cu_seqlens_q || !a->cu_seqlens_k) return fail(VAFA_ERR_INVALID, "null cu_seqlens");
  if (a->total_q > 0 && (!a->q || !a->o || !a->lse)) return fail(VAFA_ERR_INVALID, "null q/o/lse");
  if (a->total_k > 0 && (!a->k || !a->v)) return fail(VAFA_ERR_INVALID, "null k/v");
  if (bwd) {
    if (a->total_q > 0 && (!a->d_o || !a->dq)) return fail(VAFA_ERR_INVALID, "null d_o/dq");
    if (a->total_k > 0 && (!a->dk || !a->dv)) return fail(VAFA_ERR_INVALID, "null dk/dv");
  }
  if (a->split_k_block < 0 || (a->split_k_block % 128) != 0)
    return fail(VAFA_ERR_INVALID, "split_k_block %d must be 0 or a multiple of 128", a->split_k_block);
  if (a->num_kv_heads < 0 || (a->num_kv_heads > 0 && (a->num_heads % a->num_kv_heads) != 0))
    return fail(VAFA_ERR_INVALID, "num_kv_heads %d must divide num_heads %d", a->num_kv_heads, a->num_heads);
  return 0;
}

// grouped-query attention (fewer K/V heads than query heads) exists on the tensor-core kernels only
bool is_gqa(const vafa_varlen_args* a) { return a->num_kv_heads > 0 && a->num_kv_heads != a->num_heads; }

bool varlen_fwd_tc_ok(const vafa_varlen_args* a) { return sm100_varlen_fwd_supported(a); }
bool varlen_bwd_tc_ok(const vafa_varlen_args* a) { return sm100_varlen_bwd_supported(a); }

// 0 = simt, 1 = tcgen05, <0 error
int pick_impl(int impl, bool tc_ok, const char* what) {
  if (impl == VAFA_IMPL_SIMT) return 0;
  if (impl == VAFA_IMPL_TCGEN05) {
    if (!tc_ok) return fail(VAFA_ERR_UNSUPPORTED, "%s: shape/dtype not covered by the tcgen05 kernels", what);
    return 1;
  }
  if (impl != VAFA_IMPL_AUTO) return fail(VAFA_ERR_INVALID, "bad impl %d", impl);
  return tc_ok ? 1 : 0;
}

SimtAttnParams simt_from_varlen(const vafa_varlen_args* a) {
  SimtAttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = a->q; p.k = a->k; p.v = a->v; p.o = a->o; p.lse = a->lse;
  p.d_o = a->d_o; p.dq = a->dq; p.dk = a->dk; p.dv = a->dv;
  p.cu_q = a->cu_seqlens_q; p.cu_k = a->cu_seqlens_k;
  p.n_seg = a->n_seg; p.total_q = a->total_q; p.total_k = a->total_k; p.H = a->num_heads; p.D = a->head_dim;
  const int64_t hd = (int64_t)a->num_heads * a->head_dim;
  p.q_row = p.k_row = p.v_row = p.do_row = hd;
  p.q_head = p.k_head = p.v_head = p.do_head = a->head_dim;
  p.causal = a->causal; p.scale = a->scale; p.shared_kv = 0; p.dtype = a->dtype; p.do_f32 = 0;
  return p;
}

int need_ws(const void* ws, size_t have, size_t need) {
  if (need == 0) return 0;
  if (!ws || have < need) return fail(VAFA_ERR_WORKSPACE, "workspace too small: have %zu, need %zu", have, need);
  if ((reinterpret_cast<uintptr_t>(ws) & 255) != 0) return fail(VAFA_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  return 0;
}

// ---- absorb: sizes of the pieces ---------------------------------------------------------
struct AbsorbSizes {
  size_t p, u, axn;               // saved (I/O dtype)
  size_t dax, delta, du, dp;      // backward scratch
};

AbsorbSizes absorb_sizes(const vafa_absorb_args* a) {
  AbsorbSizes z;
  const size_t es = elem_size(a->dtype);
  const size_t tq = (size_t)a->total_q, H = a->num_heads, dh = a->head_dim, dkv = a->d_kv;
  z.p = align_up(tq * H * dh * es, 256);
  z.u = align_up(tq * H * dkv * es, 256);
  z.axn = align_up(tq * H * dkv * es, 256);
  z.dax = align_up(tq * H * dkv * 4, 256);
  z.delta = align_up(tq * H * 4, 256);
  z.du = align_up(tq * H * dkv * es, 256);
  z.dp = align_up(tq * H * dh * es, 256);
  return z;
}

// Row width of x / dx: d_kv unless the caller says its rows are narrower.
int x_width_of(const vafa_absorb_args* a) { return a->x_width > 0 ? a->x_width : a->d_kv; }

int check_absorb(const vafa_absorb_args* a, bool bwd, bool inner) {
  if (!a) return fail(VAFA_ERR_INVALID, "null args");
  if (!valid_dtype(a->dtype)) return fail(VAFA_ERR_INVALID, "bad dtype %d", a->dtype);
  if (a->n_seg < 1 || a->total_q < 0 || a->total_k < 0 || a->num_heads < 1 || a->d_kv < 1 || (!inner && a->d_q < 1))
    return fail(VAFA_ERR_INVALID, "bad sizes");
  const int D = a->head_dim;
  if (!(D == 16 || D == 32 || D == 64 || D == 128 || D == 256))
    return fail(VAFA_ERR_UNSUPPORTED, "D_H %d not supported (16/32/64/128/256)", D);
  if (a->d_kv > 512) return fail(VAFA_ERR_UNSUPPORTED, "d_kv %d > 512", a->d_kv);
  if (!a->cu_seqlens_q || !a->cu_seqlens_k) return fail(VAFA_ERR_INVALID, "null cu_seqlens");
  if (!a->w_v || (!inner && (!a->w_q || !a->w_k))) return fail(VAFA_ERR_INVALID, "null weights");
  if (a->total_q > 0 && (!a->q_raw || !a->o || !a->lse || !a->saved)) return fail(VAFA_ERR_INVALID, "null q_raw/o/lse/saved");
  if (a->total_k > 0 && !a->x) return fail(VAFA_ERR_INVALID, "null x");
  if (bwd) {
    if (!a->dw) return fail(VAFA_ERR_INVALID, "null dw");
    if (a->total_q > 0 && (!a->d_o || !a->dq_raw)) return fail(VAFA_ERR_INVALID, "null d_o/dq_raw");
    if (a->total_k > 0 && !a->dx) return fail(VAFA_ERR_INVALID, "null dx");
  }
  return 0;
}

// attention core of the absorb operator on the SIMT kernels: q = u [T_q,H,d_kv], k = v = X.
SimtAttnParams simt_from_absorb(const vafa_absorb_args* a, const void* u, void* axn) {
  SimtAttnParams p;
  memset(&p, 0, sizeof(p));
  p.q = u; p.k = a->x; p.v = a->x; p.o = axn; p.lse = a->lse;
  p.cu_q = a->cu_seqlens_q; p.cu_k = a->cu_seqlens_k;
  p.n_seg = a->n_seg; p.total_q = a->total_q; p.total_k = a->total_k; p.H = a->num_heads; p.D = a->d_kv;
  p.q_row = (int64_t)a->num_heads * a->d_kv; p.q_head = a->d_kv;
  p.k_row = p.v_row = a->d_kv; p.k_head = p.v_head = 0;
  p.do_row = p.q_row; p.do_head = p.q_head;
  p.causal = 0; p.scale = a->scale; p.shared_kv = 1; p.dtype = a->dtype; p.do_f32 = 1;
  return p;
}

// Which parts of the absorb forward run on the tcgen05 kernels.
struct AbsorbFast {
  bool core;      // attention over X: 16-bit, d_kv == 256, H divides 128
  bool prologue;  // u = q_raw (W_Q W_K^T): core && d_q a multiple of 256
  bool epilogue;  // O = axn W_V per head: core && H * D_H == 256 && D_H >= 32
};

AbsorbFast absorb_fast(const vafa_absorb_args* a, bool inner) {
  AbsorbFast f{false, false, false};
  if (a->impl == VAFA_IMPL_SIMT) return f;
  const int H = a->num_heads;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  f.core = (a->dtype == VAFA_BF16 || a->dtype == VAFA_F16) && a->d_kv == 256 && H >= 1 && H <= 128 && (128 % H) == 0 &&
           a->total_q > 0 && a->total_k > 0 && a->scale > 0.f && al(a->q_raw) && al(a->x) && al(a->o) && al(a->saved);
  f.prologue = f.core && !inner && a->d_q >= 256 && a->d_q % 256 == 0 && al(a->w_q) && al(a->w_k);
  f.epilogue = f.core && H * a->head_dim == 256 && a->head_dim >= 32 && al(a->w_v);
  return f;
}

// A second stream per device for the tile-list builders of the absorb operator.  The lists depend on
// cu_seqlens only and their builder is latency-bound on one or two SMs, so it runs beside the
// projections instead of in front of the attention kernels: fork() orders the side stream after
// everything already queued on the caller's stream, join() orders the caller's stream after the side
// stream.  Both are event waits (legal inside a stream capture, where the side stream joins the capture
// and is rejoined before the call returns).  Created on first use; no device memory is allocated.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t forked = nullptr, joined = nullptr;
};
constexpr int kMaxSideDevices = 64;
std::mutex g_side_mu;
SideStream g_side[kMaxSideDevices];

int side_fork(cudaStream_t s, SideStream** out) {
  int dev = -1;
  VAFA_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxSideDevices) return fail(VAFA_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_side_mu);
  SideStream& ss = g_side[dev];
  if (ss.stream == nullptr) {
    VAFA_CUDA_CHECK(cudaStreamCreateWithFlags(&ss.stream, cudaStreamNonBlocking));
    VAFA_CUDA_CHECK(cudaEventCreateWithFlags(&ss.forked, cudaEventDisableTiming));
    VAFA_CUDA_CHECK(cudaEventCreateWithFlags(&ss.joined, cudaEventDisableTiming));
  }
  // record and wait under one lock: a wait refers to the latest record of its event
  VAFA_CUDA_CHECK(cudaEventRecord(ss.forked, s));
  VAFA_CUDA_CHECK(cudaStreamWaitEvent(ss.stream, ss.forked, 0));
  *out = &ss;
  return 0;
}

// Marks the end of this call's work on the side stream.  The later wait may see a newer record of the
// same event (another call's): the side stream runs in order, so that one is behind this call's work too.
int side_done(SideStream* ss) {
  std::lock_guard<std::mutex> lk(g_side_mu);
  VAFA_CUDA_CHECK(cudaEventRecord(ss->joined, ss->stream));
  return 0;
}

int side_join(cudaStream_t s, SideStream* ss) {
  std::lock_guard<std::mutex> lk(g_side_mu);
  VAFA_CUDA_CHECK(cudaStreamWaitEvent(s, ss->joined, 0));
  return 0;
}

// Rejoins the side stream on every way out of a call (an error return included: a stream capture must
// not end with the side stream still forked).
struct SideGuard {
  cudaStream_t s;
  SideStream* ss = nullptr;
  explicit SideGuard(cudaStream_t stream) : s(stream) {}
  int join() {
    SideStream* t = ss;
    ss = nullptr;
    return t ? side_join(s, t) : 0;
  }
  ~SideGuard() { join(); }
};

size_t absorb_fwd_ws_bytes(const vafa_absorb_args* a, bool inner) {
  const AbsorbFast f = absorb_fast(a, inner);
  size_t n = 0;
  if (f.prologue) n += align_up((size_t)a->d_q * a->num_heads * a->d_kv * elem_size(a->dtype), 256);
  if (f.core) n += sm100_absorb_core_fwd_workspace_bytes(a->total_q, a->n_seg, a->num_heads);
  return n;
}

int absorb_forward(const vafa_absorb_args* a, bool inner, cudaStream_t s) {
  const AbsorbSizes z = absorb_sizes(a);
  const AbsorbFast fast = absorb_fast(a, inner);
  char* sv = (char*)a->saved;
  char* ws = (char*)a->workspace;
  const int H = a->num_heads, dh = a->head_dim, dkv = a->d_kv, Tq = a->total_q;
  const void* u;
  void* axn;
  int rc;
  // the tile list is built on the side stream while the projection runs
  SideGuard side(s);
  AbsorbCoreArgs c{nullptr, a->x, nullptr, a->lse, a->cu_seqlens_q, a->cu_seqlens_k, a->n_seg, Tq, a->total_k, H, a->dtype,
                   a->scale, a->sm_count, nullptr, a->status, x_width_of(a), 0};
  if (fast.core) {
    c.workspace = ws + ((!inner && fast.prologue) ? align_up((size_t)a->d_q * H * dkv * elem_size(a->dtype), 256) : 0);
    if (!inner) {
      if ((rc = side_fork(s, &side.ss))) return rc;
      rc = sm100_absorb_core_fwd_lists(c, side.ss->stream);
      const int rd = side_done(side.ss);
      if (rc || rd) return rc ? rc : rd;
      c.lists_built = 1;
    }
  }
  if (inner) {
    u = a->q_raw;
    axn = sv;
  } else if (fast.prologue) {
    // W_QK[a, h, kv] = sum_dd W_Q[a,h,dd] W_K[kv,h,dd]  (tiny), then u = q_raw . W_QK as one product
    void* wqk = ws;
    ws += align_up((size_t)a->d_q * H * dkv * elem_size(a->dtype), 256);
    if ((rc = absorb_wqk(a->w_q, a->w_k, wqk, a->d_q, dkv, H, dh, a->dtype, s))) return rc;
    void* ub = sv + z.p;
    axn = sv + z.p + z.u;
    GemmNNArgs g{a->q_raw, wqk, ub, Tq, H * dkv, a->d_q, H * dkv, H * dkv, a->dtype, 0, a->sm_count};
    if ((rc = sm100_gemm_nn_k256(g, s))) return rc;
    u = ub;
  } else {
    void* p = sv;
    void* ub = sv + z.p;
    axn = sv + z.p + z.u;
    // p = q_raw W_Q                      [T_q, H*D_H]
    SimtGemm g1{a->q_raw, a->w_q, p, a->dtype, a->dtype, a->dtype, Tq, H * dh, a->d_q, 1,
                a->d_q, 1, 0, (int64_t)H * dh, 1, 0, (int64_t)H * dh, 1, 0, 1.f};
    if ((rc = simt_gemm(g1, s))) return rc;
    // u_h = p_h W_K_h^T                  [T_q, H, d_kv]; batch over heads
    SimtGemm g2{p, a->w_k, ub, a->dtype, a->dtype, a->dtype, Tq, dkv, dh, H,
                (int64_t)H * dh, 1, dh, 1, (int64_t)H * dh, dh, (int64_t)H * dkv, 1, dkv, 1.f};
    if ((rc = simt_gemm(g2, s))) return rc;
    u = ub;
  }
  if ((rc = side.join())) return rc;
  if (fast.core) {
    c.u = u;
    c.axn = axn;
    if ((rc = sm100_absorb_core_fwd(c, s))) return rc;
  } else {
    SimtAttnParams p = simt_from_absorb(a, u, axn);
    if ((rc = simt_attn_fwd(p, s))) return rc;
  }
  if (fast.epilogue) {
    // rows (t, h) of axn against all of W_V, keeping for each row the D_H columns of its own head
    GemmNNArgs g{axn, a->w_v, a->o, (long long)Tq * H, H * dh, dkv, H * dh, dh, a->dtype, H, a->sm_count};
    return sm100_gemm_nn_k256(g, s);
  }
  // O_h = axn_h W_V_h                    [T_q, H, D_H]; batch over heads
  SimtGemm g3{axn, a->w_v, a->o, a->dtype, a->dtype, a->dtype, Tq, dh, dkv, H,
              (int64_t)H * dkv, 1, dkv, (int64_t)H * dh, 1, dh, (int64_t)H * dh, 1, dh, 1.f};
  return simt_gemm(g3, s);
}

// Extra backward scratch of the tcgen05 path, placed after the regions both paths share.
struct AbsorbBwdExtra {
  size_t ld, bexp, sched, tn, wqt;
};

AbsorbBwdExtra absorb_bwd_extra(const vafa_absorb_args* a) {
  AbsorbBwdExtra x;
  const size_t H = a->num_heads;
  x.ld = align_up(sm100_absorb_ld_bytes((long long)a->total_q * H), 256);
  x.bexp = align_up(H * a->head_dim * H * a->d_kv * elem_size(a->dtype), 256);
  x.sched = sm100_absorb_core_bwd_workspace_bytes(a->total_q, a->total_k, a->n_seg, a->num_heads);
  const size_t t1 = sm100_gemm_tn_workspace_bytes(a->total_q, a->num_heads, 32, a->sm_count);
  const int q_chunks = a->d_q >= 256 ? a->d_q / 256 : 1;
  const size_t t2 = sm100_gemm_tn_workspace_bytes(a->total_q, q_chunks, 256, a->sm_count);
  x.tn = t1 > t2 ? t1 : t2;
  x.wqt = align_up((size_t)256 * (a->d_q > 256 ? a->d_q : 256) * elem_size(a->dtype), 256);
  return x;
}

bool absorb_bwd_core_fast(const vafa_absorb_args* a, bool inner) {
  const AbsorbFast f = absorb_fast(a, inner);
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return f.core && f.epilogue && (64 % a->num_heads) == 0 && al(a->d_o) && al(a->dx) && al(a->dq_raw);
}

// phase: 0 = the whole backward; 1 = everything the weight gradients need (and du); 2 = the rest (dX and
// dq_raw), reading what phase 1 left in the workspace.  Only the tensor-core chain can be cut: on the
// other paths phase 1 is the whole backward and phase 2 nothing.
int absorb_backward(const vafa_absorb_args* a, bool inner, int phase, cudaStream_t s) {
  const AbsorbSizes z = absorb_sizes(a);
  char* sv = (char*)a->saved;
  char* ws = (char*)a->workspace;
  const int H = a->num_heads, dh = a->head_dim, dkv = a->d_kv, Tq = a->total_q, dq = a->d_q;
  const void* u = inner ? a->q_raw : (const void*)(sv + z.p);
  const void* p = inner ? nullptr : (const void*)sv;
  void* axn = inner ? (void*)sv : (void*)(sv + z.p + z.u);
  float* dax = (float*)ws;
  float* delta = (float*)(ws + z.dax);
  void* du = inner ? a->dq_raw : (void*)(ws + z.dax + z.delta);
  void* dp = ws + z.dax + z.delta + z.du;
  float* dWQ = a->dw;
  float* dWK = inner ? nullptr : a->dw + (size_t)dq * H * dh;
  float* dWV = inner ? a->dw : a->dw + (size_t)(dq + dkv) * H * dh;
  int rc;
  // weight-gradient chain on the tensor-core GEMMs: needs the dU/dX fast path's preconditions, D_H = 32
  // (the 64-column box trick of the token reductions) and, for the full operator, d_q = 256
  const bool fast_chain = absorb_bwd_core_fast(a, inner) && dh == 32 && (inner || (dq >= 256 && dq % 256 == 0));
  const bool cut = fast_chain && !inner && phase != 0;
  if (phase == 2 && !cut) return 0;
  // tile lists of the dU and dX kernels: built on the side stream beside the products below
  SideGuard side(s);
  AbsorbCoreBwdArgs cb{u, a->x, dax, nullptr, du, a->dx, a->cu_seqlens_q, a->cu_seqlens_k, a->n_seg, Tq, a->total_k, H,
                       a->dtype, a->scale, a->sm_count, nullptr, a->status, x_width_of(a), 0, 0};
  if (cut && phase == 2) {
    // the tile lists, the (lse, delta) rows, dax, du and dp are where phase 1 left them
    const AbsorbBwdExtra x = absorb_bwd_extra(a);
    char* ex = ws + z.dax + z.delta + z.du + z.dp;
    cb.workspace = ex + x.ld + x.bexp;
    cb.ld = ex;
    cb.lists_built = 1;
    cb.which = 2;
    if ((rc = sm100_absorb_core_bwd(cb, s))) return rc;
    void* wqt = ex + x.ld + x.bexp + x.sched + x.tn;
    if ((rc = sm100_transpose(a->w_q, wqt, dq, H * dh, a->dtype, s))) return rc;
    GemmNNArgs gq{dp, wqt, a->dq_raw, Tq, dq, H * dh, dq, dq, a->dtype, 0, a->sm_count};
    return sm100_gemm_nn_k256(gq, s);
  }
  if (absorb_bwd_core_fast(a, inner)) {
    const AbsorbBwdExtra x = absorb_bwd_extra(a);
    cb.workspace = ws + z.dax + z.delta + z.du + z.dp + x.ld + x.bexp;
    if ((rc = side_fork(s, &side.ss))) return rc;
    rc = sm100_absorb_core_bwd_lists(cb, side.ss->stream);
    const int rd = side_done(side.ss);
    if (rc || rd) return rc ? rc : rd;
    cb.lists_built = 1;
  }
  if (!inner && absorb_fast(a, false).prologue) {
    // the tcgen05 prologue goes straight to u; the weight-gradient chain below needs p = q_raw W_Q
    if (fast_chain) {
      GemmNNArgs gp{a->q_raw, a->w_q, sv, Tq, H * dh, dq, H * dh, H * dh, a->dtype, 0, a->sm_count};
      if ((rc = sm100_gemm_nn_k256(gp, s))) return rc;
    } else {
      SimtGemm gp{a->q_raw, a->w_q, sv, a->dtype, a->dtype, a->dtype, Tq, H * dh, dq, 1,
                  dq, 1, 0, (int64_t)H * dh, 1, 0, (int64_t)H * dh, 1, 0, 1.f};
      if ((rc = simt_gemm(gp, s))) return rc;
    }
  }
  if (absorb_bwd_core_fast(a, inner)) {
    // tcgen05 path: dAlphaX = dO . Bexp (one dense product over all heads), then the dU and dX kernels
    const AbsorbBwdExtra x = absorb_bwd_extra(a);
    char* ex = ws + z.dax + z.delta + z.du + z.dp;
    void* ld = ex;
    void* bexp = ex + x.ld;
    if ((rc = sm100_absorb_expand_wv(a->w_v, bexp, H, dh, dkv, a->dtype, s))) return rc;
    GemmNNArgs gd{a->d_o, bexp, dax, Tq, H * dkv, H * dh, H * dkv, H * dkv, a->dtype, 0, a->sm_count};
    if ((rc = sm100_gemm_nn_k256(gd, s))) return rc;
    if ((rc = sm100_absorb_ld(a->o, a->d_o, a->lse, ld, (long long)Tq * H, dh, a->scale, a->dtype, s))) return rc;
    cb.ld = ld;
    cb.which = cut ? 1 : 0;
    if ((rc = side.join())) return rc;
    if ((rc = sm100_absorb_core_bwd(cb, s))) return rc;
  } else {
    // dax_h = dO_h W_V_h^T                  fp32 [T_q, H, d_kv]
    SimtGemm g1{a->d_o, a->w_v, dax, a->dtype, a->dtype, VAFA_F32, Tq, dkv, dh, H,
                (int64_t)H * dh, 1, dh, 1, (int64_t)H * dh, dh, (int64_t)H * dkv, 1, dkv, 1.f};
    if ((rc = simt_gemm(g1, s))) return rc;
    if ((rc = simt_attn_delta(a->o, a->d_o, delta, Tq, H, dh, a->dtype, s))) return rc;
    SimtAttnParams ap = simt_from_absorb(a, u, axn);
    ap.d_o = dax; ap.delta = delta; ap.dq = du; ap.dk = a->dx; ap.dv = nullptr;
    if ((rc = simt_attn_dq(ap, s))) return rc;
    if ((rc = simt_attn_dkv(ap, s))) return rc;
  }
  if (fast_chain) {
    const AbsorbBwdExtra x = absorb_bwd_extra(a);
    char* ex = ws + z.dax + z.delta + z.du + z.dp + x.ld + x.bexp + x.sched;
    void* tn_ws = ex;
    void* wqt = ex + x.tn;
    // dW_V[kv,h,dd] = sum_t axn[t,h,kv] dO[t,h,dd]
    GemmTNArgs tv{axn, a->d_o, dWV, tn_ws, Tq, a->dtype, H, H, 64, 32, H * dh, dh, dh, (long long)H * dh, a->sm_count};
    if ((rc = sm100_gemm_tn(tv, s))) return rc;
    if (inner) return 0;
    // dp[(t,h), dd] = sum_kv du[t,h,kv] W_K[kv,h,dd]: stacked rows against all of W_K, own head's block kept
    GemmNNArgs gdp{du, a->w_k, dp, (long long)Tq * H, H * dh, dkv, H * dh, dh, a->dtype, H, a->sm_count};
    if ((rc = sm100_gemm_nn_k256(gdp, s))) return rc;
    // dW_K[kv,h,dd] = sum_t du[t,h,kv] p[t,h,dd]
    GemmTNArgs tk{du, p, dWK, tn_ws, Tq, a->dtype, H, H, 64, 32, H * dh, dh, dh, (long long)H * dh, a->sm_count};
    if ((rc = sm100_gemm_tn(tk, s))) return rc;
    // dW_Q[a,(h,dd)] = sum_t q_raw[t,a] dp[t,(h,dd)]: q_raw as d_q/256 column blocks ("heads") of 256,
    // one batch entry per block, all against the same dp
    const int q_chunks = dq / 256;
    GemmTNArgs tq{a->q_raw, dp, dWQ, tn_ws, Tq, a->dtype, q_chunks, q_chunks, 256, 256, H * dh, 0,
                  (long long)256 * H * dh, (long long)H * dh, a->sm_count};
    if ((rc = sm100_gemm_tn(tq, s))) return rc;
    if (cut) return 0;  // phase 1 ends with the last weight gradient
    // dq_raw = dp W_Q^T   (W_Q is [d_q, H*D_H]; its transpose [H*D_H, d_q])
    if ((rc = sm100_transpose(a->w_q, wqt, dq, H * dh, a->dtype, s))) return rc;
    GemmNNArgs gq{dp, wqt, a->dq_raw, Tq, dq, H * dh, dq, dq, a->dtype, 0, a->sm_count};
    return sm100_gemm_nn_k256(gq, s);
  }
  // dW_V_h = axn_h^T dO_h                 fp32 [d_kv, H, D_H]
  SimtGemm g2{axn, a->d_o, dWV, a->dtype, a->dtype, VAFA_F32, dkv, dh, Tq, H,
              1, (int64_t)H * dkv, dkv, (int64_t)H * dh, 1, dh, (int64_t)H * dh, 1, dh, 1.f};
  if ((rc = simt_gemm(g2, s))) return rc;
  if (inner) return 0;
  // dp_h = du_h W_K_h                     [T_q, H, D_H]
  SimtGemm g3{du, a->w_k, dp, a->dtype, a->dtype, a->dtype, Tq, dh, dkv, H,
              (int64_t)H * dkv, 1, dkv, (int64_t)H * dh, 1, dh, (int64_t)H * dh, 1, dh, 1.f};
  if ((rc = simt_gemm(g3, s))) return rc;
  // dW_K_h = du_h^T p_h                   fp32 [d_kv, H, D_H]
  SimtGemm g4{du, p, dWK, a->dtype, a->dtype, VAFA_F32, dkv, dh, Tq, H,
              1, (int64_t)H * dkv, dkv, (int64_t)H * dh, 1, dh, (int64_t)H * dh, 1, dh, 1.f};
  if ((rc = simt_gemm(g4, s))) return rc;
  // dW_Q = q_raw^T dp                     fp32 [d_q, H*D_H]
  SimtGemm g5{a->q_raw, dp, dWQ, a->dtype, a->dtype, VAFA_F32, dq, H * dh, Tq, 1,
              1, dq, 0, (int64_t)H * dh, 1, 0, (int64_t)H * dh, 1, 0, 1.f};
  if ((rc = simt_gemm(g5, s))) return rc;
  // dq_raw = dp W_Q^T                     [T_q, d_q]
  SimtGemm g6{dp, a->w_q, a->dq_raw, a->dtype, a->dtype, a->dtype, Tq, dq, H * dh, 1,
              (int64_t)H * dh, 1, 0, 1, (int64_t)H * dh, 0, dq, 1, 0, 1.f};
  return simt_gemm(g6, s);
}

}  // namespace
}  // namespace vafa

using namespace vafa;

extern "C" {

int vafa_abi_version(void) { return VAFA_ABI_VERSION; }
const char* vafa_last_error(void) { return g_err; }

size_t vafa_varlen_fwd_workspace_bytes(const vafa_varlen_args* a) {
  if (!a) return 0;
  if (a->impl != VAFA_IMPL_SIMT && varlen_fwd_tc_ok(a)) return sm100_varlen_fwd_workspace_bytes(a);
  return 0;
}

size_t vafa_varlen_bwd_workspace_bytes(const vafa_varlen_args* a) {
  if (!a) return 0;
  if (a->impl != VAFA_IMPL_SIMT && varlen_bwd_tc_ok(a)) return sm100_varlen_bwd_workspace_bytes(a);
  return align_up((size_t)a->total_q * a->num_heads * 4, 256);
}

int vafa_varlen_fwd(const vafa_varlen_args* a, vafa_stream_t stream) {
  int rc = check_varlen(a, false);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int impl = pick_impl(a->impl, varlen_fwd_tc_ok(a), "varlen_fwd");
  if (impl < 0) return impl;
  if (impl == 0 && is_gqa(a)) return fail(VAFA_ERR_UNSUPPORTED, "num_kv_heads != num_heads needs the tcgen05 kernels (bf16/fp16, head_dim 64/128)");
  if ((rc = need_ws(a->workspace, a->workspace_bytes, vafa_varlen_fwd_workspace_bytes(a)))) return rc;
  if (impl == 1) return sm100_varlen_fwd(a, s);
  return simt_attn_fwd(simt_from_varlen(a), s);
}

int vafa_varlen_fwd_noalloc(const vafa_varlen_args* a, vafa_stream_t stream) {
  int rc = check_varlen(a, false);
  if (rc) return rc;
  if (!varlen_fwd_tc_ok(a))
    return fail(VAFA_ERR_UNSUPPORTED, "vafa_varlen_fwd_noalloc covers bf16/fp16 with head_dim 64 or 128 only");
  return sm100_varlen_fwd_noalloc(a, (cudaStream_t)stream);
}

int vafa_varlen_bwd(const vafa_varlen_args* a, vafa_stream_t stream) {
  int rc = check_varlen(a, true);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int impl = pick_impl(a->impl, varlen_bwd_tc_ok(a), "varlen_bwd");
  if (impl < 0) return impl;
  if (impl == 0 && is_gqa(a)) return fail(VAFA_ERR_UNSUPPORTED, "num_kv_heads != num_heads needs the tcgen05 kernels (bf16/fp16, head_dim 64/128)");
  if ((rc = need_ws(a->workspace, a->workspace_bytes, vafa_varlen_bwd_workspace_bytes(a)))) return rc;
  if (impl == 1) return sm100_varlen_bwd(a, s);
  SimtAttnParams p = simt_from_varlen(a);
  float* delta = (float*)a->workspace;
  p.delta = delta;
  if ((rc = simt_attn_delta(a->o, a->d_o, delta, a->total_q, a->num_heads, a->head_dim, a->dtype, s))) return rc;
  if ((rc = simt_attn_dq(p, s))) return rc;
  return simt_attn_dkv(p, s);
}

size_t vafa_absorb_saved_bytes(const vafa_absorb_args* a) {
  if (!a) return 0;
  const AbsorbSizes z = absorb_sizes(a);
  return z.p + z.u + z.axn;
}
size_t vafa_absorb_fwd_workspace_bytes(const vafa_absorb_args* a) {
  if (!a) return 0;
  return absorb_fwd_ws_bytes(a, a->w_q == nullptr);
}
size_t vafa_absorb_bwd_workspace_bytes(const vafa_absorb_args* a) {
  if (!a) return 0;
  const AbsorbSizes z = absorb_sizes(a);
  size_t n = z.dax + z.delta + z.du + z.dp;
  if (a->impl != VAFA_IMPL_SIMT && a->d_kv == 256 && a->dtype != VAFA_F32) {
    const AbsorbBwdExtra x = absorb_bwd_extra(a);
    n += x.ld + x.bexp + x.sched + x.tn + x.wqt;
  }
  return n;
}

// x rows narrower than d_kv exist only for the tensor-core kernels (TMA fills the missing columns)
static int check_x_width(const vafa_absorb_args* a, bool fast) {
  const int xw = x_width_of(a);
  if (xw == a->d_kv) return 0;
  if (xw > a->d_kv || xw % 8 != 0) return fail(VAFA_ERR_INVALID, "x_width %d must be a multiple of 8 and at most d_kv %d", xw, a->d_kv);
  if (!fast) return fail(VAFA_ERR_UNSUPPORTED, "x_width %d < d_kv %d needs the tcgen05 kernels for this shape", xw, a->d_kv);
  return 0;
}

int vafa_absorb_fwd(const vafa_absorb_args* a, vafa_stream_t stream) {
  int rc = check_absorb(a, false, false);
  if (rc) return rc;
  if ((rc = check_x_width(a, absorb_fast(a, false).core))) return rc;
  const int impl = pick_impl(a->impl, absorb_fast(a, false).core, "absorb_fwd");
  if (impl < 0) return impl;
  if ((rc = need_ws(a->workspace, a->workspace_bytes, absorb_fwd_ws_bytes(a, false)))) return rc;
  return absorb_forward(a, false, (cudaStream_t)stream);
}
int vafa_absorb_bwd(const vafa_absorb_args* a, vafa_stream_t stream) {
  int rc = check_absorb(a, true, false);
  if (rc) return rc;
  if ((rc = check_x_width(a, absorb_bwd_core_fast(a, false)))) return rc;
  const int impl = pick_impl(a->impl == VAFA_IMPL_TCGEN05 ? VAFA_IMPL_AUTO : a->impl, false, "absorb_bwd");
  if (impl < 0) return impl;
  if ((rc = need_ws(a->workspace, a->workspace_bytes, vafa_absorb_bwd_workspace_bytes(a)))) return rc;
  return absorb_backward(a, false, 0, (cudaStream_t)stream);
}
int vafa_absorb_bwd_phase(const vafa_absorb_args* a, int32_t phase, vafa_stream_t stream) {
  if (phase < 0 || phase > 2) return fail(VAFA_ERR_INVALID, "bad phase %d", phase);
  int rc = check_absorb(a, true, false);
  if (rc) return rc;
  if ((rc = check_x_width(a, absorb_bwd_core_fast(a, false)))) return rc;
  const int impl = pick_impl(a->impl == VAFA_IMPL_TCGEN05 ? VAFA_IMPL_AUTO : a->impl, false, "absorb_bwd");
  if (impl < 0) return impl;
  if ((rc = need_ws(a->workspace, a->workspace_bytes, vafa_absorb_bwd_workspace_bytes(a)))) return rc;
  return absorb_backward(a, false, phase, (cudaStream_t)stream);
}
int vafa_absorb_inner_fwd(const vafa_absorb_args* a, vafa_stream_t stream) {
  int rc = check_absorb(a, false, true);
  if (rc) return rc;
  if ((rc = check_x_width(a, absorb_fast(a, true).core))) return rc;
  const int impl = pick_impl(a->impl, absorb_fast(a, true).core, "absorb_inner_fwd");
  if (impl < 0) return impl;
  if ((rc = need_ws(a->workspace, a->workspace_bytes, absorb_fwd_ws_bytes(a, true)))) return rc;
  return absorb_forward(a, true, (cudaStream_t)stream);
}
int vafa_absorb_inner_bwd(const vafa_absorb_args* a, vafa_stream_t stream) {
  int rc = check_absorb(a, true, true);
  if (rc) return rc;
  if ((rc = check_x_width(a, absorb_bwd_core_fast(a, true)))) return rc;
  const int impl = pick_impl(a->impl == VAFA_IMPL_TCGEN05 ? VAFA_IMPL_AUTO : a->impl, false, "absorb_inner_bwd");
  if (impl < 0) return impl;
  if ((rc = need_ws(a->workspace, a->workspace_bytes, vafa_absorb_bwd_workspace_bytes(a)))) return rc;
  return absorb_backward(a, true, 0, (cudaStream_t)stream);
}

int vafa_cast_from_f32(const float* src, void* dst, size_t n, int32_t dtype, vafa_stream_t stream) {
  if (n > 0 && (!src || !dst)) return fail(VAFA_ERR_INVALID, "null pointer");
  return cast_from_f32(src, dst, n, dtype, (cudaStream_t)stream);
}

long long vafa_set_wait_limit_cycles(long long cycles) {
  const long long prev = g_wait_limit_cycles.load(std::memory_order_relaxed);
  if (cycles > 0) g_wait_limit_cycles.store(cycles, std::memory_order_relaxed);
  return prev;
}

int vafa_set_varlen_bwd_mode(int mode) {
  const int prev = g_varlen_bwd_mode.load(std::memory_order_relaxed);
  if (mode == 0 || mode == 1) g_varlen_bwd_mode.store(mode, std::memory_order_relaxed);
  return prev;
}

int vafa_selftest_bounded_wait(int32_t* status, vafa_stream_t stream) {
  if (!status) return fail(VAFA_ERR_INVALID, "null status word");
  return sm100_selftest_bounded_wait(status, (cudaStream_t)stream);
}

int vafa_check_status(const int32_t* status, vafa_stream_t stream) {
  if (!status) return 0;
  int32_t h[VAFA_STATUS_WORDS] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyAsync(h, status, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(VAFA_ERR_CUDA, "status read failed: %s", cudaGetErrorString(e));
  if (h[0] == 0) return 0;
  const char* what = h[0] == 1 ? "a bounded wait ran out" : h[0] == 2 ? "bad work item" : h[0] == 3 ? "tensor memory" : "unknown";
  return fail(VAFA_ERR_DEVICE, "device error %d (%s) at site %d, detail %d", h[0], what, h[1], h[2]);
}

}  // extern "C"
