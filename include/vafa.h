/*
 * vafa.h -- C ABI of libvafa_b200.so: packed variable-length attention and absorbed
 * target attention for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, enqueues its kernels on the CUDA
 * stream it is given and returns immediately: 0 on success, a negative VAFA_ERR_* code
 * otherwise (text via vafa_last_error()).  Unless a comment says otherwise an entry
 * point never allocates or frees device memory and never synchronises; scratch memory is
 * a caller-owned workspace whose size the matching *_workspace_bytes() function returns.
 *
 * Each declaration names the reference interface it stands in for (paths are relative to
 * the reference project root).
 */
#ifndef VAFA_H_
#define VAFA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#pragma GCC visibility push(default)
#endif

#define VAFA_ABI_VERSION 3

enum vafa_dtype { VAFA_F32 = 0, VAFA_BF16 = 1, VAFA_F16 = 2 };

enum vafa_impl {
  VAFA_IMPL_AUTO = 0,    /* tcgen05 kernels when the shape is supported, else the SIMT kernels */
  VAFA_IMPL_SIMT = 1,    /* scalar CUDA kernels: any dtype, any head dim up to 512 */
  VAFA_IMPL_TCGEN05 = 2  /* tcgen05/TMA kernels only; unsupported shapes return VAFA_ERR_UNSUPPORTED */
};

enum vafa_error {
  VAFA_OK = 0,
  VAFA_ERR_INVALID = -1,     /* bad argument (null pointer, bad size, misaligned base) */
  VAFA_ERR_UNSUPPORTED = -2, /* shape or dtype the requested implementation does not cover */
  VAFA_ERR_WORKSPACE = -3,   /* workspace missing or too small */
  VAFA_ERR_CUDA = -4,        /* a CUDA runtime / driver call failed */
  VAFA_ERR_DEVICE = -5       /* a kernel reported an error through the status word */
};

typedef void* vafa_stream_t; /* a cudaStream_t */

/* Status word layout (4 x int32 in device memory, caller-zeroed once; kernels only ever
 * write non-zero codes): [0] error code (0 = none), [1] kernel/site id, [2] detail (e.g. the
 * work item), [3] reserved.  vafa_check_status() reads it after the caller has synchronised. */
#define VAFA_STATUS_WORDS 4

/* ---------------------------------------------------------------------------------------
 * Packed variable-length attention.
 * Stands in for _PackedVarlenAttnFunction.forward / .backward
 * (triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:155-250 and :253-341) together with
 * the host index builders it calls (triton_fa_varlen_v2/triton_fa_varlen_v2/chunk_indices.py:
 * 25-75, 144-287), which here run on the device inside the call.
 * ------------------------------------------------------------------------------------- */
typedef struct vafa_varlen_args {
  /* tensors, row-major contiguous: q/o/do/dq [T_q, H, D]; k/v/dk/dv [T_k, H_kv, D] (H_kv = H unless
     num_kv_heads says otherwise) */
  const void* q;
  const void* k;
  const void* v;
  void* o;              /* forward: written; backward: read */
  float* lse;           /* [T_q, H] fp32, log2 domain with the scale folded in:
                           lse = m + log2(sum exp2(s - m)), s = q.k * scale * log2(e).
                           forward: written; backward: read.  -inf for rows that see no key */
  const void* d_o;      /* backward only */
  void* dq;             /* backward only */
  void* dk;             /* backward only */
  void* dv;             /* backward only */
  const int32_t* cu_seqlens_q; /* device, [n_seg + 1] */
  const int32_t* cu_seqlens_k; /* device, [n_seg + 1] */
  int32_t n_seg;
  int32_t total_q;      /* T_q */
  int32_t total_k;      /* T_k */
  int32_t num_heads;    /* H */
  int32_t head_dim;     /* D in {16, 32, 64, 128, 256} */
  int32_t dtype;        /* enum vafa_dtype, shared by q/k/v/o/do/dq/dk/dv */
  int32_t causal;       /* 0: every key of the segment; 1: bottom-right aligned causal mask */
  float scale;          /* softmax scale (the caller resolves the 1/sqrt(D) default) */
  int32_t impl;         /* enum vafa_impl */
  int32_t split_k_block;/* 0: split factor picked from KV length and SM count;
                           >0: fixed KV slice length (multiple of 128), like the reference's 4096 */
  int32_t sm_count;     /* 0: query the current device */
  void* workspace;      /* device scratch, >= vafa_varlen_*_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  int32_t* status;      /* device, VAFA_STATUS_WORDS int32, may be NULL */
  int32_t num_kv_heads; /* ABI version 3, last field.  0 or H: one K/V head per query head, as in the reference
                           (MHA only, triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:12).  A divisor of H:
                           grouped-query attention, query head h reads K/V head h / (H / H_kv); dk and dv are
                           [T_k, H_kv, D], summed over the query heads of a group.  Tensor-core kernels only
                           (bf16/fp16, head_dim 64 or 128); other shapes return VAFA_ERR_UNSUPPORTED. */
} vafa_varlen_args;

/* Bytes of scratch built into the library for vafa_varlen_fwd_noalloc() (below). */
#define VAFA_NOALLOC_SCRATCH_BYTES (16u << 20)

size_t vafa_varlen_fwd_workspace_bytes(const vafa_varlen_args* a);
size_t vafa_varlen_bwd_workspace_bytes(const vafa_varlen_args* a);
int vafa_varlen_fwd(const vafa_varlen_args* a, vafa_stream_t stream);
int vafa_varlen_bwd(const vafa_varlen_args* a, vafa_stream_t stream);

/* Which backward vafa_varlen_bwd runs on the tensor-core path (process-wide; returns the previous mode;
 * other values only read it):
 *   0  the dQ kernel and the dK/dV kernel (the reference's own split,
 *      triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:283-338): seven matrix products per score
 *      tile, no atomics, dQ/dK/dV bit-identical from run to run like the reference's
 *      (triton_fa_varlen_v2/triton_fa_varlen_v2/test_smoke.py:496-531).  The default.
 *   1  one pass over the score tiles for head_dim 128 (five products, one exponential per score; the
 *      reference's authors sketched this as _bwd_fused_kernel, kernels.py:923-1099, and never launched
 *      it): dK and dV as before, dQ summed across key tiles by fp32 reductions in global memory, so its
 *      last bits depend on the order in which the tiles finish.  Other head dims run mode 0.
 * vafa_varlen_bwd_workspace_bytes() depends on the mode (mode 1 adds an fp32 [T_q, H, D] array): query
 * it after setting the mode. */
int vafa_set_varlen_bwd_mode(int mode);

/* Forward pass for callers that cannot provide a workspace.  No counterpart in the reference:
 * there, torch's allocator is always at hand.  Some hosts of this library are not in that
 * position -- a plugin running inside another runtime's execution callback, an inference engine
 * whose memory plan is frozen before the first request, a real-time loop that may not touch
 * the allocator -- so they cannot call cudaMalloc (or have torch do it) to size a workspace per
 * batch.  This entry point takes the same arguments as vafa_varlen_fwd but ignores `workspace`
 * and `workspace_bytes`: its tile lists and split-K partials live in a fixed
 * VAFA_NOALLOC_SCRATCH_BYTES array inside the library's device image (each GPU that loads the
 * library holds that much until the process exits).  The call itself runs no allocation routine
 * (no cudaMalloc, no cudaFree, no allocating library call).  The array is part of the library's device
 * code: the CUDA runtime creates it when it loads that code onto a GPU, which with the default lazy
 * module loading happens at the first call of this library on that GPU (or at start-up with
 * CUDA_MODULE_LOADING=EAGER).  A host with a frozen memory plan should therefore make one call per GPU
 * during its own set-up, before the plan is frozen.
 *   - tcgen05 shapes only (bf16/fp16, head_dim 64 or 128); others return VAFA_ERR_UNSUPPORTED.
 *   - Batches whose tile lists do not fit return VAFA_ERR_WORKSPACE with the sizes in the error
 *     text; the split-K partial area shrinks to whatever room is left, so long-KV batches may
 *     be split less finely than with vafa_varlen_fwd (same result up to fp32 rounding).
 *   - The first call on each device looks up the array's device address (with that device
 *     current) and caches it; make that first call outside of any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's
 *     contents; every call rewrites what it reads, so nothing has to be cleared, but two calls
 *     that may overlap on the GPU (different streams) race -- serialise them. */
int vafa_varlen_fwd_noalloc(const vafa_varlen_args* a, vafa_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Absorbed ragged target attention (u = q_raw W_Q W_K^T per head, attend over raw X,
 * project with W_V).
 * Stands in for packed_target_attn's torch prologue
 * (triton_target_attn_absorb/triton_target_attn_absorb/interface.py:434-435) and its autograd,
 * plus _TargetAttnFunction.forward / .backward (same file :153-223 and :226-321).
 * ------------------------------------------------------------------------------------- */
typedef struct vafa_absorb_args {
  const void* q_raw;    /* [T_q, d_q] */
  const void* x;        /* [T_k, d_kv] */
  const void* w_q;      /* [d_q, H, D_H] */
  const void* w_k;      /* [d_kv, H, D_H] */
  const void* w_v;      /* [d_kv, H, D_H] */
  void* o;              /* [T_q, H, D_H]; forward: written; backward: read */
  float* lse;           /* [T_q, H] fp32, log2 domain (as above) */
  void* saved;          /* caller-owned buffer of vafa_absorb_saved_bytes(): written by the
                           forward, read by the backward of the same inputs */
  const void* d_o;      /* backward: [T_q, H, D_H] */
  void* dq_raw;         /* backward outputs, I/O dtype, same shapes as the inputs */
  void* dx;
  float* dw;            /* backward: fp32 [dW_Q | dW_K | dW_V] flat, (d_q + 2 d_kv) * H * D_H floats;
                           kept fp32 so that a data-parallel caller can sum it across ranks before
                           rounding */
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  int32_t n_seg, total_q, total_k;
  int32_t d_q, d_kv, num_heads, head_dim; /* head_dim = D_H */
  int32_t dtype;
  float scale;
  int32_t impl;
  int32_t sm_count;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
  int32_t x_width;      /* row width of x and dx in elements; 0 means d_kv.  A smaller width (a multiple
                           of 8) is taken only by the tensor-core kernels: the missing columns read as
                           zero (the weights must have d_kv rows, the extra ones zero) and dx is written
                           x_width columns wide.  Lets a caller with d_kv < 256 pad only its weights. */
} vafa_absorb_args;

size_t vafa_absorb_saved_bytes(const vafa_absorb_args* a);
size_t vafa_absorb_fwd_workspace_bytes(const vafa_absorb_args* a);
size_t vafa_absorb_bwd_workspace_bytes(const vafa_absorb_args* a);
int vafa_absorb_fwd(const vafa_absorb_args* a, vafa_stream_t stream);
int vafa_absorb_bwd(const vafa_absorb_args* a, vafa_stream_t stream);

/* The backward in two calls, for data-parallel callers that all-reduce the weight gradients:
 *   phase 1 writes everything `dw` depends on (and nothing of dx / dq_raw), phase 2 the rest, so the
 *   caller can start its collective on `dw` after phase 1 and let it run under phase 2.
 *   phase 0 is vafa_absorb_bwd.  Both calls take the same arguments and the same workspace, whose
 *   contents must survive from phase 1 to phase 2.  Shapes that do not run on the tensor-core chain do
 *   all their work in phase 1; phase 2 is then a no-op.  The reference has no counterpart (it is
 *   single-GPU; its weight gradients come from torch autograd,
 *   triton_target_attn_absorb/triton_target_attn_absorb/interface.py:430-435). */
int vafa_absorb_bwd_phase(const vafa_absorb_args* a, int32_t phase, vafa_stream_t stream);

/* Inner entry on a pre-projected u [T_q, H, d_kv] (q_raw = u, w_q/w_k unused): stands in for
 * target_attn_inner (triton_target_attn_absorb/triton_target_attn_absorb/interface.py:324-354).
 * Backward writes du into dq_raw ([T_q, H, d_kv]), dX into dx and fp32 dW_V into dw. */
int vafa_absorb_inner_fwd(const vafa_absorb_args* a, vafa_stream_t stream);
int vafa_absorb_inner_bwd(const vafa_absorb_args* a, vafa_stream_t stream);

/* Round an fp32 buffer to the I/O dtype: dst[i] = (dtype) src[i].  Used after the weight
 * gradients have been summed across ranks.  Replaces the torch casts at
 * triton_target_attn_absorb/triton_target_attn_absorb/interface.py:318-319. */
int vafa_cast_from_f32(const float* src, void* dst, size_t n, int32_t dtype, vafa_stream_t stream);

/* ---- housekeeping ------------------------------------------------------------------ */
int vafa_abi_version(void);
const char* vafa_last_error(void);           /* thread-local text of the last failure */
/* Copy the status word to the host (synchronises `stream`) and translate it: returns 0 or
 * VAFA_ERR_DEVICE with the text available from vafa_last_error(). */
int vafa_check_status(const int32_t* status, vafa_stream_t stream);

/* ---- failure detection ---------------------------------------------------------------------
 * No counterpart in the reference (its Triton kernels have no device-side waits).  Every wait inside
 * the kernels of this library (mbarrier spins of the TMA / MMA / element-wise roles) gives up after a
 * clock-cycle limit: the CTA raises a shared abort flag, all its roles leave, code 1 with the kernel's
 * site id goes to the status word, tensor memory is released and the kernel returns.  Nothing traps.
 * vafa_set_wait_limit_cycles() sets that limit for all later launches of the process (values <= 0 only
 * read it) and returns the previous one; the default is 4e9 cycles, about two seconds.  The limit is
 * rounded up to a multiple of 65536 cycles.
 * vafa_selftest_bounded_wait() launches one CTA that waits, through the same code, on an mbarrier that
 * nobody arrives on: with the current limit it must come back with code 1, site 900 in `status`. */
long long vafa_set_wait_limit_cycles(long long cycles);
int vafa_selftest_bounded_wait(int32_t* status, vafa_stream_t stream);

/* ---- optional per-kernel timing and launch counters -------------------------------------
 * Not part of the reference's interface; it covers what the reference's developer tools do with
 * CUDA events around each launch (triton_fa_varlen_v2/tools/profile_v2_kernels.py:52-65).
 * Launch counters always run; event timing only after vafa_profile_enable(1) (two events per
 * launch on the launch's stream).  vafa_profile_read() waits for the recorded events. */
int vafa_profile_enable(int on);
int vafa_profile_kernel_count(void);
const char* vafa_profile_kernel_name(int id);
int vafa_profile_read(int id, double* total_ms, long long* timed_launches, long long* all_launches);
int vafa_profile_reset(void);

#ifdef __cplusplus
#pragma GCC visibility pop
}
#endif
#endif /* VAFA_H_ */
