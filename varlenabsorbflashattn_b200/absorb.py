"""packed_target_attn: ragged target attention with W_Q W_K^T absorbed into the query.

Host-side mirror of the reference's public interface
(triton_target_attn_absorb/triton_target_attn_absorb/interface.py: `packed_target_attn`
:357-445, `target_attn_inner` :324-354, `prepare_target_attn_indices` :125-138): same
arguments, same shapes (3-D weights [d, H, D_H], output [T_q, H, D_H]), same exception types.

Differences that stay behind the same signature:
  * the prologue u = q_raw W_Q W_K^T, the projection with W_V and all five gradients
    (dq_raw, dX, dW_Q, dW_K, dW_V) are computed inside libvafa_b200.so, not by torch ops and
    torch autograd around a kernel;
  * the chunk-index tensors are accepted for compatibility and ignored: tiles are derived on
    the device from cu_seqlens;
  * `weight_grad_group` (keyword-only, default None): a torch.distributed process group over
    which the fp32 weight gradients are summed before they are rounded to the I/O dtype, for
    sequence-sharded data parallel runs;
  * widths the tensor-core kernels do not take directly (the reference's production shape is
    d_q = 968, d_kv = 216, test_smoke.py:54-57) are zero-padded here to d_kv = 256 and to the next
    multiple of 256 for d_q, with differentiable torch ops, so the gradients come back in the
    caller's widths.  Zero columns of q_raw / X and zero rows of the weights change neither the
    scores nor the outputs.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib

__all__ = ["packed_target_attn", "target_attn_inner", "prepare_target_attn_indices"]

_BT_Q = 16   # chunk sizes of the reference's index tensors (interface.py:59-63)
_BT_K = 64
_SUPPORTED_D_H = (16, 32, 64, 128, 256)


def _impl_code() -> int:
    return _lib.IMPL_NAMES[os.environ.get("VAFA_IMPL", "auto").lower()]


def _check_env_modes() -> None:
    # The reference selects kernels through two environment variables and rejects bad values
    # (interface.py:66-85).  There is a single path here; the values are still checked.
    fwd = os.environ.get("TRITON_TARGET_ATTN_FWD_MODE", "alpha").lower()
    if fwd not in ("direct", "alpha"):
        raise ValueError("TRITON_TARGET_ATTN_FWD_MODE must be one of: direct, alpha")
    dx = os.environ.get("TRITON_TARGET_ATTN_DX_MODE", "auto").lower()
    if dx not in ("auto", "partial", "fused", "atomic"):
        raise ValueError("TRITON_TARGET_ATTN_DX_MODE must be one of: auto, partial, fused, atomic")


def _lengths_to_cu(seqinfo: torch.Tensor) -> torch.Tensor:
    assert seqinfo.dim() == 1 and seqinfo.numel() >= 1
    cu = torch.zeros(seqinfo.numel() + 1, dtype=torch.int64, device=seqinfo.device)
    torch.cumsum(seqinfo.to(torch.int64), 0, out=cu[1:])
    return cu.to(torch.int32)


def _check_cu(cu: torch.Tensor, total: int, name: str) -> torch.Tensor:
    # reference: interface.py:92-106
    if cu.dim() != 1 or cu.numel() < 2:
        raise ValueError(f"{name}: must be 1-D with len>=2, got {tuple(cu.shape)}")
    host = cu.detach().to("cpu", torch.int64)
    if int(host[0]) != 0:
        raise ValueError(f"{name}[0] must be 0")
    if int(host[-1]) != total:
        raise ValueError(f"{name}[-1] must equal total tokens {total}, got {int(host[-1])}")
    if bool((host[1:] < host[:-1]).any()):
        raise ValueError(f"{name} must be non-decreasing")
    return host


def _validate(cu_q, cu_k, T_q, T_k) -> None:
    assert cu_q.numel() == cu_k.numel(), "segment count mismatch q vs k"
    hq = _check_cu(cu_q, T_q, "cu_seqlens_q")
    hk = _check_cu(cu_k, T_k, "cu_seqlens_k")
    # reference: interface.py:109-116
    if bool((((hq[1:] - hq[:-1]) > 0) & ((hk[1:] - hk[:-1]) <= 0)).any()):
        raise ValueError("segments with q_len > 0 must have k_len > 0")


def _chunk_rows(cu: torch.Tensor, bt: int) -> torch.Tensor:
    """[sum ceil(L_i/bt), 2] int32 rows (segment, block-in-segment), segment order."""
    host = cu.detach().to("cpu", torch.int64)
    nblk = (host[1:] - host[:-1] + bt - 1) // bt
    seg = torch.repeat_interleave(torch.arange(nblk.numel(), dtype=torch.int64), nblk)
    first = torch.cumsum(nblk, 0) - nblk
    blk = torch.arange(int(nblk.sum()), dtype=torch.int64) - torch.repeat_interleave(first, nblk)
    return torch.stack([seg, blk], dim=1).to(torch.int32).to(cu.device)


def prepare_target_attn_indices(cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk metadata in the reference's format ((segment, block) rows for 16-row query chunks
    and 64-row key chunks).  Kept so that call sites which precompute and pass them keep
    working; the kernels here do not read them."""
    return _chunk_rows(cu_seqlens_q, _BT_Q), _chunk_rows(cu_seqlens_k, _BT_K)


def _fill(a: _lib.AbsorbArgs, device, cu_q, cu_k, T_q, T_k, d_q, d_kv, H, D_H, dtype, scale, x_width=0) -> None:
    a.x_width = 0 if x_width == d_kv else x_width
    a.cu_seqlens_q, a.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    a.n_seg, a.total_q, a.total_k = cu_q.numel() - 1, T_q, T_k
    a.d_q, a.d_kv, a.num_heads, a.head_dim = d_q, d_kv, H, D_H
    a.dtype = _lib.DTYPE_CODE[dtype]
    a.scale = float(scale)
    a.impl = _impl_code()
    a.sm_count = _lib.sm_count(device)
    a.status = _lib.status_word(device).data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _PackedTargetAttn(torch.autograd.Function):
    """q_raw, X, W_Q, W_K, W_V -> O, with all five gradients from the library."""

    @staticmethod
    def forward(ctx, q_raw, X, W_Q, W_K, W_V, cu_q, cu_k, scale, group):
        lib = _lib.load()
        T_q, d_q = q_raw.shape
        T_k, x_w = X.shape
        d_kv = W_K.shape[0]  # X may be narrower than the (padded) weights: see _padded_widths
        _, H, D_H = W_Q.shape
        dev = q_raw.device
        O = torch.empty((T_q, H, D_H), dtype=q_raw.dtype, device=dev)
        lse = torch.empty((T_q, H), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            a = _lib.AbsorbArgs()
            _fill(a, dev, cu_q, cu_k, T_q, T_k, d_q, d_kv, H, D_H, q_raw.dtype, scale, x_w)
            a.q_raw, a.x, a.w_q, a.w_k, a.w_v = (t.data_ptr() for t in (q_raw, X, W_Q, W_K, W_V))
            a.o, a.lse = O.data_ptr(), lse.data_ptr()
            saved = torch.empty(max(1, lib.vafa_absorb_saved_bytes(a)), dtype=torch.uint8, device=dev)
            a.saved = saved.data_ptr()
            ws = _lib.workspace(lib.vafa_absorb_fwd_workspace_bytes(a), dev)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            _lib.check(lib.vafa_absorb_fwd(a, _stream()), "vafa_absorb_fwd")
            _lib.maybe_check_status(dev)
        ctx.save_for_backward(q_raw, X, W_Q, W_K, W_V, O, lse, cu_q, cu_k, saved)
        ctx.scale, ctx.group = scale, group
        ctx.mark_non_differentiable(lse)
        return O, lse

    @staticmethod
    def backward(ctx, dO, _dlse):
        q_raw, X, W_Q, W_K, W_V, O, lse, cu_q, cu_k, saved = ctx.saved_tensors
        lib = _lib.load()
        T_q, d_q = q_raw.shape
        T_k, x_w = X.shape
        d_kv = W_K.shape[0]
        _, H, D_H = W_Q.shape
        dev = q_raw.device
        if dO.dtype != q_raw.dtype:
            dO = dO.to(q_raw.dtype)
        if not dO.is_contiguous():
            dO = dO.contiguous()
        dq_raw, dX = torch.empty_like(q_raw), torch.empty_like(X)
        n_wq, n_wk = d_q * H * D_H, d_kv * H * D_H
        dw = torch.empty(n_wq + 2 * n_wk, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            a = _lib.AbsorbArgs()
            _fill(a, dev, cu_q, cu_k, T_q, T_k, d_q, d_kv, H, D_H, q_raw.dtype, ctx.scale, x_w)
            a.q_raw, a.x, a.w_q, a.w_k, a.w_v = (t.data_ptr() for t in (q_raw, X, W_Q, W_K, W_V))
            a.o, a.lse, a.saved, a.d_o = O.data_ptr(), lse.data_ptr(), saved.data_ptr(), dO.data_ptr()
            a.dq_raw, a.dx, a.dw = dq_raw.data_ptr(), dX.data_ptr(), dw.data_ptr()
            ws = _lib.workspace(lib.vafa_absorb_bwd_workspace_bytes(a), dev)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            if ctx.group is None:
                _lib.check(lib.vafa_absorb_bwd(a, _stream()), "vafa_absorb_bwd")
            else:
                # weight gradients first; their all-reduce (on the process group's own stream) then runs
                # under the dX kernel and the dq_raw product, and the rounding below waits for it
                import torch.distributed as dist
                _lib.check(lib.vafa_absorb_bwd_phase(a, 1, _stream()), "vafa_absorb_bwd_phase(1)")
                work = dist.all_reduce(dw, group=ctx.group, async_op=True)
                _lib.check(lib.vafa_absorb_bwd_phase(a, 2, _stream()), "vafa_absorb_bwd_phase(2)")
                work.wait()
            _lib.maybe_check_status(dev)
            if q_raw.dtype == torch.float32:
                dwc = dw
            else:
                dwc = torch.empty(dw.numel(), dtype=q_raw.dtype, device=dev)
                _lib.check(lib.vafa_cast_from_f32(dw.data_ptr(), dwc.data_ptr(), dw.numel(),
                                                  _lib.DTYPE_CODE[q_raw.dtype], _stream()), "vafa_cast_from_f32")
        dW_Q = dwc[:n_wq].view(d_q, H, D_H)
        dW_K = dwc[n_wq:n_wq + n_wk].view(d_kv, H, D_H)
        dW_V = dwc[n_wq + n_wk:].view(d_kv, H, D_H)
        return dq_raw, dX, dW_Q, dW_K, dW_V, None, None, None, None


class _TargetAttnInner(torch.autograd.Function):
    """u, X, W_V -> O: counterpart of _TargetAttnFunction (reference interface.py:141-321)."""

    @staticmethod
    def forward(ctx, u, X, W_V, cu_q, cu_k, scale):
        lib = _lib.load()
        T_q, H, d_kv = u.shape
        T_k, x_w = X.shape
        D_H = W_V.shape[2]
        dev = u.device
        O = torch.empty((T_q, H, D_H), dtype=u.dtype, device=dev)
        lse = torch.empty((T_q, H), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            a = _lib.AbsorbArgs()
            _fill(a, dev, cu_q, cu_k, T_q, T_k, 0, d_kv, H, D_H, u.dtype, scale, x_w)
            a.q_raw, a.x, a.w_v = u.data_ptr(), X.data_ptr(), W_V.data_ptr()
            a.o, a.lse = O.data_ptr(), lse.data_ptr()
            saved = torch.empty(max(1, lib.vafa_absorb_saved_bytes(a)), dtype=torch.uint8, device=dev)
            a.saved = saved.data_ptr()
            ws = _lib.workspace(lib.vafa_absorb_fwd_workspace_bytes(a), dev)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            _lib.check(lib.vafa_absorb_inner_fwd(a, _stream()), "vafa_absorb_inner_fwd")
            _lib.maybe_check_status(dev)
        ctx.save_for_backward(u, X, W_V, O, lse, cu_q, cu_k, saved)
        ctx.scale = scale
        ctx.mark_non_differentiable(lse)
        return O, lse

    @staticmethod
    def backward(ctx, dO, _dlse):
        u, X, W_V, O, lse, cu_q, cu_k, saved = ctx.saved_tensors
        lib = _lib.load()
        T_q, H, d_kv = u.shape
        T_k, x_w = X.shape
        D_H = W_V.shape[2]
        dev = u.device
        if dO.dtype != u.dtype:
            dO = dO.to(u.dtype)
        if not dO.is_contiguous():
            dO = dO.contiguous()
        du, dX = torch.empty_like(u), torch.empty_like(X)
        dw = torch.empty(d_kv * H * D_H, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            a = _lib.AbsorbArgs()
            _fill(a, dev, cu_q, cu_k, T_q, T_k, 0, d_kv, H, D_H, u.dtype, ctx.scale, x_w)
            a.q_raw, a.x, a.w_v = u.data_ptr(), X.data_ptr(), W_V.data_ptr()
            a.o, a.lse, a.saved, a.d_o = O.data_ptr(), lse.data_ptr(), saved.data_ptr(), dO.data_ptr()
            a.dq_raw, a.dx, a.dw = du.data_ptr(), dX.data_ptr(), dw.data_ptr()
            ws = _lib.workspace(lib.vafa_absorb_bwd_workspace_bytes(a), dev)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            _lib.check(lib.vafa_absorb_inner_bwd(a, _stream()), "vafa_absorb_inner_bwd")
            _lib.maybe_check_status(dev)
        dW_V = dw.view(d_kv, H, D_H).to(u.dtype)
        return du, dX, dW_V, None, None, None


def _padded_widths(dtype: torch.dtype, d_q: Optional[int], d_kv: int, H: int) -> Optional[Tuple[Optional[int], int]]:
    """(d_q, d_kv) to pad to so that the tcgen05 kernels apply, or None to leave the inputs alone."""
    if os.environ.get("VAFA_IMPL", "auto").lower() == "simt":
        return None
    if dtype not in (torch.bfloat16, torch.float16) or d_kv > 256 or H < 1 or 128 % H != 0:
        return None
    d_q_pad = None if d_q is None else max(256, (d_q + 255) // 256 * 256)
    if d_kv == 256 and d_q_pad == d_q:
        return None
    return d_q_pad, 256


def _narrow_x_ok(x_width: int, H: int, D_H: int, T_q: int, T_k: int) -> bool:
    """X (the big tensor) can stay at its own width: the forward and backward tensor-core kernels read the
    missing columns as zero through TMA and write dX at that width (vafa_absorb_args.x_width).  The
    library takes a narrow X in the backward only where its tensor-core dU / dX kernels apply
    (H * D_H == 256, D_H >= 32, H dividing 64); every other head layout gets a padded copy of X so that
    the backward, which then runs on the general kernels, sees full-width rows."""
    return (x_width % 8 == 0 and H * D_H == 256 and D_H >= 32 and 64 % H == 0 and T_q > 0 and T_k > 0)


def _pad_last(t: torch.Tensor, width: int) -> torch.Tensor:
    return t if t.shape[-1] == width else torch.nn.functional.pad(t, (0, width - t.shape[-1]))


def _pad_first(t: torch.Tensor, rows: int) -> torch.Tensor:
    return t if t.shape[0] == rows else torch.nn.functional.pad(t, (0, 0) * (t.dim() - 1) + (0, rows - t.shape[0]))


def _next_pow2(x: int) -> int:
    if x < 1:
        raise ValueError(f"expected positive dimension, got {x}")
    return 1 << (x - 1).bit_length()


def _common_checks(dtype_tensors, device_tensors, D_H, d_kv) -> None:
    assert all(t.dtype == dtype_tensors[0].dtype for t in dtype_tensors), \
        "inputs must share dtype, got " + "/".join(str(t.dtype) for t in dtype_tensors)
    assert dtype_tensors[0].dtype in _lib.DTYPE_CODE, f"dtype {dtype_tensors[0].dtype} not supported"
    assert all(t.is_cuda for t in device_tensors), "all inputs must be CUDA"
    assert all(t.device == device_tensors[0].device for t in device_tensors), "inputs must be on same device"
    assert D_H in _SUPPORTED_D_H, f"D_H {D_H} not supported"
    assert _next_pow2(d_kv) <= 512, f"D_KV={d_kv} pads to {_next_pow2(d_kv)}, which is too large"


def target_attn_inner(
    u: torch.Tensor,
    X: torch.Tensor,
    W_V: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    scale: Optional[float] = None,
    q_chunk_indices: Optional[torch.Tensor] = None,
    k_chunk_indices: Optional[torch.Tensor] = None,
    validate: bool = True,
) -> torch.Tensor:
    """Inner entry on an already projected u = q_raw W_Q W_K^T.

    u [T_q, H, d_kv], X [T_k, d_kv], W_V [d_kv, H, D_H] -> O [T_q, H, D_H]; scale defaults to
    1/sqrt(D_H).  The chunk-index arguments are accepted and ignored.
    """
    _check_env_modes()
    T_q, H, d_kv = u.shape
    T_k, d_kv_x = X.shape
    d_kv_w, H_w, D_H = W_V.shape
    assert d_kv == d_kv_x == d_kv_w, f"D_KV mismatch: u={d_kv}, X={d_kv_x}, W_V={d_kv_w}"
    assert H == H_w, f"H mismatch: u={H}, W_V={H_w}"
    _common_checks((u, X, W_V), (u, X, W_V), D_H, d_kv)
    if scale is None:
        scale = 1.0 / math.sqrt(D_H)
    cu_q = cu_seqlens_q.to(device=u.device, dtype=torch.int32).contiguous()
    cu_k = cu_seqlens_k.to(device=u.device, dtype=torch.int32).contiguous()
    if validate:
        _validate(cu_q, cu_k, T_q, T_k)
    pad = _padded_widths(u.dtype, None, d_kv, H)
    if pad is not None:
        u, W_V = _pad_last(u, pad[1]), _pad_first(W_V, pad[1])
        if not _narrow_x_ok(d_kv, H, D_H, T_q, T_k):
            X = _pad_last(X, pad[1])
    O, _ = _TargetAttnInner.apply(u.contiguous(), X.contiguous(), W_V.contiguous(), cu_q, cu_k, float(scale))
    return O


def packed_target_attn(
    q_raw: torch.Tensor,
    X: torch.Tensor,
    W_Q: torch.Tensor,
    W_K: torch.Tensor,
    W_V: torch.Tensor,
    *,
    cu_seqlens_q: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    q_seqinfo: Optional[torch.Tensor] = None,
    k_seqinfo: Optional[torch.Tensor] = None,
    q_chunk_indices: Optional[torch.Tensor] = None,
    k_chunk_indices: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    bf16: bool = False,
    validate: bool = True,
    weight_grad_group=None,
) -> torch.Tensor:
    """O_h = softmax(scale (q_raw W_Q_h)(X W_K_h)^T) (X W_V_h) per ragged segment, computed in the
    absorbed form (attend over raw X with u_h = q_raw W_Q_h W_K_h^T, then project with W_V_h).

    q_raw [T_q, d_q] or [1, T_q, d_q]; X [T_k, d_kv] or [1, T_k, d_kv]; W_Q [d_q, H, D_H];
    W_K, W_V [d_kv, H, D_H].  cu_seqlens_* [n_seg+1] or *_seqinfo [n_seg] lengths.  bf16=True
    casts all five tensors to bfloat16 first.  Returns O [T_q, H, D_H] in the I/O dtype.

    Device-side failures are reported through the status word, not raised by this call: see
    `_lib.check_status` / `_lib.set_check_status` (VAFA_CHECK_STATUS=1).
    """
    _check_env_modes()
    if q_raw.dim() == 3:
        assert q_raw.shape[0] == 1, "batch must be 1 for packed varlen"
        q_raw = q_raw[0]
    if X.dim() == 3:
        assert X.shape[0] == 1
        X = X[0]
    T_q, d_q = q_raw.shape
    T_k, d_kv = X.shape
    d_q_w, H, D_H = W_Q.shape
    assert d_q_w == d_q, f"W_Q[0]={d_q_w} != d_q={d_q}"
    assert W_K.shape[0] == d_kv and W_V.shape[0] == d_kv, "W_K/W_V d_kv mismatch"
    assert H == W_K.shape[1] == W_V.shape[1], "H mismatch across W_Q/W_K/W_V"
    assert D_H == W_K.shape[2] == W_V.shape[2], "D_H mismatch across W_Q/W_K/W_V"
    if cu_seqlens_q is None:
        assert q_seqinfo is not None
        cu_seqlens_q = _lengths_to_cu(q_seqinfo)
    if cu_seqlens_k is None:
        assert k_seqinfo is not None
        cu_seqlens_k = _lengths_to_cu(k_seqinfo)
    if bf16:
        q_raw, X, W_Q, W_K, W_V = (t.to(torch.bfloat16) for t in (q_raw, X, W_Q, W_K, W_V))
    _common_checks((q_raw, X, W_Q, W_K, W_V), (q_raw, X, W_Q, W_K, W_V), D_H, d_kv)
    if scale is None:
        scale = 1.0 / math.sqrt(D_H)
    cu_q = cu_seqlens_q.to(device=q_raw.device, dtype=torch.int32).contiguous()
    cu_k = cu_seqlens_k.to(device=q_raw.device, dtype=torch.int32).contiguous()
    if validate:
        _validate(cu_q, cu_k, T_q, T_k)
    pad = _padded_widths(q_raw.dtype, d_q, d_kv, H)
    if pad is not None:
        q_raw, W_Q = _pad_last(q_raw, pad[0]), _pad_first(W_Q, pad[0])
        W_K, W_V = _pad_first(W_K, pad[1]), _pad_first(W_V, pad[1])
        if not _narrow_x_ok(d_kv, H, D_H, T_q, T_k):
            X = _pad_last(X, pad[1])
    O, _ = _PackedTargetAttn.apply(q_raw.contiguous(), X.contiguous(), W_Q.contiguous(), W_K.contiguous(),
                                   W_V.contiguous(), cu_q, cu_k, float(scale), weight_grad_group)
    return O
