"""packed_varlen_attn: packed variable-length attention over cu_seqlens (block-diagonal mask).

Host-side mirror of the reference's public interface
(triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:344-392, `packed_varlen_attn`, and :68-71,
`set_validate_cu_seqlens`): same positional and keyword arguments, same layout rules ([T,H,D] or
[1,T,H,D] in, same rank out), same exception types.  Two keyword-only additions default to
the reference's behaviour: `causal=False` and `split_k_block=None`.

All arithmetic happens in libvafa_b200.so; this module only checks arguments, allocates
outputs and scratch with torch, and passes raw pointers and the current CUDA stream down.
Unlike the reference no index tensors are built on the host: the tile list is built on the
device from cu_seqlens inside the call, so with validation off a call never synchronises.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib

__all__ = ["packed_varlen_attn", "packed_varlen_attn_with_lse", "set_validate_cu_seqlens", "set_impl", "set_backward_mode"]

_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128, 256)
_validate = True
_impl = _lib.IMPL_NAMES[os.environ.get("VAFA_IMPL", "auto").lower()]
LN2 = math.log(2.0)


def set_validate_cu_seqlens(enabled: bool) -> None:
    """Switch the host-side cu_seqlens check (one small device-to-host copy) on or off."""
    global _validate
    _validate = bool(enabled)


def set_impl(name: str) -> None:
    """'auto' (default), 'simt' or 'tcgen05': which kernel family the library uses."""
    global _impl
    _impl = _lib.IMPL_NAMES[name.lower()]


_BWD_MODES = {"split": 0, "fused": 1}


def set_backward_mode(name: str) -> str:
    """'split' (default): the dQ kernel and the dK/dV kernel, gradients bit-identical from run to run like
    the reference's.  'fused': one pass over the score tiles for head_dim 128 (five matrix products per tile
    instead of seven, one exponential per score instead of two); dQ is then summed across key tiles by fp32
    reductions in global memory and its last bits vary from run to run.  Returns the previous mode."""
    prev = _lib.load().vafa_set_varlen_bwd_mode(_BWD_MODES[name.lower()])
    return "fused" if prev == 1 else "split"


if os.environ.get("VAFA_BWD_MODE"):
    set_backward_mode(os.environ["VAFA_BWD_MODE"])


def _lengths_to_cu(seqinfo: torch.Tensor) -> torch.Tensor:
    # reference: interface.py:74-93 (ValueError on rank, emptiness, negatives, int32 overflow)
    if seqinfo.dim() != 1:
        raise ValueError(f"seqinfo must be 1-D [n_seg], got shape {tuple(seqinfo.shape)}")
    if seqinfo.numel() == 0:
        raise ValueError("seqinfo is empty (n_seg=0)")
    if bool((seqinfo < 0).any()):
        raise ValueError("seqinfo contains negative values")
    cu = torch.zeros(seqinfo.numel() + 1, dtype=torch.int64, device=seqinfo.device)
    torch.cumsum(seqinfo.to(torch.int64), 0, out=cu[1:])
    total = int(cu[-1])
    if total > 2**31 - 1:
        raise ValueError(f"total tokens {total} exceeds int32 range")
    return cu.to(torch.int32)


def _check_cu(cu: torch.Tensor, total: int, name: str) -> None:
    # reference: interface.py:96-118
    if not _validate:
        return
    if cu.dim() != 1:
        raise ValueError(f"{name}: must be 1-D, got shape {tuple(cu.shape)}")
    if cu.numel() < 2:
        raise ValueError(f"{name}: must have at least 2 elements (n_seg+1 with n_seg>=1)")
    host = cu.detach().to("cpu", torch.int64)
    if int(host[0]) != 0:
        raise ValueError(f"{name}[0] must be 0, got {int(host[0])}")
    if int(host[-1]) != total:
        raise ValueError(f"{name}[-1] must equal total tokens {total}, got {int(host[-1])}")
    if bool((host[1:] < host[:-1]).any()):
        raise ValueError(f"{name} must be non-decreasing (found negative segment length)")


def _as_thd(x: torch.Tensor, name: str) -> Tuple[torch.Tensor, bool]:
    # reference: interface.py:121-150
    if x.dim() == 4:
        if x.shape[0] != 1:
            raise ValueError(f"{name}: 4-D input must have batch=1 (packed varlen), got shape {tuple(x.shape)}")
        x, was4 = x[0], True
    elif x.dim() == 3:
        was4 = False
    else:
        raise ValueError(f"{name}: expected 3-D [T,H,D] or 4-D [1,T,H,D], got {x.dim()}-D")
    if not x.is_contiguous():
        x = x.contiguous()
    return x, was4


def _fill_args(q, k, v, o, lse, cu_q, cu_k, scale, causal, split_k_block) -> _lib.VarlenArgs:
    a = _lib.VarlenArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.cu_seqlens_q, a.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    a.n_seg = cu_q.numel() - 1
    a.total_q, a.num_heads, a.head_dim = q.shape
    a.total_k = k.shape[0]
    a.num_kv_heads = k.shape[1]
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal = int(bool(causal))
    a.scale = float(scale)
    a.impl = _impl
    a.split_k_block = int(split_k_block or 0)
    a.sm_count = _lib.sm_count(q.device)
    a.status = _lib.status_word(q.device).data_ptr()
    return a


class _PackedVarlenAttn(torch.autograd.Function):
    """Counterpart of _PackedVarlenAttnFunction (reference interface.py:153-341)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, scale, causal, split_k_block):
        T_q, H, D = q.shape
        T_k, H_kv = k.shape[0], k.shape[1]
        assert k.dim() == 3 and k.shape[2] == D and H_kv >= 1 and H % H_kv == 0, \
            f"K shape mismatch: {tuple(k.shape)} vs expected ({T_k},{H},{D}) (or fewer heads dividing {H})"
        assert v.shape == k.shape, f"V shape mismatch: {tuple(v.shape)} vs K {tuple(k.shape)}"
        assert q.dtype == k.dtype == v.dtype, "q/k/v must share dtype"
        assert q.dtype in _lib.DTYPE_CODE, f"q/k/v must be fp32, bf16 or fp16, got {q.dtype}"
        assert q.is_cuda, "packed_varlen_attn requires CUDA tensors (there is no CPU path)"
        assert k.device == q.device and v.device == q.device, "q/k/v must be on the same device"
        assert D in _SUPPORTED_HEAD_DIMS, f"head_dim {D} not supported (try 64/128/256)"

        cu_q = cu_q.to(device=q.device, dtype=torch.int32).contiguous()
        cu_k = cu_k.to(device=q.device, dtype=torch.int32).contiguous()
        assert cu_k.numel() == cu_q.numel(), \
            f"segment count mismatch: q has {cu_q.numel() - 1}, k has {cu_k.numel() - 1}"
        _check_cu(cu_q, T_q, "cu_seqlens_q")
        _check_cu(cu_k, T_k, "cu_seqlens_k")

        lib = _lib.load()
        o = torch.empty_like(q)
        lse = torch.empty((T_q, H), dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            a = _fill_args(q, k, v, o, lse, cu_q, cu_k, scale, causal, split_k_block)
            ws = _lib.workspace(lib.vafa_varlen_fwd_workspace_bytes(a), q.device)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            _lib.check(lib.vafa_varlen_fwd(a, torch.cuda.current_stream().cuda_stream), "vafa_varlen_fwd")
            _lib.maybe_check_status(q.device)
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k)
        ctx.scale, ctx.causal, ctx.split_k_block = scale, causal, split_k_block
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, cu_q, cu_k = ctx.saved_tensors
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        if not do.is_contiguous():
            do = do.contiguous()
        lib = _lib.load()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        with torch.cuda.device(q.device):
            a = _fill_args(q, k, v, o, lse, cu_q, cu_k, ctx.scale, ctx.causal, ctx.split_k_block)
            a.d_o, a.dq, a.dk, a.dv = do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
            ws = _lib.workspace(lib.vafa_varlen_bwd_workspace_bytes(a), q.device)
            a.workspace, a.workspace_bytes = _lib.ptr(ws), 0 if ws is None else ws.numel()
            _lib.check(lib.vafa_varlen_bwd(a, torch.cuda.current_stream().cuda_stream), "vafa_varlen_bwd")
            _lib.maybe_check_status(q.device)
        return dq, dk, dv, None, None, None, None, None


def _prepare(q, k, v, cu_seqlens_q, cu_seqlens_k, q_seqinfo, k_seqinfo, scale):
    q3, q4 = _as_thd(q, "q")
    k3, _ = _as_thd(k, "k")
    v3, _ = _as_thd(v, "v")
    if cu_seqlens_q is None:
        if q_seqinfo is None:
            raise ValueError("must provide either cu_seqlens_q or q_seqinfo")
        cu_seqlens_q = _lengths_to_cu(q_seqinfo)
    if cu_seqlens_k is None:
        if k_seqinfo is None:
            raise ValueError("must provide either cu_seqlens_k or k_seqinfo")
        cu_seqlens_k = _lengths_to_cu(k_seqinfo)
    if scale is None:
        scale = 1.0 / math.sqrt(q3.shape[-1])
    if k3.dim() == 3 and q3.dim() == 3 and k3.shape[1] != q3.shape[1]:
        k3, v3 = _expand_kv_heads(q3, k3, v3)
    return q3, k3, v3, cu_seqlens_q, cu_seqlens_k, float(scale), q4


def packed_varlen_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    cu_seqlens_q: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    q_seqinfo: Optional[torch.Tensor] = None,
    k_seqinfo: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    causal: bool = False,
    split_k_block: Optional[int] = None,
) -> torch.Tensor:
    """Attention where token t of segment i attends only to the keys of segment i.

    q: [1, T_q, H, D] or [T_q, H, D]; k, v: [1, T_k, H, D] or [T_k, H, D] (fp32, bf16 or fp16).
    k and v may carry fewer heads, H_kv dividing H (grouped-query / multi-query attention; the reference is
    multi-head only): query head h then attends over K/V head h // (H // H_kv), and dk, dv come back with
    H_kv heads.
    cu_seqlens_q / cu_seqlens_k: [n_seg+1] prefix sums (any integer dtype, any device), or
    q_seqinfo / k_seqinfo: [n_seg] per-segment lengths.  scale defaults to 1/sqrt(D).
    causal: bottom-right aligned causal mask inside each segment (row i sees keys
    j <= i + Lk - Lq); False reproduces the reference.  split_k_block: None lets the library
    pick the split-K factor from the KV lengths; an integer (multiple of 128) fixes the KV
    slice length the way the reference's constant 4096 does.  The result does not depend on it
    beyond fp32 rounding.

    Returns o with the layout of q.  A query row that sees no key (empty KV segment, or masked
    out entirely) yields zeros.

    Failures found on the device (a wait inside a kernel that ran out, a tile list that outgrew its
    buffer) do not raise here: the call only enqueues work.  They are written to a per-device status
    word; `_lib.check_status(device)` reads it (it synchronises), and `_lib.set_check_status(True)` or
    VAFA_CHECK_STATUS=1 makes every call do so.
    """
    q3, k3, v3, cu_q, cu_k, scale, was4 = _prepare(q, k, v, cu_seqlens_q, cu_seqlens_k, q_seqinfo, k_seqinfo, scale)
    o, _ = _PackedVarlenAttn.apply(q3, k3, v3, cu_q, cu_k, scale, bool(causal), split_k_block)
    return o.unsqueeze(0) if was4 else o


def _expand_kv_heads(q3, k3, v3):
    """Grouped-query inputs on shapes the tensor-core kernels do not take (fp32, head dims other than 64/128):
    the K/V heads are repeated to one per query head with a differentiable torch op, so the gradients come back
    summed over each group.  The tensor-core kernels read the shared heads in place instead."""
    H, H_kv = q3.shape[1], k3.shape[1]
    if H_kv == H or H % max(H_kv, 1) != 0:
        return k3, v3
    native = q3.dtype in (torch.bfloat16, torch.float16) and q3.shape[2] in (64, 128) and _impl != _lib.IMPL_SIMT
    if native:
        return k3, v3
    g = H // H_kv
    return k3.repeat_interleave(g, dim=1), v3.repeat_interleave(g, dim=1)


def packed_varlen_attn_with_lse(q, k, v, *, cu_seqlens_q=None, cu_seqlens_k=None, q_seqinfo=None,
                                k_seqinfo=None, scale=None, causal=False, split_k_block=None):
    """As packed_varlen_attn, and also returns the natural-log LSE [T_q, H] (fp32).

    The reference keeps the same quantity in the log2 domain as an internal saved tensor
    (triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:164-166); this is that value times ln 2.
    """
    q3, k3, v3, cu_q, cu_k, scale, was4 = _prepare(q, k, v, cu_seqlens_q, cu_seqlens_k, q_seqinfo, k_seqinfo, scale)
    o, lse2 = _PackedVarlenAttn.apply(q3, k3, v3, cu_q, cu_k, scale, bool(causal), split_k_block)
    return (o.unsqueeze(0) if was4 else o), lse2 * LN2
