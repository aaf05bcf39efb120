"""fp32 (or fp64) CPU restatements of the two operators.  Test infrastructure only.

Varlen attention follows the reference's own torch oracle
(triton_fa_varlen_v2/triton_fa_varlen_v2/test_smoke.py:73-164: per segment, explicit
`matmul -> softmax -> matmul`, autograd for the gradients) and adds what the reference
kernels compute but its oracle does not return: the log-sum-exp (natural log here; the
kernels keep `m + log2(l)` in the log2 domain, triton_fa_varlen_v2/triton_fa_varlen_v2/
kernels.py:164-166, which is this value divided by ln 2), an optional causal mask
(bottom-right aligned like flash-attn: row i of a segment sees keys j <= i + Lk - Lq) and
a defined result for rows that see no key (O = 0, LSE = -inf).

Target attention follows `reference_target_attn`
(triton_target_attn_absorb/triton_target_attn_absorb/test_smoke.py:111-147): the
un-absorbed formulation with explicit K = X W_K and V = X W_V per segment and head, with
autograd for the gradients of all five inputs.  Unlike that function the probabilities
are not rounded to the I/O dtype, so the oracle is the exact-arithmetic answer for the
(already rounded) inputs.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _lens(cu) -> list:
    c = [int(x) for x in (cu.tolist() if isinstance(cu, torch.Tensor) else cu)]
    return [c[i + 1] - c[i] for i in range(len(c) - 1)]


def _segment_attn(qi, ki, vi, scale: float, causal: bool):
    """qi [Lq,H,D], ki/vi [Lk,H,D] (compute dtype).  Returns o [Lq,H,D], lse [Lq,H] (natural log)."""
    Lq, H, D = qi.shape
    Lk = ki.shape[0]
    qh = qi.transpose(0, 1).contiguous()   # [H, Lq, D], the layout the reference's oracle multiplies in
    kh = ki.transpose(0, 1).contiguous()
    vh = vi.transpose(0, 1).contiguous()
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        row = torch.arange(Lq).view(Lq, 1)
        col = torch.arange(Lk).view(1, Lk)
        dead = col > row + (Lk - Lq)
        s = s.masked_fill(dead.unsqueeze(0), float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m_safe)
    l = p.sum(dim=-1, keepdim=True)
    lse = (m_safe + torch.log(l)).squeeze(-1)            # -inf where l == 0
    pn = p / torch.where(l == 0, torch.ones_like(l), l)
    o = torch.matmul(pn, vh).transpose(0, 1)
    return o, lse.transpose(0, 1)


def varlen_attn_ref(q, k, v, cu_seqlens_q, cu_seqlens_k, scale: Optional[float] = None,
                    causal: bool = False, compute_dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward only.  Returns (o [T_q,H,D] compute dtype, lse [T_q,H] natural log)."""
    Tq, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ql, kl = _lens(cu_seqlens_q), _lens(cu_seqlens_k)
    assert len(ql) == len(kl)
    o = torch.zeros(Tq, H, D, dtype=compute_dtype)
    lse = torch.full((Tq, H), float("-inf"), dtype=compute_dtype)
    qo = ko = 0
    for Lq, Lk in zip(ql, kl):
        if Lq > 0 and Lk > 0:
            oi, li = _segment_attn(q[qo:qo + Lq].to(compute_dtype), k[ko:ko + Lk].to(compute_dtype),
                                   v[ko:ko + Lk].to(compute_dtype), scale, causal)
            o[qo:qo + Lq] = oi
            lse[qo:qo + Lq] = li
        qo += Lq
        ko += Lk
    return o, lse


def varlen_attn_ref_fwd_bwd(q, k, v, do, cu_seqlens_q, cu_seqlens_k, scale: Optional[float] = None,
                            causal: bool = False, compute_dtype=torch.float32):
    """Forward + autograd backward, one throw-away graph per segment.

    Returns (o, lse, dq, dk, dv) in the compute dtype.
    """
    Tq, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ql, kl = _lens(cu_seqlens_q), _lens(cu_seqlens_k)
    o = torch.zeros(Tq, H, D, dtype=compute_dtype)
    lse = torch.full((Tq, H), float("-inf"), dtype=compute_dtype)
    dq = torch.zeros(q.shape, dtype=compute_dtype)
    dk = torch.zeros(k.shape, dtype=compute_dtype)
    dv = torch.zeros(v.shape, dtype=compute_dtype)
    qo = ko = 0
    for Lq, Lk in zip(ql, kl):
        if Lq > 0 and Lk > 0:
            qi = q[qo:qo + Lq].detach().to(compute_dtype).requires_grad_(True)
            ki = k[ko:ko + Lk].detach().to(compute_dtype).requires_grad_(True)
            vi = v[ko:ko + Lk].detach().to(compute_dtype).requires_grad_(True)
            oi, li = _segment_attn(qi, ki, vi, scale, causal)
            oi.backward(do[qo:qo + Lq].detach().to(compute_dtype))
            o[qo:qo + Lq] = oi.detach()
            lse[qo:qo + Lq] = li.detach()
            dq[qo:qo + Lq] = qi.grad
            dk[ko:ko + Lk] = ki.grad
            dv[ko:ko + Lk] = vi.grad
        qo += Lq
        ko += Lk
    return o, lse, dq, dk, dv


def lse_combine_ref(partial_o: torch.Tensor, partial_lse: torch.Tensor):
    """Merge split-K partials: partial_o [S, R, D] normalised per split, partial_lse [S, R]
    natural log.  Follows triton_fa_varlen_v2/triton_fa_varlen_v2/kernels.py:639-648."""
    m = partial_lse.max(dim=0).values
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(partial_lse - m_safe)
    den = w.sum(0)
    o = (partial_o * w.unsqueeze(-1)).sum(0) / torch.where(den == 0, torch.ones_like(den), den).unsqueeze(-1)
    return o, m_safe + torch.log(den)


def _target_segments(q_raw, X, W_Q, W_K, W_V, ql, kl, scale, compute_dtype, do=None):
    Tq = q_raw.shape[0]
    _, H, D_H = W_Q.shape
    O = torch.zeros(Tq, H, D_H, dtype=compute_dtype)
    lse = torch.full((Tq, H), float("-inf"), dtype=compute_dtype)
    outs = []
    qo = ko = 0
    for Lq, Lk in zip(ql, kl):
        if Lq > 0 and Lk > 0:
            qi = q_raw[qo:qo + Lq]
            xi = X[ko:ko + Lk]
            qp = torch.einsum("qa,ahd->qhd", qi, W_Q)
            kp = torch.einsum("ka,ahd->khd", xi, W_K)
            vp = torch.einsum("ka,ahd->khd", xi, W_V)
            oi, li = _segment_attn(qp, kp, vp, scale, False)
            outs.append((qo, Lq, oi, li))
        qo += Lq
        ko += Lk
    return outs


def target_attn_ref(q_raw, X, W_Q, W_K, W_V, cu_seqlens_q, cu_seqlens_k, scale: Optional[float] = None,
                    compute_dtype=torch.float32):
    """Forward only.  Returns (O [T_q,H,D_H], lse [T_q,H] natural log) in the compute dtype."""
    _, H, D_H = W_Q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D_H)
    args = [t.detach().to(compute_dtype) for t in (q_raw, X, W_Q, W_K, W_V)]
    O = torch.zeros(q_raw.shape[0], H, D_H, dtype=compute_dtype)
    lse = torch.full((q_raw.shape[0], H), float("-inf"), dtype=compute_dtype)
    for qo, Lq, oi, li in _target_segments(*args, _lens(cu_seqlens_q), _lens(cu_seqlens_k), scale, compute_dtype):
        O[qo:qo + Lq] = oi
        lse[qo:qo + Lq] = li
    return O, lse


def target_attn_ref_fwd_bwd(q_raw, X, W_Q, W_K, W_V, dO, cu_seqlens_q, cu_seqlens_k,
                            scale: Optional[float] = None, compute_dtype=torch.float32):
    """Forward + autograd backward.  Returns (O, lse, dq_raw, dX, dW_Q, dW_K, dW_V)."""
    _, H, D_H = W_Q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D_H)
    leaves = [t.detach().to(compute_dtype).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
    O = torch.zeros(q_raw.shape[0], H, D_H, dtype=compute_dtype)
    lse = torch.full((q_raw.shape[0], H), float("-inf"), dtype=compute_dtype)
    dOc = dO.detach().to(compute_dtype)
    loss = None
    for qo, Lq, oi, li in _target_segments(*leaves, _lens(cu_seqlens_q), _lens(cu_seqlens_k), scale, compute_dtype):
        O[qo:qo + Lq] = oi.detach()
        lse[qo:qo + Lq] = li.detach()
        term = (oi * dOc[qo:qo + Lq]).sum()
        loss = term if loss is None else loss + term
    grads = [torch.zeros_like(t) for t in leaves]
    if loss is not None:
        loss.backward()
        grads = [t.grad if t.grad is not None else torch.zeros_like(t) for t in leaves]
    return (O, lse, *grads)
