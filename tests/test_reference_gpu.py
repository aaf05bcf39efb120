"""The library beside the reference's own GPU kernels and flash-attn, on identical seeded inputs.

`baseline/_ref` holds the unmodified reference packages (installed by baseline/install_ref.sh; the
folder is not part of the repository's history, so these tests skip where it is absent).  Each case
runs three implementations on the same device tensors -- this library, the reference's Triton
kernels through their public API, and flash-attn's `flash_attn_varlen_func` -- and holds all of
them to the fp32 CPU oracle.  The assertion is the second half of the parity criterion: this
library's error is no worse than the reference's on the same inputs (within a factor of 1.3 in rel-L2 and 1.5 in max-abs, or
within 1.5x of the error that rounding the exact result to bf16 causes, whichever is larger), for
O, the LSE and every gradient.

Shapes stay far below 2^31 elements per tensor: the reference's kernels compute element offsets in
32 bits and are not run beyond that.  The reference has no causal mode, so causal is compared with
flash-attn alone.  The reference keeps its LSE (log2 domain) as saved tensor 4 of the autograd node
(triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:245-248).

With VAFA_PARITY_REPORT=<path> the measured errors are also written there as JSON.
"""
import json
import math
import os
import sys

import pytest
import torch

import varlenabsorbflashattn_b200 as vb
from oracle import (bf16_floor, log_uniform_lengths, make_absorb_inputs, make_varlen_inputs, max_abs, rel_l2,
                    target_attn_ref_fwd_bwd, varlen_attn_ref_fwd_bwd)

pytestmark = pytest.mark.gpu
DEV = "cuda"
LN2 = math.log(2.0)
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
_REPORT = {}


def _ref_pkgs():
    if not os.path.isdir(os.path.join(REF_DIR, "triton_fa_varlen_v2")):
        pytest.skip("baseline/_ref is absent (bash baseline/install_ref.sh <reference checkout>)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    # the reference must be compiled for the GPU here, not run by Triton's CPU interpreter
    assert os.environ.get("TRITON_INTERPRET", "0") in ("", "0"), "TRITON_INTERPRET is set in this process"
    import triton_fa_varlen_v2 as R
    import triton_target_attn_absorb as RA
    return R, RA


def _fa2():
    try:
        from flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"flash_attn is not importable: {e}")


def _errs(got, ref):
    return {"max_abs": max_abs(got.float(), ref), "rel_l2": rel_l2(got.float(), ref), "floor": bf16_floor(ref)}


def _no_worse(name, ours, theirs, who):
    assert theirs["rel_l2"] < 0.1, f"{name}: {who} itself is off by rel-L2 {theirs['rel_l2']:.3e}: the comparison is void"
    bound = max(1.3 * theirs["rel_l2"], 1.5 * ours["floor"], 1e-3)
    assert ours["rel_l2"] <= bound, f"{name}: rel-L2 {ours['rel_l2']:.3e} vs {who} {theirs['rel_l2']:.3e} (floor {ours['floor']:.3e})"
    bound_abs = max(1.5 * theirs["max_abs"], 2e-2)
    assert ours["max_abs"] <= bound_abs, f"{name}: max-abs {ours['max_abs']:.3e} vs {who} {theirs['max_abs']:.3e}"


def _flush_report():
    path = os.environ.get("VAFA_PARITY_REPORT")
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as fh:
            json.dump(_REPORT, fh, indent=1)


def _varlen_three_ways(ql, kl, H, D, causal, seed):
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, torch.bfloat16, seed)
    ref = varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=causal)   # o, lse (natural), dq, dk, dv
    dq_, dk_, dv_, ddo = (t.to(DEV) for t in (q, k, v, do))
    cq, ck = cu_q.to(DEV), cu_k.to(DEV)
    out = {}

    def run(fn, lse_of):
        g = [t.detach().clone().requires_grad_(True) for t in (dq_, dk_, dv_)]
        o = fn(*g)
        o_main = o[0] if isinstance(o, tuple) else o
        lse = lse_of(o)
        grads = torch.autograd.grad(o_main, g, ddo)
        torch.cuda.synchronize()
        return o_main.detach(), lse, grads

    o, lse, gr = run(lambda a, b, c: vb.packed_varlen_attn_with_lse(a, b, c, cu_seqlens_q=cq, cu_seqlens_k=ck, causal=causal),
                     lambda r: r[1].detach())
    out["ours"] = (o, lse, gr)
    if not causal:
        R, _ = _ref_pkgs()
        o, lse, gr = run(lambda a, b, c: R.packed_varlen_attn(a, b, c, cu_seqlens_q=cq, cu_seqlens_k=ck),
                         lambda r: r.grad_fn.saved_tensors[4].detach() * LN2)
        out["triton"] = (o, lse, gr)
    fa = _fa2()
    o, lse, gr = run(lambda a, b, c: fa(a, b, c, cq, ck, max(ql), max(kl), causal=causal, return_attn_probs=True),
                     lambda r: r[1].detach().transpose(0, 1).contiguous())      # [H, T] -> [T, H], natural log
    out["fa2"] = (o, lse, gr)

    live = torch.isfinite(ref[1])
    metrics = {}
    for who, (o, lse, gr) in out.items():
        m = {"o": _errs(o.cpu(), ref[0]), "dq": _errs(gr[0].cpu(), ref[2]), "dk": _errs(gr[1].cpu(), ref[3]),
             "dv": _errs(gr[2].cpu(), ref[4]),
             "lse_max_abs": float((lse.float().cpu()[live] - ref[1][live]).abs().max()) if lse.shape == ref[1].shape else None}
        metrics[who] = m
    return metrics


@pytest.mark.parametrize("name,ql,kl,H,D", [
    ("ragged_h4_d128", log_uniform_lengths(12, 1, 1500, 3), None, 4, 128),
    ("cross_lengths_h4_d64", [500, 500, 129], [19, 800, 257], 4, 64),
])
def test_varlen_noncausal_against_triton_reference_and_fa2(name, ql, kl, H, D):
    kl = kl or list(ql)
    m = _varlen_three_ways(ql, kl, H, D, False, seed=21)
    _REPORT["varlen_noncausal_" + name] = m
    _flush_report()
    for t in ("o", "dq", "dk", "dv"):
        _no_worse(f"{name}.{t}", m["ours"][t], m["triton"][t], "reference Triton")
        _no_worse(f"{name}.{t}", m["ours"][t], m["fa2"][t], "flash-attn")
    assert m["ours"]["lse_max_abs"] <= 1e-4
    assert m["ours"]["lse_max_abs"] <= max(2.0 * m["triton"]["lse_max_abs"], 1e-4)


def test_varlen_causal_against_fa2():
    ql = log_uniform_lengths(12, 1, 1500, 5)
    m = _varlen_three_ways(ql, list(ql), 4, 128, True, seed=22)
    _REPORT["varlen_causal"] = m
    _flush_report()
    for t in ("o", "dq", "dk", "dv"):
        _no_worse(f"causal.{t}", m["ours"][t], m["fa2"][t], "flash-attn")
    assert m["ours"]["lse_max_abs"] <= 1e-4


@pytest.mark.parametrize("name,ql,kl", [
    ("ragged_real", [7, 8, 6, 9], [2048, 1024, 1536, 512]),
    ("mixed_tails", [1, 16, 5, 12, 3], [123, 257, 999, 64, 2048]),
])
def test_absorb_against_triton_reference(name, ql, kl):
    """Production widths d_q = 968, d_kv = 216 (reference test_smoke.py:54-57), bf16, all five gradients
    (test_smoke.py:611-625)."""
    _, RA = _ref_pkgs()
    ins = make_absorb_inputs(ql, kl, 968, 216, 8, 32, torch.bfloat16, 7, x_std=0.1, w_std=0.1)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    ref = target_attn_ref_fwd_bwd(q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k)   # O, lse, 5 grads
    cq, ck = cu_q.to(DEV), cu_k.to(DEV)
    res = {}
    for who, fn in (("ours", lambda *g: vb.packed_target_attn(*g, cu_seqlens_q=cq, cu_seqlens_k=ck)),
                    ("triton", lambda *g: RA.packed_target_attn(*g, cu_seqlens_q=cq, cu_seqlens_k=ck))):
        g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
        O = fn(*g)
        grads = torch.autograd.grad(O, g, dO.to(DEV))
        torch.cuda.synchronize()
        res[who] = {"O": _errs(O.detach().cpu(), ref[0])}
        for nm, t, r in zip(("dq_raw", "dX", "dW_Q", "dW_K", "dW_V"), grads, ref[2:]):
            res[who][nm] = _errs(t.cpu(), r)
    _REPORT["absorb_" + name] = res
    _flush_report()
    for t in ("O", "dq_raw", "dX", "dW_Q", "dW_K", "dW_V"):
        _no_worse(f"{name}.{t}", res["ours"][t], res["triton"][t], "reference Triton")
