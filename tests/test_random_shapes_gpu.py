"""Seeded random-shape sweeps of both operators on the GPU (through the C ABI).

The reference tests fixed lists of shapes (triton_fa_varlen_v2/triton_fa_varlen_v2/test_smoke.py:222-531,
triton_target_attn_absorb/triton_target_attn_absorb/test_smoke.py:2295-2338).  The sweeps draw segment lists
with empty, one-row, tile-edge and multi-block lengths, head counts, grouped K/V heads, head dims, dtypes,
causal flags, split-K blocks and both backward modes, and hold every output and gradient to the CPU oracle.

Absorb: a user with a single key has an exactly zero score gradient, so dq_raw, dW_Q and dW_K of a batch of
such users are mostly rounding noise of the 16-bit O that delta = rowsum(dO * O) is formed from, and a
relative bound against their small true value has no meaning (the reference's kernels show the same figures
on the same inputs).  Those three are therefore bounded in absolute terms here and, when the installed
reference is present, by the reference kernels' own error against the oracle on the same inputs."""
import os
import random
import sys

import pytest
import torch

import varlenabsorbflashattn_b200 as vb
from varlenabsorbflashattn_b200 import _lib
from oracle import (bf16_floor, make_absorb_inputs, make_varlen_inputs, max_abs, rel_l2, target_attn_ref_fwd_bwd,
                    varlen_attn_ref_fwd_bwd)
from helpers import check_close, check_lse, LN2

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def _draw_len(r):
    u = r.random()
    if u < 0.10:
        return 0
    if u < 0.30:
        return r.randint(1, 8)
    if u < 0.55:
        return r.randint(9, 140)
    if u < 0.85:
        return r.randint(100, 400)
    return r.randint(300, 1400)


def varlen_case(seed):
    r = random.Random(seed)
    n = r.randint(1, 10)
    same = r.random() < 0.4
    ql, kl = [], []
    for _ in range(n):
        a = _draw_len(r)
        ql.append(a)
        kl.append(a if same else _draw_len(r))
    if sum(ql) == 0:
        ql[0] = 3
    if sum(kl) == 0:
        kl[0] = 5
    H = r.choice([1, 2, 3, 4, 6, 8])
    G = r.choice([g for g in (1, 1, 2, 3, 4, 8) if H % g == 0])
    D = r.choice([64, 128])
    return dict(ql=ql, kl=kl, H=H, G=G, D=D, dtype=r.choice([torch.bfloat16, torch.float16]),
                causal=r.random() < 0.5, split=r.choice([None, None, 128, 256, 512]),
                fused=D == 128 and G == 1 and r.random() < 0.25)


@pytest.mark.parametrize("seed", range(48))
def test_varlen_random_shapes(seed):
    c = varlen_case(seed)
    ql, kl, H, G, D, dtype, causal = c["ql"], c["kl"], c["H"], c["G"], c["D"], c["dtype"], c["causal"]
    q, _, _, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, dtype, seed)
    Hk = H // G
    g = torch.Generator().manual_seed(seed + 99)
    k = torch.randn(sum(kl), Hk, D, generator=g).to(dtype)
    v = torch.randn(sum(kl), Hk, D, generator=g).to(dtype)
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    vb.set_backward_mode("fused" if c["fused"] else "split")
    try:
        o, lse = vb.packed_varlen_attn_with_lse(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal,
                                                split_k_block=c["split"])
        o.backward(do.to(DEV))
        torch.cuda.synchronize()
    finally:
        vb.set_backward_mode("split")
    _lib.check_status(torch.device("cuda", 0))
    ke, ve = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)
    ro, rlse, rdq, rdk, rdv = varlen_attn_ref_fwd_bwd(q, ke, ve, do, cu_q, cu_k, causal=causal)
    Tk = rdk.shape[0]
    check_close("o", o, ro, dtype)
    check_lse(lse / LN2, rlse)
    check_close("dq", qg.grad, rdq, dtype, scale_abs=True)
    check_close("dk", kg.grad, rdk.view(Tk, Hk, G, D).sum(2), dtype, scale_abs=True)
    check_close("dv", vg.grad, rdv.view(Tk, Hk, G, D).sum(2), dtype, scale_abs=True)


def absorb_case(seed):
    r = random.Random(10_000 + seed)
    n = r.randint(1, 24)
    ql = [0 if r.random() < 0.1 else r.randint(1, r.choice([4, 18, 40])) for _ in range(n)]
    kl = [0 if r.random() < 0.1 else r.randint(1, r.choice([30, 300, 2048])) for _ in range(n)]
    kl = [max(b, 1) if a > 0 else b for a, b in zip(ql, kl)]   # a user with queries has at least one key
    if sum(ql) == 0:
        ql[0], kl[0] = 2, max(kl[0], 7)
    d_q, d_kv = r.choice([(968, 216), (968, 216), (256, 256), (1024, 256), (512, 128), (200, 96)])
    H, D_H = r.choice([(8, 32), (8, 32), (4, 64), (16, 16), (2, 32)])
    dtype = r.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32])
    return dict(ql=ql, kl=kl, d_q=d_q, d_kv=d_kv, H=H, D_H=D_H, dtype=dtype)


def _reference_absorb():
    """The installed reference's operator, or None (the comparison with it is then left out)."""
    if not os.path.isdir(os.path.join(REF_DIR, "triton_target_attn_absorb")):
        return None
    if os.environ.get("TRITON_INTERPRET", "0") not in ("", "0"):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import triton_target_attn_absorb as RA
    return RA.packed_target_attn


NAMES = ("O", "dq_raw", "dX", "dW_Q", "dW_K", "dW_V")
NOISE_BOUND = ("dq_raw", "dW_Q", "dW_K")


@pytest.mark.parametrize("seed", range(48))
def test_absorb_random_shapes(seed):
    c = absorb_case(seed)
    dtype = c["dtype"]
    ins = make_absorb_inputs(c["ql"], c["kl"], c["d_q"], c["d_kv"], c["H"], c["D_H"], dtype, seed, x_std=0.1, w_std=0.1)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    ref = target_attn_ref_fwd_bwd(*ins)
    refs = (ref[0],) + tuple(ref[2:])
    cq, ck = cu_q.to(DEV), cu_k.to(DEV)

    def run(fn):
        g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
        O = fn(*g, cu_seqlens_q=cq, cu_seqlens_k=ck)
        grads = torch.autograd.grad(O, g, dO.to(DEV))
        torch.cuda.synchronize()
        return (O.detach(),) + tuple(grads)

    ours = run(vb.packed_target_attn)
    _lib.check_status(torch.device("cuda", 0))
    theirs_fn = _reference_absorb()
    theirs = run(theirs_fn) if theirs_fn is not None else None
    for i, (name, mine, r) in enumerate(zip(NAMES, ours, refs)):
        if name not in NOISE_BOUND:
            check_close(name, mine, r, dtype, scale_abs=True)
            continue
        got = mine.float().cpu()
        assert torch.isfinite(got).all(), name
        abs_tol = (2e-4 if dtype == torch.float32 else 2e-2) * max(1.0, r.abs().max().item())
        assert max_abs(got, r) <= abs_tol, f"{name}: max-abs {max_abs(got, r):.3e} > {abs_tol:.3e}"
        if theirs is not None:
            t = theirs[i].float().cpu()
            assert max_abs(got, r) <= max(2.0 * max_abs(t, r), 1e-5), \
                f"{name}: max-abs {max_abs(got, r):.3e} vs reference kernels {max_abs(t, r):.3e}"
            if rel_l2(t, r) < 0.1:   # else the true value is (nearly) zero and only the absolute bounds mean anything
                bound = max(1.3 * rel_l2(t, r), 1.5 * bf16_floor(r, dtype), 1e-3)
                assert rel_l2(got, r) <= bound, \
                    f"{name}: rel-L2 {rel_l2(got, r):.3e} vs reference kernels {rel_l2(t, r):.3e}"
