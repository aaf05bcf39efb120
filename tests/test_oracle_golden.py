"""Pin the CPU oracle against the stored outputs of the reference's own Triton kernels.

The .npz files under tests/golden/ were produced by tests/golden/make_golden.py, which runs
the reference kernels (fp32) under the Triton interpreter on inputs regenerated here from
the same seeds.  fp32 kernels vs an fp32 restatement: agreement to ~1e-5.
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import VARLEN_CASES, ABSORB_CASES  # noqa: E402
from oracle import (make_varlen_inputs, make_absorb_inputs, varlen_attn_ref_fwd_bwd,
                    target_attn_ref_fwd_bwd, max_abs)

LN2 = math.log(2.0)


@pytest.mark.parametrize("name", sorted(VARLEN_CASES))
def test_varlen_oracle_matches_reference_kernels(name, golden_dir):
    ql, kl, H, D, seed, bwd = VARLEN_CASES[name]
    g = np.load(os.path.join(golden_dir, f"varlen_{name}.npz"))
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, torch.float32, seed)
    o, lse, dq, dk, dv = varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=False,
                                                 compute_dtype=torch.float64)
    # rows whose segment has no keys: the reference yields NaN/-inf there, the oracle 0/-inf
    live = torch.isfinite(lse)
    go, glse = torch.from_numpy(g["o"]), torch.from_numpy(g["lse_log2"]) * LN2
    assert max_abs(o[live], go[live]) < 2e-5
    assert max_abs(lse[live], glse[live]) < 2e-5
    if bwd:
        assert max_abs(dq[live], torch.from_numpy(g["dq"])[live]) < 5e-5
        assert max_abs(dk, torch.from_numpy(g["dk"])) < 5e-5
        assert max_abs(dv, torch.from_numpy(g["dv"])) < 5e-5


@pytest.mark.parametrize("name", sorted(ABSORB_CASES))
def test_absorb_oracle_matches_reference_kernels(name, golden_dir):
    ql, kl, d_q, d_kv, H, D_H, seed = ABSORB_CASES[name]
    g = np.load(os.path.join(golden_dir, f"absorb_{name}.npz"))
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs(
        ql, kl, d_q, d_kv, H, D_H, torch.float32, seed, x_std=0.5)
    O, lse, dq_raw, dX, dW_Q, dW_K, dW_V = target_attn_ref_fwd_bwd(
        q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k, compute_dtype=torch.float64)
    assert max_abs(O, torch.from_numpy(g["O"])) < 2e-5
    assert max_abs(lse, torch.from_numpy(g["lse_log2"]) * LN2) < 2e-5
    for mine, key in ((dq_raw, "dq_raw"), (dX, "dX"), (dW_Q, "dW_Q"), (dW_K, "dW_K"), (dW_V, "dW_V")):
        ref = torch.from_numpy(g[key])
        assert max_abs(mine, ref) < 1e-4 * max(1.0, ref.abs().max().item()), key
