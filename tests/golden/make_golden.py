"""Generate the golden vectors under tests/golden/ from the reference's own kernels.

Run once, in a container that holds the reference checkout (it is not needed afterwards):

    TRITON_INTERPRET=1 PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The reference's public wrappers refuse CPU tensors, so this script replays their launch
sequence (triton_fa_varlen_v2/triton_fa_varlen_v2/interface.py:187-236 and :268-338;
triton_target_attn_absorb/triton_target_attn_absorb/interface.py:203-216 and :243-319,
prologue :434-435) on CPU tensors with the Triton interpreter.  Inputs are regenerated from
seeds by `oracle.gen`; only the reference's OUTPUTS are stored (fp32, .npz).
"""
from __future__ import annotations

import math
import os
import sys

if __name__ == "__main__":
    # only when generating: the tests import this module for its case tables, in a process that may
    # also run the reference's kernels on a GPU, where the interpreter must stay off
    os.environ.setdefault("TRITON_INTERPRET", "1")
    sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.gen import make_varlen_inputs, make_absorb_inputs  # noqa: E402

LN2 = math.log(2.0)

# name -> (q_lens, k_lens, H, D, seed, with_backward)
VARLEN_CASES = {
    "c1": ([17, 64, 128, 255], [17, 64, 128, 255], 8, 64, 0, False),
    "tiny": ([7, 11], [19, 5], 4, 64, 0, True),
    "cross_block": ([129, 257], [33, 130], 2, 64, 1, True),
    "split": ([3, 40], [4500, 70], 1, 16, 2, True),
    "empty_seg": ([5, 0, 9], [12, 6, 0 + 31], 2, 16, 3, True),
}
# name -> (q_lens, k_lens, d_q, d_kv, H, D_H, seed)
ABSORB_CASES = {
    "short_k": ([1, 2, 4, 8], [1, 3, 7, 15], 64, 48, 4, 16, 0),
    "smoke": ([4], [64], 968, 216, 8, 32, 1),
    "tails": ([17, 3, 33], [70, 129, 64], 128, 256, 8, 32, 2),
}


def run_varlen(ref_root: str, out_dir: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "triton_fa_varlen_v2"))
    from triton_fa_varlen_v2 import kernels as K
    from triton_fa_varlen_v2.chunk_indices import prepare_split_indices, prepare_k_chunk_indices

    BT, BS = 128, 32
    for name, (ql, kl, H, D, seed, bwd) in VARLEN_CASES.items():
        q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, torch.float32, seed)
        scale = 1.0 / math.sqrt(D)
        Tq, Tk = q.shape[0], k.shape[0]
        o = torch.zeros_like(q)
        lse = torch.zeros(Tq, H, dtype=torch.float32)
        si = prepare_split_indices(cu_q, cu_k, BT=BT, SPLIT_K_BLOCK=4096, SPLIT_THRESHOLD=4096)
        if si.short.shape[0] > 0:
            K._fwd_kernel[(si.short.shape[0], H)](q, k, v, o, lse, cu_q, cu_k, si.short, scale,
                                                  H=H, D=D, BT=BT, BS=BS)
        if si.n_split_progs > 0:
            po = torch.zeros(si.n_split_progs, H, BT, D, dtype=torch.float32)
            pl = torch.zeros(si.n_split_progs, H, BT, dtype=torch.float32)
            K._fwd_split_kernel[(si.n_split_progs, H)](q, k, v, po, pl, cu_q, cu_k, si.split, scale,
                                                       H=H, D=D, BT=BT, BS=BS, SPLIT_K_BLOCK=4096)
            K._fwd_combine_kernel[(si.n_combine_progs, H)](po, pl, o, lse, cu_q, si.combine, H=H, D=D, BT=BT)
        rec = {"o": o.numpy(), "lse_log2": lse.numpy()}
        if bwd:
            delta = torch.zeros(Tq, H, dtype=torch.float32)
            K._bwd_preprocess_kernel[((Tq + BT - 1) // BT, H)](o, do, delta, Tq, H=H, D=D, BT=BT)
            dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
            if si.short.shape[0] > 0:
                K._bwd_dq_kernel[(si.short.shape[0], H)](q, k, v, do, dq, lse, delta, cu_q, cu_k, si.short, scale,
                                                         H=H, D=D, BT=BT, BS=BS)
            if si.n_split_progs > 0:
                pdq = torch.zeros(si.n_split_progs, H, BT, D, dtype=torch.float32)
                K._bwd_dq_split_kernel[(si.n_split_progs, H)](q, k, v, do, pdq, lse, delta, cu_q, cu_k, si.split,
                                                              scale, H=H, D=D, BT=BT, BS=BS, SPLIT_K_BLOCK=4096)
                K._bwd_dq_combine_kernel[(si.n_combine_progs, H)](pdq, dq, cu_q, si.combine, scale,
                                                                  H=H, D=D, BT=BT)
            k_idx = prepare_k_chunk_indices(cu_k, 128)
            if k_idx.shape[0] > 0:
                K._bwd_dkv_kernel[(k_idx.shape[0], H)](q, k, v, do, dk, dv, lse, delta, cu_q, cu_k, k_idx, scale,
                                                       H=H, D=D, BT=128, BS=32)
            rec.update(dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())
        np.savez(os.path.join(out_dir, f"varlen_{name}.npz"), **rec)
        print("varlen", name, "done", flush=True)
    sys.path.pop(0)


def run_absorb(ref_root: str, out_dir: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "triton_target_attn_absorb"))
    from triton_target_attn_absorb import kernels as K
    from triton_target_attn_absorb.chunk_indices import prepare_q_chunk_indices, prepare_k_chunk_indices

    for name, (ql, kl, d_q, d_kv, H, D_H, seed) in ABSORB_CASES.items():
        q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs(
            ql, kl, d_q, d_kv, H, D_H, torch.float32, seed, x_std=0.5)
        scale = 1.0 / math.sqrt(D_H)
        Tq, Tk = q_raw.shape[0], X.shape[0]
        q_raw.requires_grad_(True)
        W_Q.requires_grad_(True)
        W_K.requires_grad_(True)
        q_proj = (q_raw @ W_Q.reshape(d_q, H * D_H)).view(Tq, H, D_H)
        u_t = torch.einsum("thd,khd->thk", q_proj, W_K)
        u = u_t.detach().contiguous()
        B_DKV = 1 << (d_kv - 1).bit_length()
        qi = prepare_q_chunk_indices(cu_q, 16)
        ki = prepare_k_chunk_indices(cu_k, 64)
        O = torch.zeros(Tq, H, D_H, dtype=torch.float32)
        LSE = torch.zeros(Tq, H, dtype=torch.float32)
        K._fwd_alpha_kernel[(qi.shape[0], H)](u, X, W_V, O, LSE, cu_q, cu_k, qi, scale,
                                              H=H, D_KV=d_kv, B_DKV=B_DKV, D_H=D_H, BT_Q=16, BT_K=64)
        delta = torch.zeros(Tq, H, dtype=torch.float32)
        K._bwd_preprocess_kernel[((Tq + 15) // 16, H)](O, dO, delta, Tq, H=H, D_H=D_H, BT=16)
        du = torch.zeros_like(u)
        dax = torch.zeros(Tq, H, d_kv, dtype=torch.float32)
        dWV = torch.zeros(d_kv, H, D_H, dtype=torch.float32)
        dX = torch.zeros(Tk, d_kv, dtype=torch.float32)
        K._bwd_du_kernel[(qi.shape[0], H)](u, X, W_V, dO, du, dax, dWV, LSE, delta, cu_q, cu_k, qi, scale,
                                           H=H, D_KV=d_kv, B_DKV=B_DKV, D_H=D_H, BT_Q=16, BT_K=64)
        K._bwd_dx_fused_heads_kernel[(ki.shape[0],)](u, X, dax, dX, LSE, delta, cu_q, cu_k, ki, scale,
                                                     H=H, D_KV=d_kv, B_DKV=B_DKV, D_H=D_H, BT_K=64, BT_Q=16)
        u_t.backward(du)
        np.savez(os.path.join(out_dir, f"absorb_{name}.npz"), O=O.numpy(), lse_log2=LSE.numpy(),
                 dq_raw=q_raw.grad.numpy(), dX=dX.numpy(), dW_Q=W_Q.grad.numpy(),
                 dW_K=W_K.grad.numpy(), dW_V=dWV.numpy())
        print("absorb", name, "done", flush=True)
    sys.path.pop(0)


if __name__ == "__main__":
    root = sys.argv[1]
    torch.set_num_threads(1)
    run_varlen(root, HERE)
    run_absorb(root, HERE)
