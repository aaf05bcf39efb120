"""GPU parity of packed_target_attn / target_attn_inner (through the C ABI) against the CPU
oracle (explicit K = X W_K, V = X W_V formulation) and the stored outputs of the reference
kernels.  Cases follow triton_target_attn_absorb/triton_target_attn_absorb/test_smoke.py:2295-2338."""
import math
import os
import sys

import numpy as np
import pytest
import torch

import varlenabsorbflashattn_b200 as vb
from oracle import make_absorb_inputs, target_attn_ref_fwd_bwd, uniform_lengths, log_uniform_lengths
from helpers import check_close, check_lse

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import ABSORB_CASES  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (q_lens, k_lens) of the reference's correctness list, production dims d_q=968, d_kv=216
REF_CASES = {
    "smoke": ([4], [64]),
    "single_segment": ([7], [256]),
    "uniform4": ([8, 8, 8, 8], [128, 128, 128, 128]),
    "ragged_real": ([7, 8, 6, 9], [2048, 1024, 1536, 512]),
    "k_tail": ([5, 5, 5], [123, 257, 999]),
    "q_tail": ([33, 65, 129], [64, 64, 64]),
    "short_k": ([1, 2, 4, 8], [1, 3, 7, 15]),
    "nq1": ([1], [512]),
    "empty_users": ([3, 0, 0, 5], [40, 0, 17, 9]),
}


def _run(ql, kl, d_q, d_kv, H, D_H, dtype, seed, x_std=0.1, w_std=0.1):
    ins = make_absorb_inputs(ql, kl, d_q, d_kv, H, D_H, dtype, seed, x_std=x_std, w_std=w_std)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
    O = vb.packed_target_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    O.backward(dO.to(DEV))
    torch.cuda.synchronize()
    return ins, O, [t.grad for t in g]


def _compare(ins, O, grads, dtype):
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    ref = target_attn_ref_fwd_bwd(q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k)
    check_close("O", O, ref[0], dtype, scale_abs=True)
    for name, mine, r in zip(("dq_raw", "dX", "dW_Q", "dW_K", "dW_V"), grads, ref[2:]):
        check_close(name, mine, r, dtype, scale_abs=True)


@pytest.mark.parametrize("name", sorted(REF_CASES))
def test_reference_cases_fp32(name):
    ql, kl = REF_CASES[name]
    ins, O, grads = _run(ql, kl, 968, 216, 8, 32, torch.float32, 0)
    _compare(ins, O, grads, torch.float32)


@pytest.mark.parametrize("name", ["smoke", "ragged_real", "k_tail", "q_tail", "short_k", "empty_users"])
def test_reference_cases_bf16(name):
    ql, kl = REF_CASES[name]
    ins, O, grads = _run(ql, kl, 968, 216, 8, 32, torch.bfloat16, 0)
    _compare(ins, O, grads, torch.bfloat16)


def test_production_dims_run_on_the_tensor_core_kernels():
    """d_q = 968, d_kv = 216 (the reference's production shape) are zero-padded to 1024 / 256 on the way
    in, so forward and backward run on the tcgen05 kernels and not on the SIMT attention kernels."""
    from varlenabsorbflashattn_b200 import _lib
    ql = uniform_lengths(24, 1, 16, 3)
    kl = log_uniform_lengths(24, 8, 700, 4)
    _lib.profile_reset()
    ins, O, grads = _run(ql, kl, 968, 216, 8, 32, torch.bfloat16, 1)
    launched = {name for name, v in _lib.profile_read().items() if v[2] > 0}
    assert {"varlen_fwd_kernel<absorb>", "varlen_bwd_kernel<absorb dU>", "varlen_bwd_kernel<absorb dX>",
            "gemm_nn_k256_kernel", "gemm_tn_kernel"} <= launched, launched
    assert not ({"simt_fwd_kernel", "simt_dq_kernel", "simt_dkv_kernel"} & launched), launched
    assert grads[0].shape == (sum(ql), 968) and grads[1].shape == (sum(kl), 216)
    assert grads[2].shape == (968, 8, 32) and grads[3].shape == (216, 8, 32) and grads[4].shape == (216, 8, 32)
    _compare(ins, O, grads, torch.bfloat16)


def test_benchmark_dims_bf16():
    """d_q = d_kv = 256, H = 8, D_H = 32 with the benchmark's value distributions
    (q_raw, X ~ N(0,1); W ~ N(0, 1/256)), a scaled-down draw of configuration 4."""
    ql = uniform_lengths(40, 1, 16, 0)
    kl = log_uniform_lengths(40, 8, 600, 1)
    ins, O, grads = _run(ql, kl, 256, 256, 8, 32, torch.bfloat16, 0, x_std=1.0, w_std=None)
    _compare(ins, O, grads, torch.bfloat16)


@pytest.mark.parametrize("name", sorted(ABSORB_CASES))
def test_golden_against_reference_kernels(name, golden_dir):
    ql, kl, d_q, d_kv, H, D_H, seed = ABSORB_CASES[name]
    ins = make_absorb_inputs(ql, kl, d_q, d_kv, H, D_H, torch.float32, seed, x_std=0.5)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
    O = vb.packed_target_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    O.backward(dO.to(DEV))
    gold = np.load(os.path.join(golden_dir, f"absorb_{name}.npz"))
    assert (O.detach().cpu() - torch.from_numpy(gold["O"])).abs().max().item() < 5e-5
    for t, key in zip(g, ("dq_raw", "dX", "dW_Q", "dW_K", "dW_V")):
        ref = torch.from_numpy(gold[key])
        assert (t.grad.cpu() - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item()), key


def test_inner_entry_matches_full_op():
    ql, kl = [7, 8, 6, 9], [200, 100, 150, 50]
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs(ql, kl, 64, 48, 4, 16, torch.float32, 3, x_std=0.3)
    d = [t.to(DEV) for t in (q_raw, X, W_Q, W_K, W_V)]
    O_full = vb.packed_target_attn(*d, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    p = (d[0] @ d[2].reshape(64, -1)).view(-1, 4, 16)
    u = torch.einsum("thd,khd->thk", p, d[3]).contiguous().requires_grad_(True)
    Xg, Wg = d[1].clone().requires_grad_(True), d[4].clone().requires_grad_(True)
    qi, ki = vb.prepare_target_attn_indices(cu_q, cu_k)
    O_in = vb.target_attn_inner(u, Xg, Wg, cu_q, cu_k, q_chunk_indices=qi, k_chunk_indices=ki, validate=False)
    assert (O_in - O_full).abs().max().item() < 1e-5
    O_in.backward(dO.to(DEV))
    # oracle for du/dX/dW_V: autograd of the absorbed formulation in fp64
    u64 = u.detach().double().cpu().requires_grad_(True)
    X64 = X.double().requires_grad_(True)
    W64 = W_V.double().requires_grad_(True)
    outs = []
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for i in range(len(ql)):
        s = torch.einsum("qha,ka->hqk", u64[cq[i]:cq[i + 1]], X64[ck[i]:ck[i + 1]]) / math.sqrt(16)
        ax = torch.einsum("hqk,ka->qha", s.softmax(-1), X64[ck[i]:ck[i + 1]])
        outs.append(torch.einsum("qha,ahd->qhd", ax, W64))
    torch.cat(outs).backward(dO.double())
    for name, mine, r in (("du", u.grad, u64.grad), ("dX", Xg.grad, X64.grad), ("dW_V", Wg.grad, W64.grad)):
        check_close(name, mine, r, torch.float32, scale_abs=True)


def test_bf16_flag_and_3d_inputs():
    ql, kl = [4, 9], [64, 33]
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs(ql, kl, 64, 64, 8, 32, torch.float32, 4, x_std=0.3)
    d = [t.to(DEV) for t in (q_raw, X, W_Q, W_K, W_V)]
    O = vb.packed_target_attn(d[0][None], d[1][None], *d[2:], q_seqinfo=torch.tensor(ql), k_seqinfo=torch.tensor(kl),
                              bf16=True)
    assert O.dtype == torch.bfloat16 and O.shape == (13, 8, 32)
    ref = target_attn_ref_fwd_bwd(*[t.to(torch.bfloat16) for t in (q_raw, X, W_Q, W_K, W_V)], dO, cu_q, cu_k)[0]
    check_close("O", O, ref, torch.bfloat16, scale_abs=True)


def test_validation_raises_on_gpu_inputs():
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs([3, 2], [5, 4], 32, 32, 2, 16, torch.float32, 5)
    d = [t.to(DEV) for t in (q_raw, X, W_Q, W_K, W_V)]
    with pytest.raises(ValueError, match="k_len > 0"):
        vb.packed_target_attn(*d, cu_seqlens_q=cu_q, cu_seqlens_k=torch.tensor([0, 9, 9], dtype=torch.int32))


def test_forward_backward_inside_a_cuda_graph():
    """The call forks a library-owned side stream for the tile-list builder and rejoins it before it
    returns, which must be legal inside a stream capture: a captured forward+backward replays to the
    same bits as the eager call."""
    ql = uniform_lengths(40, 1, 16, 0)
    kl = log_uniform_lengths(40, 8, 600, 1)
    ins = make_absorb_inputs(ql, kl, 256, 256, 8, 32, torch.bfloat16, 0, x_std=1.0, w_std=None)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
    cu_q, cu_k, dO = cu_q.to(DEV), cu_k.to(DEV), dO.to(DEV)

    def step():
        O = vb.packed_target_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, validate=False)
        return (O,) + torch.autograd.grad(O, g, dO)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            eager = [t.clone() for t in step()]
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    for name, a, b in zip(("O", "dq_raw", "dX", "dW_Q", "dW_K", "dW_V"), captured, eager):
        assert torch.equal(a, b), name


@pytest.mark.parametrize("H,D_H", [(4, 32), (8, 16), (2, 64)])
def test_head_dims_off_the_fused_projection_path(H, D_H):
    """d_kv = 256 keeps the tensor-core forward core while H * D_H != 256 sends the output projection, the
    backward and the weight gradients through the general kernels."""
    ql, kl = [3, 9, 16, 1], [70, 300, 129, 5]
    ins, O, grads = _run(ql, kl, 256, 256, H, D_H, torch.bfloat16, 3, x_std=1.0, w_std=None)
    _compare(ins, O, grads, torch.bfloat16)


@pytest.mark.parametrize("H,D_H", [(4, 32), (8, 16), (2, 64)])
def test_narrow_x_off_the_fused_backward_path(H, D_H):
    """d_kv = 216 with head layouts whose backward does not run on the tensor-core dU/dX kernels: the
    forward may take X at its own width, the backward needs full-width rows, so the wrapper has to pad X
    for these layouts.  Forward and backward against the oracle."""
    ins, O, grads = _run([5, 9, 3], [100, 33, 260], 512, 216, H, D_H, torch.bfloat16, 3)
    _compare(ins, O, grads, torch.bfloat16)


def test_weight_grad_group_path_matches_the_plain_backward():
    """packed_target_attn(weight_grad_group=pg) cuts its backward in two library calls around the
    all-reduce of the fp32 weight gradients.  With a one-rank group the sum is the identity, so all five
    gradients must equal those of the plain call bit for bit."""
    import torch.distributed as dist
    import tempfile
    ql, kl = uniform_lengths(64, 1, 16, 0), log_uniform_lengths(64, 8, 2048, 1)
    ins = make_absorb_inputs(ql, kl, 256, 256, 8, 32, torch.bfloat16, 0)
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = ins
    created = False
    if not dist.is_initialized():
        store = tempfile.mktemp(prefix="vafa_pg_")
        dist.init_process_group("nccl", init_method=f"file://{store}", rank=0, world_size=1,
                                device_id=torch.device("cuda", 0))
        created = True
    try:
        outs = []
        for group in (None, dist.group.WORLD):
            g = [t.to(DEV).requires_grad_(True) for t in (q_raw, X, W_Q, W_K, W_V)]
            O = vb.packed_target_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, weight_grad_group=group)
            O.backward(dO.to(DEV))
            torch.cuda.synchronize()
            outs.append([O] + [t.grad for t in g])
        for a, b in zip(*outs):
            assert torch.equal(a, b)
    finally:
        if created:
            dist.destroy_process_group()
