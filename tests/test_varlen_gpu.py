"""GPU parity of packed_varlen_attn (through the C ABI) against the CPU oracle and the stored
outputs of the reference kernels.  Cases follow the reference's own list
(triton_fa_varlen_v2/triton_fa_varlen_v2/test_smoke.py:222-531) plus causal, empty-segment and
split-K cases."""
import os
import sys

import numpy as np
import pytest
import torch

import varlenabsorbflashattn_b200 as vb
from varlenabsorbflashattn_b200 import varlen as V
from oracle import make_varlen_inputs, varlen_attn_ref_fwd_bwd, varlen_attn_ref, config_lengths
from helpers import check_close, check_lse, LN2

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import VARLEN_CASES  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"

CASES = {
    "tiny": ([7, 11], [19, 5]),
    "cross_block": ([129, 257], [33, 130]),
    "stage1_like": ([500, 500], [19, 800]),
    "stage2_like": ([512, 512], [500, 500]),
    "single_seg": ([400], [400]),
    "block_aligned": ([256, 256], [128, 128]),
    "ones": ([1, 1, 1, 2], [1, 2, 129, 1]),
    "empty_q_and_k": ([5, 0, 9, 4], [12, 6, 0, 31]),
}


@pytest.fixture(params=["simt", "tcgen05"])
def impl(request):
    V.set_impl(request.param)
    yield request.param
    V.set_impl("auto")


def _supported(impl, dtype, D):
    if impl == "tcgen05":
        return dtype in (torch.bfloat16, torch.float16) and D in (64, 128)
    return True


def _run(ql, kl, H, D, dtype, causal, seed=0, split=None, bwd=True):
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, dtype, seed)
    qg, kg, vg = (t.to(DEV).requires_grad_(bwd) for t in (q, k, v))
    o, lse = vb.packed_varlen_attn_with_lse(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k,
                                            causal=causal, split_k_block=split)
    grads = None
    if bwd:
        o.backward(do.to(DEV))
        grads = (qg.grad, kg.grad, vg.grad)
    torch.cuda.synchronize()
    return (q, k, v, do, cu_q, cu_k), o, lse, grads


def _compare(inputs, o, lse, grads, dtype, causal):
    q, k, v, do, cu_q, cu_k = inputs
    ro, rlse, rdq, rdk, rdv = varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=causal)
    check_close("o", o, ro, dtype)
    check_lse(lse / LN2, rlse)
    if grads is not None:
        check_close("dq", grads[0], rdq, dtype, scale_abs=True)
        check_close("dk", grads[1], rdk, dtype, scale_abs=True)
        check_close("dv", grads[2], rdv, dtype, scale_abs=True)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_cases_bf16(impl, name, causal):
    ql, kl = CASES[name]
    ins, o, lse, grads = _run(ql, kl, 4, 64, torch.bfloat16, causal)
    _compare(ins, o, lse, grads, torch.bfloat16, causal)


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 128), (torch.float16, 64),
                                     (torch.float32, 64), (torch.bfloat16, 32), (torch.float32, 16),
                                     (torch.bfloat16, 256)])
def test_dtypes_and_head_dims(impl, dtype, D):
    if not _supported(impl, dtype, D):
        pytest.skip("shape not covered by this kernel family")
    ins, o, lse, grads = _run([129, 257, 3], [33, 130, 300], 2, D, dtype, False, seed=1)
    _compare(ins, o, lse, grads, dtype, False)
    ins, o, lse, grads = _run([130, 64, 3], [130, 64, 300], 2, D, dtype, True, seed=2)
    _compare(ins, o, lse, grads, dtype, True)


def test_config_c1_fp32_against_reference_kernels(golden_dir):
    """Benchmark configuration 1: fp32, H=8, D=64, lengths 17/64/128/255, seed 0."""
    V.set_impl("auto")
    ql, kl, H, D, seed, _ = VARLEN_CASES["c1"]
    ins, o, lse, _ = _run(ql, kl, H, D, torch.float32, False, seed=seed, bwd=False)
    g = np.load(os.path.join(golden_dir, "varlen_c1.npz"))
    assert (o.cpu() - torch.from_numpy(g["o"])).abs().max().item() < 2e-5
    assert (lse.cpu() / LN2 - torch.from_numpy(g["lse_log2"])).abs().max().item() < 2e-5
    ro, rlse = varlen_attn_ref(*ins[:3], ins[4], ins[5])
    check_close("o", o, ro, torch.float32, max_abs_tol=2e-5)


@pytest.mark.parametrize("name", ["tiny", "cross_block", "split"])
def test_golden_fp32_with_grads(name, golden_dir):
    V.set_impl("auto")
    ql, kl, H, D, seed, _ = VARLEN_CASES[name]
    ins, o, lse, grads = _run(ql, kl, H, D, torch.float32, False, seed=seed)
    g = np.load(os.path.join(golden_dir, f"varlen_{name}.npz"))
    assert (o.cpu() - torch.from_numpy(g["o"])).abs().max().item() < 3e-5
    for mine, key in zip(grads, ("dq", "dk", "dv")):
        assert (mine.cpu() - torch.from_numpy(g[key])).abs().max().item() < 1e-4, key


def test_layout_4d_and_noncontiguous(impl):
    ql, kl = [129, 70], [200, 70]
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 4, 64, torch.bfloat16, 3)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    o3 = vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    o4 = vb.packed_varlen_attn(q[None], k[None], v[None], cu_seqlens_q=cu_q.to(DEV), cu_seqlens_k=cu_k.long())
    assert o4.shape == (1,) + o3.shape and torch.equal(o4[0], o3)
    big = torch.zeros(q.shape[0], 4, 128, dtype=q.dtype, device=DEV)
    big[:, :, ::2] = q
    o5 = vb.packed_varlen_attn(big[:, :, ::2], k, v, q_seqinfo=torch.tensor(ql), k_seqinfo=torch.tensor(kl))
    assert torch.equal(o5, o3)


def test_no_grad_equals_grad_and_is_repeatable(impl):
    ql, kl = [300, 45, 128], [300, 500, 128]
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 4, 64, torch.bfloat16, 4)
    outs = []
    for rep in range(2):
        qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
        o = vb.packed_varlen_attn(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=True)
        o.backward(do.to(DEV))
        outs.append((o.detach(), qg.grad, kg.grad, vg.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b), "run-to-run results differ"
    with torch.no_grad():
        o_ng = vb.packed_varlen_attn(q.to(DEV), k.to(DEV), v.to(DEV), cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=True)
    assert torch.equal(o_ng, outs[0][0])


def test_partial_grad(impl):
    ql, kl = [64, 200], [100, 260]
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 4, 64, torch.bfloat16, 5)
    qg = q.to(DEV).requires_grad_(True)
    o = vb.packed_varlen_attn(qg, k.to(DEV), v.to(DEV), cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    o.backward(do.to(DEV))
    _, _, rdq, _, _ = varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k)
    check_close("dq", qg.grad, rdq, torch.bfloat16, scale_abs=True)


@pytest.mark.parametrize("split", [128, 256, 4096])
def test_split_k_invariance(impl, split):
    """Any KV slice length gives the un-split answer (to fp32 rounding of the merge)."""
    ql, kl = [3, 140, 1], [4500, 700, 129]
    ins, o, lse, grads = _run(ql, kl, 2, 128, torch.bfloat16, False, seed=6, split=split)
    _compare(ins, o, lse, grads, torch.bfloat16, False)
    _, o0, lse0, _ = _run(ql, kl, 2, 128, torch.bfloat16, False, seed=6, split=None, bwd=False)
    assert (o.float() - o0.float()).abs().max().item() <= 2e-2
    assert (lse - lse0).abs().max().item() <= 1e-4


def test_decode_like_split(impl):
    """One query row per segment over long KV (the split-K + LSE-combine shape)."""
    kl = [8192, 9000, 12345, 300]
    ins, o, lse, _ = _run([1] * 4, kl, 8, 128, torch.bfloat16, False, seed=7, bwd=False)
    ro, rlse = varlen_attn_ref(*ins[:3], ins[4], ins[5])
    check_close("o", o, ro, torch.bfloat16)
    check_lse(lse / LN2, rlse)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_ragged_random_causal_fwd_bwd(impl, seed):
    """A scaled-down draw of benchmark configuration 2 (log-uniform lengths, H=16->4, D=128)."""
    from oracle import log_uniform_lengths
    L = log_uniform_lengths(12, 1, 700, seed)
    ins, o, lse, grads = _run(L, L, 4, 128, torch.bfloat16, True, seed=seed)
    _compare(ins, o, lse, grads, torch.bfloat16, True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gain", [1.0, 6.0])
def test_backward_large_scores_and_dead_rows(dtype, gain):
    """The dK/dV kernel receives lse and delta as sums of three 16-bit pieces inside its score products:
    large |lse| (q scaled up, so that |scale * s| reaches several hundred) must not cost accuracy, and
    query rows that see no key (causal, more queries than keys) must leave dQ exactly zero and add
    nothing to dK/dV."""
    V.set_impl("tcgen05")
    try:
        ql, kl = [300, 200, 140, 129], [300, 70, 140, 640]
        q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 2, 128, dtype, 5)
        q = (q.float() * gain).to(dtype)
        for causal in (False, True):
            qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
            o, lse = vb.packed_varlen_attn_with_lse(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)
            o.backward(do.to(DEV))
            _compare((q, k, v, do, cu_q, cu_k), o, lse, (qg.grad, kg.grad, vg.grad), dtype, causal)
            if causal:
                # segment 1 has 200 queries over 70 keys: its first 130 rows see nothing
                dead = qg.grad[300:430]
                assert torch.count_nonzero(dead).item() == 0
                assert torch.isinf(lse[300:430]).all()
    finally:
        V.set_impl("auto")


def test_sequence_sharding_is_bitwise_equivalent():
    """Running each rank's shard of a packed batch on its own gives, row for row, the bits of the
    full-batch run (no sequence crosses ranks and no result depends on its neighbours)."""
    from varlenabsorbflashattn_b200.sharding import partition_segments, shard_rows, unshard_rows, local_cu_seqlens
    V.set_impl("auto")
    from oracle import log_uniform_lengths
    L = log_uniform_lengths(24, 1, 600, 5)
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(L, L, 4, 128, torch.bfloat16, 5)

    def run(q, k, v, do, cu_q, cu_k):
        g = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
        o = vb.packed_varlen_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=True)
        o.backward(do.to(DEV))
        return [o.detach().cpu()] + [t.grad.cpu() for t in g]

    full = run(q, k, v, do, cu_q, cu_k)
    for world in (2, 3):
        part = partition_segments(L, L, world)
        outs = [run(*(shard_rows(t, L, part, r) for t in (q, k, v, do)), local_cu_seqlens(L, part, r),
                    local_cu_seqlens(L, part, r)) for r in range(world)]
        for i in range(4):
            assert torch.equal(unshard_rows([o[i] for o in outs], L, part), full[i])


def test_forward_backward_inside_a_cuda_graph():
    """With validation off the op neither synchronises nor reads lengths on the host, so a forward+backward
    (split-K forward included) can be captured into a CUDA graph; the replay reproduces the eager bits."""
    ql, kl = [300, 45, 128, 1], [300, 9000, 128, 7]
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 4, 128, torch.bfloat16, 6)
    g = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    cu_q, cu_k, do = cu_q.to(DEV), cu_k.to(DEV), do.to(DEV)
    vb.set_validate_cu_seqlens(False)
    try:
        def step():
            o = vb.packed_varlen_attn(*g, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
            return (o,) + torch.autograd.grad(o, g, do)

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
        for name, a, b in zip(("o", "dq", "dk", "dv"), captured, eager):
            assert torch.equal(a, b), name
    finally:
        vb.set_validate_cu_seqlens(True)


def test_nan_in_q_reaches_o_lse_and_dq():
    """A NaN must not vanish: the reference's kernels propagate it through the softmax, so a diverged run
    shows.  One NaN in a query row makes that row of O, its LSE and its dQ row NaN; the other rows of
    the segment stay finite in O."""
    V.set_impl("tcgen05")
    try:
        ql, kl = [200, 64], [200, 300]
        q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, 2, 128, torch.bfloat16, 5)
        q[37, 1, 5] = float("nan")
        qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
        o, lse = vb.packed_varlen_attn_with_lse(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
        o.backward(do.to(DEV))
        assert torch.isnan(o[37, 1]).all() and torch.isnan(lse[37, 1])
        assert torch.isnan(qg.grad[37, 1]).all()
        others = torch.ones(o.shape[0], dtype=torch.bool, device=DEV)
        others[37] = False
        assert torch.isfinite(o[others].float()).all() and torch.isfinite(o[37, 0].float()).all()
    finally:
        V.set_impl("auto")


def test_bounded_wait_runs_out_and_is_reported():
    """Failure detection without a fault: with the wait limit at about a million cycles, a CTA that waits on
    a barrier nobody arrives on comes back by itself, the status word reads code 1 at the self-test's site,
    vafa_check_status turns that into VAFA_ERR_DEVICE, and the next ordinary call works."""
    import ctypes as C
    from varlenabsorbflashattn_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    prev = lib.vafa_set_wait_limit_cycles(1_000_000)
    try:
        st = torch.zeros(4, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        assert lib.vafa_selftest_bounded_wait(st.data_ptr(), stream) == 0
        rc = lib.vafa_check_status(st.data_ptr(), stream)
        assert rc == -5, lib.vafa_last_error()
        host = st.cpu().tolist()
        assert host[0] == 1 and host[1] == 900, host
        assert b"bounded wait" in lib.vafa_last_error()
    finally:
        assert lib.vafa_set_wait_limit_cycles(prev) >= 1_000_000
    assert lib.vafa_set_wait_limit_cycles(0) == prev  # reads back, sets nothing
    ins, o, lse, grads = _run([130, 7], [130, 260], 2, 128, torch.bfloat16, True)
    _compare(ins, o, lse, grads, torch.bfloat16, True)
    _lib.check_status(dev)


def test_status_check_after_every_call_is_opt_in():
    from varlenabsorbflashattn_b200 import _lib
    _lib.set_check_status(True)
    try:
        ins, o, lse, grads = _run([70], [90], 2, 64, torch.bfloat16, False)
        _compare(ins, o, lse, grads, torch.bfloat16, False)
    finally:
        _lib.set_check_status(False)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("name", ["cross_block", "stage1_like", "stage2_like", "empty_q_and_k", "ones", "long"])
def test_fused_backward_mode(name, causal):
    """The one-pass backward (opt-in, head dim 128): same tolerances against the oracle as the default kernel
    pair; dK and dV are bit-identical to the pair's (same products in the same order), dQ is summed across
    key tiles in global memory and agrees to rounding."""
    ql, kl = CASES[name] if name in CASES else ([700, 45, 1300], [1500, 45, 1300])
    V.set_impl("tcgen05")
    try:
        vb.set_backward_mode("split")
        ins, o, lse, gs = _run(ql, kl, 2, 128, torch.bfloat16, causal, seed=3)
        assert vb.set_backward_mode("fused") == "split"
        _, o2, _, gf = _run(ql, kl, 2, 128, torch.bfloat16, causal, seed=3)
    finally:
        vb.set_backward_mode("split")
        V.set_impl("auto")
    _compare(ins, o2, lse, gf, torch.bfloat16, causal)
    assert torch.equal(gs[1], gf[1]) and torch.equal(gs[2], gf[2])
    ref = float(gs[0].float().abs().max())
    assert float((gs[0].float() - gf[0].float()).abs().max()) <= 2e-2 * max(1.0, ref)


def test_fused_backward_mode_leaves_other_head_dims_to_the_kernel_pair():
    V.set_impl("tcgen05")
    try:
        vb.set_backward_mode("fused")
        ins, o, lse, grads = _run([200, 64], [200, 300], 2, 64, torch.float16, True)
    finally:
        vb.set_backward_mode("split")
        V.set_impl("auto")
    _compare(ins, o, lse, grads, torch.float16, True)


def _gqa_reference(q, k, v, do, cu_q, cu_k, G, causal):
    """Oracle for grouped-query attention: K/V heads repeated to one per query head, dK/dV summed per group."""
    ke, ve = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)
    ro, rlse, rdq, rdk, rdv = varlen_attn_ref_fwd_bwd(q, ke, ve, do, cu_q, cu_k, causal=causal)
    Tk, H, D = rdk.shape
    return ro, rlse, rdq, rdk.view(Tk, H // G, G, D).sum(2), rdv.view(Tk, H // G, G, D).sum(2)


@pytest.mark.parametrize("H,H_kv,D,dtype,causal", [
    (8, 2, 128, torch.bfloat16, True), (8, 2, 128, torch.bfloat16, False), (4, 1, 64, torch.float16, True),
    (6, 3, 128, torch.bfloat16, False), (4, 2, 32, torch.float32, True)])
def test_grouped_query_heads(H, H_kv, D, dtype, causal):
    """Fewer K/V heads than query heads (the reference is multi-head only): query head h reads K/V head
    h // (H // H_kv); dK and dV are sums over the group.  The last case (fp32, head dim 32) runs through the
    wrapper's head expansion, the others on the tensor-core kernels with the shared heads read in place."""
    ql, kl = [300, 45, 128, 2, 700], [300, 500, 128, 9, 700]
    G = H // H_kv
    torch.manual_seed(7)
    q, _, _, do, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, dtype, 7)
    k = torch.randn(sum(kl), H_kv, D).to(dtype)
    v = torch.randn(sum(kl), H_kv, D).to(dtype)
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    o, lse = vb.packed_varlen_attn_with_lse(qg, kg, vg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)
    o.backward(do.to(DEV))
    torch.cuda.synchronize()
    assert kg.grad.shape == k.shape and vg.grad.shape == v.shape
    ro, rlse, rdq, rdk, rdv = _gqa_reference(q, k, v, do, cu_q, cu_k, G, causal)
    check_close("o", o, ro, dtype)
    check_lse(lse / LN2, rlse)
    check_close("dq", qg.grad, rdq, dtype, scale_abs=True)
    check_close("dk", kg.grad, rdk, dtype, scale_abs=True)
    check_close("dv", vg.grad, rdv, dtype, scale_abs=True)


def test_grouped_query_decode_reads_shared_heads():
    """Decode shape with multi-query attention: one query row per sequence, 16 query heads on one K/V head,
    long KV (split across CTAs)."""
    ql, kl = [1] * 6, [9000, 300, 4097, 12000, 128, 6000]
    q, _, _, _, cu_q, cu_k = make_varlen_inputs(ql, kl, 16, 128, torch.bfloat16, 9, with_do=False)
    k = torch.randn(sum(kl), 1, 128).to(torch.bfloat16)
    v = torch.randn(sum(kl), 1, 128).to(torch.bfloat16)
    with torch.no_grad():
        o, lse = vb.packed_varlen_attn_with_lse(q.to(DEV), k.to(DEV), v.to(DEV), cu_seqlens_q=cu_q, cu_seqlens_k=cu_k)
    ro, rlse = varlen_attn_ref(q, k.repeat_interleave(16, dim=1), v.repeat_interleave(16, dim=1), cu_q, cu_k)
    check_close("o", o, ro, torch.bfloat16)
    check_lse(lse / LN2, rlse)


def test_two_tile_forward_kernel_opt_in():
    """VAFA_FWD_PAIR=1 (read once per process) sends batches of long query segments to the forward kernel that
    works on two 128-row query tiles per CTA; the reference's shape cases, the split-K cases and the ragged
    causal cases must pass with it exactly as with the default kernel."""
    import subprocess
    env = dict(os.environ, VAFA_FWD_PAIR="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sel = ("(test_reference_cases_bf16 or test_split_k_invariance or test_ragged_random_causal_fwd_bwd "
           "or test_dtypes_and_head_dims or test_grouped_query_heads) and not simt")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_varlen_gpu.py"), "-q", "-x",
                        "-m", "gpu", "-k", sel, "-p", "no:cacheprovider"],
                       env=env, cwd=root, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
