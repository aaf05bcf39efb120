"""Host-side argument handling of the two public wrappers (no GPU): the same exception
types as the reference for the same mistakes."""
import os

import pytest
import torch

import varlenabsorbflashattn_b200 as vb
from varlenabsorbflashattn_b200 import varlen, absorb


def test_seqinfo_errors():
    with pytest.raises(ValueError, match="1-D"):
        varlen._lengths_to_cu(torch.zeros(2, 2, dtype=torch.int32))
    with pytest.raises(ValueError, match="empty"):
        varlen._lengths_to_cu(torch.zeros(0, dtype=torch.int32))
    with pytest.raises(ValueError, match="negative"):
        varlen._lengths_to_cu(torch.tensor([3, -1]))
    with pytest.raises(ValueError, match="int32"):
        varlen._lengths_to_cu(torch.tensor([2**31 - 1, 5], dtype=torch.int64))
    cu = varlen._lengths_to_cu(torch.tensor([3, 0, 5]))
    assert cu.dtype == torch.int32 and cu.tolist() == [0, 3, 3, 8]


def test_cu_seqlens_validation():
    with pytest.raises(ValueError, match=r"\[0\] must be 0"):
        varlen._check_cu(torch.tensor([1, 4]), 4, "cu_seqlens_q")
    with pytest.raises(ValueError, match="must equal total tokens"):
        varlen._check_cu(torch.tensor([0, 4]), 5, "cu_seqlens_q")
    with pytest.raises(ValueError, match="non-decreasing"):
        varlen._check_cu(torch.tensor([0, 5, 4]), 4, "cu_seqlens_q")
    with pytest.raises(ValueError, match="at least 2"):
        varlen._check_cu(torch.tensor([0]), 0, "cu_seqlens_q")
    vb.set_validate_cu_seqlens(False)
    try:
        varlen._check_cu(torch.tensor([1, 4]), 4, "cu_seqlens_q")
    finally:
        vb.set_validate_cu_seqlens(True)


def test_layout_errors():
    with pytest.raises(ValueError, match="batch=1"):
        varlen._as_thd(torch.zeros(2, 3, 1, 16), "q")
    with pytest.raises(ValueError, match="expected 3-D"):
        varlen._as_thd(torch.zeros(3, 16), "q")
    x, was4 = varlen._as_thd(torch.zeros(1, 3, 2, 16), "q")
    assert was4 and x.shape == (3, 2, 16)
    y, _ = varlen._as_thd(torch.zeros(3, 2, 32)[:, :, ::2], "q")
    assert y.is_contiguous()


def test_missing_lengths():
    q = torch.zeros(3, 1, 16)
    with pytest.raises(ValueError, match="cu_seqlens_q or q_seqinfo"):
        vb.packed_varlen_attn(q, q, q)
    with pytest.raises(ValueError, match="cu_seqlens_k or k_seqinfo"):
        vb.packed_varlen_attn(q, q, q, cu_seqlens_q=torch.tensor([0, 3]))


def test_cpu_tensors_refused():
    q = torch.zeros(3, 1, 16)
    cu = torch.tensor([0, 3], dtype=torch.int32)
    with pytest.raises(AssertionError, match="CUDA"):
        vb.packed_varlen_attn(q, q, q, cu_seqlens_q=cu, cu_seqlens_k=cu)
    with pytest.raises(AssertionError, match="CUDA"):
        vb.packed_target_attn(torch.zeros(3, 8), torch.zeros(3, 8), torch.zeros(8, 2, 16), torch.zeros(8, 2, 16),
                              torch.zeros(8, 2, 16), cu_seqlens_q=cu, cu_seqlens_k=cu)


def test_absorb_shape_asserts_and_env(monkeypatch):
    cu = torch.tensor([0, 3], dtype=torch.int32)
    with pytest.raises(AssertionError, match="W_Q"):
        vb.packed_target_attn(torch.zeros(3, 8), torch.zeros(3, 8), torch.zeros(9, 2, 16), torch.zeros(8, 2, 16),
                              torch.zeros(8, 2, 16), cu_seqlens_q=cu, cu_seqlens_k=cu)
    with pytest.raises(AssertionError, match="H mismatch"):
        vb.packed_target_attn(torch.zeros(3, 8), torch.zeros(3, 8), torch.zeros(8, 2, 16), torch.zeros(8, 3, 16),
                              torch.zeros(8, 2, 16), cu_seqlens_q=cu, cu_seqlens_k=cu)
    monkeypatch.setenv("TRITON_TARGET_ATTN_DX_MODE", "bogus")
    with pytest.raises(ValueError, match="TRITON_TARGET_ATTN_DX_MODE"):
        vb.packed_target_attn(torch.zeros(3, 8), torch.zeros(3, 8), torch.zeros(8, 2, 16), torch.zeros(8, 2, 16),
                              torch.zeros(8, 2, 16), cu_seqlens_q=cu, cu_seqlens_k=cu)


def test_absorb_validation():
    with pytest.raises(ValueError, match="k_len > 0"):
        absorb._validate(torch.tensor([0, 2, 3]), torch.tensor([0, 0, 4]), 3, 4)
    with pytest.raises(ValueError, match="non-decreasing"):
        absorb._validate(torch.tensor([0, 3, 2]), torch.tensor([0, 1, 4]), 2, 4)
    absorb._validate(torch.tensor([0, 0, 3]), torch.tensor([0, 0, 4]), 3, 4)


def test_prepare_indices_format():
    qi, ki = vb.prepare_target_attn_indices(torch.tensor([0, 17, 17, 20]), torch.tensor([0, 130, 131, 131]))
    assert qi.dtype == torch.int32 and qi.tolist() == [[0, 0], [0, 1], [2, 0]]
    assert ki.tolist() == [[0, 0], [0, 1], [0, 2], [1, 0]]


def test_absorb_padding_of_production_widths():
    """The host layer pads d_q = 968 / d_kv = 216 (the reference's production shape) to 1024 / 256 for
    the tensor-core kernels, with zero columns / rows and differentiable ops; other cases stay as given."""
    import torch
    from varlenabsorbflashattn_b200.absorb import _padded_widths, _pad_first, _pad_last
    assert _padded_widths(torch.bfloat16, 968, 216, 8) == (1024, 256)
    assert _padded_widths(torch.float16, 256, 216, 8) == (256, 256)
    assert _padded_widths(torch.bfloat16, 100, 256, 4) == (256, 256)
    assert _padded_widths(torch.bfloat16, None, 216, 8) == (None, 256)
    assert _padded_widths(torch.bfloat16, 256, 256, 8) is None      # already fits
    assert _padded_widths(torch.float32, 968, 216, 8) is None        # fp32 runs on the SIMT kernels
    assert _padded_widths(torch.bfloat16, 968, 216, 6) is None       # 6 heads do not stack into 128 rows
    assert _padded_widths(torch.bfloat16, 968, 300, 8) is None       # wider than one tile
    W = torch.randn(5, 2, 3, requires_grad=True)
    X = torch.randn(4, 5, requires_grad=True)
    Wp, Xp = _pad_first(W, 8), _pad_last(X, 8)
    assert Wp.shape == (8, 2, 3) and Xp.shape == (4, 8)
    assert torch.equal(Wp[:5], W) and Wp[5:].abs().sum() == 0 and Xp[:, 5:].abs().sum() == 0
    (Wp.sum() * 2 + Xp.sum() * 3).backward()
    assert W.grad.shape == W.shape and torch.all(W.grad == 2) and torch.all(X.grad == 3)


def test_production_shape_fixtures_load_and_are_consistent():
    """The reference's two logged-shape fixtures (stage-1 varlen shapes; production absorb batches), stored
    gzip-compressed beside the golden vectors, as bench.py's `stage1:<row>` / `absorb-prod:<i>` workloads
    read them.  Same consistency rules as the reference's loaders
    (tools/benchmark_packed_varlen_flash_attn.py:900-954; triton_target_attn_absorb/test_smoke.py:502-534)."""
    import gzip
    import json
    import bench
    gd = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    rows = [json.loads(l) for l in gzip.open(os.path.join(gd, "stage1_shapes.jsonl.gz"), "rt") if l.strip()]
    assert len(rows) == 958
    for r in rows:
        assert r["users"] == len(r["q_lens"]) == len(r["k_lens"])
        assert r["tq"] == sum(r["q_lens"]) and r["tk"] == sum(r["k_lens"])
        assert min(r["q_lens"]) > 0 and min(r["k_lens"]) > 0
    recs = json.load(gzip.open(os.path.join(gd, "real_shape_all.json.gz"), "rt"))["records"]
    assert len(recs) == 100
    for r in recs:
        assert r["n_seg"] == len(r["q_lens"]) == len(r["k_lens"])
        assert r["sum_q"] == sum(r["q_lens"]) and r["sum_k"] == sum(r["k_lens"])
        assert r["raw_q_shape"][-1] == 968 and r["raw_k_shape"][-1] == 216
    w = bench.workload("stage1:0")
    assert w["kind"] == "varlen" and sum(w["ql"]) == rows[0]["tq"] and w["H"] == 4 and w["D"] == 64
    w = bench.workload("absorb-prod:99")
    assert w["kind"] == "absorb" and sum(w["kl"]) == recs[99]["sum_k"] and (w["d_q"], w["d_kv"]) == (968, 216)


def test_bench_partition_balances_tokens_and_cells():
    import bench
    w = bench.workload("C5")
    assert sum(w["ql"]) == 1_000_000 and len(w["ql"]) == 520
    for n in (2, 4, 8):
        part, info = bench.partition_report(w["ql"], w["kl"], n, True)
        owned = sorted(i for seg in part.assignment for i in seg)
        assert owned == list(range(520))                       # every sequence exactly once, none split
        assert info["used_balance"]["token_imbalance"] <= 1.01 and info["used_balance"]["cell_imbalance"] <= 1.01
