"""Seeded length and value generators for the benchmark configurations.

Test infrastructure only.  Lengths come from a CPU `torch.Generator` in float64 so
that every machine draws the same ragged batch; values are drawn in fp32 on the CPU
and cast, so the oracle and the GPU see identical bits.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def log_uniform_lengths(n: int, lo: int, hi: int, seed: int) -> List[int]:
    u = torch.rand(n, generator=_gen(seed), dtype=torch.float64)
    a, b = math.log(lo), math.log(hi + 1)
    L = torch.floor(torch.exp(a + u * (b - a))).to(torch.int64).clamp_(lo, hi)
    return L.tolist()


def uniform_lengths(n: int, lo: int, hi: int, seed: int) -> List[int]:
    return torch.randint(lo, hi + 1, (n,), generator=_gen(seed)).tolist()


def log_uniform_until(total: int, lo: int, hi: int, seed: int) -> List[int]:
    """Draw log-uniform lengths one at a time; truncate the last so the sum is `total`."""
    g = _gen(seed)
    a, b = math.log(lo), math.log(hi + 1)
    out: List[int] = []
    s = 0
    while s < total:
        u = torch.rand(1, generator=g, dtype=torch.float64).item()
        L = int(min(max(math.floor(math.exp(a + u * (b - a))), lo), hi))
        L = min(L, total - s)
        out.append(L)
        s += L
    return out


def lengths_to_cu(lengths) -> torch.Tensor:
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int64)
    cu[1:] = torch.tensor(list(lengths), dtype=torch.int64).cumsum(0)
    return cu.to(torch.int32)


# name -> description of the five benchmark configurations (C1..C5) plus variants.
CONFIGS: Dict[str, dict] = {
    "C1": dict(kind="varlen", H=8, D=64, dtype="fp32", causal=False),
    "C2": dict(kind="varlen", H=16, D=128, dtype="bf16", causal=True),
    "C2b": dict(kind="varlen", H=16, D=128, dtype="bf16", causal=True),
    "C3": dict(kind="varlen", H=8, D=128, dtype="bf16", causal=False),
    "C4": dict(kind="absorb", H=8, D_H=32, d_q=256, d_kv=256, dtype="bf16"),
    "C5v": dict(kind="varlen", H=32, D=128, dtype="bf16", causal=True),
    "C5a": dict(kind="absorb", H=8, D_H=32, d_q=256, d_kv=256, dtype="bf16"),
    # production-like training shape of the varlen operator: few users, 500 queries each, very long key
    # histories (the reference's fixture of 958 logged batches, triton_fa_varlen_v2/fixtures/
    # stage1_shapes.jsonl: 16-30 users, q = 500, k up to 102 400 with more than half of the users at the
    # cap; its harness defaults to 4 heads of 64, tools/benchmark_packed_varlen_flash_attn.py:1497-1498)
    "S1": dict(kind="varlen", H=4, D=64, dtype="bf16", causal=False),
}


def config_lengths(name: str, seed: int = 0) -> Tuple[List[int], List[int]]:
    """(q_lens, k_lens) of a named configuration."""
    if name == "C1":
        L = [17, 64, 128, 255]
        return L, list(L)
    if name == "C2":
        L = log_uniform_lengths(64, 1, 4096, seed)
        return L, list(L)
    if name == "C2b":
        L = log_uniform_lengths(128, 1, 4096, seed)
        return L, list(L)
    if name == "C3":
        return [1] * 256, log_uniform_lengths(256, 8192, 32768, seed)
    if name == "C4":
        return uniform_lengths(1024, 1, 16, seed), log_uniform_lengths(1024, 8, 2048, seed + 1)
    if name == "C5v":
        L = log_uniform_until(1_000_000, 128, 8192, seed)
        return L, list(L)
    if name == "S1":
        g = torch.Generator(device="cpu").manual_seed(seed)
        n = 23
        capped = torch.rand(n, generator=g, dtype=torch.float64) < 0.55
        tail = log_uniform_lengths(n, 1, 102400, seed + 1)
        return [500] * n, [102400 if c else t for c, t in zip(capped.tolist(), tail)]
    if name == "C5a":
        return uniform_lengths(16384, 1, 16, seed), log_uniform_lengths(16384, 8, 2048, seed + 1)
    raise KeyError(name)


_DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def make_varlen_inputs(q_lens, k_lens, H: int, D: int, dtype, seed: int = 0, with_do: bool = True):
    """q, k, v, dO ~ N(0,1) drawn in fp32 on the CPU (order q, k, v, dO) and cast."""
    if isinstance(dtype, str):
        dtype = _DT[dtype]
    torch.manual_seed(seed)
    Tq, Tk = int(sum(q_lens)), int(sum(k_lens))
    q = torch.randn(Tq, H, D, dtype=torch.float32).to(dtype)
    k = torch.randn(Tk, H, D, dtype=torch.float32).to(dtype)
    v = torch.randn(Tk, H, D, dtype=torch.float32).to(dtype)
    do = torch.randn(Tq, H, D, dtype=torch.float32).to(dtype) if with_do else None
    return q, k, v, do, lengths_to_cu(q_lens), lengths_to_cu(k_lens)


def make_absorb_inputs(q_lens, k_lens, d_q: int, d_kv: int, H: int, D_H: int, dtype, seed: int = 0,
                       x_std: float = 1.0, w_std: float | None = None):
    """q_raw, X ~ N(0, x_std^2); W_* ~ N(0, w_std^2) (default 1/sqrt(d)); dO ~ N(0,1)."""
    if isinstance(dtype, str):
        dtype = _DT[dtype]
    torch.manual_seed(seed)
    Tq, Tk = int(sum(q_lens)), int(sum(k_lens))
    wq_std = w_std if w_std is not None else 1.0 / math.sqrt(d_q)
    wk_std = w_std if w_std is not None else 1.0 / math.sqrt(d_kv)
    q_raw = (torch.randn(Tq, d_q) * x_std).to(dtype)
    X = (torch.randn(Tk, d_kv) * x_std).to(dtype)
    W_Q = (torch.randn(d_q, H, D_H) * wq_std).to(dtype)
    W_K = (torch.randn(d_kv, H, D_H) * wk_std).to(dtype)
    W_V = (torch.randn(d_kv, H, D_H) * wk_std).to(dtype)
    dO = torch.randn(Tq, H, D_H).to(dtype)
    return q_raw, X, W_Q, W_K, W_V, dO, lengths_to_cu(q_lens), lengths_to_cu(k_lens)
