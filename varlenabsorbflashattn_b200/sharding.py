"""Sequence-sharded data parallelism for packed batches (one process per GPU).

Attention here is block-diagonal over segments, so whole segments are the unit of distribution:
no segment is ever split across ranks and the data path needs no collective.  The only exchanged
data are the absorb operator's weight gradients (`packed_target_attn(..., weight_grad_group=pg)`
all-reduces them in fp32 before rounding).

The reference has no multi-GPU code; this module is the host-side plumbing a data-parallel caller
needs around the two operators: a token-balanced partition of the segments and the packing /
unpacking of per-rank slices.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

__all__ = ["Partition", "partition_segments", "shard_rows", "unshard_rows", "local_cu_seqlens"]


@dataclass
class Partition:
    """assignment[r] = segment indices (ascending) owned by rank r."""
    assignment: List[List[int]]
    load: List[int]

    @property
    def world_size(self) -> int:
        return len(self.assignment)

    def imbalance(self) -> float:
        """max load / mean load (1.0 = perfectly balanced)."""
        mean = sum(self.load) / max(1, len(self.load))
        return max(self.load) / mean if mean > 0 else 1.0


def partition_segments(q_lens: Sequence[int], k_lens: Sequence[int], world_size: int,
                       weight: Optional[Callable[[int, int], int]] = None) -> Partition:
    """Greedy longest-processing-time assignment of whole segments to ranks.

    weight(Lq, Lk) is the cost of a segment; the default is its token count Lq + Lk
    ("token-balanced").  Pass e.g. `lambda a, b: a * b` to balance attention cells instead.
    Deterministic: ties go to the lower segment index and the lower rank.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    if len(q_lens) != len(k_lens):
        raise ValueError("q_lens and k_lens must have the same number of segments")
    w = weight or (lambda a, b: a + b)
    cost = [int(w(int(a), int(b))) for a, b in zip(q_lens, k_lens)]
    order = sorted(range(len(cost)), key=lambda i: (-cost[i], i))
    load = [0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (load[j], j))
        owned[r].append(i)
        load[r] += cost[i]
    for lst in owned:
        lst.sort()
    return Partition(owned, load)


def _starts(lens: Sequence[int]) -> List[int]:
    out, s = [], 0
    for L in lens:
        out.append(s)
        s += int(L)
    return out


def _row_index(lens: Sequence[int], segs: Sequence[int]) -> torch.Tensor:
    st = _starts(lens)
    parts = [torch.arange(st[i], st[i] + int(lens[i]), dtype=torch.int64) for i in segs]
    return torch.cat(parts) if parts else torch.empty(0, dtype=torch.int64)


def shard_rows(x: torch.Tensor, lens: Sequence[int], part: Partition, rank: int) -> torch.Tensor:
    """Rows of the packed tensor x ([T, ...], segments laid out by `lens`) that rank owns, re-packed
    contiguously in ascending segment order."""
    idx = _row_index(lens, part.assignment[rank]).to(x.device)
    return x.index_select(0, idx)


def local_cu_seqlens(lens: Sequence[int], part: Partition, rank: int) -> torch.Tensor:
    cu = torch.zeros(len(part.assignment[rank]) + 1, dtype=torch.int64)
    if part.assignment[rank]:
        cu[1:] = torch.tensor([int(lens[i]) for i in part.assignment[rank]], dtype=torch.int64).cumsum(0)
    return cu.to(torch.int32)


def unshard_rows(shards: Sequence[torch.Tensor], lens: Sequence[int], part: Partition) -> torch.Tensor:
    """Inverse of shard_rows over all ranks: shards[r] are rank r's rows; returns the packed tensor."""
    total = int(sum(int(L) for L in lens))
    ref = shards[0]
    out = torch.empty((total,) + tuple(ref.shape[1:]), dtype=ref.dtype, device=ref.device)
    for r, sh in enumerate(shards):
        idx = _row_index(lens, part.assignment[r]).to(ref.device)
        out.index_copy_(0, idx, sh.to(ref.device))
    return out
