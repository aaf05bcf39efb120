"""Multi-rank host logic on CPU: the token-balanced partition, pack/unpack round trips, and a
world_size-2 gloo run in which each rank processes its shard (with the CPU oracle standing in for
the kernels) and the weight gradients are all-reduced exactly as the absorb wrapper does on GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import (config_lengths, make_absorb_inputs, make_varlen_inputs, target_attn_ref_fwd_bwd,
                    varlen_attn_ref_fwd_bwd)
from varlenabsorbflashattn_b200.sharding import (local_cu_seqlens, partition_segments, shard_rows, unshard_rows)


def test_partition_is_complete_deterministic_and_balanced():
    ql, kl = config_lengths("C5v")
    for n in (1, 2, 4, 8):
        p = partition_segments(ql, kl, n)
        flat = sorted(i for lst in p.assignment for i in lst)
        assert flat == list(range(len(ql)))
        assert p == partition_segments(ql, kl, n)
        assert p.imbalance() < 1.02, (n, p.imbalance())
    cells = partition_segments(ql, kl, 8, weight=lambda a, b: a * b)
    assert cells.imbalance() < 1.05


def test_partition_edge_cases():
    p = partition_segments([5, 0, 3], [5, 0, 3], 4)
    assert sorted(i for lst in p.assignment for i in lst) == [0, 1, 2]
    with pytest.raises(ValueError):
        partition_segments([1], [1, 2], 2)
    with pytest.raises(ValueError):
        partition_segments([1], [1], 0)


def test_shard_round_trip():
    ql = [3, 0, 7, 2, 9]
    x = torch.arange(sum(ql) * 4, dtype=torch.float32).view(sum(ql), 2, 2)
    p = partition_segments(ql, ql, 3)
    shards = [shard_rows(x, ql, p, r) for r in range(3)]
    assert sum(s.shape[0] for s in shards) == x.shape[0]
    assert torch.equal(unshard_rows(shards, ql, p), x)
    for r in range(3):
        assert int(local_cu_seqlens(ql, p, r)[-1]) == shards[r].shape[0]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    # absorb: shard users, compute local gradients, sum the fp32 weight gradients over ranks
    ql, kl = [3, 5, 1, 7, 2, 4], [20, 9, 33, 12, 5, 17]
    q_raw, X, W_Q, W_K, W_V, dO, cu_q, cu_k = make_absorb_inputs(ql, kl, 16, 24, 2, 8, torch.float32, 0, x_std=0.5)
    part = partition_segments(ql, kl, world)
    lq, lX, ldO = shard_rows(q_raw, ql, part, rank), shard_rows(X, kl, part, rank), shard_rows(dO, ql, part, rank)
    res = target_attn_ref_fwd_bwd(lq, lX, W_Q, W_K, W_V, ldO, local_cu_seqlens(ql, part, rank),
                                  local_cu_seqlens(kl, part, rank), compute_dtype=torch.float64)
    dw = torch.cat([res[4].flatten(), res[5].flatten(), res[6].flatten()])
    dist.all_reduce(dw)
    # varlen: no collective; gather the shards' outputs to rank 0
    vq, vk = [5, 130, 2, 64], [9, 130, 40, 64]
    q, k, v, do, _, _ = make_varlen_inputs(vq, vk, 2, 16, torch.float32, 1)
    vp = partition_segments(vq, vk, world)
    o, _, dq, dk, dv = varlen_attn_ref_fwd_bwd(shard_rows(q, vq, vp, rank), shard_rows(k, vk, vp, rank),
                                               shard_rows(v, vk, vp, rank), shard_rows(do, vq, vp, rank),
                                               local_cu_seqlens(vq, vp, rank), local_cu_seqlens(vk, vp, rank), causal=True)
    gathered = [None] * world
    dist.all_gather_object(gathered, (res[0], res[2], res[3], o, dq, dk))
    if rank == 0:
        torch.save({"dw": dw, "gathered": gathered}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_equivalence(tmp_path):
    world, out = 2, str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = torch.load(out, weights_only=False)
    ql, kl = [3, 5, 1, 7, 2, 4], [20, 9, 33, 12, 5, 17]
    ins = make_absorb_inputs(ql, kl, 16, 24, 2, 8, torch.float32, 0, x_std=0.5)
    full = target_attn_ref_fwd_bwd(*ins[:5], ins[5], ins[6], ins[7], compute_dtype=torch.float64)
    part = partition_segments(ql, kl, world)
    O = unshard_rows([g[0] for g in got["gathered"]], ql, part)
    dq_raw = unshard_rows([g[1] for g in got["gathered"]], ql, part)
    dX = unshard_rows([g[2] for g in got["gathered"]], kl, part)
    assert torch.allclose(O, full[0], atol=1e-12) and torch.allclose(dq_raw, full[2], atol=1e-12)
    assert torch.allclose(dX, full[3], atol=1e-12)
    ref_dw = torch.cat([full[4].flatten(), full[5].flatten(), full[6].flatten()])
    assert torch.allclose(got["dw"], ref_dw, atol=1e-10)
    vq, vk = [5, 130, 2, 64], [9, 130, 40, 64]
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(vq, vk, 2, 16, torch.float32, 1)
    fo, _, fdq, fdk, _ = varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=True)
    vp = partition_segments(vq, vk, world)
    assert torch.equal(unshard_rows([g[3] for g in got["gathered"]], vq, vp), fo)
    assert torch.equal(unshard_rows([g[4] for g in got["gathered"]], vq, vp), fdq)
    assert torch.equal(unshard_rows([g[5] for g in got["gathered"]], vk, vp), fdk)
