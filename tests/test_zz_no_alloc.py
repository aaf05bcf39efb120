"""vafa_varlen_fwd_noalloc: the forward entry point for hosts that cannot allocate.

Some programs that embed this library cannot hand it a per-batch workspace: a plugin called from
inside another runtime's execution callback, a serving engine whose device-memory plan is frozen
at start-up, a real-time loop that must stay off the allocator.  For them the library carries a
fixed scratch array in its own device image and this entry point uses it instead of a workspace.

The test drives both entry points through the C ABI with raw pointers (the only torch use is to
own the input and output buffers) and requires the same results from the built-in scratch as from
a caller-owned workspace, twice in a row: the second call sees the first call's leftovers in the
shared array and must not be disturbed by them.  Both results are also held to the CPU oracle.
Tolerance as everywhere in this suite for 16-bit outputs: max-abs 2e-2 on O, 1e-4 on the
(natural-log) LSE; the two paths normally agree exactly, except in the last case, where the
built-in array is too small for the split-K partials the forced slice length asks for, so the
library has to split less finely there than with a workspace.  This file sorts last on purpose so
that a run that stops at the first failure has already run every other test.
"""
import ctypes as C
import math

import pytest
import torch

from varlenabsorbflashattn_b200 import _lib
from oracle import make_varlen_inputs, varlen_attn_ref

pytestmark = pytest.mark.gpu
LN2 = math.log(2.0)


def _args(q, k, v, o, lse, cu_q, cu_k, causal, split_k_block=0):
    a = _lib.VarlenArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.cu_seqlens_q, a.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    a.n_seg = cu_q.numel() - 1
    a.total_q, a.num_heads, a.head_dim = q.shape
    a.total_k = k.shape[0]
    a.dtype = _lib.DTYPE_CODE[q.dtype]
    a.causal = int(causal)
    a.scale = 1.0 / math.sqrt(q.shape[-1])
    a.impl = _lib.IMPL_TCGEN05
    a.split_k_block = split_k_block
    a.sm_count = 0
    a.status = _lib.status_word(q.device).data_ptr()
    return a


def _both(lib, ql, kl, H, D, dtype, causal, seed, split_k_block=0):
    dev = torch.device("cuda", 0)
    q, k, v, _, cu_q, cu_k = make_varlen_inputs(ql, kl, H, D, dtype, seed, with_do=False)
    o_cpu, lse_cpu = varlen_attn_ref(q, k, v, cu_q, cu_k, causal=causal)
    q, k, v, cu_q, cu_k = (t.to(dev) for t in (q, k, v, cu_q, cu_k))
    stream = torch.cuda.current_stream(dev).cuda_stream
    # existing entry point, caller-owned workspace
    o_ref = torch.empty_like(q)
    lse_ref = torch.empty(q.shape[0], H, dtype=torch.float32, device=dev)
    a = _args(q, k, v, o_ref, lse_ref, cu_q, cu_k, causal, split_k_block)
    ws = torch.empty(max(1, lib.vafa_varlen_fwd_workspace_bytes(C.byref(a))), dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(lib.vafa_varlen_fwd(C.byref(a), stream), "vafa_varlen_fwd")
    # new entry point: no workspace at all
    o_new = torch.full_like(q, float("nan"))
    lse_new = torch.full_like(lse_ref, float("nan"))
    b = _args(q, k, v, o_new, lse_new, cu_q, cu_k, causal, split_k_block)
    b.workspace, b.workspace_bytes = None, 0
    _lib.check(lib.vafa_varlen_fwd_noalloc(C.byref(b), stream), "vafa_varlen_fwd_noalloc")
    torch.cuda.synchronize(dev)
    _lib.check_status(dev)
    assert torch.isfinite(o_new.float()).all()
    assert (o_new.float() - o_ref.float()).abs().max().item() <= 2e-2
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse_new), fin)
    assert ((lse_new[fin] - lse_ref[fin]).abs().max().item() * LN2) <= 1e-4
    # and against the fp32 CPU oracle (natural-log LSE there, log2 domain here)
    for o_gpu, lse_gpu in ((o_ref, lse_ref), (o_new, lse_new)):
        assert (o_gpu.float().cpu() - o_cpu.float()).abs().max().item() <= 2e-2
        live = torch.isfinite(lse_cpu)
        assert torch.equal(torch.isfinite(lse_gpu.cpu()), live)
        assert (lse_gpu.cpu()[live] * LN2 - lse_cpu[live]).abs().max().item() <= 1e-4


def test_noalloc_forward_matches_workspace_forward_twice():
    lib = _lib.load()
    with torch.cuda.device(0):
        # first call: ragged causal batch plus one long-KV segment that is split across CTAs
        _both(lib, [300, 45, 128, 2], [300, 500, 128, 9000], 4, 128, torch.bfloat16, False, seed=11)
        # second call, different shape and dtype, on top of the first call's leftovers
        _both(lib, [7, 130, 1], [19, 130, 5000], 2, 64, torch.float16, True, seed=12)


def test_noalloc_splits_less_finely_when_the_partials_do_not_fit():
    """Forced 128-key slices on 128 query rows x 4096 keys x 16 heads ask for 32 x 128 partial rows of
    16 x 129 floats each, about 34 MB: twice the built-in 16 MiB.  The workspace path takes the slices
    as asked; the built-in array has to double them until the partials fit.  Same answer either way."""
    lib = _lib.load()
    H, D = 16, 128
    need = 32 * 128 * H * (D + 1) * 4
    assert need > 2 * (16 << 20)
    with torch.cuda.device(0):
        _both(lib, [128, 40], [4096, 300], H, D, torch.bfloat16, False, seed=13, split_k_block=128)
        _both(lib, [128, 40], [4096, 300], H, D, torch.bfloat16, False, seed=14, split_k_block=128)


def test_noalloc_rejects_oversized_batches_and_unsupported_shapes():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    n_seg = 400_000                                    # tile lists alone exceed the built-in scratch
    cu = torch.arange(n_seg + 1, dtype=torch.int32, device=dev)
    q = torch.zeros(n_seg, 1, 64, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(n_seg, 1, dtype=torch.float32, device=dev)
    a = _args(q, q, q, torch.empty_like(q), lse, cu, cu, False)
    rc = lib.vafa_varlen_fwd_noalloc(C.byref(a), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -3 and b"built-in" in lib.vafa_last_error()
    q32 = torch.zeros(4, 1, 64, dtype=torch.float32, device=dev)
    cu4 = torch.tensor([0, 4], dtype=torch.int32, device=dev)
    b = _args(q32, q32, q32, torch.empty_like(q32), lse[:4], cu4, cu4, False)
    assert lib.vafa_varlen_fwd_noalloc(C.byref(b), torch.cuda.current_stream(dev).cuda_stream) == -2
