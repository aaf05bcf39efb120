#!/usr/bin/env python
"""Benchmark of the packed variable-length attention hot path (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C2]

One step = one forward + backward pass of `packed_varlen_attn` over one packed batch of
benchmark configuration 2 (64 sequences, lengths log-uniform in [1, 4096] from a fixed seed,
H=16, D=128, bf16, causal; synthetic N(0,1) values).  FLOPs use the reference harness's
convention, 4*H*D*cells for the forward (cells = L(L+1)/2 under the causal mask) and 2.5x
that for the backward.  With N > 1 (torchrun, one rank per GPU) every rank runs its own batch
of the same configuration (the same length list on every rank, values from seed r): packed batches shard
by sequence with no data-path collective, so this is weak scaling and `value` is the sum over
ranks divided by the slowest rank's time.

The JSON line also carries: `e2e` (same metric, host pinned buffers in, host buffers out, copies
inside the timed region), `roofline` of the dominant kernel (event-timed inside this run),
`cpu_baseline` (the fp32 torch CPU restatement of the reference's own oracle, timed on a bounded
sample on this box's host cores), `absorb` (target-attention keys/s on configuration 4 and on the
production-like shape: forward, forward+backward, and the forward+backward step replayed from a CUDA
graph, which leaves the host's launch rate out) and the GPU clocks sampled during the timed regions.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum)
# from the ncu capture summarised under profiles/ for the same kernel, or None when no capture
# exists for this workload.
NCU_TRAFFIC_BYTES = {
    # profiles/varlen_kernels_C2_ncu_full.md (dram__bytes_read.sum + dram__bytes_write.sum, one launch)
    ("C2", "varlen_bwd_kernel<dKV>"): 574_531_328 + 231_917_056,
    ("C2", "varlen_bwd_kernel<dQ>"): 540_098_816 + 116_789_504,
    ("C2", "varlen_fwd_kernel"): 400_167_424 + 113_049_344,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def causal_cells(ql, kl):
    tot = 0
    for a, b in zip(ql, kl):
        if a == b:
            tot += a * (a + 1) // 2
        else:
            off = b - a
            tot += sum(max(0, min(b, i + off + 1)) for i in range(a))
    return tot


def cells_of(ql, kl, causal):
    return causal_cells(ql, kl) if causal else sum(a * b for a, b in zip(ql, kl))


class ClockSampler:
    """nvidia-smi in the background while the timed regions run (read-only query)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="vafa_clocks_", suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons, power = [], [], set(), []
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def make_batch(workload: str, seed: int):
    from oracle import CONFIGS, config_lengths
    cfg = CONFIGS[workload]
    # every rank gets the configuration's own length list (seed 0): weak scaling means the same work per
    # GPU, and `value` divides by the slowest rank's time, so ranks with different draws of the lengths
    # (whose cell counts differ by tens of percent) would measure the draw, not the scaling.  The values
    # differ per rank.
    ql, kl = config_lengths(workload, 0)
    g = torch.Generator(device="cpu").manual_seed(seed)
    H, D = cfg["H"], cfg["D"]
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[cfg["dtype"]]
    Tq, Tk = sum(ql), sum(kl)

    def rnd(T):
        return torch.randn(T, H, D, generator=g, dtype=torch.float32).to(dt).pin_memory()
    return cfg, ql, kl, rnd(Tq), rnd(Tk), rnd(Tk), rnd(Tq)


def cpu_reference_sample(workload: str, budget_cells: float, threads: int):
    """Time the fp32 torch CPU path (per segment, autograd backward) on a leading sample."""
    from oracle import CONFIGS, config_lengths, make_varlen_inputs, varlen_attn_ref_fwd_bwd
    cfg = CONFIGS[workload]
    ql, kl = config_lengths(workload, 0)
    tot, n = 0, 0
    for a, b in zip(ql, kl):
        if n > 0 and tot + a * b > budget_cells:
            break
        tot += a * b
        n += 1
    ql, kl = ql[:n], kl[:n]
    torch.set_num_threads(threads)
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(ql, kl, cfg["H"], cfg["D"], cfg["dtype"], 0)
    t0 = time.perf_counter()
    varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=cfg["causal"])
    dt = time.perf_counter() - t0
    flops = 3.5 * 4 * cfg["H"] * cfg["D"] * cells_of(ql, kl, cfg["causal"])
    all_cells = cells_of(*config_lengths(workload, 0), cfg["causal"])
    frac = cells_of(ql, kl, cfg["causal"]) / max(1, all_cells)
    return flops / dt / 1e12, dt, f"first {n} of {len(config_lengths(workload, 0)[0])} sequences of {workload} seed 0 ({100 * frac:.0f}% of its cells), fwd+bwd, fp32 torch on CPU"


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    sample = ""
    for i in range(args.warmup + args.steps):
        v, dt, sample = cpu_reference_sample(args.workload, args.ref_cells, threads)
        if i >= args.warmup:
            vals.append((v, dt))
    value = sum(v for v, _ in vals) / len(vals)
    ms = 1e3 * sum(d for _, d in vals) / len(vals)
    from oracle import CONFIGS
    cfg = CONFIGS[args.workload]
    line = {
        "impl": "reference", "metric": "varlen-attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: packed varlen {'causal' if cfg['causal'] else 'non-causal'} attention fwd+bwd, H={cfg['H']} D={cfg['D']}",
                   "note": "reference's torch CPU path (per-segment fp32 matmul-softmax-matmul, autograd backward); each step is a bounded sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def production_lengths(seed=0):
    """Synthetic stand-in for the reference's production length lists (its fixture of 100 logged
    batches: 1103-1174 users, 2.2-2.35 M keys; 96-98 % of the users have exactly 2048 keys, the rest
    anything from 1 up; 1-18 queries per user, mean 5.3)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = 1137
    q = torch.clamp((torch.empty(n, dtype=torch.float64).exponential_(1 / 4.8, generator=g)).floor().long() + 1, 1, 18)
    full = torch.rand(n, generator=g, dtype=torch.float64) < 0.969
    k = torch.where(full, torch.full((n,), 2048), torch.randint(1, 2048, (n,), generator=g))
    return [int(x) for x in q], [int(x) for x in k]


def absorb_leg(dev, steps, warmup, group, production=False):
    """Target attention on configuration 4 (or the production-like shape: d_q = 968, d_kv = 216):
    keys/s forward and forward+backward."""
    import varlenabsorbflashattn_b200 as vb
    from oracle import config_lengths, lengths_to_cu
    ql, kl = production_lengths(0) if production else config_lengths("C4", 0)
    d_q, d_kv = (968, 216) if production else (256, 256)
    Tq, Tk = sum(ql), sum(kl)
    g = torch.Generator(device="cpu").manual_seed(0)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std).to(torch.bfloat16).to(dev)
    q_raw, X = mk(Tq, d_q), mk(Tk, d_kv)
    W = [mk(d, 8, 32, std=1 / 16).requires_grad_(True) for d in (d_q, d_kv, d_kv)]
    q_raw.requires_grad_(True); X.requires_grad_(True)
    dO = mk(Tq, 8, 32)
    cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)

    def fwd():
        return vb.packed_target_attn(q_raw, X, *W, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, validate=False,
                                     weight_grad_group=group)

    def fb():
        torch.autograd.grad(fwd(), (q_raw, X, *W), dO)

    out = {}
    for name, fn in (("fwd", fwd), ("fwd_bwd", fb)):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[name + "_ms"] = ms
        out[name + "_keys_per_s"] = Tk / (ms * 1e-3)
    # The same forward+backward replayed from a CUDA graph: a step of this size is some 25 short launches,
    # so the eager number above contains the host's launch rate; the replay is the device time.
    if group is None:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fb()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fb()
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out["fwd_bwd_graph_ms"] = ms
        out["fwd_bwd_graph_keys_per_s"] = Tk / (ms * 1e-3)
    out["workload"] = ("production-like: 1137 users, 97 % with 2048 keys, q 1-18 (mean 5.3), d_q=968, d_kv=216, "
                       f"H=8, D_H=32, bf16 ({Tq} queries, {Tk} keys)" if production else
                       "C4: 1024 users, q U[1,16], k logU[8,2048], d=256, H=8, D_H=32, bf16")
    out["unit"] = "keys/s"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2")
    ap.add_argument("--ref-cells", type=float, default=None,
                    help="cell budget (sum of Lq*Lk) of the CPU sample; default 2.5e7 for the cpu_baseline leg, 6e6 per step for --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-absorb", action="store_true")
    ap.add_argument("--e2e-groups", type=int, default=8,
                    help="sequence groups (streams) the end-to-end leg overlaps copies and kernels over")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        args.ref_cells = args.ref_cells or 6e6
        run_reference(args, rank, world)
        return
    args.ref_cells = args.ref_cells or 2.5e7

    import torch.distributed as dist
    import varlenabsorbflashattn_b200 as vb
    from varlenabsorbflashattn_b200 import _lib
    from varlenabsorbflashattn_b200 import build as vbuild
    from oracle import lengths_to_cu

    if rank == 0:
        vbuild.build()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
        dist.barrier()
    _lib.load()
    vb.set_validate_cu_seqlens(False)

    cfg, ql, kl, hq, hk, hv, hdo = make_batch(args.workload, rank)
    causal = cfg["causal"]
    H, D = cfg["H"], cfg["D"]
    cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)
    fwd_flops = 4.0 * H * D * cells_of(ql, kl, causal)
    step_flops = 3.5 * fwd_flops

    q = hq.to(dev).requires_grad_(True)
    k = hk.to(dev).requires_grad_(True)
    v = hv.to(dev).requires_grad_(True)
    do = hdo.to(dev)

    def step():
        o = vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)
        return (o,) + torch.autograd.grad(o, (q, k, v), do)

    def fwd_only():
        with torch.no_grad():
            return vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    def total_over_ranks(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    _lib.profile_reset()
    ms_step = timed(step, args.steps, args.warmup)
    launches = sum(v[2] for v in _lib.profile_read().values())
    launches_per_step = launches // (args.steps + args.warmup)
    ms_fwd = timed(fwd_only, args.steps, 2)
    total_flops = total_over_ranks(step_flops)
    total_fwd_flops = total_over_ranks(fwd_flops)
    value = total_flops / (ms_step * 1e-3) / 1e12
    fwd_value = total_fwd_flops / (ms_fwd * 1e-3) / 1e12

    # ---- end to end: pinned host -> device, fwd+bwd through the public API, results -> host.
    # Sequences are independent, so the batch is cut into contiguous groups of sequences, each on its
    # own stream: the copy of one group (either direction) runs while another group computes, and the
    # two copy directions run at the same time.  Every byte of the step's inputs and results still
    # crosses the bus inside the timed region.
    ho = torch.empty_like(hq).pin_memory()
    hdq, hdk, hdv = torch.empty_like(hq).pin_memory(), torch.empty_like(hk).pin_memory(), torch.empty_like(hv).pin_memory()
    dq_ = torch.empty_like(q.detach()); dk_ = torch.empty_like(k.detach()); dv_ = torch.empty_like(v.detach()); ddo_ = torch.empty_like(do)
    n_groups = max(1, min(args.e2e_groups, len(ql)))
    groups = []
    tot_q, seq0, tq0, tk0 = sum(ql), 0, 0, 0
    for gi in range(n_groups):
        seq1, tq1, tk1 = seq0, tq0, tk0
        target = tot_q * (gi + 1) / n_groups
        while seq1 < len(ql) and (tq1 < target or gi == n_groups - 1):
            tq1 += ql[seq1]; tk1 += kl[seq1]; seq1 += 1
        if seq1 > seq0:
            groups.append({"q": (tq0, tq1), "k": (tk0, tk1), "stream": torch.cuda.Stream(device=dev),
                           "cu_q": lengths_to_cu(ql[seq0:seq1]).to(dev), "cu_k": lengths_to_cu(kl[seq0:seq1]).to(dev)})
        seq0, tq0, tk0 = seq1, tq1, tk1

    def e2e_step():
        cur = torch.cuda.current_stream()
        for g in groups:
            st = g["stream"]
            st.wait_stream(cur)
            (q0, q1), (k0, k1) = g["q"], g["k"]
            with torch.cuda.stream(st):
                a, b, c, d = dq_[q0:q1], dk_[k0:k1], dv_[k0:k1], ddo_[q0:q1]
                a.copy_(hq[q0:q1], non_blocking=True); b.copy_(hk[k0:k1], non_blocking=True)
                c.copy_(hv[k0:k1], non_blocking=True); d.copy_(hdo[q0:q1], non_blocking=True)
                a = a.detach().requires_grad_(True); b = b.detach().requires_grad_(True); c = c.detach().requires_grad_(True)
                o = vb.packed_varlen_attn(a, b, c, cu_seqlens_q=g["cu_q"], cu_seqlens_k=g["cu_k"], causal=causal)
                ga, gb, gc = torch.autograd.grad(o, (a, b, c), d)
                ho[q0:q1].copy_(o.detach(), non_blocking=True); hdq[q0:q1].copy_(ga, non_blocking=True)
                hdk[k0:k1].copy_(gb, non_blocking=True); hdv[k0:k1].copy_(gc, non_blocking=True)
        for g in groups:
            cur.wait_stream(g["stream"])

    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps, 2)
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv))

    # ---- per-kernel durations (events around every launch) for the roofline of the top kernel
    _lib.profile_reset()
    _lib.profile_enable(True)
    for _ in range(max(3, min(args.steps, 10))):
        step()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    _lib.profile_enable(False)
    clocks = sampler.stop() if rank == 0 else None

    absorb = None
    if not args.no_absorb:
        try:
            absorb = absorb_leg(dev, max(3, min(args.steps, 10)), 3, group)
        except Exception as e:  # the headline line must still print
            absorb = {"error": str(e)[:200]}
        try:
            absorb["production_shape"] = absorb_leg(dev, max(3, min(args.steps, 10)), 3, group, production=True)
        except Exception as e:
            absorb["production_shape"] = {"error": str(e)[:200]}
    _lib.check_status(dev)

    if rank == 0:
        peaks, peak_src = load_peaks()
        kern = {n: (ms / max(1, nt)) for n, (ms, nt, na) in prof.items() if nt}
        share = {n: ms for n, (ms, nt, na) in prof.items()}
        tot_ms = sum(share.values()) or 1.0
        top = max(share, key=share.get)
        cells = cells_of(ql, kl, causal)
        # matmul FLOPs each kernel performs on the visible cells: 2*D per cell per product
        products = {"varlen_fwd_kernel": 2, "varlen_bwd_kernel<dQ>": 3, "varlen_bwd_kernel<dKV>": 4}
        roofline = None
        if top in products:
            algo = products[top] * 2.0 * H * D * cells
            ach = algo / (kern[top] * 1e-3) / 1e12
            peak = peaks["bf16_tflops_sustained"]
            roofline = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                        "frac": ach / peak, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, top)),
                        "peak_source": f"{peak_src} sustained bf16 (kernel timed inside a long step)",
                        "avg_launch_ms": kern[top], "share_of_step": share[top] / tot_ms,
                        "algorithmic_flops_per_launch": algo,
                        "kernel_shares": {n: round(v / tot_ms, 4) for n, v in sorted(share.items(), key=lambda x: -x[1])}}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v_cpu, dt_cpu, sample = cpu_reference_sample(args.workload, args.ref_cells, threads)
            cpu = {"value": v_cpu, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample,
                   "seconds": dt_cpu}
        line = {
            "metric": "varlen-attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: packed varlen {'causal' if causal else 'non-causal'} attention fwd+bwd, {len(ql)} sequences/rank, "
                                   f"{sum(ql)} tokens/rank, H={H} D={D} bf16",
                       "flops_convention": "fwd 4*H*D*cells (visible cells), bwd 2.5x fwd",
                       "l2": "inputs larger than L2 (q, dO, o, dq: %.0f MB each; k, v, dk, dv: %.0f MB each)" % (hq.numel() * 2 / 1e6, hk.numel() * 2 / 1e6),
                       "parallelism": f"dp{world} by sequence, no data-path collective"},
            "fwd_only": {"value": fwd_value, "unit": "TFLOP/s", "ms": ms_fwd},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "sequence_groups": len(groups),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches_per_step * args.steps),
            "roofline": roofline, "cpu_baseline": cpu, "absorb": absorb, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
