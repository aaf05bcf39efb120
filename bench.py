#!/usr/bin/env python
"""Benchmark of the two hot paths on the box-scale configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C5]

Default workload, configuration 5 ("C5"): ONE packed batch of 1 000 000 tokens (520 sequences, lengths
log-uniform in [128, 8192] from a fixed seed, H=32, D=128, bf16, causal) through `packed_varlen_attn`
forward + backward -- this is `value`, in TFLOP/s -- plus ONE batch of 16 384 users through
`packed_target_attn` forward + backward, reported under `absorb` in keys/s.  Values are synthetic
N(0,1), drawn on the device (the host copy of the batch alone would be 33 GB).  FLOPs use the reference
harness's convention: forward 4*H*D*cells (cells = visible (query, key) pairs, L(L+1)/2 per causal
sequence), backward 2.5x that.

With N > 1 (torchrun, one rank per GPU) the SAME batch is cut by whole sequences with
`sharding.partition_segments` and each rank runs its shard: strong scaling.  `value` is the whole
batch's FLOPs divided by the slowest rank's device time.  The varlen path exchanges nothing; the absorb
operator all-reduces its fp32 weight gradients over NCCL inside the timed step.

The JSON line also carries `e2e` (the same metric through the public API with pinned host buffers in
and out, copies inside the timed region, on a stated slice of the batch), `roofline` of the dominant
kernel (event-timed inside this run), `cpu_baseline` (the fp32 torch CPU restatement of the reference's
own oracle on a bounded sample, N=1 only), `vs_reference_gpu` (N=1 only: the reference's Triton kernels
and flash-attn timed in a child process on the same GPU and the same seeded inputs, on the shapes their
32-bit indexing can address) and the GPU clocks sampled during the timed regions.

Other workloads: C5s (the leading 1/16 of C5, for profiler captures), C2, C2b, S1 (named length generators), `stage1:<row>` (a row of the reference's logged
production shapes, tests/golden/stage1_shapes.jsonl.gz) for the varlen operator, and `absorb-prod:<i>`
(record i of tests/golden/real_shape_all.json.gz; d_q=968, d_kv=216) / `C4` for the absorb operator
alone.
"""
from __future__ import annotations

import argparse
import gzip
import json
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
GOLDEN = os.path.join(ROOT, "tests", "golden")
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# matrix products each varlen kernel performs per visible (query, key) cell
PRODUCTS = {"varlen_fwd_kernel": 2, "varlen_bwd_kernel<dQ>": 3, "varlen_bwd_kernel<dKV>": 4,
            "varlen_bwd_kernel<fused>": 5}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def load_dram_traffic():
    """Rows `| workload | kernel | bytes per launch | tokens |` of profiles/dram_traffic.md: DRAM bytes
    (read + write) one launch moved in an ncu capture, and the token count of the captured batch."""
    out = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(path):
        return out
    for line in open(path):
        f = [x.strip() for x in line.strip().strip("|").split("|")]
        if len(f) >= 4 and f[2].replace("_", "").isdigit() and f[3].replace("_", "").isdigit():
            out.setdefault(f[1].strip("`"), []).append((f[0], int(f[2].replace("_", "")), int(f[3].replace("_", ""))))
    return out


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


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
def _golden_lines(name):
    with gzip.open(os.path.join(GOLDEN, name), "rt", encoding="utf-8") as fh:
        return fh.read()


def stage1_row(i: int):
    rows = [json.loads(l) for l in _golden_lines("stage1_shapes.jsonl.gz").splitlines() if l.strip()]
    r = rows[i]
    return r["name"], [int(x) for x in r["q_lens"]], [int(x) for x in r["k_lens"]]


def absorb_prod_record(i: int):
    rec = json.loads(_golden_lines("real_shape_all.json.gz"))["records"][i]
    return rec["tag"] + f"#{i}", [int(x) for x in rec["q_lens"]], [int(x) for x in rec["k_lens"]]


def workload(name: str) -> dict:
    """kind 'varlen': q/k lengths + H, D, causal; kind 'absorb': lengths + d_q, d_kv."""
    from oracle import CONFIGS, config_lengths
    if name == "C5":
        ql, kl = config_lengths("C5v", 0)
        c = CONFIGS["C5v"]
        return dict(kind="varlen", name="C5", ql=ql, kl=kl, H=c["H"], D=c["D"], causal=c["causal"], absorb="C5a",
                    label="C5: one packed batch, lengths logU[128,8192] seed 0, causal")
    if name == "C5s":
        # the leading sequences of C5 that hold 1/16 of its tokens: the same kernels and head count on a few GB,
        # small enough for a profiler capture
        ql, _ = config_lengths("C5v", 0)
        n, acc = 0, 0
        while acc + ql[n] <= 62_500:
            acc += ql[n]; n += 1
        c = CONFIGS["C5v"]
        return dict(kind="varlen", name="C5s", ql=ql[:n], kl=ql[:n], H=c["H"], D=c["D"], causal=c["causal"], absorb=None,
                    label=f"C5s: the first {n} sequences of C5")
    if name in ("C2", "C2b", "S1", "C3"):
        ql, kl = config_lengths(name, 0)
        c = CONFIGS[name]
        return dict(kind="varlen", name=name, ql=ql, kl=kl, H=c["H"], D=c["D"], causal=c["causal"],
                    absorb="C4" if name.startswith("C2") else None, label=f"{name}: named length generator, seed 0")
    if name.startswith("stage1:"):
        nm, ql, kl = stage1_row(int(name.split(":")[1]))
        return dict(kind="varlen", name=name, ql=ql, kl=kl, H=4, D=64, causal=False, absorb=None,
                    label=f"{nm}: logged production shape (q=500 per user, keys up to 102 400)")
    if name in ("C4", "C5a"):
        ql, kl = config_lengths(name, 0)
        return dict(kind="absorb", name=name, ql=ql, kl=kl, d_q=256, d_kv=256, label=f"{name}: q U[1,16], k logU[8,2048]")
    if name.startswith("absorb-prod:"):
        nm, ql, kl = absorb_prod_record(int(name.split(":")[1]))
        return dict(kind="absorb", name=name, ql=ql, kl=kl, d_q=968, d_kv=216, label=f"{nm}: logged production batch")
    raise SystemExit(f"unknown workload {name}")


def balanced_partition(ql, kl, world, causal):
    """Whole sequences to ranks, balancing tokens AND attention cells at once: sequences in descending
    cell order, each to the rank whose larger normalised load (tokens, cells) stays smallest.  Tokens set
    the memory and HBM traffic of a shard, cells its tensor-core time."""
    from varlenabsorbflashattn_b200.sharding import Partition
    tok = [a + b for a, b in zip(ql, kl)]
    cel = [cells_of([a], [b], causal) for a, b in zip(ql, kl)]
    tt, tc = max(1, sum(tok)), max(1, sum(cel))
    order = sorted(range(len(ql)), key=lambda i: (-cel[i], i))
    lt, lc = [0] * world, [0] * world
    owned = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (max((lt[j] + tok[i]) / tt, (lc[j] + cel[i]) / tc), j))
        owned[r].append(i); lt[r] += tok[i]; lc[r] += cel[i]
    for o in owned:
        o.sort()
    return Partition(owned, lt), lt, lc


def _imb(load):
    m = sum(load) / max(1, len(load))
    return round(max(load) / m, 4) if m > 0 else 1.0


def partition_report(ql, kl, world, causal):
    from varlenabsorbflashattn_b200.sharding import partition_segments
    cel = lambda a, b: cells_of([a], [b], causal)
    p_tok = partition_segments(ql, kl, world)
    p_cel = partition_segments(ql, kl, world, weight=cel)
    part, lt, lc = balanced_partition(ql, kl, world, causal)

    def both(p):
        t = [sum(ql[i] + kl[i] for i in seg) for seg in p.assignment]
        c = [sum(cel(ql[i], kl[i]) for i in seg) for seg in p.assignment]
        return {"token_imbalance": _imb(t), "cell_imbalance": _imb(c)}
    return part, {"used": "tokens+cells (vector greedy)", "used_balance": {"token_imbalance": _imb(lt), "cell_imbalance": _imb(lc)},
                  "token_balanced_lpt": both(p_tok), "cell_balanced_lpt": both(p_cel)}


def device_randn(shape, seed, dev, dtype=torch.bfloat16, std=1.0):
    g = torch.Generator(device=dev)
    g.manual_seed(int(seed))
    t = torch.randn(shape, generator=g, device=dev, dtype=dtype)
    return t if std == 1.0 else t * std


def shard_of(full, lens, part, rank, world):
    if world == 1:
        return full
    from varlenabsorbflashattn_b200.sharding import shard_rows
    return shard_rows(full, lens, part, rank)


# ---------------------------------------------------------------------------------------------
# CPU baseline / reference arm
# ---------------------------------------------------------------------------------------------
def cpu_reference_sample(wl: dict, budget_cells: float, threads: int):
    """Time the fp32 torch CPU path (per segment, autograd backward) on a leading sample of the batch."""
    from oracle import make_varlen_inputs, varlen_attn_ref_fwd_bwd
    ql, kl = wl["ql"], wl["kl"]
    # sequences in batch order, each taken if it still fits the budget of Lq*Lk cells (the oracle computes
    # the full rectangle, masked or not); at least one sequence (the smallest) is always taken
    tot, pick = 0, []
    for i, (a, b) in enumerate(zip(ql, kl)):
        if tot + a * b <= budget_cells:
            tot += a * b
            pick.append(i)
        if tot >= 0.9 * budget_cells:
            break
    if not pick:
        pick = [min(range(len(ql)), key=lambda i: ql[i] * kl[i])]
    sq, sk = [ql[i] for i in pick], [kl[i] for i in pick]
    n = len(pick)
    torch.set_num_threads(threads)
    q, k, v, do, cu_q, cu_k = make_varlen_inputs(sq, sk, wl["H"], wl["D"], "bf16", 0)
    t0 = time.perf_counter()
    varlen_attn_ref_fwd_bwd(q, k, v, do, cu_q, cu_k, causal=wl["causal"])
    dt = time.perf_counter() - t0
    flops = 3.5 * 4 * wl["H"] * wl["D"] * cells_of(sq, sk, wl["causal"])
    frac = cells_of(sq, sk, wl["causal"]) / max(1, cells_of(ql, kl, wl["causal"]))
    return flops / dt / 1e12, dt, (f"{n} of the {len(ql)} sequences of {wl['name']} (in batch order, those that fit a budget of "
                                   f"{budget_cells:.1e} Lq*Lk cells; lengths {min(sq)}-{max(sq)}; {100 * frac:.2f}% of the batch's cells), "
                                   "fwd+bwd, fp32 torch on CPU")


def run_reference(args, rank):
    if rank != 0:
        return
    wl = workload(args.workload)
    if wl["kind"] != "varlen":
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm times the varlen operator's CPU path only"}))
        return
    threads = os.cpu_count() or 1
    vals, sample = [], ""
    for i in range(args.warmup + args.steps):
        v, dt, sample = cpu_reference_sample(wl, args.ref_cells, threads)
        if i >= args.warmup:
            vals.append((v, dt))
    value = sum(v for v, _ in vals) / len(vals)
    ms = 1e3 * sum(d for _, d in vals) / len(vals)
    line = {
        "impl": "reference", "metric": "varlen-attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": varlen_config(wl, 1, None),
        "note": "the reference's torch CPU path (per-segment fp32 matmul-softmax-matmul, autograd backward) on this "
                "box's host cores; each step is a bounded leading sample of the workload",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def varlen_config(wl, world, part_info):
    ql = wl["ql"]
    mb = sum(ql) * wl["H"] * wl["D"] * 2 / 1e6
    cfg = {"workload": f"{wl['label']}; packed varlen {'causal' if wl['causal'] else 'non-causal'} attention fwd+bwd, "
                       f"{len(ql)} sequences, {sum(ql)} tokens, H={wl['H']} D={wl['D']} bf16",
           "flops_convention": "fwd 4*H*D*cells (visible cells), bwd 2.5x fwd",
           "l2": f"inputs larger than L2 (q, k, v, dO: {mb:.0f} MB each over the whole batch)",
           "parallelism": f"dp{world} by whole sequence: one batch cut across ranks, no data-path collective "
                          "(absorb leg: NCCL all-reduce of the fp32 weight gradients inside the step)"}
    if part_info is not None:
        cfg["partition"] = part_info
    return cfg


# ---------------------------------------------------------------------------------------------
# absorb leg
# ---------------------------------------------------------------------------------------------
def production_lengths(seed=0):
    """Synthetic stand-in with the distribution of the reference's logged production batches
    (1103-1174 users, 96-98 % of them with exactly 2048 keys, 1-18 queries per user, mean 5.3)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = 1137
    q = torch.clamp((torch.empty(n, dtype=torch.float64).exponential_(1 / 4.8, generator=g)).floor().long() + 1, 1, 18)
    full = torch.rand(n, generator=g, dtype=torch.float64) < 0.969
    k = torch.where(full, torch.full((n,), 2048), torch.randint(1, 2048, (n,), generator=g))
    return [int(x) for x in q], [int(x) for x in k]


def absorb_inputs(ql, kl, d_q, d_kv, dev, seed=0, dtype=torch.bfloat16):
    Tq, Tk = sum(ql), sum(kl)
    q_raw = device_randn((Tq, d_q), seed * 16 + 1, dev, dtype)
    X = device_randn((Tk, d_kv), seed * 16 + 2, dev, dtype)
    W = [device_randn((d, 8, 32), seed * 16 + 3 + i, dev, dtype, std=1 / 16) for i, d in enumerate((d_q, d_kv, d_kv))]
    dO = device_randn((Tq, 8, 32), seed * 16 + 6, dev, dtype)
    return q_raw, X, W, dO


def absorb_leg(dev, ql, kl, d_q, d_kv, steps, warmup, timed, rank, world, group, label, graph=False, shard_check=False):
    """packed_target_attn forward and forward+backward on one batch (cut across ranks by whole users):
    keys/s = keys of the whole batch / slowest rank's time."""
    import varlenabsorbflashattn_b200 as vb
    from oracle import lengths_to_cu
    from varlenabsorbflashattn_b200.sharding import partition_segments, local_cu_seqlens
    Tk = sum(kl)
    q_raw, X, W, dO = absorb_inputs(ql, kl, d_q, d_kv, dev)
    part = partition_segments(ql, kl, world) if world > 1 else None
    if world > 1:
        lq = shard_of(q_raw, ql, part, rank, world).contiguous()
        lx = shard_of(X, kl, part, rank, world).contiguous()
        ldo = shard_of(dO, ql, part, rank, world).contiguous()
        cu_q = local_cu_seqlens(ql, part, rank).to(dev)
        cu_k = local_cu_seqlens(kl, part, rank).to(dev)
    else:
        lq, lx, ldo = q_raw, X, dO
        cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)
    lq.requires_grad_(True); lx.requires_grad_(True)
    Wg = [w.clone().requires_grad_(True) for w in W]

    def fwd():
        return vb.packed_target_attn(lq, lx, *Wg, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, validate=False,
                                     weight_grad_group=group)

    def fb():
        return torch.autograd.grad(fwd(), (lq, lx, *Wg), ldo)

    out = {"workload": label, "unit": "keys/s", "users": len(ql), "queries": sum(ql), "keys": Tk, "d_q": d_q, "d_kv": d_kv}
    ms_f = timed(lambda: fwd(), steps, warmup)
    ms_fb = timed(fb, steps, warmup)
    out.update(fwd_ms=ms_f, fwd_keys_per_s=Tk / (ms_f * 1e-3), fwd_bwd_ms=ms_fb, fwd_bwd_keys_per_s=Tk / (ms_fb * 1e-3))
    if world > 1:
        t = [sum(ql[i] + kl[i] for i in seg) for seg in part.assignment]
        out["partition"] = {"used": "token-balanced LPT by user", "token_imbalance": _imb(t)}
    if graph and world == 1:
        # The same step replayed from a CUDA graph: a step of a small batch is some 25 short launches, so the
        # eager number contains the host's launch rate; the replay is the device time.
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fb()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fb()
        ms_g = timed(g.replay, steps, warmup)
        out.update(fwd_bwd_graph_ms=ms_g, fwd_bwd_graph_keys_per_s=Tk / (ms_g * 1e-3))
    if shard_check and world > 1:
        # value check of the sharded operator: the all-reduced weight gradients of the shards against the
        # whole batch run on this rank alone
        sh = fb()
        q_full = q_raw.detach().requires_grad_(True); x_full = X.detach().requires_grad_(True)
        Wf = [w.clone().requires_grad_(True) for w in W]
        o = vb.packed_target_attn(q_full, x_full, *Wf, cu_seqlens_q=lengths_to_cu(ql).to(dev),
                                  cu_seqlens_k=lengths_to_cu(kl).to(dev), validate=False)
        full = torch.autograd.grad(o, Wf, dO)
        err = max(float((a.float() - b.float()).abs().max()) for a, b in zip(sh[2:], full))
        ref = max(float(b.float().abs().max()) for b in full)
        out["shard_check_max_abs"] = err
        out["shard_check_max_ref"] = ref
    return out


# ---------------------------------------------------------------------------------------------
# child process: the reference's Triton kernels and flash-attn beside the library, same GPU, same inputs
# ---------------------------------------------------------------------------------------------
def compare_leg():
    res = {}
    if not os.path.isdir(os.path.join(REF_DIR, "triton_fa_varlen_v2")):
        print(json.dumps({"unavailable": "baseline/_ref is missing (bash baseline/install_ref.sh <reference checkout> installs the reference there)"}))
        return
    sys.path.insert(0, REF_DIR)
    import varlenabsorbflashattn_b200 as vb
    from oracle import config_lengths, lengths_to_cu
    vb.set_validate_cu_seqlens(False)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        import triton_fa_varlen_v2 as R
        import triton_target_attn_absorb as RA
        R.set_validate_cu_seqlens(False)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"unavailable": f"reference import failed: {str(e)[:160]}"}))
        return
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception:  # noqa: BLE001
        flash_attn_varlen_func = None

    def t_ms(fn, n=5, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def ratio(a, b):
        return {k: round(b[k] / a[k], 3) for k in ("fwd_ms", "fwd_bwd_ms") if k in a and k in b}

    def varlen_case(name, ql, kl, H, D):
        # every tensor stays far below 2^31 elements: the reference kernels index in 32 bits
        assert max(sum(ql), sum(kl)) * H * D < 2**31
        q, k, v, do = (device_randn((T, H, D), 11 + i, dev).requires_grad_(i < 3)
                       for i, T in enumerate((sum(ql), sum(kl), sum(kl), sum(ql))))
        cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)
        mq, mk = max(ql), max(kl)
        impls = {("noncausal", "ours"): lambda: vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k),
                 ("noncausal", "triton"): lambda: R.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k),
                 ("causal", "ours"): lambda: vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=True)}
        if flash_attn_varlen_func is not None:
            impls[("noncausal", "fa2")] = lambda: flash_attn_varlen_func(q, k, v, cu_q, cu_k, mq, mk, causal=False)
            impls[("causal", "fa2")] = lambda: flash_attn_varlen_func(q, k, v, cu_q, cu_k, mq, mk, causal=True)
        out = {}
        for (mode, who), f in impls.items():
            try:
                with torch.no_grad():
                    tf = t_ms(f)
                tfb = t_ms(lambda: torch.autograd.grad(f(), (q, k, v), do))
                out.setdefault(mode, {})[who] = {"fwd_ms": round(tf, 4), "fwd_bwd_ms": round(tfb, 4)}
            except Exception as e:  # noqa: BLE001
                out.setdefault(mode, {})[who] = {"error": str(e)[:120]}
        for mode, d in out.items():
            fl = 4.0 * H * D * cells_of(ql, kl, mode == "causal")
            for who, r in d.items():
                if "fwd_ms" in r:
                    r["fwd_tflops"] = round(fl / r["fwd_ms"] / 1e9, 1)
                    r["fwd_bwd_tflops"] = round(3.5 * fl / r["fwd_bwd_ms"] / 1e9, 1)
            if "ours" in d and "fwd_ms" in d["ours"]:
                for who in ("triton", "fa2"):
                    if who in d and "fwd_ms" in d[who]:
                        d["vs_" + who] = {"fwd": round(d[who]["fwd_ms"] / d["ours"]["fwd_ms"], 3),
                                          "fwd_bwd": round(d[who]["fwd_bwd_ms"] / d["ours"]["fwd_bwd_ms"], 3)}
        res[name] = out

    def absorb_case(name, ql, kl, d_q, d_kv, dtype=torch.bfloat16):
        q_raw, X, W, dO = absorb_inputs(ql, kl, d_q, d_kv, dev, dtype=dtype)
        q_raw.requires_grad_(True); X.requires_grad_(True)
        W = [w.requires_grad_(True) for w in W]
        cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)
        qi, ki = RA.prepare_target_attn_indices(cu_q, cu_k)
        impls = {"ours": lambda: vb.packed_target_attn(q_raw, X, *W, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, validate=False),
                 "triton": lambda: RA.packed_target_attn(q_raw, X, *W, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k,
                                                         q_chunk_indices=qi, k_chunk_indices=ki, validate=False)}
        out = {}
        for who, f in impls.items():
            try:
                with torch.no_grad():
                    tf = t_ms(f)
                tfb = t_ms(lambda: torch.autograd.grad(f(), (q_raw, X, *W), dO))
                out[who] = {"fwd_ms": round(tf, 4), "fwd_bwd_ms": round(tfb, 4),
                            "fwd_keys_per_s": sum(kl) / (tf * 1e-3), "fwd_bwd_keys_per_s": sum(kl) / (tfb * 1e-3)}
            except Exception as e:  # noqa: BLE001
                out[who] = {"error": str(e)[:120]}
        if all("fwd_ms" in out.get(w, {}) for w in ("ours", "triton")):
            out["vs_triton"] = {"fwd": round(out["triton"]["fwd_ms"] / out["ours"]["fwd_ms"], 3),
                                "fwd_bwd": round(out["triton"]["fwd_bwd_ms"] / out["ours"]["fwd_bwd_ms"], 3)}
        res[name] = out

    ql, kl = config_lengths("C2", 0)
    varlen_case("C2", ql, kl, 16, 128)
    ql, kl = config_lengths("C2b", 0)
    varlen_case("C2b", ql, kl, 16, 128)
    ql, kl = config_lengths("C4", 0)
    absorb_case("C4", ql, kl, 256, 256)
    ql, kl = production_lengths(0)
    absorb_case("absorb_production_shape", ql, kl, 968, 216)
    # fp32 inputs are the reference's default for packed_target_attn (IEEE fp32 dots in its kernels); here they
    # run on the scalar kernels
    ql, kl = config_lengths("C4", 0)
    absorb_case("C4_fp32", ql[:256], kl[:256], 256, 256, dtype=torch.float32)
    res["note"] = ("ratios are reference time / this library's time (> 1: this library is faster); the reference has no "
                   "causal mode, so causal is compared with flash-attn only; shapes whose tensors reach 2^31 elements "
                   "(C3, C5) are not run on the reference: its 32-bit indexing faulted there")
    print(json.dumps(res), flush=True)


# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C5")
    ap.add_argument("--leg", default="main", choices=["main", "compare"])
    ap.add_argument("--ref-cells", type=float, default=None,
                    help="cell budget (sum of Lq*Lk) of the CPU sample; default 2.5e7 for the cpu_baseline leg, 6e6 per step for --impl reference")
    ap.add_argument("--e2e-fraction", type=float, default=0.125,
                    help="share of the batch's tokens (leading sequences) the end-to-end leg moves through pinned host memory")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-absorb", action="store_true")
    ap.add_argument("--no-compare", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-groups", type=int, default=8,
                    help="sequence groups (streams) the end-to-end leg overlaps copies and kernels over")
    args = ap.parse_args()
    if args.leg == "compare":
        compare_leg()
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        args.ref_cells = args.ref_cells or 6e6
        run_reference(args, rank)
        return
    args.ref_cells = args.ref_cells or 2.5e7

    import torch.distributed as dist
    import varlenabsorbflashattn_b200 as vb
    from varlenabsorbflashattn_b200 import _lib
    from varlenabsorbflashattn_b200 import build as vbuild
    from varlenabsorbflashattn_b200.sharding import local_cu_seqlens
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

    wl = workload(args.workload)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    small_steps = max(3, min(args.steps, 10))

    if wl["kind"] == "absorb":
        res = absorb_leg(dev, wl["ql"], wl["kl"], wl["d_q"], wl["d_kv"], args.steps, args.warmup, timed, rank, world, group,
                         wl["label"], graph=True, shard_check=True)
        _lib.check_status(dev)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            print(json.dumps({"metric": "absorb target-attn fwd+bwd keys/s", "value": res["fwd_bwd_keys_per_s"], "unit": "keys/s",
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["fwd_bwd_ms"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                              "data": "synthetic", "config": {"workload": wl["label"]}, "absorb": res, "clocks": clocks}), flush=True)
        if world > 1:
            dist.barrier(); dist.destroy_process_group()
        return

    # ---- the batch, cut across ranks by whole sequences ----
    ql, kl, H, D, causal = wl["ql"], wl["kl"], wl["H"], wl["D"], wl["causal"]
    part, part_info = partition_report(ql, kl, world, causal) if world > 1 else (None, None)
    mine = part.assignment[rank] if world > 1 else list(range(len(ql)))
    my_ql, my_kl = [ql[i] for i in mine], [kl[i] for i in mine]
    if world > 1:
        cu_q, cu_k = local_cu_seqlens(ql, part, rank).to(dev), local_cu_seqlens(kl, part, rank).to(dev)
    else:
        cu_q, cu_k = lengths_to_cu(ql).to(dev), lengths_to_cu(kl).to(dev)
    Tq, Tk = sum(ql), sum(kl)
    # every rank draws the whole tensor from the same seed and keeps its rows: one batch, whatever N is
    q = shard_of(device_randn((Tq, H, D), 1, dev), ql, part, rank, world).requires_grad_(True)
    k = shard_of(device_randn((Tk, H, D), 2, dev), kl, part, rank, world).requires_grad_(True)
    v = shard_of(device_randn((Tk, H, D), 3, dev), kl, part, rank, world).requires_grad_(True)
    do = shard_of(device_randn((Tq, H, D), 4, dev), ql, part, rank, world)
    torch.cuda.empty_cache()
    fwd_flops = 4.0 * H * D * cells_of(ql, kl, causal)           # the whole batch
    step_flops = 3.5 * fwd_flops
    my_cells = cells_of(my_ql, my_kl, causal)

    def step():
        o = vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)
        return (o,) + torch.autograd.grad(o, (q, k, v), do)

    def fwd_only():
        with torch.no_grad():
            return vb.packed_varlen_attn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, causal=causal)

    _lib.profile_reset()
    ms_step = timed(step, args.steps, args.warmup)
    launches = sum(x[2] for x in _lib.profile_read().values())
    launches_per_step = launches // (args.steps + args.warmup)
    ms_fwd = timed(fwd_only, small_steps, 2)
    value = step_flops / (ms_step * 1e-3) / 1e12
    fwd_value = fwd_flops / (ms_fwd * 1e-3) / 1e12

    # ---- per-kernel durations (events around every launch) for the roofline of the top kernel
    _lib.profile_reset()
    _lib.profile_enable(True)
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    _lib.profile_enable(False)
    _lib.profile_reset()
    del q, k, v, do
    torch.cuda.empty_cache()

    # ---- end to end: pinned host -> device, fwd+bwd through the public API, results -> host, on the leading
    # sequences that hold --e2e-fraction of the tokens (the whole batch is 33 GB each way per step).  The
    # slice is cut across ranks like the batch.  Sequences are independent, so a rank's share is cut into
    # groups of sequences, each on its own stream: one group's copies (either direction) run under another
    # group's kernels.  Every byte of the slice's inputs and results crosses the bus inside the timed region.
    e2e = None
    if not args.no_e2e:
        n_e2e, acc = 0, 0
        for a in ql:
            if n_e2e > 0 and acc + a > args.e2e_fraction * Tq:
                break
            acc += a; n_e2e += 1
        eq, ek = ql[:n_e2e], kl[:n_e2e]
        epart = balanced_partition(eq, ek, world, causal)[0] if world > 1 else None
        emine = epart.assignment[rank] if world > 1 else list(range(n_e2e))
        mq, mk = [eq[i] for i in emine], [ek[i] for i in emine]
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        hq, hk, hv, hdo = (torch.randn(T, H, D, generator=g, dtype=torch.float32).to(torch.bfloat16).pin_memory()
                           for T in (sum(mq), sum(mk), sum(mk), sum(mq)))
        ho, hdq, hdk, hdv = (torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv))
        dq_, dk_, dv_, ddo_ = (torch.empty(t.shape, dtype=t.dtype, device=dev) for t in (hq, hk, hv, hdo))
        n_groups = max(1, min(args.e2e_groups, len(mq)))
        groups, tot_q, s0, tq0, tk0 = [], sum(mq), 0, 0, 0
        for gi in range(n_groups):
            s1, tq1, tk1 = s0, tq0, tk0
            target = tot_q * (gi + 1) / n_groups
            while s1 < len(mq) and (tq1 < target or gi == n_groups - 1):
                tq1 += mq[s1]; tk1 += mk[s1]; s1 += 1
            if s1 > s0:
                groups.append({"q": (tq0, tq1), "k": (tk0, tk1), "stream": torch.cuda.Stream(device=dev),
                               "cu_q": lengths_to_cu(mq[s0:s1]).to(dev), "cu_k": lengths_to_cu(mk[s0:s1]).to(dev)})
            s0, tq0, tk0 = s1, tq1, tk1

        def e2e_step():
            cur = torch.cuda.current_stream()
            for gr in groups:
                st = gr["stream"]
                st.wait_stream(cur)
                (q0, q1), (k0, k1) = gr["q"], gr["k"]
                with torch.cuda.stream(st):
                    a, b, c, d = dq_[q0:q1], dk_[k0:k1], dv_[k0:k1], ddo_[q0:q1]
                    a.copy_(hq[q0:q1], non_blocking=True); b.copy_(hk[k0:k1], non_blocking=True)
                    c.copy_(hv[k0:k1], non_blocking=True); d.copy_(hdo[q0:q1], non_blocking=True)
                    a = a.detach().requires_grad_(True); b = b.detach().requires_grad_(True); c = c.detach().requires_grad_(True)
                    o = vb.packed_varlen_attn(a, b, c, cu_seqlens_q=gr["cu_q"], cu_seqlens_k=gr["cu_k"], causal=causal)
                    ga, gb, gc = torch.autograd.grad(o, (a, b, c), d)
                    ho[q0:q1].copy_(o.detach(), non_blocking=True); hdq[q0:q1].copy_(ga, non_blocking=True)
                    hdk[k0:k1].copy_(gb, non_blocking=True); hdv[k0:k1].copy_(gc, non_blocking=True)
            for gr in groups:
                cur.wait_stream(gr["stream"])

        ms_e2e = timed(e2e_step, small_steps, 2)
        e2e_flops = 3.5 * 4.0 * H * D * cells_of(eq, ek, causal)

        def total(x):
            t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return int(t.item())
        h2d = total(sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo)))
        d2h = total(sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv)))
        e2e = {"value": e2e_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "sequence_groups_per_rank": len(groups),
               "config": f"the first {n_e2e} sequences of the batch ({sum(eq)} tokens, {100 * sum(eq) / Tq:.1f}% of its tokens), "
                         f"cut across {world} rank(s); host buffers pinned; bytes are summed over ranks"}
        del hq, hk, hv, hdo, ho, hdq, hdk, hdv, dq_, dk_, dv_, ddo_
        torch.cuda.empty_cache()

    # ---- absorb operator
    absorb = None
    if not args.no_absorb and wl.get("absorb"):
        from oracle import config_lengths
        try:
            name = wl["absorb"]
            aq, ak = config_lengths(name, 0)
            absorb = absorb_leg(dev, aq, ak, 256, 256, small_steps, 3, timed, rank, world, group,
                                f"{name}: {len(aq)} users, q U[1,16], k logU[8,2048], d=256, H=8, D_H=32, bf16; one batch cut "
                                f"across {world} rank(s) by whole users", graph=True, shard_check=True)
        except Exception as e:  # the headline line must still print
            absorb = {"error": str(e)[:300]}
        if world == 1:
            for key, (lens, dq_, dkv_, label) in {
                    "C4": (config_lengths("C4", 0), 256, 256, "C4: 1024 users, q U[1,16], k logU[8,2048], d=256, H=8, D_H=32, bf16"),
                    "production_shape": (production_lengths(0), 968, 216,
                                         "production-like: 1137 users, 97 % with 2048 keys, q 1-18 (mean 5.3), d_q=968, d_kv=216, H=8, D_H=32, bf16")}.items():
                if key == wl["absorb"]:
                    continue
                try:
                    absorb[key] = absorb_leg(dev, lens[0], lens[1], dq_, dkv_, small_steps, 3, timed, rank, world, group, label, graph=True)
                except Exception as e:  # noqa: BLE001
                    absorb[key] = {"error": str(e)[:300]}
    _lib.check_status(dev)
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peaks, peak_src = load_peaks()
        kern = {n: (ms / max(1, nt)) for n, (ms, nt, na) in prof.items() if nt}
        share = {n: ms for n, (ms, nt, na) in prof.items()}
        tot_ms = sum(share.values()) or 1.0
        top = max(share, key=share.get)
        roofline = None
        if top in PRODUCTS:
            algo = PRODUCTS[top] * 2.0 * H * D * my_cells      # this rank's launch
            ach = algo / (kern[top] * 1e-3) / 1e12
            peak = peaks["bf16_tflops_sustained"]
            traffic, traffic_note = None, "no ncu capture on file for this kernel"
            rows = load_dram_traffic().get(top)
            if rows:
                src, nbytes, toks = rows[-1]
                traffic = int(nbytes * (sum(my_ql) / toks))
                traffic_note = (f"ncu capture of {src} ({toks} tokens, H={H}): {nbytes} bytes per launch, scaled by tokens "
                                f"to this launch ({sum(my_ql)} tokens)")
            roofline = {"bound": "tensor", "kernel": top, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                        "frac": ach / peak, "traffic": traffic, "traffic_source": traffic_note,
                        "peak_source": f"{peak_src} sustained bf16 (kernel timed inside a long step)",
                        "avg_launch_ms": kern[top], "share_of_step": share[top] / tot_ms,
                        "algorithmic_flops_per_launch": algo,
                        "step_frac": value / world / peak,
                        "kernel_shares": {n: round(x / tot_ms, 4) for n, x in sorted(share.items(), key=lambda x: -x[1])}}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v_cpu, dt_cpu, sample = cpu_reference_sample(wl, args.ref_cells, threads)
            cpu = {"value": v_cpu, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample, "seconds": dt_cpu}
        compare = None
        if world == 1 and not args.no_compare:
            try:
                r = subprocess.run([sys.executable, os.path.abspath(__file__), "--leg", "compare"], capture_output=True,
                                   text=True, timeout=900)
                last = [l for l in r.stdout.splitlines() if l.startswith("{")]
                compare = json.loads(last[-1]) if last else {"unavailable": (r.stderr or "no output")[-300:]}
            except Exception as e:  # noqa: BLE001
                compare = {"unavailable": str(e)[:300]}
        line = {
            "metric": "varlen-attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": varlen_config(wl, world, part_info),
            "fwd_only": {"value": fwd_value, "unit": "TFLOP/s", "ms": ms_fwd},
            "e2e": e2e, "gpu_launches": int(launches_per_step * args.steps),
            "roofline": roofline, "cpu_baseline": cpu, "absorb": absorb, "vs_reference_gpu": compare, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
