#!/usr/bin/env python
"""Benchmark of the compressed-weight matmul hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

Default workload (N=1): batch-1 decode over every projection of a SmolLM3-3B-shaped model stored as
trellis 3INST at 4 bits per weight — 36 layers x (q, k, v, o, gate, up, down), 1.406 GB of packed
bit-streams, all distinct buffers (far larger than the 126 MB L2, so nothing is re-read from cache
between steps).  One step = one pass over all 252 projections with seeded synthetic bit-streams,
sign vectors, scales and bf16 activations.  The metric is compressed bytes read per second.

With N > 1 every projection is split tensor-parallel (rows of q/k/v/gate/up, columns of o/down, each
shard a GLQ layer of its own) and the o/down outputs are summed with an NCCL all-reduce; the total
work is fixed ("strong" scaling).

`--impl reference` times the CPU restatement of the reference's decode-then-matmul path
(oracle/glq_oracle.c, all host threads) on one decoder layer per step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode matvec compressed-byte HBM GB/s (bs=1)"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# workload construction
# --------------------------------------------------------------------------------------------------
def build_trellis_decode(device, world, rank, bits=(4,), n_layers=None):
    """All projections of the SmolLM3-3B shape as one sweep plan; returns plan + buffers + bookkeeping."""
    import torch
    from glq_b200 import synth
    from glq_b200.plan import Plan

    from glq_b200 import tp

    cfg = synth.SMOLLM3_3B
    gen = torch.Generator(device=device)
    gen.manual_seed(1234 + rank)
    layout = tp.build_layout(cfg["proj"], n_layers or cfg["layers"], world, rank)
    layers, specs = [], []
    for e in layout.entries:
        L = synth.trellis_layer(f"L{e.layer}.{e.name}", e.m, e.n, list(bits), gen, device)
        layers.append(L)
        specs.append(L.spec(batch=1, x_offset=e.x_offset, y_offset=e.y_offset, x_stride=e.n, y_stride=e.m))
    plan = Plan(specs)
    gx = torch.Generator(device=device)
    gx.manual_seed(99)
    x = torch.randn(layout.x_elems, generator=gx, device=device, dtype=torch.float32).to(torch.bfloat16)
    y = torch.zeros(layout.y_elems, device=device, dtype=torch.bfloat16)
    return dict(plan=plan, x=x, y=y, layers=layers, layout=layout,
                code_bytes=plan.code_bytes, name="smollm3-3b trellis-3inst %dbpw decode bs=1" % sum(bits))


WORKLOADS = {
    # name: (model shape, format, bits-or-stages, default tokens, default layers, metric)
    "decode_trellis": ("SMOLLM3_3B", "trellis", (4,), 1, 36, METRIC),
    "decode_trellis_6bpw": ("SMOLLM3_3B", "trellis", (4, 2), 1, 36, METRIC),
    "decode_e8": ("LLAMA3_8B", "e8", 2, 1, 8, METRIC),
    "prefill_e8": ("LLAMA3_8B", "e8", 2, 2048, 2, "prefill TFLOP/s per layer"),
    "prefill_trellis": ("SMOLLM3_3B", "trellis", (4,), 2048, 4, "prefill TFLOP/s per layer"),
    # 62-layer dense decoder (hidden 5376, intermediate 21504): E8 stages cycle 2/3/3 per layer (nominal
    # 4/5/6 bpw; every stage is stored as int16, so the stored rate is 4/6/6 bits per weight)
    "decode_e8_62l": ("DENSE_62L", "e8", [2, 3, 3], 1, 6, METRIC),
    "prefill_e8_62l": ("DENSE_62L", "e8", [2, 3, 3], 2048, 3, "prefill TFLOP/s per layer"),
}


def build_workload(name, device, world, rank, tokens=None, n_layers=None):
    """Plan over n_layers x 7 projections of the named shape; q/k/v and gate/up share their input."""
    import torch
    from glq_b200 import synth, tp
    from glq_b200.plan import Plan

    shape, fmt, par, d_tokens, d_layers, metric = WORKLOADS[name]
    cfg = getattr(synth, shape)
    T = tokens or d_tokens
    nl = n_layers or d_layers
    gen = torch.Generator(device=device)
    gen.manual_seed(4321 + rank)
    table = synth.load_e8_table(device) if fmt == "e8" else None
    col_mult = 8 if fmt == "e8" else 32
    specs, layers = [], []
    x_elems = y_elems = 0
    reduce_spans = []
    pending = []
    for li in range(nl):
        x_of = {}
        for pname, m, n in cfg["proj"]:
            ms, ns = tp.shard_shape(pname, m, n, world, 32 if fmt == "trellis" else 16, col_mult)
            group = {"q": "attn_in", "k": "attn_in", "v": "attn_in", "gate": "mlp_in", "up": "mlp_in"}.get(pname, pname)
            if group not in x_of:
                x_of[group] = x_elems
                x_elems += T * ns
            stages = par[li % len(par)] if isinstance(par, list) else par
            L = (synth.trellis_layer(f"L{li}.{pname}", ms, ns, list(par), gen, device) if fmt == "trellis"
                 else synth.e8_layer(f"L{li}.{pname}", ms, ns, stages, table, gen, device))
            if group == "attn_in" and pname != "q":
                L.sv = layers[-1].sv if pname == "k" else layers[-2].sv      # fused shards share the input signs
            if pname == "up":
                L.sv = layers[-1].sv
            layers.append(L)
            pending.append((L, x_of[group], ns, ms, pname in tp.ROW_PARALLEL))
    # outputs: column-parallel layers first, row-parallel ones as one contiguous tail, so that the partial sums
    # of a step are added over the ranks by ONE all-reduce (the layers of the sweep do not depend on each other)
    y_at = {}
    for want_row in (False, True):
        if want_row:
            tail_begin = y_elems
        for i, (L, xo, ns, ms, is_row) in enumerate(pending):
            if is_row == want_row:
                y_at[i] = y_elems
                y_elems += T * ms
    for i, (L, xo, ns, ms, is_row) in enumerate(pending):
        specs.append(L.spec(batch=T, x_offset=xo, y_offset=y_at[i], x_stride=ns, y_stride=ms))
    if world > 1 and y_elems > tail_begin:
        reduce_spans.append((tail_begin, y_elems - tail_begin))
    plan = Plan(specs)
    gx = torch.Generator(device=device)
    gx.manual_seed(77)
    x = torch.randn(x_elems, generator=gx, device=device, dtype=torch.float32).to(torch.bfloat16)
    y = torch.zeros(y_elems, device=device, dtype=torch.bfloat16)
    return dict(plan=plan, x=x, y=y, layers=layers, layout=None, reduce_spans=reduce_spans, tokens=T, n_layers=nl,
                code_bytes=plan.code_bytes, flops=plan.flops, metric=metric, shape=shape, fmt=fmt, par=par)


def build_moe(device, tokens, skew=None, E=128, top_k=8, hidden=2048, inter=768, bits=(4,), world=1, rank=0):
    """MoE step of BASELINE config 3: 128 experts, top-8, hidden 2048, expert intermediate 768 (gate/up fused
    2048->1536, down 768->2048), trellis 4 bpw, gelu-tanh gating.  Router logits N(0,1) (near-uniform loads) or
    a Zipf(1.2) popularity over experts."""
    import torch
    from glq_b200 import ops
    from glq_b200.plan import block_decompose
    from glq_b200 import tp
    E_all = E
    e0, e1 = tp.expert_range(E_all, world, rank)
    E = e1 - e0                                    # experts held by this rank
    gen = torch.Generator(device=device)
    gen.manual_seed(2025 + rank)                   # weights: every rank its own experts
    ri = lambda *shape: torch.randint(-32768, 32768, shape, generator=gen, device=device, dtype=torch.int32).to(torch.int16)
    sg = lambda *shape: (torch.randint(0, 2, shape, generator=gen, device=device, dtype=torch.int32) * 2 - 1).to(torch.float16)
    K = bits[0]
    w13_out = 2 * inter
    Wt = dict(w13=ri(E, (w13_out // 16) * (hidden // 16), 16 * K), w2=ri(E, (hidden // 16) * (inter // 16), 16 * K),
              su13=sg(E, w13_out), sv13=sg(hidden), su2=sg(E, hidden), sv2=sg(inter),
              ws13=(0.5 + torch.rand(E, generator=gen, device=device)) * 0.02,
              ws2=(0.5 + torch.rand(E, generator=gen, device=device)) * 0.02)
    gen = torch.Generator(device=device)
    gen.manual_seed(77)                            # tokens and routing: replicated on all ranks
    x = torch.randn(tokens, hidden, generator=gen, device=device).to(torch.bfloat16)
    logits = torch.randn(tokens, E_all, generator=gen, device=device)
    if skew:
        ranks = torch.arange(1, E_all + 1, device=device, dtype=torch.float32)
        logits = logits * 0.0 + torch.log(ranks.pow(-skew))[None, :] - torch.log(-torch.log(torch.rand(tokens, E_all, generator=gen, device=device)))
    topw, topi = torch.topk(torch.softmax(logits, -1), top_k, dim=-1)
    topw = (topw / topw.sum(-1, keepdim=True)).float().contiguous()
    sentinel = torch.zeros(E, 1, 1, dtype=torch.int16, device=device)
    bl = lambda n: torch.tensor(block_decompose(n))

    def run_local(xin, ids, tw):
        return ops.fused_moe_trellis_3inst(
            xin, ids, tw, Wt["w13"], sentinel, Wt["su13"], Wt["sv13"], Wt["ws13"], Wt["ws13"],
            Wt["w2"], sentinel, Wt["su2"], Wt["sv2"], Wt["ws2"], Wt["ws2"], hidden, inter, w13_out,
            hidden, w13_out, inter, hidden, bl(hidden), bl(w13_out), None, None, bl(inter), bl(hidden), None, None, 1)

    def run(xin):
        # expert parallel: this rank's experts for all tokens, then one all-reduce of (tokens, hidden)
        return tp.moe_expert_parallel(run_local, xin, topi, topw, E_all)

    code_bytes = (Wt["w13"].numel() * 2 + Wt["w2"].numel() * 2) * world     # all ranks together
    flops = 2 * tokens * top_k * (w13_out * hidden + hidden * inter)
    return dict(run=run, x=x, code_bytes=code_bytes, flops=flops, keep=Wt, tokens=tokens)


def bench_moe(args, device):
    """Separate, simpler driver for the MoE workloads (expert parallel under torchrun): time K steps of the op on resident inputs,
    then with host activations copied in and the result copied out."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    skew = 1.2 if "zipf" in args.workload else None
    T = args.tokens or 256
    W = build_moe(device, T, skew, world=world, rank=rank)
    x = W["x"]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        y = W["run"](x)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        y = W["run"](x)
    e1.record()
    sync()
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop()
    hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True); hx.copy_(x)
    hy = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
    e0.record()
    for _ in range(args.steps):
        x.copy_(hx, non_blocking=True)
        y = W["run"](x)
        hy.copy_(y, non_blocking=True)
    e1.record()
    sync()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    if rank != 0:
        return 0
    peak, kind = measured_peaks()
    peak *= world
    gbs = W["code_bytes"] / (ms * 1e-3) / 1e9
    line = {"metric": "MoE grouped expert matmul: compressed-byte GB/s and TFLOP/s", "value": gbs, "unit": "GB/s",
            "tflops": W["flops"] / (ms * 1e-3) / 1e12, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: 128 experts top-8, hidden 2048, expert intermediate 768, trellis 4 bpw, "
                                   f"{T} tokens, {'Zipf(1.2) expert popularity' if skew else 'near-uniform routing'}",
                       "cache": "302 MB of expert weights per step, larger than L2",
                       "parallelism": f"ep{world}: experts sharded over ranks, one all-reduce of (tokens, hidden)" if world > 1 else "single"},
            "e2e": {"value": W["code_bytes"] / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": x.numel() * 2, "d2h_bytes_per_step": y.numel() * 2},
            "gpu_launches": (6 if T * 8 < 8192 else 8) * args.steps, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "peak_kind": f"of {kind}", "unit": "GB/s",
                         "frac": gbs / peak, "note": "whole step (six kernels, eight from 8192 routings); all expert weights read once"}}
    print(json.dumps(line))
    return 0


def cpu_layer_sample(threads_note=True):
    """One SmolLM3-3B decoder layer (7 projections, 39,059,456 packed bytes) for the CPU restatement."""
    import numpy as np
    from glq_b200 import synth
    rng = np.random.default_rng(0)
    out = []
    for name, m, n in synth.SMOLLM3_3B["proj"]:
        packed = rng.integers(0, 65536, size=((m // 16) * (n // 16), 64), dtype=np.uint16).view(np.int16)
        su = (rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)
        sv = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
        x = rng.standard_normal((1, n)).astype(np.float32)
        out.append((name, m, n, packed, su, sv, x))
    return out


def run_cpu_layer(sample):
    from oracle import c_oracle as CO
    from oracle import glq_oracle as O
    nbytes = 0
    for name, m, n, packed, su, sv, x in sample:
        CO.trellis_linear(x, packed, 4, None, 0, 0.0, m, n, su, sv, 0.02, O.block_decompose(n), O.block_decompose(m))
        nbytes += packed.nbytes
    return nbytes


def cpu_baseline(budget_s=12.0):
    sample = cpu_layer_sample()
    run_cpu_layer(sample)                      # warm-up (builds the library on first use)
    t0 = time.perf_counter()
    reps, nbytes = 0, 0
    while True:
        nbytes += run_cpu_layer(sample)
        reps += 1
        if time.perf_counter() - t0 >= budget_s or reps >= 64:
            break
    dt = time.perf_counter() - t0
    threads = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{reps} x one SmolLM3-3B decoder layer (7 projections, {nbytes // reps} packed bytes), "
                      "decode + fp32 matvec + Hadamard transforms, oracle/glq_oracle.c with OpenMP"}


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode_trellis_sweep",
                    help="decode_trellis_sweep (default, the headline) or one of: " + ", ".join(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None,
                    help="decoder layers to build (default: all 36); smaller values are for profiler captures only")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "trellis 3INST 4 bpw decode matvec, batch 1, SmolLM3-3B projections "
                          "(36 layers x q/k/v/o/gate/up/down), L=16 K=4, 16x16 tiles",
              "cache": "inputs larger than L2 (1.4 GB of distinct packed weights per step)",
              "parallelism": f"tp{args.gpus}" if args.gpus > 1 else "single"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        # torchrun exports OMP_NUM_THREADS=1 to every worker; the CPU arm is meant to use all host threads
        # (the OpenMP runtime reads the variable when the oracle library is loaded, which happens below)
        if world > 1 and os.environ.get("OMP_NUM_THREADS") == "1":
            os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
        sample = cpu_layer_sample()
        for _ in range(max(1, min(args.warmup, 3))):
            run_cpu_layer(sample)
        t0 = time.perf_counter()
        nbytes = 0
        for _ in range(args.steps):
            nbytes += run_cpu_layer(sample)
        dt = time.perf_counter() - t0
        v = nbytes / dt / 1e9
        threads = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
                "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                                 "sample": "each step = one SmolLM3-3B decoder layer (7 projections, 39,059,456 packed "
                                           "bytes): decode + fp32 matvec + Hadamard transforms on the host cores"},
                "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in glq_b200)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.workload.startswith("moe"):
        return bench_moe(args, device)
    generic = args.workload != "decode_trellis_sweep"
    if generic:
        W = build_workload(args.workload, device, world, rank, args.tokens, args.layers)
        config = {"workload": f"{args.workload}: {W['shape']} projections, {W['fmt']} {W['par']}, {W['tokens']} tokens, "
                              f"{W['n_layers']} decoder layers per step (weights {W['code_bytes'] / 1e6:.0f} MB, cycled)",
                  "cache": "distinct weight buffers per layer; working set larger than L2",
                  "parallelism": f"tp{args.gpus}" if args.gpus > 1 else "single"}
    else:
        W = build_trellis_decode(device, world, rank, n_layers=args.layers)
        if args.layers:
            config["layers_built"] = args.layers
    plan, x, y = W["plan"], W["x"], W["y"]
    total_code_bytes = W["code_bytes"]
    total_flops = W.get("flops", 0)
    if world > 1:
        t = torch.tensor([total_code_bytes, total_flops], device=device, dtype=torch.int64)
        dist.all_reduce(t)
        total_code_bytes, total_flops = int(t[0].item()), int(t[1].item())

    from glq_b200 import tp

    def step():
        plan.run(x, y)
        # row-parallel outputs (o, down) are partial sums over ranks: one NCCL all-reduce over the
        # contiguous tail of y (the sweep has no dependency between layers, so the per-layer
        # reductions of a real decode step are issued as one)
        if W["layout"] is not None:
            tp.all_reduce_row_parallel(y, W["layout"])
        elif world > 1:
            for off, ln in W["reduce_spans"]:
                dist.all_reduce(y[off:off + ln])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    plan.set_timing(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync()
    ms_total = e0.elapsed_time(e1)
    kern_ms, kern_runs = plan.kernel_ms()
    plan.set_timing(False)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = total_code_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end: host buffers in, host buffers out, through the same public call
    hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    hx.copy_(x)
    hy = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
    for _ in range(3):
        x.copy_(hx, non_blocking=True); step(); hy.copy_(y, non_blocking=True)
    sync()
    e0.record()
    for _ in range(args.steps):
        x.copy_(hx, non_blocking=True)
        step()
        hy.copy_(y, non_blocking=True)
    e1.record()
    sync()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = total_code_bytes / (e2e_ms / args.steps * 1e-3) / 1e9

    if rank == 0:
        peak, peak_kind = measured_peaks()
        kern_ms_avg = kern_ms / max(1, kern_runs)
        achieved = W["code_bytes"] / (kern_ms_avg * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": x.numel() * x.element_size(),
                    "d2h_bytes_per_step": y.numel() * y.element_size()},
            "gpu_launches": plan.launches * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "trellis_mv_kernel<4,0,1>", "achieved": achieved, "peak": peak,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "kernel_ms": kern_ms_avg, "bytes_per_launch": W["code_bytes"],
                         # dram__bytes_read+write of one launch: captured with ncu on the 4-layer case
                         # (160.9 MB for 156.2 MB of packed bytes, profiles/trellis_mv_kernel_decode_smollm3.md)
                         # and scaled by the packed bytes of this launch (traffic grows with the layers read)
                         "traffic": int(W["code_bytes"] * 160.93 / 156.24) if not generic else None},
        }
        if generic and "prefill" in args.workload:
            # per-layer TFLOP/s, against the bf16 tensor peak
            flops_layer = total_flops / W["n_layers"]          # all ranks
            tf = flops_layer / (ms_step / W["n_layers"] * 1e-3) / 1e12
            tf_kernel = W["flops"] / (kern_ms_avg * 1e-3) / 1e12
            try:
                tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
                tkind = "of measured"
            except Exception:
                tpeak, tkind = 1590.0, "of fallback"
            line.update({"metric": W["metric"], "value": tf, "unit": "TFLOP/s", "dtype": "f16",
                         "ms_per_layer": ms_step / W["n_layers"]})
            line["e2e"]["value"] = flops_layer / (e2e_ms / args.steps / W["n_layers"] * 1e-3) / 1e12
            line["e2e"]["unit"] = "TFLOP/s"
            kname = "glq_gemm_kernel"
            if W["fmt"] == "e8" and W["tokens"] >= 129:
                kname = "e8_tiles_kernel + glq_gemm_kernel (weight tiles decoded once, then the copy-fed GEMM)"
            line["roofline"] = {"bound": "tensor", "kernel": kname, "achieved": tf_kernel, "peak": tpeak,
                                "peak_kind": tkind, "unit": "TFLOP/s", "frac": tf_kernel / tpeak,
                                "kernel_ms": kern_ms_avg, "flops_per_launch": W["flops"], "traffic": None}
        elif generic:
            line["metric"] = W["metric"]
        if args.gpus == 1 and not args.no_cpu_baseline and not generic:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
