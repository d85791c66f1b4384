#!/usr/bin/env python
"""Benchmark of the compressed-weight matmul hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME] [--no-subs]

Headline workload (the JSON line's `value`): batch-1 decode over every projection of a SmolLM3-3B-shaped
model stored as trellis 3INST at 4 bits per weight — 36 layers x (q, k, v, o, gate, up, down), 1.406 GB of
packed bit-streams, all distinct buffers (far larger than the 126 MB L2, so nothing is re-read from cache
between steps).  One step = one pass over all 252 projections with seeded synthetic bit-streams, sign
vectors, scales and bf16 activations.  The metric is compressed bytes read per second.

The same line carries, under "sub", one record per other benchmark configuration (each with its own
roofline and end-to-end figure): E8 two-stage decode (1 and 16 tokens) and prefill (256 and 2048 tokens) on
Llama-3-8B shapes, trellis prefill, the 128-expert MoE step (256 and 4096 tokens, near-uniform and Zipf
routing), the 62-layer mixed-rate E8 shapes, a dependent decode chain through the operator layer, and the
latency of one 2048 x 2048 linear.  `--workload NAME` runs one of them alone; `--no-subs` only the headline.

With N > 1 every projection is split tensor-parallel (rows of q/k/v/gate/up, columns of o/down, each shard
a GLQ layer of its own); the row-parallel outputs are fp32 partial sums added over the ranks with NCCL, and
after the timed region one layer's per-rank partials are gathered and summed in rank order to check the
reduced output ("tp_check").  MoE is expert-parallel.  Total work is fixed ("strong" scaling).

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
PREFILL_METRIC = "prefill TFLOP/s per layer"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0


def measured_peaks():
    """(hbm GB/s, bf16 TFLOP/s burst, 'measured' | 'fallback')"""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


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
# distributed helpers
# --------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self, device):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.device = device

    def sync(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, v: float) -> float:
        if self.world == 1:
            return v
        import torch
        import torch.distributed as dist
        t = torch.tensor([v], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_int(self, *vals):
        if self.world == 1:
            return [int(v) for v in vals]
        import torch
        import torch.distributed as dist
        t = torch.tensor(list(vals), device=self.device, dtype=torch.int64)
        dist.all_reduce(t)
        return [int(v) for v in t.tolist()]


def timed(D: Dist, step, steps: int, before=None, after=None):
    """K steps bracketed by a barrier + synchronize on both sides; CUDA events on the current stream; max over
    ranks.  `before` / `after` run inside the timed region around every step (host<->device copies)."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    D.sync()
    e0.record()
    for _ in range(steps):
        if before:
            before()
        step()
        if after:
            after()
    e1.record()
    D.sync()
    return D.max(e0.elapsed_time(e1)) / steps


# --------------------------------------------------------------------------------------------------
# workloads built from plans of independent linears
# --------------------------------------------------------------------------------------------------
WORKLOADS = {
    # name: (model shape, format, bits-or-stages, default tokens, default layers, metric)
    "decode_trellis_sweep": ("SMOLLM3_3B", "trellis", (4,), 1, 36, METRIC),
    "decode_trellis": ("SMOLLM3_3B", "trellis", (4,), 1, 36, METRIC),
    "decode_trellis_6bpw": ("SMOLLM3_3B", "trellis", (4, 2), 1, 36, METRIC),
    "decode_e8": ("LLAMA3_8B", "e8", 2, 1, 8, METRIC),
    "prefill_e8": ("LLAMA3_8B", "e8", 2, 2048, 2, PREFILL_METRIC),
    "prefill_trellis": ("SMOLLM3_3B", "trellis", (4,), 2048, 4, PREFILL_METRIC),
    # 62-layer dense decoder (hidden 5376, intermediate 21504): E8 stages cycle 2/3/3 per layer (nominal
    # 4/5/6 bpw; every stage is stored as int16, so the stored rate is 4/6/6 bits per weight)
    "decode_e8_62l": ("DENSE_62L", "e8", [2, 3, 3], 1, 6, METRIC),
    "prefill_e8_62l": ("DENSE_62L", "e8", [2, 3, 3], 2048, 3, PREFILL_METRIC),
}


def build_workload(name, device, world, rank, tokens=None, n_layers=None):
    """Plan over n_layers x 7 projections of the named shape.  In the sweep every projection has its own input;
    elsewhere q/k/v and gate/up share theirs.  Column-parallel outputs are bf16; row-parallel outputs (o, down)
    are fp32 partial sums in one contiguous tail of the result buffer, added over the ranks by one all-reduce
    (the layers of a step do not depend on each other)."""
    import torch
    from glq_b200 import synth, tp
    from glq_b200.plan import Plan

    shape, fmt, par, d_tokens, d_layers, metric = WORKLOADS[name]
    cfg = getattr(synth, shape)
    T = tokens or d_tokens
    nl = n_layers or d_layers
    sweep = name == "decode_trellis_sweep"
    gen = torch.Generator(device=device)
    gen.manual_seed((1234 if sweep else 4321) + rank)
    table = synth.load_e8_table(device) if fmt == "e8" else None
    col_mult = 8 if fmt == "e8" else 32
    layers, pending = [], []
    x_elems = 0
    for li in range(nl):
        x_of = {}
        for pname, m, n in cfg["proj"]:
            ms, ns = tp.shard_shape(pname, m, n, world, 32 if fmt == "trellis" else 16, col_mult)
            group = pname if sweep else {"q": "attn_in", "k": "attn_in", "v": "attn_in", "gate": "mlp_in",
                                         "up": "mlp_in"}.get(pname, pname)
            if group not in x_of:
                x_of[group] = x_elems
                x_elems += T * ns
            stages = par[li % len(par)] if isinstance(par, list) else par
            L = (synth.trellis_layer(f"L{li}.{pname}", ms, ns, list(par), gen, device) if fmt == "trellis"
                 else synth.e8_layer(f"L{li}.{pname}", ms, ns, stages, table, gen, device))
            if not sweep:
                if group == "attn_in" and pname != "q":
                    L.sv = layers[-1].sv if pname == "k" else layers[-2].sv      # fused shards share the input signs
                if pname == "up":
                    L.sv = layers[-1].sv
            layers.append(L)
            pending.append((L, x_of[group], ns, ms, pname in tp.ROW_PARALLEL and world > 1, pname))
    # result buffer (bytes): bf16 outputs first, then the fp32 partial sums of the row-parallel layers
    col_bytes = sum(T * ms * 2 for (_, _, _, ms, rp, _) in pending if not rp)
    col_bytes = (col_bytes + 255) // 256 * 256
    row_bytes = sum(T * ms * 4 for (_, _, _, ms, rp, _) in pending if rp)
    y = torch.zeros(col_bytes + row_bytes, device=device, dtype=torch.uint8)
    specs, y_at = [], []
    c_off, r_off = 0, col_bytes
    for (L, xo, ns, ms, rp, pname) in pending:
        if rp:
            specs.append(L.spec(batch=T, x_offset=xo, y_offset=r_off // 4, x_stride=ns, y_stride=ms, y_dtype=torch.float32))
            y_at.append((r_off, T * ms * 4, True))
            r_off += T * ms * 4
        else:
            specs.append(L.spec(batch=T, x_offset=xo, y_offset=c_off // 2, x_stride=ns, y_stride=ms))
            y_at.append((c_off, T * ms * 2, False))
            c_off += T * ms * 2
    plan = Plan(specs)
    gx = torch.Generator(device=device)
    gx.manual_seed(99 if sweep else 77)
    x = torch.randn(x_elems, generator=gx, device=device, dtype=torch.float32).to(torch.bfloat16)
    reduce_view = y[col_bytes:].view(torch.float32) if row_bytes else None
    return dict(plan=plan, x=x, y=y, layers=layers, specs=specs, pending=pending, y_at=y_at, reduce_view=reduce_view,
                tokens=T, n_layers=nl, code_bytes=plan.code_bytes, flops=plan.flops, metric=metric, shape=shape,
                fmt=fmt, par=par)


def kernel_name(W):
    """The kernel the plan's timing events bracket (what `roofline` describes)."""
    T, fmt, par = W["tokens"], W["fmt"], W["par"]
    ns = max(par) if isinstance(par, list) else par
    if T > 64:
        tn = 128 if T <= 128 else 256
        if fmt == "trellis":
            return f"glq_gemm_kernel<trellis,{par[0]},{par[1] if len(par) > 1 else 0},{tn},4>"
        if T >= 129:
            return f"e8_tiles_smem_kernel<{ns}> + glq_gemm_kernel<tiles,{tn},4> (weight tiles decoded once, then the copy-fed GEMM)"
        return f"glq_gemm_kernel<e8,{ns},{tn},4>"
    nb = 1 if T <= 8 else 2 if T <= 16 else 4 if T <= 32 else 8
    if fmt == "trellis":
        # large single-stage batch-1 launches take the table form (two of eight states per lane looked up)
        lut = nb == 1 and len(par) == 1 and W["code_bytes"] >= int(os.environ.get("GLQB_TRELLIS_LUT_MIN_BYTES", str(48 << 20)))
        return f"trellis_mv_kernel<{par[0]},{par[1] if len(par) > 1 else 0},{nb}{',2' if lut else ''}>"
    resident = W["code_bytes"] >= int(os.environ.get("GLQB_E8_SMEM_MIN_BYTES", str(48 << 20))) and nb <= 2
    return f"e8_mv_smem_kernel<{ns},{nb}>" if resident else f"e8_mv_kernel<{ns},{nb}>"


_COMM = {}


def rank_comm(D: Dist):
    """The communicator of the library's own sums over ranks (glq_b200.comm), built once per process; None (and the
    reason in _COMM["why"]) when the peers' memory cannot be mapped here, in which case NCCL does the sums."""
    if "c" not in _COMM:
        _COMM["c"], _COMM["why"] = None, None
        if D.world > 1 and os.environ.get("GLQB_BENCH_NCCL") != "1":
            try:
                from glq_b200.comm import Comm
                _COMM["c"] = Comm.from_process_group(max_floats=1 << 20, device=D.device)
            except Exception as e:          # e.g. CUDA IPC closed to this container
                _COMM["why"] = f"{type(e).__name__}: {e}"
        elif D.world > 1:
            _COMM["why"] = "GLQB_BENCH_NCCL=1"
    return _COMM["c"]


def tp_check(D: Dist, W):
    """One row-parallel layer: every rank's fp32 partial is gathered, the partials are added in rank order
    0..G-1, and the all-reduced output must equal that sum within 2e-3 of its largest value."""
    import torch
    import torch.distributed as dist
    if D.world == 1 or W["reduce_view"] is None:
        return None
    from glq_b200.plan import Plan
    i = next(k for k, p in enumerate(W["pending"]) if p[4])
    L, xo, ns, ms, _, pname = W["pending"][i]
    T = W["tokens"]
    part = torch.zeros(T * ms, dtype=torch.float32, device=D.device)
    one = Plan([L.spec(batch=T, x_offset=xo, y_offset=0, x_stride=ns, y_stride=ms, y_dtype=torch.float32)])
    one.run(W["x"], part)
    parts = [torch.empty_like(part) for _ in range(D.world)]
    dist.all_gather(parts, part)
    fixed = torch.zeros_like(part)
    for p in parts:                       # rank order
        fixed += p
    off, nbytes, _ = W["y_at"][i]
    got = W["y"][off:off + nbytes].view(torch.float32)
    err = ((got - fixed).abs().max() / fixed.abs().max().clamp_min(1e-30)).item()
    one.close()
    return {"layer": pname, "max_rel_diff": err, "result": "ok" if err <= 2e-3 else "FAILED"}


def run_plan_bench(name, D: Dist, args, steps, tokens=None, layers=None, clocks=False, check=False):
    import torch
    import torch.distributed as dist
    W = build_workload(name, D.device, D.world, D.rank, tokens, layers)
    plan, x, y = W["plan"], W["x"], W["y"]
    code_bytes, flops = D.sum_int(W["code_bytes"], W["flops"])

    comm = rank_comm(D) if W["reduce_view"] is not None else None
    if comm is not None and W["reduce_view"].numel() > comm.max_floats:
        comm = None                                   # prefill-sized sums stay with NCCL

    def step():
        plan.run(x, y)
        if W["reduce_view"] is not None:
            if comm is not None:
                comm.all_reduce_(W["reduce_view"])    # one launch: stores into every rank's area, flags, fixed-order sum
            else:
                dist.all_reduce(W["reduce_view"])

    for _ in range(max(args.warmup, 3)):
        step()
    D.sync()
    sampler = ClockSampler(D.device.index or 0) if (clocks and D.rank == 0) else None
    if sampler:
        sampler.start()
    plan.set_timing(True)
    ms_step = timed(D, step, steps)
    kern_ms, kern_runs = plan.kernel_ms()
    plan.set_timing(False)
    clock_rec = sampler.stop() if sampler else None
    checked = tp_check(D, W) if check else None

    hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    hx.copy_(x)
    hy = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
    for _ in range(2):
        x.copy_(hx, non_blocking=True); step(); hy.copy_(y, non_blocking=True)
    ms_e2e = timed(D, step, steps, before=lambda: x.copy_(hx, non_blocking=True),
                   after=lambda: hy.copy_(y, non_blocking=True))
    hbm, tens, kind = measured_peaks()
    kern_ms_avg = D.max(kern_ms / max(1, kern_runs))
    prefill = W["metric"] == PREFILL_METRIC
    nl = W["n_layers"]
    rec = {"workload": name, "metric": W["metric"], "ms_per_step": ms_step, "n_gpus": D.world,
           "config": f"{W['shape']} projections, {W['fmt']} {W['par']}, {W['tokens']} tokens, {nl} decoder layers per step "
                     f"({code_bytes / 1e6:.0f} MB of codes, distinct buffers, larger than L2)",
           "gpu_launches": plan.launches * steps}
    if prefill:
        rec.update({"value": flops / nl / (ms_step / nl * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_layer": ms_step / nl,
                    "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                            "h2d_bytes_per_step": x.numel() * x.element_size(), "d2h_bytes_per_step": y.numel()},
                    "roofline": {"bound": "tensor", "kernel": kernel_name(W), "achieved": W["flops"] / (kern_ms_avg * 1e-3) / 1e12,
                                 "peak": tens, "peak_kind": f"of {kind}", "unit": "TFLOP/s",
                                 "frac": W["flops"] / (kern_ms_avg * 1e-3) / 1e12 / tens, "kernel_ms": kern_ms_avg,
                                 "flops_per_launch": W["flops"], "whole_step_frac": flops / (ms_step * 1e-3) / 1e12 / (tens * D.world),
                                 "traffic": None}})
    else:
        ach = W["code_bytes"] / (kern_ms_avg * 1e-3) / 1e9
        rec.update({"value": code_bytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
                    "e2e": {"value": code_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                            "h2d_bytes_per_step": x.numel() * x.element_size(), "d2h_bytes_per_step": y.numel()},
                    "roofline": {"bound": "hbm", "kernel": kernel_name(W), "achieved": ach, "peak": hbm,
                                 "peak_kind": f"of {kind}", "unit": "GB/s", "frac": ach / hbm, "kernel_ms": kern_ms_avg,
                                 "bytes_per_launch": W["code_bytes"],
                                 # dram bytes of one launch, from an ncu capture of the 4-layer case scaled by the
                                 # packed bytes of this launch (160.9 MB for 156.2 MB of codes; traffic grows with
                                 # the layers read); only captured for the trellis sweep
                                 "traffic": int(W["code_bytes"] * 160.93 / 156.24) if name.startswith("decode_trellis") and len(W["par"]) == 1 else None}})
    if clock_rec:
        rec["clocks"] = clock_rec
    if checked:
        rec["tp_check"] = checked
    if W["reduce_view"] is not None:
        rec["rank_sum"] = ("glqb_comm_all_reduce (one launch, NVLink stores, fixed rank order)" if comm is not None
                           else "ncclAllReduce" + (f" ({_COMM.get('why')})" if _COMM.get("why") else " (message larger than the communicator's area)"))
        if comm is not None:
            comm.check_status()
    plan.close()
    del W, plan, x, y
    torch.cuda.empty_cache()
    return rec


# --------------------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------------------
def build_moe(device, tokens, skew=None, E=128, top_k=8, hidden=2048, inter=768, bits=(4,), world=1, rank=0, comm=None):
    """MoE step of the benchmark configuration: 128 experts, top-8, hidden 2048, expert intermediate 768 (gate/up
    fused 2048->1536, down 768->2048), trellis 4 bpw, gelu-tanh gating.  Router logits N(0,1) (near-uniform
    loads) or a Zipf(1.2) popularity over experts.  Expert parallel: fp32 partial results, one all-reduce."""
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
    odt = torch.float32 if world > 1 else None

    def run_local(xin, ids, tw):
        return ops.fused_moe_trellis_3inst(
            xin, ids, tw, Wt["w13"], sentinel, Wt["su13"], Wt["sv13"], Wt["ws13"], Wt["ws13"],
            Wt["w2"], sentinel, Wt["su2"], Wt["sv2"], Wt["ws2"], Wt["ws2"], hidden, inter, w13_out,
            hidden, w13_out, inter, hidden, bl(hidden), bl(w13_out), None, None, bl(inter), bl(hidden), None, None, 1,
            out_dtype=odt)

    def run(xin):
        # expert parallel: this rank's experts for all tokens, then one all-reduce of (tokens, hidden)
        return tp.moe_expert_parallel(run_local, xin, topi, topw, E_all, comm=comm)

    code_bytes = (Wt["w13"].numel() * 2 + Wt["w2"].numel() * 2) * world     # all ranks together
    flops = 2 * tokens * top_k * (w13_out * hidden + hidden * inter)
    return dict(run=run, x=x, code_bytes=code_bytes, flops=flops, keep=Wt, tokens=tokens)


def run_moe_bench(name, D: Dist, args, steps, tokens=None):
    import torch
    from glq_b200 import ops
    skew = 1.2 if "zipf" in name else None
    T = tokens or 256
    W = build_moe(D.device, T, skew, world=D.world, rank=D.rank, comm=rank_comm(D))
    x = W["x"]
    for _ in range(max(args.warmup, 3)):
        y = W["run"](x)
    D.sync()
    plans = [p for p in ops._PLAN_CACHE.values() if isinstance(p, ops.MoePlan)]
    for p in plans:
        p.set_timing(True)
    ms = timed(D, lambda: W["run"](x), steps)
    kern_ms = sum(p.kernel_ms()[0] for p in plans) / steps
    for p in plans:
        p.set_timing(False)
    kern_ms = D.max(kern_ms)
    hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True); hx.copy_(x)
    hy = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
    box = {}

    def step():
        box["y"] = W["run"](x)
    ms_e2e = timed(D, step, steps, before=lambda: x.copy_(hx, non_blocking=True),
                   after=lambda: hy.copy_(box["y"], non_blocking=True))
    hbm, tens, kind = measured_peaks()
    gbs = W["code_bytes"] / (ms * 1e-3) / 1e9
    tf = W["flops"] / (ms * 1e-3) / 1e12
    gemm = T * 8 >= 128 * 64
    rec = {"workload": name, "metric": "MoE grouped expert matmul: compressed-byte GB/s and TFLOP/s", "value": gbs,
           "unit": "GB/s", "tflops": tf, "ms_per_step": ms, "n_gpus": D.world,
           "config": f"128 experts top-8, hidden 2048, expert intermediate 768, trellis 4 bpw, {T} tokens, "
                     f"{'Zipf(1.2) expert popularity' if skew else 'near-uniform routing'}; 302 MB of expert weights, larger than L2"
                     + (f"; ep{D.world}: experts sharded over ranks, one fp32 sum of (tokens, hidden) over the ranks "
                        f"({'glqb_comm_all_reduce' if (rank_comm(D) is not None and T * 2048 <= min(rank_comm(D).max_floats, 1 << 18)) else 'ncclAllReduce'})" if D.world > 1 else ""),
           "e2e": {"value": W["code_bytes"] / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                   "h2d_bytes_per_step": x.numel() * 2, "d2h_bytes_per_step": hy.numel() * hy.element_size()},
           "gpu_launches": (6 if T * 8 < 8192 else 8) * steps}
    if gemm:     # tensor-core form: the two grouped GEMMs against the tensor peak
        ach = W["flops"] / D.world / (kern_ms * 1e-3) / 1e12
        rec["roofline"] = {"bound": "tensor", "kernel": "glq_gemm_kernel<trellis,4,0,128,4> (w13 + w2 grouped GEMMs)",
                           "achieved": ach, "peak": tens, "peak_kind": f"of {kind}", "unit": "TFLOP/s", "frac": ach / tens,
                           "kernel_ms": kern_ms, "flops_per_launch": W["flops"] // D.world,
                           "whole_step_frac": tf / (tens * D.world), "traffic": None}
    else:        # streaming form: expert codes read once by the two grouped decode kernels
        ach = W["code_bytes"] / D.world / (kern_ms * 1e-3) / 1e9
        rec["roofline"] = {"bound": "hbm", "kernel": "trellis_moe_mv_kernel<4,0,4> (w13 + w2)", "achieved": ach, "peak": hbm,
                           "peak_kind": f"of {kind}", "unit": "GB/s", "frac": ach / hbm, "kernel_ms": kern_ms,
                           "bytes_per_launch": W["code_bytes"] // D.world, "whole_step_frac": gbs / (hbm * D.world),
                           "traffic": None}
    ops.clear_caches()
    del W
    torch.cuda.empty_cache()
    return rec


# --------------------------------------------------------------------------------------------------
# dependent chain through the operator layer, and the latency of one linear
# --------------------------------------------------------------------------------------------------
def run_chain_bench(D: Dist, args, steps, n_layers=36, e8=False, dense62=False):
    """Batch-1 decode where every projection consumes the previous output, through glq_b200.ops (the calls a
    drop-in user makes), captured in one CUDA graph: per layer  qkv(h) -> o(attention stand-in) -> residual ->
    gate/up(h) -> silu(gate) * up -> down -> residual.  SmolLM3-3B shapes, trellis 4 bpw.  The attention itself
    is replaced by a shape-correct stand-in (the first 2048 of the qkv outputs), the metric counts the linears'
    compressed bytes.  Tensor parallel ranks all-reduce after o and down (fp32), as a served model does."""
    import torch
    import torch.distributed as dist
    from glq_b200 import ops, synth, tp
    cfg = synth.DENSE_62L if dense62 else synth.LLAMA3_8B if e8 else synth.SMOLLM3_3B
    stage_cycle = [2, 3, 3] if dense62 else [2]          # nominal 4 / 5 / 6 bpw
    dev = D.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(555 + D.rank)
    shapes = {p: tp.shard_shape(p, m, n, D.world, 16 if e8 else 32, 8 if e8 else 32) for p, m, n in cfg["proj"]}
    Ls = []
    table = synth.load_e8_table(dev) if e8 else None
    cb16 = None
    if e8:
        # the operator functions take the fp16 codebook the reference passes around; they pack it once
        import numpy as np
        nib = table.cpu().numpy().astype(np.uint32)
        cb16 = torch.from_numpy((((nib[:, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).astype(np.float32) * 0.5 - 3.0)
                                .astype(np.float16)).to(dev)
    for li in range(n_layers):
        if e8:
            d = {p: synth.e8_layer(f"L{li}.{p}", *shapes[p], stage_cycle[li % len(stage_cycle)], table, gen, dev) for p, _, _ in cfg["proj"]}
        else:
            d = {p: synth.trellis_layer(f"L{li}.{p}", *shapes[p], [4], gen, dev) for p, _, _ in cfg["proj"]}
        d["k"].sv = d["v"].sv = d["q"].sv
        d["up"].sv = d["gate"].sv
        Ls.append(d)
    code_bytes = sum(L.code_bytes() for d in Ls for L in d.values())
    hidden = cfg["hidden"]
    h0 = torch.randn(1, hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.bfloat16)
    world = D.world

    norm1 = [torch.ones(hidden, device=dev, dtype=torch.bfloat16) for _ in Ls]
    norm2 = [torch.ones(hidden, device=dev, dtype=torch.bfloat16) for _ in Ls]

    comm = rank_comm(D)

    ei = torch.empty(0, dtype=torch.int16, device=dev)
    eh = torch.empty(0, dtype=torch.float16, device=dev)

    def lin(L, x, **kw):
        if e8:
            tail = []
            for st in range(1, 4):
                tail += [L.codes[st], cb16, L.stage_scale[st - 1]] if st < len(L.codes) else [ei, eh, 0.0]
            return ops.fused_linear_block_diag(x, L.sv, L.su, L.codes[0], cb16, L.wscale, L.n, L.m, L.n, L.m, None, None, None, None,
                                               *tail, **kw)
        return ops.fused_linear_trellis_3inst(x, L.sv, L.su, L.codes[0], None, None, None, None, L.wscale,
                                              L.n, L.m, L.n, L.m, **kw)

    def shards(x, group, norm_w):
        if e8:
            return ops.fused_linear_e8_shards(x, group[0].sv, [(L.su, L.codes, L.stage_scale, L.wscale, L.m) for L in group], cb16,
                                              in_norm_weight=norm_w, in_norm_eps=1e-6)
        return ops.fused_linear_trellis_3inst_shards(x, group[0].sv, [(L.su, L.codes[0], None, L.wscale, 0.0, L.m) for L in group],
                                                     in_norm_weight=norm_w, in_norm_eps=1e-6)

    def forward(h0_):
        h = h0_.clone()
        for d, w1, w2 in zip(Ls, norm1, norm2):
            qkv = shards(h, (d["q"], d["k"], d["v"]), w1)             # RMSNorm + q/k/v: one launch
            a = qkv[:, :d["q"].m]                                     # attention stand-in: a view, (1, 2048 / world)
            if world == 1:
                lin(d["o"], a, accumulate_into=h)                     # o projection + residual add: one launch
            elif comm is not None:
                lin(d["o"], a, accumulate_into=h, reduce_over=comm)   # ... and the sum over ranks, same launch
            else:
                o = lin(d["o"], a, out_dtype=torch.float32)
                dist.all_reduce(o)
                h.add_(o.to(h.dtype))
            gu = shards(h, (d["gate"], d["up"]), w2)                  # RMSNorm + gate/up: one launch
            if world == 1:
                lin(d["down"], gu, gated_act=0, accumulate_into=h)    # silu(gate) * up + down + residual: one launch
            elif comm is not None:
                lin(d["down"], gu, gated_act=0, accumulate_into=h, reduce_over=comm)
            else:
                dn = lin(d["down"], gu, gated_act=0, out_dtype=torch.float32)
                dist.all_reduce(dn)
                h.add_(dn.to(h.dtype))
        return h

    for _ in range(3):
        out = forward(h0)
    D.sync()
    graph = None
    if world == 1 or comm is not None:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = forward(h0)
            graph = g
        except Exception:
            graph = None
            torch.cuda.synchronize()
    step = (lambda: graph.replay()) if graph is not None else (lambda: forward(h0))
    for _ in range(3):
        step()
    ms = timed(D, step, steps)
    hh = torch.empty(h0.shape, dtype=h0.dtype, pin_memory=True); hh.copy_(h0)
    ho = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
    ms_e2e = timed(D, step, steps, before=lambda: h0.copy_(hh, non_blocking=True),
                   after=lambda: ho.copy_(out, non_blocking=True))
    hbm, tens, kind = measured_peaks()
    total_bytes = D.sum_int(code_bytes)[0]
    gbs = total_bytes / (ms * 1e-3) / 1e9
    glq_launches = sum(p.launches for p in ops._PLAN_CACHE.values() if hasattr(p, "launches"))
    model = ("decoder layers of the 62-layer dense shape (hidden 5376, intermediate 21504), E8 shell 2 / 3 / 3 stages" if dense62 else
             "Llama-3-8B decoder layers, E8 shell two-stage (4 bpw)" if e8 else "SmolLM3-3B decoder layers, trellis 4 bpw")
    rec = {"workload": "decode_chain_62l" if dense62 else "decode_chain_e8" if e8 else "decode_chain", "metric": METRIC, "value": gbs, "unit": "GB/s", "ms_per_step": ms, "n_gpus": world,
           "us_per_layer": ms * 1e3 / n_layers, "us_per_linear": ms * 1e3 / (7 * n_layers),
           "config": f"{n_layers} {model}, batch 1, every projection consumes the previous "
                     f"output through glq_b200.ops: per layer RMSNorm + q/k/v, o + residual, RMSNorm + gate/up, "
                     f"silu(gate) * up + down + residual as four calls (attention replaced by a view of the q output; "
                     f"{'one CUDA graph' if graph is not None else 'eager launches'}); "
                     f"{total_bytes / 1e6:.0f} MB of codes per step, larger than L2"
                     + ((f"; tp{world}: o and down summed over the ranks inside their decode kernels (glq_b200.comm)" if comm is not None
                         else f"; tp{world}: fp32 NCCL all-reduce after o and down ({_COMM.get('why')})") if world > 1 else ""),
           "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h0.numel() * 2,
                   "d2h_bytes_per_step": out.numel() * 2},
           "gpu_launches": glq_launches * steps, "glq_launches_per_layer": glq_launches / n_layers,
           "roofline": {"bound": "hbm", "kernel": ("whole chain: e8_fused_kernel for the launches of up to 16 MB of indices, rht_in + e8_mv(_smem)_kernel + rht_out above" if e8 else
                                                  "whole chain: 4 trellis_fused_kernel<4,0> launches (+ 1 rht_in_kernel for down) per layer")
                                                 + " for its 7 linears, norms, activation and residual adds",
                        "achieved": gbs / world, "peak": hbm, "peak_kind": f"of {kind}", "unit": "GB/s",
                        "frac": gbs / world / hbm, "kernel_ms": ms, "bytes_per_launch": code_bytes, "traffic": None}}
    if world > 1:
        # every rank must hold the same hidden state; and one o projection summed inside the kernel must equal the
        # rank-ordered sum of the ranks' own fp32 outputs
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(outs, out)
        same = all(torch.equal(outs[0], o) for o in outs) and bool(torch.isfinite(out.float()).all())
        chk = {"chain_output_identical_on_all_ranks": same}
        if comm is not None:
            d0 = Ls[0]
            a = h0[:, :d0["o"].n].contiguous()
            mine = lin(d0["o"], a, out_dtype=torch.float32)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            fixed = torch.zeros_like(mine)
            for p_ in parts:
                fixed += p_
            got = lin(d0["o"], a, out_dtype=torch.float32, reduce_over=comm)
            torch.cuda.synchronize()
            chk["in_kernel_sum_max_rel_diff"] = ((got - fixed).abs().max() / fixed.abs().max().clamp_min(1e-30)).item()
            same = same and chk["in_kernel_sum_max_rel_diff"] <= 2e-3
            comm.check_status()
        chk["result"] = "ok" if same else "FAILED"
        rec["tp_check"] = chk
    del graph
    ops.clear_caches()
    torch.cuda.empty_cache()
    return rec


def run_linear_latency(D: Dist, args, steps=200):
    """One 2048 x 2048 trellis 4 bpw linear, batch 1, called through glq_b200.ops again and again on the same
    input (the weights stay in L2: this is launch and dependency latency, not bandwidth)."""
    import torch
    from glq_b200 import ops, synth
    dev = D.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    L = synth.trellis_layer("lat", 2048, 2048, [4], gen, dev)
    x = torch.randn(1, 2048, device=dev).to(torch.bfloat16)
    call = lambda: ops.fused_linear_trellis_3inst(x, L.sv, L.su, L.codes[0], None, None, None, None, L.wscale, 2048, 2048, 2048, 2048)
    for _ in range(5):
        call()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(20):
            call()
    g.replay()
    ms = timed(D, g.replay, steps) / 20
    ms_eager = timed(D, call, steps)
    del g
    # the same for an E8-shell layer of the reference's own CPU-runnable configuration (2048 x 2048, 2 stages), through
    # a plan (the call underneath ops.fused_linear_block_diag)
    from glq_b200.plan import Plan
    E = synth.e8_layer("lat_e8", 2048, 2048, 2, synth.load_e8_table(dev), gen, dev)
    y = torch.empty(1, 2048, device=dev, dtype=torch.bfloat16)
    plan = Plan([E.spec(batch=1, x_stride=2048, y_stride=2048)])
    call_e8 = lambda: plan.run(x, y)
    for _ in range(5):
        call_e8()
    torch.cuda.synchronize()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2):
        for _ in range(20):
            call_e8()
    g2.replay()
    ms_e8 = timed(D, g2.replay, steps) / 20
    e8_launches = plan.launches
    del g2
    plan.close()
    ops.clear_caches()
    return {"workload": "linear_call_latency", "metric": "time per call of one 2048x2048 trellis 4 bpw linear, batch 1",
            "value": ms * 1e3, "unit": "us", "higher_is_better": False, "eager_us": ms_eager * 1e3,
            "e8_2stage_us": ms_e8 * 1e3, "e8_launches_per_call": e8_launches,
            "config": "20 back-to-back calls in one CUDA graph (value; e8_2stage_us: the same for a 2048x2048 two-stage E8-shell "
                      "layer) and eager Python calls (eager_us); weights L2-resident"}


# --------------------------------------------------------------------------------------------------
# CPU arm
# --------------------------------------------------------------------------------------------------
def cpu_layer_sample():
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


def cpu_config0():
    """The reference's own CPU-runnable case: one E8 layer, in = out = 2048, 2 bpw (single stage), fp32 activations,
    batch 1 and 16, decode-then-matmul on the host cores (oracle/glq_oracle.c)."""
    import numpy as np
    from oracle import c_oracle as CO
    rng = np.random.default_rng(1)
    m = n = 2048
    q = rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16)
    table = np.load(os.path.join(ROOT, "glq_b200", "data", "e8_shell_packed.npy"))
    su = (rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)
    sv = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
    out = {}
    for B in (1, 16):
        x = rng.standard_normal((B, n)).astype(np.float32)
        CO.e8_linear(x, [q], [table], [], m, n, su, sv, 0.02, [n], [m], m)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 1.5:
            CO.e8_linear(x, [q], [table], [], m, n, su, sv, 0.02, [n], [m], m)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        out[f"batch{B}_ms"] = dt * 1e3
        out[f"batch{B}_GBps"] = q.nbytes / dt / 1e9
    return out


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
    rec = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": f"{reps} x one SmolLM3-3B decoder layer (7 projections, {nbytes // reps} packed bytes), "
                     "decode + fp32 matvec + Hadamard transforms, oracle/glq_oracle.c with OpenMP"}
    try:
        rec["e8_2048x2048_2bpw"] = cpu_config0()
    except Exception as e:          # the headline CPU figure stands on its own
        rec["e8_2048x2048_2bpw"] = {"error": str(e)}
    return rec


def reference_arm(args, world, rank):
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
            "dtype": "f32", "data": "synthetic", "config": headline_config(args.gpus),
            "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": "each step = one SmolLM3-3B decoder layer (7 projections, 39,059,456 packed "
                                       "bytes): decode + fp32 matvec + Hadamard transforms on the host cores"},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


def headline_config(gpus):
    return {"workload": "trellis 3INST 4 bpw decode matvec, batch 1, SmolLM3-3B projections "
                        "(36 layers x q/k/v/o/gate/up/down), L=16 K=4, 16x16 tiles",
            "cache": "inputs larger than L2 (1.4 GB of distinct packed weights per step)",
            "parallelism": f"tp{gpus}: rows of q/k/v/gate/up and columns of o/down split over ranks, fp32 partial sums "
                           "of o/down added by one NCCL all-reduce per step" if gpus > 1 else "single"}


# sub-records of the default run: (kind, workload, tokens, layers)
DEFAULT_SUBS = [
    ("plan", "decode_e8", 1, 8), ("plan", "decode_e8", 16, 8),
    ("plan", "prefill_e8", 2048, 2), ("plan", "prefill_e8", 256, 2),
    ("plan", "prefill_trellis", 2048, 4),
    ("plan", "decode_e8_62l", 1, 6), ("plan", "prefill_e8_62l", 2048, 3),
    ("moe", "moe", 256, None), ("moe", "moe", 4096, None), ("moe", "moe_zipf", 256, None), ("moe", "moe_zipf", 4096, None),
    ("chain", "decode_chain", 1, 36), ("chain", "decode_chain_e8", 1, 32), ("chain", "decode_chain_62l", 1, 62),
    ("latency", "linear_call_latency", 1, None),
]


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-subs", action="store_true", help="only the headline workload, no sub-records")
    ap.add_argument("--workload", default="decode_trellis_sweep",
                    help="decode_trellis_sweep (default, the headline with sub-records) or one of: "
                         + ", ".join(list(WORKLOADS) + ["moe", "moe_zipf", "decode_chain", "decode_chain_e8", "decode_chain_62l", "linear_call_latency"]))
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None,
                    help="decoder layers to build (default: per workload); smaller values are for profiler captures only")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return reference_arm(args, world, rank)

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in glq_b200)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    D = Dist(device)
    steps = args.steps

    def run_one(kind, name, tokens, layers, clocks=False, check=False, n_steps=None):
        n_steps = n_steps or steps
        if kind == "plan":
            return run_plan_bench(name, D, args, n_steps, tokens, layers, clocks=clocks, check=check)
        if kind == "moe":
            return run_moe_bench(name, D, args, n_steps, tokens)
        if kind == "chain":
            dense62 = name == "decode_chain_62l"
            e8 = name == "decode_chain_e8" or dense62
            return run_chain_bench(D, args, n_steps, layers or (62 if dense62 else 32 if e8 else 36), e8=e8, dense62=dense62)
        return run_linear_latency(D, args)

    if args.workload != "decode_trellis_sweep":
        kind = ("moe" if args.workload.startswith("moe") else "chain" if args.workload.startswith("decode_chain")
                else "latency" if args.workload == "linear_call_latency" else "plan")
        rec = run_one(kind, args.workload, args.tokens, args.layers, clocks=True, check=True)
        if rank == 0:
            line = {"metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "n_gpus": args.gpus, "steps": steps,
                    "warmup": max(args.warmup, 3), "ms_per_step": rec.get("ms_per_step"),
                    "higher_is_better": rec.get("higher_is_better", True), "scaling": "strong" if args.gpus > 1 else "weak",
                    "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                    "config": {"workload": f"{args.workload}: {rec['config']}", "parallelism": f"tp{args.gpus}" if args.gpus > 1 else "single"}}
            line.update({k: v for k, v in rec.items() if k not in ("metric", "value", "unit", "config", "workload", "n_gpus")})
            print(json.dumps(line))
    else:
        head = run_one("plan", "decode_trellis_sweep", None, args.layers, clocks=True, check=True)
        subs = []
        if not args.no_subs and not args.layers:
            sub_steps = max(3, min(steps, 10))
            failed = False
            for kind, name, tokens, layers in DEFAULT_SUBS:
                if world > 1 and kind == "latency":
                    continue
                if world > 1:
                    # ranks agree before every sub-record: after a failure on any rank all of them stop here (a
                    # sub-record must not take the headline down with it, nor leave ranks waiting for each other)
                    flag = torch.tensor([1.0 if failed else 0.0], device=device)
                    dist.all_reduce(flag)
                    if flag.item() > 0:
                        subs.append({"workload": name, "tokens": tokens, "error": "skipped after an earlier failure"})
                        failed = True
                        continue
                try:
                    subs.append(run_one(kind, name, tokens, layers, check=(kind == "plan"), n_steps=sub_steps))
                except Exception as e:
                    subs.append({"workload": name, "tokens": tokens, "error": f"{type(e).__name__}: {e}"})
                    failed = True
                    try:
                        torch.cuda.synchronize()
                    except Exception:
                        pass
        if rank == 0:
            config = headline_config(args.gpus)
            if args.layers:
                config["layers_built"] = args.layers
            line = {"metric": METRIC, "value": head["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
                    "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f16",
                    "data": "synthetic", "config": config, "e2e": head["e2e"], "gpu_launches": head["gpu_launches"],
                    "clocks": head.get("clocks"), "roofline": head["roofline"]}
            if "tp_check" in head:
                line["tp_check"] = head["tp_check"]["result"]
                line["tp_check_detail"] = head["tp_check"]
            if subs:
                line["sub"] = subs
            if args.gpus == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline()
            print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
