#!/usr/bin/env python
"""Benchmark of the fused-MoE layer call (router -> align -> gate/up GEMM+silu -> down GEMM -> sum).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config mixtral] [--tokens T]

One step = one `fused_moe` call on one batch of T synthetic tokens of the named layer.  Prints ONE JSON
line.  `value` is tokens/s with the inputs resident in HBM, device-timed with CUDA events; `e2e` is the
same call with host buffers (pinned) copied in and the result copied out inside the timed region.
The headline is the Mixtral-8x7B layer at T=4096; the same line carries the per-T sweep of that layer and,
under "qwen3", "refbench" (the reference's own benchmark shapes) and "dsv3", the sweeps of the other
configurations, a parity figure against the CPU oracle ("parity") and a same-box timing of the reference's
Triton path ("vs_triton").  With N > 1 (torchrun) the experts are sharded E/N per GPU and tokens are
exchanged over NVLink (expert parallel, weak scaling: T tokens per rank).  `--impl reference` times the CPU
restatement of the reference path (oracle/) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# decode-sized batches are replayed from a CUDA graph (launch-bound otherwise); larger ones run eagerly
GRAPH_MAX_TOKENS = 256
METRIC = "fused_moe tokens/s"
UNIT = "tokens/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.idx)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------------------------
# reference arm: CPU restatement of the reference path, timed on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_sample_tokens(cfg, T):
    # about 10-30 s of CPU work in total: the weight up-cast dominates for small samples
    return min(T, 64 if cfg.dtype != "fp8" else 8)


def workload_name(cfg, T):
    router = "softmax top-k renormalised" if cfg.router == "softmax" else "grouped top-k"
    return f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, T={T}, {router}"


def run_cpu_oracle(cfg, T, steps, warmup, seed=0, gpu=None):
    """Times the CPU oracle on the first tokens of the batch -> (tokens/s, ms, sample text, cores, output, Ts).

    Weights are restricted to the experts the sample routes to.  With `gpu` = (weights, tokens) of the product
    arm the sample is a copy of those tensors, so that the oracle's output can be compared with the GPU's."""
    import dataclasses

    from flaggems_sglang_b200 import workloads as W
    from oracle import experts as OE
    from oracle import routing as OR

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Ts = cpu_sample_tokens(cfg, T)
    if gpu is None:
        tok = W.make_tokens(cfg, Ts, "cpu", seed=seed)
    else:
        tok = {k: v[:Ts].cpu() if v.dim() == 2 else v.cpu() for k, v in gpu[1].items()}
    if cfg.router == "grouped":
        tw, ti = OR.grouped_topk(tok["logits"], tok["correction_bias"], cfg.top_k, cfg.n_group, cfg.topk_group, True, None)
    else:
        tw, ti = OR.softmax_topk(tok["logits"], cfg.top_k, True)
    used = sorted(set(ti.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    ti_local = torch.tensor([[remap[int(e)] for e in row] for row in ti], dtype=torch.int32)
    if gpu is None:
        parts = [W.make_weights(dataclasses.replace(cfg), "cpu", seed=seed, num_experts=1, expert_offset=e) for e in used]
        w = {key: torch.cat([p[key] for p in parts]) for key in parts[0]}
    else:
        sel = torch.tensor(used, device=gpu[0]["w1"].device)
        w = {key: val[sel].cpu() for key, val in gpu[0].items()}

    def step():
        if cfg.dtype == "fp8":
            fn = OE.fused_experts_fp8_per_channel if cfg.fp8_scales == "channel" else OE.fused_experts_fp8
            return fn(tok["hidden"], w["w1"], w["w1_scale"], w["w2"], w["w2_scale"], tw, ti_local,
                      routed_scaling_factor=cfg.routed_scaling_factor)
        return OE.fused_experts(tok["hidden"], w["w1"], w["w2"], tw, ti_local)

    out = None
    for _ in range(warmup):
        out = step()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = step()
    dt = (time.perf_counter() - t0) / max(1, steps)
    sample = (f"first {Ts} tokens of the T={T} batch, {len(used)} experts touched, torch fp32 matmul on up-cast weights, "
              f"{steps} steps")
    return Ts / dt, dt * 1e3, sample, cores, out, Ts


def reference_arm(args, cfg):
    """`--impl reference`: the CPU oracle port on all host cores, K steps after W warm-up steps, each step a
    bounded sample (the first tokens) of the product arm's batch."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    val, ms, sample, cores, _, _ = run_cpu_oracle(cfg, args.tokens, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": cfg.dtype, "data": "synthetic",
        "config": {"workload": workload_name(cfg, args.tokens), "tokens_per_step": args.tokens},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# product arm
# ----------------------------------------------------------------------------------------------
def layer_kwargs(cfg, wts):
    kw = {}
    if cfg.dtype == "fp8" and cfg.fp8_scales == "channel":
        kw = dict(use_fp8_w8a8=True, per_channel_quant=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"])
    elif cfg.dtype == "fp8":
        kw = dict(use_fp8_w8a8=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"], block_shape=[128, 128])
    return kw


def make_step(cfg, wts, tok):
    import flaggems_sglang_b200 as fg

    kw = layer_kwargs(cfg, wts)

    def step(hidden=None, logits=None):
        h = tok["hidden"] if hidden is None else hidden
        lg = tok["logits"] if logits is None else logits
        return fg.fused_moe(h, wts["w1"], wts["w2"], lg, cfg.top_k, True, use_grouped_topk=cfg.router == "grouped",
                            num_expert_group=cfg.n_group, topk_group=cfg.topk_group,
                            correction_bias=tok.get("correction_bias"),
                            routed_scaling_factor=cfg.routed_scaling_factor, **kw)

    return step


def graphed(step, warmup=3):
    """Capture one call into a CUDA graph (the layer call has no host sync) -> replay function."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(warmup):
            step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    return g.replay


_FLUSH = None


def flush_l2():
    """Overwrite a buffer of twice the L2 size, so that the next step finds none of its inputs in L2."""
    global _FLUSH
    if _FLUSH is None:
        l2 = torch.cuda.get_device_properties(0).L2_cache_size
        _FLUSH = torch.empty(2 * l2, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_steps(step, steps, warmup, flush=False):
    """Device time of `steps` calls (CUDA events on the current stream) -> ms per step.  With `flush` every step
    is timed by its own event pair and L2 is flushed before it, outside the timed interval."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if flush:
        pairs = []
        for _ in range(steps):
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step()
            b.record()
            pairs.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def stage_times(step, steps):
    """Average device time per stage (ms) with events around each launch, in a pass of its own (the kernels are
    launched one by one from Python): used for the CUDA-graph / L2-flushed points, whose timed loop cannot
    carry events."""
    import importlib

    FM = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")

    FM.STAGE_EVENTS = []
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    acc = {}
    for name, a, b in FM.STAGE_EVENTS:
        acc.setdefault(name, []).append(a.elapsed_time(b))
    FM.STAGE_EVENTS = None
    return {k: sum(v) / len(v) for k, v in acc.items()}


def time_steps_staged(step, steps, warmup, names):
    """Device time of `steps` production calls AND the average duration of every stage inside those same calls:
    the library records caller-provided events at its stage boundaries (fmoe_debug_stage_events), so the
    per-kernel times and the step time come from one timed region."""
    import ctypes

    from flaggems_sglang_b200 import _C

    lib = _C.lib()
    n = 7
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(n)] for _ in range(steps)]
    for row in evs:
        for e in row:
            e.record()  # creates the underlying handle
    torch.cuda.synchronize()
    arrs = [(ctypes.c_void_p * n)(*[e.cuda_event for e in row]) for row in evs]
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        _C.check(lib.fmoe_debug_stage_events(arrs[i], n))
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    st = {}
    for j, name in enumerate(names):
        if name is None:
            continue
        st[name] = sum(row[j].elapsed_time(row[j + 1]) for row in evs) / steps
    return ms, st


def stage_names(cfg, T):
    from flaggems_sglang_b200.ops.fused_moe import _pick_variant

    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn}[cfg.dtype]
    name, _ = _pick_variant(dt, T * cfg.top_k, cfg.E, cfg.I, cfg.H, None)
    fp8 = cfg.dtype == "fp8"
    if fp8 and cfg.fp8_scales == "channel":
        name = "tcgen05"  # the only kernel family of the per-channel format
    g = ("gemm1_fp8_" if fp8 else "gemm1_") + name, ("gemm2_fp8_" if fp8 else "gemm2_") + name
    prep = "quant_input" if fp8 else ("gather_rows" if name.startswith("tcgen05") else None)
    return ["align", prep, g[0], "quant_act" if fp8 else None, g[1], "moe_sum"]


def measure_point(cfg, wts, T, steps, warmup, peaks, seed=0, skew=False):
    """One (config, T) point -> dict with ms, tokens/s, roofline of the whole call and of the dominant kernel."""
    from flaggems_sglang_b200 import workloads as W

    tok = W.make_tokens(cfg, T, "cuda", seed=seed, skew=skew)
    step = make_step(cfg, wts, tok)
    use_graph = T <= GRAPH_MAX_TOKENS
    _, ids = W.route(cfg, tok)
    active = int(torch.unique(ids).numel())
    nbytes, flops = W.algorithmic_bytes_flops(cfg, T, active)
    # inputs smaller than twice the L2 could be served from L2 on the next iteration: flush before every step
    flush = nbytes < 2 * torch.cuda.get_device_properties(0).L2_cache_size
    if use_graph or flush:
        ms = time_steps(graphed(step) if use_graph else step, steps, warmup, flush=flush)
        st = stage_times(step, max(3, steps // 2))
        st_src = "separate pass, one launch per stage from the host"
    else:
        ms, st = time_steps_staged(step, steps, warmup, stage_names(cfg, T))
        st_src = "events inside the timed loop"
    p_tensor = peaks["bf16_tflops"] * (2.0 if cfg.dtype == "fp8" else 1.0)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_tc = flops / (p_tensor * 1e12)
    bound = "tensor" if t_tc > t_hbm else "hbm"
    t_roof = max(t_hbm, t_tc)
    return {"T": T, "ms": ms, "cuda_graph": use_graph, "l2_flush": flush, "tokens_per_s": T / (ms * 1e-3), "active_experts": active, "bound": bound,
            "roofline_ms": t_roof * 1e3, "roofline_frac": t_roof / (ms * 1e-3),
            "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "achieved_tflops": flops / (ms * 1e-3) / 1e12,
            "stages_ms": st, "stages_source": st_src, "alg_bytes": nbytes, "alg_flops": flops, "skew": skew, "tok": tok}


# DRAM traffic of the gate/up GEMM per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture; the
# summaries with the full commands are under profiles/).  Keyed by (config, T).
MEASURED_TRAFFIC = {
    ("mixtral", 4096): (2.19e9, "profiles/grouped_gemm_tcgen05_bf16_mixtral.md, full-size capture of the same launch"),
}


def dominant_kernel_roofline(cfg, T, point, peaks):
    """Roofline of the gate/up GEMM (2/3 of the flops and of the weight bytes)."""
    st = point["stages_ms"]
    name = next((k for k in st if k.startswith("gemm1")), None)
    if name is None:
        return None
    t = st[name] * 1e-3
    bw = 1 if cfg.dtype == "fp8" else 2
    M = T * cfg.top_k
    flops = 4.0 * M * cfg.H * cfg.I
    nbytes = point["active_experts"] * 2 * cfg.I * cfg.H * bw + T * cfg.H * bw + M * cfg.I * bw
    traffic, traffic_src = MEASURED_TRAFFIC.get((cfg.name, T), (None, None))
    common = {"kernel": name, "launch_ms": st[name], "timing": point["stages_source"], "traffic": traffic,
              "traffic_source": traffic_src, "alg_flops_per_launch": flops, "alg_bytes_per_launch": nbytes}
    if point["bound"] == "tensor":
        peak = peaks["bf16_tflops"] * (2.0 if cfg.dtype == "fp8" else 1.0)
        ach = flops / t / 1e12
        return {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "peak_source": peaks["source"] + " (burst cuBLAS bf16" + (", x2 nominal for fp8)" if cfg.dtype == "fp8" else ")"),
                **common}
    ach = nbytes / t / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"] + " (copy bandwidth)", **common}


def e2e_run(cfg, wts, T, steps, warmup, seed=0):
    """Same call from pinned host buffers: H2D of hidden+logits and D2H of the result inside the timed region.

    The copies run on two side streams and are double-buffered: while step i computes, the inputs of step i+1
    are already on their way in and the result of step i-1 on its way out (the three engines of the GPU work
    at the same time); every step's input copy, compute and output copy are ordered by events."""
    from flaggems_sglang_b200 import workloads as W

    tok = W.make_tokens(cfg, T, "cuda", seed=seed)
    h_host = tok["hidden"].cpu().pin_memory()
    l_host = tok["logits"].cpu().pin_memory()
    odt = torch.bfloat16 if cfg.dtype != "fp32" else torch.float32
    out_host = [torch.empty(T, cfg.H, dtype=odt).pin_memory() for _ in range(2)]
    h_dev = [torch.empty_like(tok["hidden"]) for _ in range(2)]
    l_dev = [torch.empty_like(tok["logits"]) for _ in range(2)]
    o_dev = [None, None]
    step = make_step(cfg, wts, tok)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]

    def copy_in(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])  # the compute that last read this buffer has finished
            h_dev[b].copy_(h_host, non_blocking=True)
            l_dev[b].copy_(l_host, non_blocking=True)
            ev_in[b].record(s_in)

    def run(n):
        for b in range(2):
            ev_free[b].record(main)
        copy_in(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                copy_in(i + 1)
            main.wait_event(ev_in[b])
            o_dev[b] = step(h_dev[b], l_dev[b])
            ev_free[b].record(main)
            ev_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                out_host[b].copy_(o_dev[b], non_blocking=True)
                o_dev[b].record_stream(s_out)
        main.wait_stream(s_out)

    run(max(warmup, 2))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    h2d = h_host.numel() * h_host.element_size() + l_host.numel() * l_host.element_size()
    d2h = out_host[0].numel() * out_host[0].element_size()
    return ms, h2d, d2h


def launches_per_step(cfg, T):
    from flaggems_sglang_b200.ops.fused_moe import _pick_variant

    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn}[cfg.dtype]
    name, _ = _pick_variant(dt, T * cfg.top_k, cfg.E, cfg.I, cfg.H, None)
    numel = T * cfg.top_k
    n = 1 + (3 if numel >= 8192 else 1) + 2 + 1  # router, align (count/scan/scatter above 8192 slots), two GEMMs, sum
    if cfg.dtype == "fp8":
        n += 1  # quantisation of the input rows
        if name == "tcgen05" and cfg.top_k >= 2 and cfg.H % 512 == 0:
            n += 2  # token rows quantised once, then bytes and scales copied into the sorted order
        n += 1  # quantisation of the activations between the two GEMMs
    elif name == "tcgen05":
        n += 1  # row gather into sorted order
    return n


def sweep_entry(cfg, T, pt, peaks):
    dom = dominant_kernel_roofline(cfg, T, pt, peaks)
    return {"T": T, "routing": "zipf-1.2" if pt["skew"] else "uniform", "ms": round(pt["ms"], 4),
            "tokens_per_s": round(pt["tokens_per_s"], 1), "cuda_graph": pt["cuda_graph"], "l2_flush": pt["l2_flush"],
            "bound": pt["bound"], "roofline_frac": round(pt["roofline_frac"], 4),
            "gemm1_frac": None if dom is None else round(dom["frac"], 4), "active_experts": pt["active_experts"],
            "stages_ms": {k: round(v, 4) for k, v in pt["stages_ms"].items()}, "stages_source": pt["stages_source"]}


def config_sweep(name, peaks, steps, extra_T=(), skew_T=()):
    """Sweep of one more configuration (its own weights, freed afterwards) -> list of sweep entries."""
    from flaggems_sglang_b200 import workloads as W

    cfg = W.CONFIGS[name]
    wts = W.make_weights(cfg, "cuda", seed=0)
    out = []
    try:
        for T, skew in [(t, False) for t in sorted(set(cfg.sweep_T) | set(extra_T))] + [(t, True) for t in skew_T]:
            pt = measure_point(cfg, wts, T, steps, 3, peaks, skew=skew)
            out.append(sweep_entry(cfg, T, pt, peaks))
    finally:
        del wts
        torch.cuda.empty_cache()
    return out


def parity_vs_oracle(cfg, wts, tok, T):
    """CPU oracle on the first tokens of the product arm's batch: its timing is the cpu_baseline, its output is
    compared with the GPU's for those tokens."""
    step = make_step(cfg, wts, tok)
    got = step()
    torch.cuda.synchronize()
    val, ms, sample, cores, ref, Ts = run_cpu_oracle(cfg, T, 2, 1, gpu=(wts, tok))
    g, r = got[:Ts].float().cpu(), ref.float()
    parity = {"tokens": Ts, "against": "CPU oracle (oracle/experts.py) on the same weights and tokens",
              "rel_l2": float((g - r).norm() / r.norm()), "max_abs_frac": float((g - r).abs().max() / r.abs().max())}
    return {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}, parity


def _interleaved_ms(fns, rounds=40, warmup=5):
    """Median device time of each callable when they are called in turn (a, b, a, b, ...), every call preceded by an
    L2 flush outside its timed interval: both sides see the same clocks, temperature and power state, which
    back-to-back blocks of calls do not (the GPU sheds speed within a second of sustained load)."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(rounds)]
           for _ in fns]
    for i in range(warmup + rounds):
        for j, fn in enumerate(fns):
            flush.zero_()
            if i >= warmup:
                evs[j][i - warmup][0].record()
            fn()
            if i >= warmup:
                evs[j][i - warmup][1].record()
    torch.cuda.synchronize()
    return [statistics.median(a.elapsed_time(b) for a, b in ev) for ev in evs]


def vs_triton(cfg, wts, tokens):
    """Same box, same inputs: the REAL reference operator (`flaggems_sglang.triton_kernel_fused_experts` from the
    offline install under baseline/_ref, running the `triton_kernels` copy vLLM vendors) against this package,
    both timed with the reference's own method (triton.testing.do_bench, median; ref
    benchmark/performance_utils.py:365-377).  bf16 only (the reference rejects fp8).  Outside every timed region
    of the headline."""
    import tempfile

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flaggems_sglang")):
        return {"unavailable": "no reference install under baseline/_ref"}
    try:
        import vllm

        stub = tempfile.mkdtemp()
        os.makedirs(os.path.join(stub, "sgl_kernel"))
        with open(os.path.join(stub, "sgl_kernel", "__init__.py"), "w") as f:
            f.write("def gelu_and_mul(x, out):\n    raise NotImplementedError\n")
        os.environ.setdefault("DNN_VENDOR", "nvidia")
        sys.path[:0] = [ref_dir, os.path.join(os.path.dirname(vllm.__file__), "third_party"), stub]
        import flaggems_sglang
        import triton
        from flaggems_sglang.ops import fused_moe as ref_fm
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}
    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import workloads as W

    out = {"reference": "flaggems_sglang.triton_kernel_fused_experts (baseline/_ref) on vLLM's triton_kernels",
           "timing": "triton.testing.do_bench median, L2 flushed between calls (blocks of calls: reference, reference "
                     "with routing, this package); 'interleaved': alternating calls, median of 40 each; "
                     "'same_arguments': this package's triton_kernel_fused_experts called with the reference's own "
                     "argument list ([E,H,2I] / [E,I,H] weights, its routing objects)", "points": []}
    w1r = wts["w1"].transpose(1, 2).contiguous()  # the reference's [E,H,2I] / [E,I,H] layouts, prepared once
    w2r = wts["w2"].transpose(1, 2).contiguous()
    for T in tokens:
        rec = {"T": T}
        try:
            tok = W.make_tokens(cfg, T, "cuda", seed=0)
            tw, ti = W.route(cfg, tok)
            x = tok["hidden"]
            tables = ref_fm._standard_topk_to_triton_kernels(tw, ti, cfg.E)

            def ref_experts():
                return flaggems_sglang.triton_kernel_fused_experts(x, w1r, w2r, *tables)

            def ref_with_routing():
                return flaggems_sglang.triton_kernel_fused_experts(
                    x, w1r, w2r, *ref_fm._standard_topk_to_triton_kernels(tw, ti, cfg.E))

            def ours():
                return fg.fused_experts(x, wts["w1"], wts["w2"], tw, ti)

            def ours_entry():  # the drop-in call: the reference's own arguments, weights [E,H,2I] / [E,I,H] read in place
                return fg.triton_kernel_fused_experts(x, w1r, w2r, *tables)

            r, g = ref_experts().float(), ours().float()
            rec["rel_l2"] = float((g - r).norm() / r.norm())
            rec["reference_experts_ms"] = triton.testing.do_bench(ref_experts, warmup=20, rep=100, return_mode="median")
            rec["reference_routing_plus_experts_ms"] = triton.testing.do_bench(ref_with_routing, warmup=20, rep=100,
                                                                                return_mode="median")
            rec["ours_ms"] = triton.testing.do_bench(ours, warmup=20, rep=100, return_mode="median")
            rec["rel_l2_same_arguments"] = float((ours_entry().float() - r).norm() / r.norm())
            rec["ours_same_arguments_ms"] = triton.testing.do_bench(ours_entry, warmup=20, rep=100, return_mode="median")
            rec["speedup_experts"] = rec["reference_experts_ms"] / rec["ours_ms"]
            rec["speedup_with_routing"] = rec["reference_routing_plus_experts_ms"] / rec["ours_ms"]
            a, b, c = _interleaved_ms([ref_experts, ours, ours_entry])
            rec["interleaved"] = {"reference_experts_ms": a, "ours_ms": b, "ours_same_arguments_ms": c,
                                  "speedup_experts": a / b, "speedup_same_arguments": a / c}
        except Exception as e:  # noqa: BLE001  (the vendored third-party copy is not pinned by the reference)
            rec["error"] = f"{type(e).__name__}: {e}"[:300]
        out["points"].append(rec)
    del w1r, w2r
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="mixtral")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-T sweeps (this configuration's and the others')")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / parity leg")
    ap.add_argument("--no-triton", action="store_true", help="skip the same-box timing of the reference's Triton path")
    ap.add_argument("--triton-tokens", default="", help="comma-separated batch sizes for that comparison (default 64,1024,4096)")
    ap.add_argument("--skew", action="store_true", help="Zipf(1.2)-skewed routing for the headline point")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: token exchange by this package's P2P-store kernels (default) or by NCCL all-to-all")
    ap.add_argument("--no-c5", action="store_true", help="N>1: skip the DeepSeek-V3 fp8 expert-parallel block")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    from flaggems_sglang_b200 import workloads as W

    cfg = W.CONFIGS[args.config]
    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    rank, world, local = dist_env()
    # a rank that blocks (a collective a peer never joins) ends the run with a Python traceback of every thread
    # instead of holding the GPUs until an outer limit: FMOE_BENCH_WATCHDOG seconds (default 780 for N > 1)
    watchdog = int(os.environ.get("FMOE_BENCH_WATCHDOG", "780" if world > 1 else "0"))
    if watchdog > 0:
        import faulthandler

        faulthandler.dump_traceback_later(watchdog, exit=True)
    if world > 1:
        from flaggems_sglang_b200 import ep_bench

        args.peaks = load_peaks()
        ep_bench.run(args, cfg, rank, world, local, clock_sampler=ClockSampler(local))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(0)
    peaks = load_peaks()
    T = args.tokens
    wts = W.make_weights(cfg, "cuda", seed=0)

    sampler = ClockSampler(0)
    sampler.start()
    point = measure_point(cfg, wts, T, args.steps, args.warmup, peaks, skew=args.skew)
    clocks = sampler.stop()
    e2e_ms, h2d, d2h = e2e_run(cfg, wts, T, args.steps, args.warmup)

    sweep_steps = max(5, args.steps // 2)
    sweep = []
    if not args.no_sweep:
        for Ts in cfg.sweep_T:
            pt = point if (Ts == T and not args.skew) else measure_point(cfg, wts, Ts, sweep_steps, 3, peaks)
            sweep.append(sweep_entry(cfg, Ts, pt, peaks))

    cpu = parity = None
    if not args.no_cpu:
        cpu, parity = parity_vs_oracle(cfg, wts, point["tok"], T)

    triton_cmp = None
    if not args.no_triton and cfg.dtype == "bf16":
        triton_T = [int(t) for t in args.triton_tokens.split(",") if t] or [t for t in (64, 1024, 4096) if t in cfg.sweep_T]
        triton_cmp = vs_triton(cfg, wts, triton_T or [T])

    others = {}
    if not args.no_sweep and args.config == "mixtral":
        del wts
        torch.cuda.empty_cache()
        # the other configurations of the metric; DeepSeek-V3 also at the per-rank sizes of the expert-parallel
        # runs (128, 4096), so that weak-scaling efficiency can be read against one GPU doing the same tokens
        others["qwen3"] = config_sweep("qwen3", peaks, sweep_steps, skew_T=(512, 8192))
        others["refbench"] = config_sweep("refbench", peaks, sweep_steps)
        others["dsv3"] = config_sweep("dsv3", peaks, sweep_steps, extra_T=(128, 4096), skew_T=(4096,))
        others["dsv3_channel"] = config_sweep("dsv3_channel", peaks, sweep_steps)

    from flaggems_sglang_b200 import _C

    _C.check_device_status()
    line = {
        "metric": METRIC, "value": point["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": point["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
        "config": {"workload": workload_name(cfg, T), "tokens_per_step": T,
                   "routing": "zipf-1.2 skew" if args.skew else "uniform",
                   "l2": ("flushed before every step" if point["l2_flush"]
                          else "weights re-read every step exceed L2 (no flush needed)"),
                   "active_experts": point["active_experts"]},
        "roofline": dominant_kernel_roofline(cfg, T, point, peaks),
        "layer_roofline": {"bound": point["bound"], "frac": point["roofline_frac"], "roofline_ms": point["roofline_ms"],
                           "achieved_tflops": point["achieved_tflops"], "achieved_gbs": point["achieved_gbs"],
                           "peaks": peaks},
        "cpu_baseline": cpu,
        "parity": parity,
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "copies": "pinned host buffers, side streams, double-buffered"},
        "gpu_launches": launches_per_step(cfg, T) * args.steps,
        "clocks": clocks,
        "stages_ms": {k: round(v, 4) for k, v in point["stages_ms"].items()},
        "sweep": sweep,
        **others,
        "vs_triton": triton_cmp,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
