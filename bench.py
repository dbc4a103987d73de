#!/usr/bin/env python
"""Benchmark of the fused-MoE layer call (router -> align -> gate/up GEMM+silu -> down GEMM -> sum).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config mixtral] [--tokens T]

One step = one `fused_moe` call on one batch of T synthetic tokens of the named layer.  Prints ONE JSON
line.  `value` is tokens/s with the inputs resident in HBM, device-timed with CUDA events; `e2e` is the
same call with host buffers (pinned) copied in and the result copied out inside the timed region.
With N > 1 (torchrun) the experts are sharded E/N per GPU and tokens are exchanged with NCCL all-to-all
(expert parallel, weak scaling: T tokens per rank).  `--impl reference` times the CPU restatement of the
reference path (oracle/) on the host cores on a bounded sample of the same workload.
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


def run_cpu_oracle(cfg, T, steps, warmup, seed=0):
    """-> (tokens/s, sample description, cores).  Weights are restricted to the experts the sample routes to."""
    from flaggems_sglang_b200 import workloads as W
    from oracle import experts as OE
    from oracle import routing as OR

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Ts = cpu_sample_tokens(cfg, T)
    tok = W.make_tokens(cfg, Ts, "cpu", seed=seed)
    if cfg.router == "grouped":
        tw, ti = OR.grouped_topk(tok["logits"], tok["correction_bias"], cfg.top_k, cfg.n_group, cfg.topk_group, True, None)
    else:
        tw, ti = OR.softmax_topk(tok["logits"], cfg.top_k, True)
    used = sorted(set(ti.reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    ti_local = torch.tensor([[remap[int(e)] for e in row] for row in ti], dtype=torch.int32)
    import dataclasses

    parts = [W.make_weights(dataclasses.replace(cfg), "cpu", seed=seed, num_experts=1, expert_offset=e) for e in used]
    w = {key: torch.cat([p[key] for p in parts]) for key in parts[0]}

    def step():
        if cfg.dtype == "fp8":
            return OE.fused_experts_fp8(tok["hidden"], w["w1"], w["w1_scale"], w["w2"], w["w2_scale"], tw, ti_local,
                                        routed_scaling_factor=cfg.routed_scaling_factor)
        return OE.fused_experts(tok["hidden"], w["w1"], w["w2"], tw, ti_local)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, steps)
    sample = (f"first {Ts} tokens of the T={T} batch, {len(used)} experts touched, torch fp32 matmul on up-cast weights, "
              f"{steps} steps")
    return Ts / dt, dt * 1e3, sample, cores


def reference_arm(args, cfg):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    warmup = max(0, min(args.warmup, 1))
    val, ms, sample, cores = run_cpu_oracle(cfg, args.tokens, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": cfg.dtype, "data": "synthetic",
        "config": {"workload": f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, T={args.tokens}",
                   "tokens_per_step": args.tokens},
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
    if cfg.dtype == "fp8":
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
    """Average device time per stage (ms) with events around each GEMM launch, over `steps` calls."""
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


def measure_point(cfg, wts, T, steps, warmup, peaks, seed=0):
    """One (config, T) point -> dict with ms, tokens/s, roofline of the whole call and of the dominant kernel."""
    from flaggems_sglang_b200 import workloads as W

    tok = W.make_tokens(cfg, T, "cuda", seed=seed)
    step = make_step(cfg, wts, tok)
    use_graph = T <= GRAPH_MAX_TOKENS
    _, ids = W.route(cfg, tok)
    active = int(torch.unique(ids).numel())
    nbytes, flops = W.algorithmic_bytes_flops(cfg, T, active)
    # inputs smaller than twice the L2 could be served from L2 on the next iteration: flush before every step
    flush = nbytes < 2 * torch.cuda.get_device_properties(0).L2_cache_size
    ms = time_steps(graphed(step) if use_graph else step, steps, warmup, flush=flush)
    st = stage_times(step, max(3, steps // 2))
    p_tensor = peaks["bf16_tflops"] * (2.0 if cfg.dtype == "fp8" else 1.0)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    t_tc = flops / (p_tensor * 1e12)
    bound = "tensor" if t_tc > t_hbm else "hbm"
    t_roof = max(t_hbm, t_tc)
    return {"T": T, "ms": ms, "cuda_graph": use_graph, "l2_flush": flush, "tokens_per_s": T / (ms * 1e-3), "active_experts": active, "bound": bound,
            "roofline_ms": t_roof * 1e3, "roofline_frac": t_roof / (ms * 1e-3),
            "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "achieved_tflops": flops / (ms * 1e-3) / 1e12,
            "stages_ms": st, "alg_bytes": nbytes, "alg_flops": flops}


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
    if point["bound"] == "tensor":
        peak = peaks["bf16_tflops"] * (2.0 if cfg.dtype == "fp8" else 1.0)
        ach = flops / t / 1e12
        return {"kernel": name, "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "traffic": None, "peak_source": peaks["source"] + " (burst cuBLAS bf16" + (", x2 nominal for fp8)" if cfg.dtype == "fp8" else ")"),
                "launch_ms": st[name], "alg_flops_per_launch": flops}
    ach = nbytes / t / 1e9
    return {"kernel": name, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": ach / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"] + " (copy bandwidth)",
            "launch_ms": st[name], "alg_bytes_per_launch": nbytes}


def e2e_run(cfg, wts, T, steps, warmup, seed=0):
    """Same call from pinned host buffers: H2D of hidden+logits and D2H of the result inside the timed region."""
    from flaggems_sglang_b200 import workloads as W

    tok = W.make_tokens(cfg, T, "cuda", seed=seed)
    h_host = tok["hidden"].cpu().pin_memory()
    l_host = tok["logits"].cpu().pin_memory()
    out_host = torch.empty(T, cfg.H, dtype=torch.bfloat16 if cfg.dtype != "fp32" else torch.float32).pin_memory()
    step = make_step(cfg, wts, tok)

    def one():
        h = h_host.to("cuda", non_blocking=True)
        lg = l_host.to("cuda", non_blocking=True)
        out = step(h, lg)
        out_host.copy_(out, non_blocking=True)

    ms = time_steps(one, steps, warmup)
    h2d = h_host.numel() * h_host.element_size() + l_host.numel() * l_host.element_size()
    d2h = out_host.numel() * out_host.element_size()
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="mixtral")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-T sweep of the configuration")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="N>1: token exchange by this package's P2P-store kernels (default) or by NCCL all-to-all")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    from flaggems_sglang_b200 import workloads as W

    cfg = W.CONFIGS[args.config]
    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    rank, world, local = dist_env()
    if world > 1:
        from flaggems_sglang_b200 import ep_bench

        ep_bench.run(args, cfg, rank, world, local, clock_sampler=ClockSampler(local))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(0)
    peaks = load_peaks()
    T = args.tokens
    wts = W.make_weights(cfg, "cuda", seed=0)

    sampler = ClockSampler(0)
    sampler.start()
    point = measure_point(cfg, wts, T, args.steps, args.warmup, peaks)
    clocks = sampler.stop()
    e2e_ms, h2d, d2h = e2e_run(cfg, wts, T, args.steps, args.warmup)

    sweep = []
    if not args.no_sweep:
        for Ts in cfg.sweep_T:
            pt = point if Ts == T else measure_point(cfg, wts, Ts, max(5, args.steps // 2), 3, peaks)
            dom = dominant_kernel_roofline(cfg, Ts, pt, peaks)
            sweep.append({"T": Ts, "ms": round(pt["ms"], 4), "tokens_per_s": round(pt["tokens_per_s"], 1),
                          "cuda_graph": pt["cuda_graph"], "l2_flush": pt["l2_flush"], "bound": pt["bound"], "roofline_frac": round(pt["roofline_frac"], 4),
                          "gemm1_frac": None if dom is None else round(dom["frac"], 4),
                          "active_experts": pt["active_experts"],
                          "stages_ms": {k: round(v, 4) for k, v in pt["stages_ms"].items()}})

    cpu = None
    if not args.no_cpu:
        val, ms, sample, cores = run_cpu_oracle(cfg, T, 2, 1)
        cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    from flaggems_sglang_b200 import _C

    _C.check_device_status()
    line = {
        "metric": METRIC, "value": point["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": point["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
        "config": {"workload": f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, T={T}, "
                               f"softmax top-k renormalised" if cfg.router == "softmax" else
                               f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, T={T}, grouped top-k",
                   "tokens_per_step": T, "l2": ("flushed before every step" if point["l2_flush"]
                          else "weights re-read every step exceed L2 (no flush needed)"),
                   "active_experts": point["active_experts"]},
        "roofline": dominant_kernel_roofline(cfg, T, point, peaks),
        "layer_roofline": {"bound": point["bound"], "frac": point["roofline_frac"], "roofline_ms": point["roofline_ms"],
                           "achieved_tflops": point["achieved_tflops"], "achieved_gbs": point["achieved_gbs"],
                           "peaks": peaks},
        "cpu_baseline": cpu,
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step(cfg, T) * args.steps,
        "clocks": clocks,
        "sweep": sweep,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
