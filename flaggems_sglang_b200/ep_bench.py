"""Multi-GPU leg of bench.py: expert-parallel fused MoE, one process per GPU (torchrun), NCCL over NVLink.

Weak scaling: every rank holds T tokens and E/N experts of the same global layer; tokens are dispatched to
the ranks that own their experts and combined back (flaggems_sglang_b200.ep).  Timing: CUDA events around K
steps between barriers, maximum over ranks; value = N*T / that time.

The headline stays the configuration bench.py was asked for (Mixtral bf16 by default); the same JSON line
carries under "c5" the DeepSeek-V3 fp8 expert-parallel block: T per rank in {128, 4096}, uniform and
Zipf(1.2)-skewed routing, P2P and NCCL exchange, and a parity figure of rank 0's output against the
single-GPU operator on the full layer.
"""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist


def _timed(step, steps, warmup, dev):
    """K steps between barriers, CUDA events, max over ranks -> ms per step."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def _layer_kwargs(cfg, wts):
    if cfg.dtype == "fp8":
        return dict(use_fp8_w8a8=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"], block_shape=[128, 128])
    return {}


def _make_step(ep, cfg, wts, tok, xc):
    kw = _layer_kwargs(cfg, wts)

    def step(hidden=None, logits=None):
        return ep.ep_fused_moe(tok["hidden"] if hidden is None else hidden, wts["w1"], wts["w2"],
                               tok["logits"] if logits is None else logits, cfg.top_k, cfg.E, True,
                               use_grouped_topk=cfg.router == "grouped", num_expert_group=cfg.n_group,
                               topk_group=cfg.topk_group, correction_bias=tok.get("correction_bias"),
                               routed_scaling_factor=cfg.routed_scaling_factor, exchange=xc, **kw)

    return step


def _parity_rank0(cfg, tok, out, rank):
    """Rank 0: the single-GPU operator on the FULL layer (all experts, built here for the check) on this rank's
    whole batch, so that both sides pick the same kernel family, against the expert-parallel output.  Outside
    every timed region; the other ranks wait in the barrier."""
    res = None
    if rank == 0:
        import flaggems_sglang_b200 as fg
        from . import workloads as W

        full = W.make_weights(cfg, out.device, seed=0)
        ref = fg.fused_moe(tok["hidden"], full["w1"], full["w2"], tok["logits"], cfg.top_k, True,
                           use_grouped_topk=cfg.router == "grouped", num_expert_group=cfg.n_group,
                           topk_group=cfg.topk_group, correction_bias=tok.get("correction_bias"),
                           routed_scaling_factor=cfg.routed_scaling_factor, **_layer_kwargs(cfg, full)).float()
        got = out.float()
        res = {"tokens": int(out.shape[0]), "against": "single-GPU fused_moe on the full layer, same tokens",
               "rel_l2": float((got - ref).norm() / ref.norm()),
               "max_abs_frac": float((got - ref).abs().max() / ref.abs().max()), "bit_equal": bool(torch.equal(got, ref))}
        del full
        torch.cuda.empty_cache()
    dist.barrier()
    return res


def _exchange(ep, mode, T, cfg, dtype, rank):
    """-> (PeerExchange or None, mode actually used)."""
    if mode != "p2p":
        return None, "nccl"
    try:
        world = dist.get_world_size()
        return ep.PeerExchange(None, T, cfg.top_k, cfg.H, dtype, num_local_experts=cfg.E // world,
                               intermediate_size=cfg.I, fp8=cfg.dtype == "fp8"), "p2p"
    except RuntimeError as e:  # raised on every rank together (see PeerExchange): use the NCCL exchange
        if rank == 0:
            print(f"# P2P exchange unavailable, using NCCL all-to-all: {e}", flush=True)
        return None, "nccl"


def c5_block(args, rank, world, dev):
    """DeepSeek-V3 fp8 expert parallel: T per rank x routing x exchange -> list of records (all ranks take part)."""
    from . import ep, workloads as W

    cfg = W.CONFIGS["dsv3"]
    if cfg.E % world:
        return {"unavailable": f"{cfg.E} experts do not divide over {world} GPUs"}
    e_local = cfg.E // world
    wts = W.make_weights(cfg, dev, seed=0, num_experts=e_local, expert_offset=rank * e_local)
    steps = max(5, args.steps // 2)
    points, parity, parity_done = [], None, False
    for T in (128, 4096):
        for mode in ("p2p", "nccl"):
            xc, used = _exchange(ep, mode, T, cfg, torch.bfloat16, rank)
            for skew in (False, True):
                tok = W.make_tokens(cfg, T, dev, seed=rank, skew=skew)
                step = _make_step(ep, cfg, wts, tok, xc)
                ms = _timed(step, steps, 3, dev)
                points.append({"T_local": T, "routing": "zipf-1.2" if skew else "uniform", "exchange": used,
                               "ms": round(ms, 4), "tokens_per_s": round(world * T / (ms * 1e-3), 1)})
                if not parity_done and T == 4096 and not skew:  # once, on every rank (only rank 0 gets a result)
                    parity = _parity_rank0(cfg, tok, step(), rank)
                    parity_done = True
            if xc is not None:
                xc.close()
    del wts
    torch.cuda.empty_cache()
    return {"workload": f"dsv3 fp8 w8a8 128x128 MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, grouped top-k, "
                        f"{e_local} experts per GPU", "steps": steps, "points": points, "parity": parity}


def run(args, cfg, rank: int, world: int, local: int, clock_sampler=None) -> None:
    """`clock_sampler`: object with start()/stop() -> dict; rank 0 samples its GPU's clocks from the warm-up to
    the end of the timed regions (they are tens of milliseconds, shorter than one nvidia-smi sample)."""
    from . import ep, workloads as W
    from . import _C

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        if cfg.E % world:
            raise SystemExit(f"{cfg.E} experts do not divide over {world} GPUs")
        e_local = cfg.E // world
        T = args.tokens
        wts = W.make_weights(cfg, dev, seed=0, num_experts=e_local, expert_offset=rank * e_local)
        tok = W.make_tokens(cfg, T, dev, seed=rank, skew=getattr(args, "skew", False))

        # rows travel by P2P stores of this package's kernels into IPC-mapped receive areas ("p2p"), or by
        # NCCL all-to-all ("nccl")
        xc, mode = _exchange(ep, getattr(args, "ep_exchange", "p2p"), T, cfg, tok["hidden"].dtype, rank)
        step = _make_step(ep, cfg, wts, tok, xc)

        if clock_sampler is not None and rank == 0:
            clock_sampler.start()
        warm = max(args.warmup, 3)
        t_wall = time.perf_counter()
        ms_v = _timed(step, args.steps, warm, dev)
        t_wall = time.perf_counter() - t_wall
        _C.check_device_status(dev)

        # end-to-end: pinned host inputs in, result out, inside the timed region; copies on side streams,
        # double-buffered, so that step i's copies overlap the neighbouring steps' compute
        h_host = tok["hidden"].cpu().pin_memory()
        l_host = tok["logits"].cpu().pin_memory()
        out_host = [torch.empty(T, cfg.H, dtype=tok["hidden"].dtype).pin_memory() for _ in range(2)]
        h_dev = [torch.empty_like(tok["hidden"]) for _ in range(2)]
        l_dev = [torch.empty_like(tok["logits"]) for _ in range(2)]
        s_in, s_out, main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]
        counter = [0]

        def copy_in(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[b])
                h_dev[b].copy_(h_host, non_blocking=True)
                l_dev[b].copy_(l_host, non_blocking=True)
                ev_in[b].record(s_in)

        def e2e_prologue():
            counter[0] = 0
            for b in range(2):
                ev_free[b].record(main)
            copy_in(0)

        def e2e_step():
            i = counter[0]
            counter[0] += 1
            b = i & 1
            copy_in(i + 1)  # the next step's inputs (one surplus copy after the last step, inside the timed region)
            main.wait_event(ev_in[b])
            out = step(h_dev[b], l_dev[b])
            ev_free[b].record(main)
            ev_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                out_host[b].copy_(out, non_blocking=True)
                out.record_stream(s_out)

        def e2e_pass(n):
            e2e_prologue()
            for _ in range(n):
                e2e_step()
            main.wait_stream(s_out)
            main.wait_stream(s_in)

        e2e_pass(3)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_pass(args.steps)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms2 = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        clocks = clock_sampler.stop() if clock_sampler is not None and rank == 0 else None

        # phases of the exchange and the two GEMMs, timed in five extra steps (events around every phase; the
        # GEMM events sit inside the "experts" phase): median over the steps, then max over ranks
        phases_ms, roofline = None, None
        ep.PHASE_EVENTS = []
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        names, samples = [], {}
        for name, a, b in ep.PHASE_EVENTS:
            if name not in samples:
                names.append(name)
            samples.setdefault(name, []).append(a.elapsed_time(b))
        acc = {n: sorted(v)[len(v) // 2] for n, v in samples.items()}
        ep.PHASE_EVENTS = None
        if names:
            vec = torch.tensor([acc[n] for n in names], device=dev)
            own_gemm1 = acc.get("gemm1")
            dist.all_reduce(vec, op=dist.ReduceOp.MAX)
            phases_ms = {n: round(float(v), 4) for n, v in zip(names, vec.tolist())}
            if xc is not None and own_gemm1 and getattr(args, "peaks", None):
                used = int(xc.npp.item())
                rows = int((xc.sorted_ids[:used] < xc.capacity).sum().item())  # rows this rank's experts received
                flops = 4.0 * rows * cfg.H * cfg.I
                peak = args.peaks["bf16_tflops"] * (2.0 if cfg.dtype == "fp8" else 1.0)
                ach = flops / (own_gemm1 * 1e-3) / 1e12
                roofline = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                            "peak_source": args.peaks["source"], "kernel": f"gemm1 on rank 0 of {world} ({rows} rows received)",
                            "launch_ms": own_gemm1, "timing": "events around the launch, median of five extra steps",
                            "traffic": None, "alg_flops_per_launch": flops}

        parity = _parity_rank0(cfg, tok, step(), rank)
        if xc is not None:
            xc.close()
            xc = None
        del wts
        torch.cuda.empty_cache()
        c5 = None
        if not getattr(args, "no_c5", False) and cfg.name != "dsv3":
            c5 = c5_block(args, rank, world, dev)
        _C.check_device_status(dev)

        if rank == 0:
            T_all = T * world
            ms2_v = float(ms2.item())
            line = {
                "metric": "fused_moe tokens/s", "value": T_all / (ms_v * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": warm, "ms_per_step": ms_v, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
                "config": {"workload": f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, "
                                       f"T={T} tokens per rank, experts sharded {e_local} per GPU, "
                                       + ("dispatch/combine by P2P stores into IPC-mapped receive areas"
                                          if mode == "p2p" else "NCCL all-to-all dispatch/combine"),
                           "tokens_per_step": T_all, "parallelism": f"ep{world}",
                           "l2": "weights re-read every step exceed L2 (no flush needed)"},
                "roofline": roofline, "phases_ms": phases_ms, "cpu_baseline": None, "parity": parity,
                "e2e": {"value": T_all / (ms2_v * 1e-3), "unit": "tokens/s", "ms_per_step": ms2_v,
                        "h2d_bytes_per_step": (h_host.numel() * h_host.element_size() + l_host.numel() * 4) * world,
                        "d2h_bytes_per_step": out_host[0].numel() * out_host[0].element_size() * world,
                        "copies": "pinned host buffers, side streams, double-buffered"},
                # router, route, sort, dispatch, mask, align, row copy, 2 GEMMs, combine, sum (NCCL's not counted)
                "gpu_launches": (11 if mode == "p2p" else 9) * args.steps * world,
                "wall_ms_per_step": t_wall * 1e3 / (args.steps + warm),
                "clocks": clocks,
                "c5": c5,
            }
            print(json.dumps(line), flush=True)
    finally:
        dist.destroy_process_group()
