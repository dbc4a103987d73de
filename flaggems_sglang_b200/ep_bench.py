"""Multi-GPU leg of bench.py: expert-parallel fused MoE, one process per GPU (torchrun), NCCL over NVLink.

Weak scaling: every rank holds T tokens and E/N experts of the same global layer; tokens are dispatched to
the ranks that own their experts and combined back (flaggems_sglang_b200.ep).  Timing: CUDA events around K
steps between barriers, maximum over ranks; value = N*T / that time.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist


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
        wts = W.make_weights(cfg, dev, seed=0, num_experts=e_local, expert_offset=rank * e_local)
        tok = W.make_tokens(cfg, args.tokens, dev, seed=rank)
        kw = {}
        if cfg.dtype == "fp8":
            kw = dict(use_fp8_w8a8=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"], block_shape=[128, 128])

        # rows travel by P2P stores of this package's kernels into IPC-mapped receive areas ("p2p"), or by
        # NCCL all-to-all ("nccl")
        mode = getattr(args, "ep_exchange", "p2p")
        xc = None
        if mode == "p2p":
            try:
                xc = ep.PeerExchange(None, args.tokens, cfg.top_k, cfg.H, tok["hidden"].dtype)
            except RuntimeError as e:  # raised on every rank together (see PeerExchange): use the NCCL exchange
                mode = "nccl"
                if rank == 0:
                    print(f"# P2P exchange unavailable, using NCCL all-to-all: {e}", flush=True)

        def step():
            return ep.ep_fused_moe(tok["hidden"], wts["w1"], wts["w2"], tok["logits"], cfg.top_k, cfg.E, True,
                                   use_grouped_topk=cfg.router == "grouped", num_expert_group=cfg.n_group,
                                   topk_group=cfg.topk_group, correction_bias=tok.get("correction_bias"),
                                   routed_scaling_factor=cfg.routed_scaling_factor, exchange=xc, **kw)

        if clock_sampler is not None and rank == 0:
            clock_sampler.start()
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t_wall = time.perf_counter() - t_wall
        ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        _C.check_device_status(dev)

        # end-to-end: pinned host inputs in, result out, inside the timed region
        h_host = tok["hidden"].cpu().pin_memory()
        l_host = tok["logits"].cpu().pin_memory()
        out_host = torch.empty(args.tokens, cfg.H, dtype=tok["hidden"].dtype).pin_memory()

        def e2e_step():
            tok["hidden"].copy_(h_host, non_blocking=True)
            tok["logits"].copy_(l_host, non_blocking=True)
            out_host.copy_(step(), non_blocking=True)

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms2 = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        clocks = clock_sampler.stop() if clock_sampler is not None and rank == 0 else None

        if rank == 0:
            T_all = args.tokens * world
            ms_v, ms2_v = float(ms.item()), float(ms2.item())
            line = {
                "metric": "fused_moe tokens/s", "value": T_all / (ms_v * 1e-3), "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_v, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": cfg.dtype, "data": "synthetic",
                "config": {"workload": f"{cfg.name} MoE layer H={cfg.H} I={cfg.I} E={cfg.E} top_k={cfg.top_k}, "
                                       f"T={args.tokens} tokens per rank, experts sharded {e_local} per GPU, "
                                       + ("dispatch/combine by P2P stores into IPC-mapped receive areas"
                                          if mode == "p2p" else "NCCL all-to-all dispatch/combine"),
                           "tokens_per_step": T_all, "parallelism": f"ep{world}",
                           "l2": "weights re-read every step exceed L2 (no flush needed)"},
                "roofline": None, "cpu_baseline": None,
                "e2e": {"value": T_all / (ms2_v * 1e-3), "unit": "tokens/s", "ms_per_step": ms2_v,
                        "h2d_bytes_per_step": (h_host.numel() * h_host.element_size() + l_host.numel() * 4) * world,
                        "d2h_bytes_per_step": out_host.numel() * out_host.element_size() * world},
                # router, route, sort, dispatch, mask, align, row copy, 2 GEMMs, combine, sum (NCCL's not counted)
                "gpu_launches": (11 if mode == "p2p" else 9) * args.steps * world,
                "wall_ms_per_step": t_wall * 1e3 / args.steps,
                "clocks": clocks,
            }
            print(json.dumps(line), flush=True)
        if xc is not None:
            xc.close()
    finally:
        dist.destroy_process_group()
