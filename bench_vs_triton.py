#!/usr/bin/env python
"""Same-box comparison with the reference's GPU data path.

The reference op (FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:197-232) is three calls: the
third-party `triton_kernels.matmul_ogs` (gather + grouped GEMM), a Triton silu-and-mul pass, and
`matmul_ogs` again (grouped GEMM * gate weight + grouped reduce), fed by routing tables built with torch
ops (:119-146).  The reference checkout itself is not available on the GPU box, so this script restates
that call sequence on top of the `triton_kernels` copy that vLLM vendors in this image (Triton lowers it to
tcgen05 on sm_100) and times it next to this package on identical inputs, with the reference's own timing
method (`triton.testing.do_bench`, median).  It also prints the relative L2 difference of the two outputs.

    python bench_vs_triton.py [--config mixtral|qwen3|refbench] [--tokens 1,16,64,...]

Prints one JSON line per token count.  bf16 only (the reference rejects fp8).  Weights are given to the
Triton path in its own [E,H,2I]/[E,I,H] layout, prepared once outside the timed region (the reference's
SGLang hook re-does that transpose on every call, fused_moe.py:342-343; `--with-transpose` adds it).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


def _import_triton_kernels():
    try:
        import triton_kernels  # noqa: F401
    except ImportError:
        import vllm

        sys.path.insert(0, os.path.join(os.path.dirname(vllm.__file__), "third_party"))
    import triton
    import triton.language as tl
    from triton_kernels.matmul_ogs import matmul_ogs
    from triton_kernels.routing import GatherIndx, RoutingData, ScatterIndx, compute_expt_data_torch

    @triton.jit
    def silu_mul_kernel(x_ptr, y_ptr, half, BLOCK: tl.constexpr):
        row = tl.program_id(0)
        cols = tl.program_id(1) * BLOCK + tl.arange(0, BLOCK)
        m = cols < half
        g = tl.load(x_ptr + row * 2 * half + cols, mask=m, other=0.0).to(tl.float32)
        u = tl.load(x_ptr + row * 2 * half + half + cols, mask=m, other=0.0).to(tl.float32)
        tl.store(y_ptr + row * half + cols, (g / (1.0 + tl.exp(-g))) * u, mask=m)

    def routing_tables(tw, ti, E):
        T, k = tw.shape
        ids2, perm = torch.sort(ti, dim=1)
        w2 = torch.gather(tw, 1, perm)
        expt = ids2.reshape(-1).to(torch.int32)
        topk_indx = torch.argsort(expt, stable=True).to(torch.int32)
        gate_indx = torch.argsort(topk_indx, stable=True).to(torch.int32)
        gate_scal = w2.reshape(-1)[topk_indx.long()]
        hist = torch.histc(expt.float(), bins=E, max=E - 1).int()
        ed = compute_expt_data_torch(hist, E, T * k)
        return (RoutingData(gate_scal, hist, E, k, ed), GatherIndx(src_indx=topk_indx, dst_indx=gate_indx),
                ScatterIndx(src_indx=gate_indx, dst_indx=topk_indx))

    def experts(x, w1r, w2r, rd, gi, si):
        y1 = matmul_ogs(x, w1r, None, rd, gather_indx=gi)
        rows, two_i = y1.shape[-2], y1.shape[-1]
        act = y1.new_empty((rows, two_i // 2))
        block = 2048 if rows <= 128 else 1024
        silu_mul_kernel[(rows, triton.cdiv(two_i // 2, block))](y1, act, two_i // 2, BLOCK=block,
                                                               num_warps=8 if rows <= 128 else 4)
        out = matmul_ogs(act, w2r, None, rd, scatter_indx=si, gammas=rd.gate_scal)
        return out.view(x.shape[0], x.shape[1])

    return routing_tables, experts, triton


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="mixtral")
    ap.add_argument("--tokens", default="")
    ap.add_argument("--with-transpose", action="store_true")
    ap.add_argument("--plain-reps", type=int, default=0,
                    help="run each path this many times back to back without do_bench (for a profiler's launch list)")
    args = ap.parse_args()

    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import workloads as W

    cfg = W.CONFIGS[args.config]
    assert cfg.dtype == "bf16", "the reference path is bf16 only"
    routing_tables, tk_experts, triton = _import_triton_kernels()
    torch.cuda.set_device(0)
    wts = W.make_weights(cfg, "cuda", seed=0)
    w1r = wts["w1"].transpose(1, 2).contiguous()  # [E,H,2I]
    w2r = wts["w2"].transpose(1, 2).contiguous()  # [E,I,H]
    tokens = [int(t) for t in args.tokens.split(",")] if args.tokens else list(cfg.sweep_T)
    for T in tokens:
        tok = W.make_tokens(cfg, T, "cuda", seed=0)
        tw, ti = W.route(cfg, tok)
        x = tok["hidden"]

        def ours_experts():
            return fg.fused_experts(x, wts["w1"], wts["w2"], tw, ti)

        def ours_layer():
            return fg.fused_moe(x, wts["w1"], wts["w2"], tok["logits"], cfg.top_k, True)

        def ref_experts_only(tables=routing_tables(tw, ti, cfg.E)):
            return tk_experts(x, w1r, w2r, *tables)

        def ref_with_routing():
            a, b = (wts["w1"].transpose(1, 2).contiguous(), wts["w2"].transpose(1, 2).contiguous()) \
                if args.with_transpose else (w1r, w2r)
            return tk_experts(x, a, b, *routing_tables(tw, ti, cfg.E))

        rec = {"config": cfg.name, "T": T}
        if args.plain_reps:
            for _ in range(args.plain_reps):
                ref_experts_only()
            for _ in range(args.plain_reps):
                ours_experts()
            torch.cuda.synchronize()
            print(json.dumps({"config": cfg.name, "T": T, "plain_reps": args.plain_reps}), flush=True)
            continue
        try:
            ref = ref_experts_only()
            got = ours_experts()
            rec["rel_l2_vs_triton"] = float((got.float() - ref.float()).norm() / ref.float().norm())
            rec["triton_experts_ms"] = triton.testing.do_bench(ref_experts_only, warmup=50, rep=200, return_mode="median")
            rec["triton_routing_plus_experts_ms"] = triton.testing.do_bench(ref_with_routing, warmup=50, rep=200,
                                                                             return_mode="median")
        except Exception as e:  # the vendored copy is not pinned by the reference; report instead of failing
            rec["triton_error"] = f"{type(e).__name__}: {e}"[:300]
        rec["ours_experts_ms"] = triton.testing.do_bench(ours_experts, warmup=50, rep=200, return_mode="median")
        rec["ours_router_plus_experts_ms"] = triton.testing.do_bench(ours_layer, warmup=50, rep=200, return_mode="median")
        if "triton_experts_ms" in rec:
            rec["speedup_experts"] = rec["triton_experts_ms"] / rec["ours_experts_ms"]
            rec["speedup_with_routing"] = rec["triton_routing_plus_experts_ms"] / rec["ours_experts_ms"]
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
