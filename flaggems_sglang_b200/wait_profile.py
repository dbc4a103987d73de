"""Where the cycles of a tcgen05 grouped GEMM go: per-role wait counters kept by the instrumented kernels.

    FMOE_TC_PROFILE=1 python -m flaggems_sglang_b200.wait_profile [--config mixtral] [--tokens 4096]

Runs the layer's expert computation a few times with the library's stage events, then reads the counters of the
LAST launches with `fmoe_debug_wait_profile` and prints them per tile (bf16 kernels: MMA warp waiting for its
accumulator / for TMA data, producer waiting for a free stage, epilogue wait and busy) or per K block (e4m3 kernel:
fold warps waiting for the MMAs / busy, per tile: wait for staged scales, epilogue).  With `FMOE_TC_DEBUG=1` the bf16
kernels skip their TMA loads and the MMA warp never waits for data (results are wrong; the time is the pure MMA
stream), with bit 1 (`=2`) they issue no MMAs (the TMA ring alone), with bit 2 (`=4`, `=5`) B is read as an N-major
operand; `FMOE_TC_MAX_CTAS=<n>` caps the grid.  `FMOE_FP8_DEBUG=<bits>` does the same kind of experiment on the e4m3
kernel (see gemm_tcgen05_fp8.cu).
Reading the clock inside the e4m3 fold loop distorts it: use those figures for proportions, the stage times for speed.
"""
from __future__ import annotations

import argparse
import ctypes
import os

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="mixtral")
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    if not any(os.environ.get(v) for v in ("FMOE_TC_PROFILE", "FMOE_FP8_DEBUG", "FMOE_TC_DEBUG", "FMOE_TC_MAX_CTAS")):
        raise SystemExit("set FMOE_TC_PROFILE=1 (counters) or FMOE_TC_DEBUG / FMOE_FP8_DEBUG=<bits> / FMOE_TC_MAX_CTAS=<n> "
                         "(timing experiments) first")

    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import _C, workloads as W

    cfg = W.CONFIGS[args.config]
    wts = W.make_weights(cfg, "cuda", seed=0)
    tok = W.make_tokens(cfg, args.tokens, "cuda", seed=0)
    tw, ti = W.route(cfg, tok)
    kw = {}
    if cfg.dtype == "fp8":
        kw = dict(use_fp8_w8a8=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"], block_shape=[128, 128])
    lib = _C.lib()
    n = 7
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
    for e in evs:
        e.record()
    torch.cuda.synchronize()
    arr = (ctypes.c_void_p * n)(*[e.cuda_event for e in evs])
    for _ in range(args.steps):
        _C.check(lib.fmoe_debug_stage_events(arr, n))
        fg.fused_experts(tok["hidden"], wts["w1"], wts["w2"], tw, ti, variant="tcgen05", **kw)
    torch.cuda.synchronize()
    _C.check_device_status()
    g1, g2 = evs[2].elapsed_time(evs[3]), evs[4].elapsed_time(evs[5])
    try:
        mhz = f", SM clock now {torch.cuda.clock_rate()} MHz"
    except Exception:  # noqa: BLE001  (needs NVML)
        mhz = ""
    print(f"{cfg.name} T={args.tokens} tcgen05: gate/up GEMM {g1:.3f} ms, down GEMM {g2:.3f} ms (last of {args.steps} calls){mhz}")
    if not os.environ.get("FMOE_TC_PROFILE"):
        return
    sms = lib.fmoe_sm_count()
    if cfg.dtype == "fp8":
        buf = (ctypes.c_int64 * 4096)()
        _C.check(lib.fmoe_debug_wait_profile(-_C.VARIANTS["tcgen05"], buf, 4096))
        both = np.array(buf).reshape(2, 256, 8)[:, :sms]
        for name, a, kb in (("gate/up", both[1], cfg.H // 128), ("down", both[0], cfg.I // 128)):
            tiles = a[:, 0].sum()
            print(f"  {name}: {a[:, 0].mean():.1f} tiles per CTA, {kb} K blocks per tile, kernel {a[:, 5].mean():.0f} clock ticks per CTA")
            print("    per K block: fold waits %.0f, fold busy %.0f; per tile: waits for staged scales %.0f, epilogue %.0f"
                  % (a[:, 1].sum() / tiles / kb, a[:, 2].sum() / tiles / kb, a[:, 3].sum() / tiles, a[:, 4].sum() / tiles))
        return
    buf = (ctypes.c_int64 * (sms * 8))()
    _C.check(lib.fmoe_debug_wait_profile(_C.VARIANTS["tcgen05"], buf, sms * 8))  # the last launch: the down GEMM
    a = np.array(buf).reshape(sms, 8)
    lead = a[a[:, 0] > 0]
    tiles = lead[:, 0].sum()
    all_tiles = tiles * (sms / len(lead))
    print(f"  down GEMM: {len(lead)} CTAs issue MMAs, {tiles / len(lead):.1f} tiles each; per tile (clock cycles):")
    print("    MMA warp waits for its accumulator %.0f, for TMA data %.0f; producer waits for a free stage %.0f; "
          "epilogue waits %.0f, busy %.0f" % (lead[:, 1].sum() / tiles, lead[:, 2].sum() / tiles, a[:, 3].sum() / all_tiles,
                                             a[:, 4].sum() / all_tiles, a[:, 5].sum() / all_tiles))


if __name__ == "__main__":
    main()
