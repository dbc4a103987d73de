"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configurations.

No model checkpoint or dataset is involved: hidden ~ N(0,1), w1 [E,2I,H] ~ N(0,1)/sqrt(H),
w2 [E,H,I] ~ N(0,1)/sqrt(I), router logits ~ N(0,1) fp32, generated with a seeded
torch.Generator on the requested device (weights expert by expert, so that the largest
configuration never holds more than one expert in fp32).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class MoEConfig:
    name: str
    H: int
    I: int
    E: int
    top_k: int
    dtype: str = "bf16"              # "fp32" | "bf16" | "fp8"
    router: str = "softmax"          # "softmax" | "grouped"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: Optional[float] = None
    sweep_T: tuple = field(default_factory=tuple)
    fp8_scales: str = "block128"     # fp8: "block128" (128x128 weight blocks, 1x128 activation groups) | "channel"


CONFIGS = {
    # Tiny fp32 layer (plumbing / correctness)
    "tiny": MoEConfig("tiny", H=256, I=512, E=8, top_k=2, dtype="fp32", sweep_T=(16,)),
    # Mixtral-8x7B MoE layer, bf16
    "mixtral": MoEConfig("mixtral", H=4096, I=14336, E=8, top_k=2, dtype="bf16", sweep_T=(1, 16, 64, 256, 1024, 4096)),
    # Qwen3-30B-A3B style, bf16
    "qwen3": MoEConfig("qwen3", H=2048, I=768, E=128, top_k=8, dtype="bf16", sweep_T=(1, 32, 512, 8192)),
    # DeepSeek-V3 style, fp8 w8a8 with 128x128 block scales, grouped router
    "dsv3": MoEConfig("dsv3", H=7168, I=2048, E=256, top_k=8, dtype="fp8", router="grouped", n_group=8,
                      topk_group=4, routed_scaling_factor=2.5, sweep_T=(1, 64, 1024, 16384)),
    # 32-expert cut of the DeepSeek-V3 layer (1.4 GB of weights): same tile shapes, small enough to profile
    # the same layer with per-output-channel weight scales and per-token activation scales (`per_channel_quant`)
    "dsv3_channel": MoEConfig("dsv3_channel", H=7168, I=2048, E=256, top_k=8, dtype="fp8", router="grouped", n_group=8,
                              topk_group=4, routed_scaling_factor=2.5, sweep_T=(64, 1024, 4096, 16384),
                              fp8_scales="channel"),
    "dsv3_channel_small": MoEConfig("dsv3_channel_small", H=7168, I=2048, E=32, top_k=8, dtype="fp8", router="grouped",
                                    n_group=8, topk_group=4, routed_scaling_factor=2.5, sweep_T=(64, 2048),
                                    fp8_scales="channel"),
    "dsv3_small": MoEConfig("dsv3_small", H=7168, I=2048, E=32, top_k=8, dtype="fp8", router="grouped", n_group=8,
                            topk_group=4, routed_scaling_factor=2.5, sweep_T=(64, 2048)),
    # shapes of the reference's own test/benchmark list (M,1280,3072,64,8)
    "refbench": MoEConfig("refbench", H=1280, I=3072, E=64, top_k=8, dtype="bf16", sweep_T=(1, 4, 17, 64, 1024, 2048, 4096)),
}

TORCH_DTYPE = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp8": torch.bfloat16}


def zipf_logit_bias(E: int, s: float, gen: torch.Generator, device) -> torch.Tensor:
    """log of a Zipf(s) pmf over a seeded random expert->rank permutation (hot and near-empty experts)."""
    ranks = torch.randperm(E, generator=gen, device=device).float() + 1.0
    pmf = ranks.pow(-s)
    pmf = pmf / pmf.sum()
    return pmf.log()


def make_weights(cfg: MoEConfig, device, seed: int = 0, num_experts: Optional[int] = None, expert_offset: int = 0):
    """-> dict(w1, w2[, w1_scale, w2_scale]).  `num_experts`/`expert_offset` build one rank's shard of the
    same global layer (expert e always gets the same values)."""
    from .ops.quant import quant_weight_block128, quant_weight_per_channel

    E = cfg.E if num_experts is None else num_experts
    dt = TORCH_DTYPE[cfg.dtype]
    fp8 = cfg.dtype == "fp8"
    wdt = torch.float8_e4m3fn if fp8 else dt
    w1 = torch.empty(E, 2 * cfg.I, cfg.H, dtype=wdt, device=device)
    w2 = torch.empty(E, cfg.H, cfg.I, dtype=wdt, device=device)
    out = {"w1": w1, "w2": w2}
    channel = fp8 and cfg.fp8_scales == "channel"
    if channel:
        out["w1_scale"] = torch.empty(E, 2 * cfg.I, dtype=torch.float32, device=device)
        out["w2_scale"] = torch.empty(E, cfg.H, dtype=torch.float32, device=device)
    elif fp8:
        out["w1_scale"] = torch.empty(E, 2 * cfg.I // 128, cfg.H // 128, dtype=torch.float32, device=device)
        out["w2_scale"] = torch.empty(E, cfg.H // 128, cfg.I // 128, dtype=torch.float32, device=device)
    for i in range(E):
        gen = torch.Generator(device=device)
        gen.manual_seed(seed * 1000003 + 7919 * (expert_offset + i) + 1)
        a = (torch.randn(2 * cfg.I, cfg.H, generator=gen, device=device) / math.sqrt(cfg.H)).to(dt)
        b = (torch.randn(cfg.H, cfg.I, generator=gen, device=device) / math.sqrt(cfg.I)).to(dt)
        if channel:
            qa, sa = quant_weight_per_channel(a)
            qb, sb = quant_weight_per_channel(b)
            w1[i], out["w1_scale"][i] = qa, sa
            w2[i], out["w2_scale"][i] = qb, sb
        elif fp8:
            if torch.device(device).type == "cuda":
                qa, sa = quant_weight_block128(a)
                qb, sb = quant_weight_block128(b)
            else:
                qa, sa = _quant_weight_cpu(a)
                qb, sb = _quant_weight_cpu(b)
            w1[i], out["w1_scale"][i] = qa, sa
            w2[i], out["w2_scale"][i] = qb, sb
        else:
            w1[i], w2[i] = a, b
    return out


def _quant_weight_cpu(w: torch.Tensor):
    N, K = w.shape
    blk = w.float().reshape(N // 128, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / torch.full_like(amax, 448.0), torch.ones_like(amax))
    q = (blk / scale[:, None, :, None]).clamp(-448.0, 448.0).reshape(N, K)
    return q.to(torch.float8_e4m3fn), scale.contiguous()


def make_tokens(cfg: MoEConfig, T: int, device, seed: int = 0, skew: bool = False):
    """-> dict(hidden [T,H], logits [T,E] f32[, correction_bias [E] f32])."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 7907 + 13)
    dt = TORCH_DTYPE[cfg.dtype]
    hidden = torch.randn(T, cfg.H, generator=gen, device=device).to(dt)
    logits = torch.randn(T, cfg.E, generator=gen, device=device, dtype=torch.float32)
    out = {"hidden": hidden, "logits": logits}
    if skew:
        out["logits"] = logits + zipf_logit_bias(cfg.E, 1.2, gen, device)[None, :]
    if cfg.router == "grouped":
        out["correction_bias"] = torch.randn(cfg.E, generator=gen, device=device) * 0.1  # N(0, 0.01) variance
    return out


def route(cfg: MoEConfig, tokens: dict):
    """Routing of `tokens` with the configuration's router -> (topk_weights, topk_ids)."""
    from .ops.topk import topk

    return topk(tokens["hidden"], tokens["logits"], cfg.top_k, True, cfg.router == "grouped", cfg.n_group,
                cfg.topk_group, tokens.get("correction_bias"), None)


def algorithmic_bytes_flops(cfg: MoEConfig, T: int, active_experts: int):
    """Bytes that must cross HBM and flops of one layer call (intermediates and re-reads are not algorithmic)."""
    bw = 1 if cfg.dtype == "fp8" else (4 if cfg.dtype == "fp32" else 2)
    ba = bw
    H, I, k = cfg.H, cfg.I, cfg.top_k
    b = active_experts * 3 * H * I * bw + T * H * ba + T * H * 2 + T * k * 8
    if cfg.dtype == "fp8" and cfg.fp8_scales == "channel":
        b += active_experts * (2 * I + H) * 4 + T * 4
    elif cfg.dtype == "fp8":
        b += active_experts * ((2 * I // 128) * (H // 128) + (H // 128) * (I // 128)) * 4 + T * (H // 128) * 4
    return b, 6 * T * k * H * I
