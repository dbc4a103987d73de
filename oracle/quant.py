"""Oracle (test infrastructure): fp8-e4m3 block quantisation on CPU.

The reference rejects fp8 (ref:src/flaggems_sglang/ops/fused_moe.py:170-185),
so these contracts are builder-defined ("parity unpinned").  They follow the
usual w8a8 block-quant convention: weights carry one fp32 scale per 128x128
block, activations one fp32 scale per token per 128 channels.
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
GROUP = 128


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to e4m3 with saturation at +-448."""
    return x.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def quant_weight_block128(w: torch.Tensor):
    """w [..., N, K] (N, K multiples of 128) -> (q e4m3 same shape, scale f32 [..., N/128, K/128]).

    scale = amax(block)/448 (1.0 for an all-zero block); q = rne(w / scale).
    """
    *lead, N, K = w.shape
    wf = w.detach().cpu().to(torch.float32)
    blk = wf.reshape(*lead, N // GROUP, GROUP, K // GROUP, GROUP)
    amax = blk.abs().amax(dim=(-3, -1))  # [..., N/128, K/128]
    scale = torch.where(amax > 0, amax / torch.full_like(amax, FP8_MAX), torch.ones_like(amax))
    q = blk / scale[..., :, None, :, None]
    return to_e4m3(q.reshape(*lead, N, K)), scale.contiguous()


def dequant_weight_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    *lead, N, K = q.shape
    blk = q.detach().cpu().to(torch.float32).reshape(*lead, N // GROUP, GROUP, K // GROUP, GROUP)
    return (blk * scale.cpu()[..., :, None, :, None]).reshape(*lead, N, K)


def quant_act_group128(x: torch.Tensor):
    """x [rows, K] -> (q e4m3 [rows, K], scale f32 [rows, K/128]).

    scale = max(amax(group), 1e-10)/448; q = rne(clamp(x / scale, +-448)),
    the division done in fp32.
    """
    rows, K = x.shape
    xf = x.detach().cpu().to(torch.float32).reshape(rows, K // GROUP, GROUP)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-10)
    scale = amax / torch.full_like(amax, FP8_MAX)
    q = xf / scale[..., None]
    return to_e4m3(q.reshape(rows, K)), scale.contiguous()


def dequant_act_group128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    xf = q.detach().cpu().to(torch.float32).reshape(rows, K // GROUP, GROUP)
    return (xf * scale.cpu()[..., None]).reshape(rows, K)


# ---- per-channel w8a8: one scale per output channel of the weights, one dynamic scale per activation row ----
# (`per_channel_quant`, asserted off in the reference at src/flaggems_sglang/ops/fused_moe.py:173-175; the rule below
# is the one vLLM's dynamic per-token quantiser and its fp8 MoE kernels follow: parity unpinned against the reference,
# cross-checked against vLLM on the GPU.)
MIN_TOKEN_SCALE = 1.0 / (FP8_MAX * 512.0)


def quant_weight_per_channel(w: torch.Tensor):
    """w [..., N, K] -> (q e4m3 same shape, scale f32 [..., N]); scale = amax(row)/448 (1.0 for a zero row)."""
    wf = w.detach().cpu().to(torch.float32)
    amax = wf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, FP8_MAX), torch.ones_like(amax))
    return to_e4m3(wf / scale[..., None]), scale.contiguous()


def quant_act_per_token(x: torch.Tensor):
    """x [rows, K] -> (q e4m3 [rows, K], scale f32 [rows]); scale = max(amax/448, 1/(448*512)), q = rne(x/scale)."""
    xf = x.detach().cpu().to(torch.float32)
    amax = xf.abs().amax(dim=-1)
    scale = (amax / torch.full_like(amax, FP8_MAX)).clamp_min(MIN_TOKEN_SCALE)
    return to_e4m3(xf / scale[:, None]), scale.contiguous()
