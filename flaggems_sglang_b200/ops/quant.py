"""fp8-e4m3 block quantisation helpers (w8a8, 128x128 weight blocks, 1x128 activation groups).

The reference rejects fp8 (FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:170-185);
these follow the usual serving-side convention.
"""
from __future__ import annotations

import torch

from .. import _C

FP8_MAX = 448.0


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128):
    """x [rows, K] (bf16 or fp32) -> (q e4m3 [rows, K], scale f32 [rows, K/128]); CUDA kernel."""
    dev = _C.require_cuda(x)
    if group_size != 128:
        raise NotImplementedError("only group_size=128 is implemented")
    if x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("x must be a 2-D bf16 or fp32 tensor")
    x = x.contiguous()
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty(rows, K // 128, dtype=torch.float32, device=dev)
    _C.check(_C.lib().fmoe_quant_fp8_group128(x.data_ptr(), _C.DTYPE_CODE[x.dtype], rows, K, None, 1, 0, None,
                                              q.data_ptr(), s.data_ptr(), _C.stream_ptr(dev)))
    return q, s


def quant_weight_block128(w: torch.Tensor):
    """One-time weight preparation (torch ops, not on the per-token path):
    w [..., N, K] -> (q e4m3, scale f32 [..., N/128, K/128]), scale = amax(block)/448."""
    *lead, N, K = w.shape
    if N % 128 or K % 128:
        raise ValueError("N and K must be multiples of 128")
    if lead and w.shape[0] > 1:  # one slice at a time keeps the fp32 temporaries small
        parts = [quant_weight_block128(w[i]) for i in range(w.shape[0])]
        return torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts])
    blk = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    amax = blk.abs().amax(dim=(-3, -1))
    # tensor / tensor is an IEEE division on every device (tensor / python-scalar may multiply by a reciprocal)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, FP8_MAX), torch.ones_like(amax))
    q = (blk / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(*lead, N, K)
    return q.to(torch.float8_e4m3fn), scale.contiguous()


def per_token_quant_fp8(x: torch.Tensor):
    """x [rows, K] bf16 -> (q e4m3 [rows, K], scale f32 [rows]): one dynamic scale per row,
    scale = max(amax / 448, 1 / (448 * 512)); CUDA kernel.  The activation side of per-channel w8a8."""
    dev = _C.require_cuda(x)
    if x.dim() != 2 or x.dtype != torch.bfloat16:
        raise ValueError("x must be a 2-D bf16 tensor")
    x = x.contiguous()
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty(rows, dtype=torch.float32, device=dev)
    _C.check(_C.lib().fmoe_quant_fp8_per_token(x.data_ptr(), _C.BF16, rows, K, None, 1, 0, None, q.data_ptr(),
                                               s.data_ptr(), _C.stream_ptr(dev)))
    return q, s


def quant_weight_per_channel(w: torch.Tensor):
    """One-time weight preparation (torch ops): w [..., N, K] -> (q e4m3, scale f32 [..., N]),
    one scale per output channel, scale = amax(row)/448 (1 for an all-zero row)."""
    wf = w.float()
    amax = wf.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, FP8_MAX), torch.ones_like(amax))
    qv = (wf / scale[..., None]).clamp(-FP8_MAX, FP8_MAX)
    return qv.to(torch.float8_e4m3fn), scale.contiguous()


__all__ = ["per_token_group_quant_fp8", "quant_weight_block128", "per_token_quant_fp8", "quant_weight_per_channel"]
