"""moe_sum: reduce the top-k expert outputs of every token.

Takes over the grouped reduce that ends the reference's second grouped GEMM
(FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:224-231): fp32 adds in
ascending slot order, one rounding to the output dtype.
"""
from __future__ import annotations

import torch

from .. import _C


def moe_sum(input: torch.Tensor, output: torch.Tensor, routed_scaling_factor: float | None = None,
            shared_output: torch.Tensor | None = None) -> torch.Tensor:
    """``output[t] = sum_j input[t, j]`` for ``input [T, k, H]``; writes and returns ``output [T, H]``.
    ``routed_scaling_factor`` multiplies the rounded sum; ``shared_output [T, H]`` (the shared expert's result) is
    then added with one more rounding — the two steps a caller would otherwise run as separate passes."""
    dev = _C.require_cuda(input, output, shared_output)
    if shared_output is not None and (shared_output.shape != output.shape or shared_output.dtype != output.dtype
                                      or not shared_output.is_contiguous()):
        raise ValueError("shared_output must be a contiguous [T,H] tensor of the output dtype")
    if input.dim() != 3 or output.dim() != 2 or input.shape[0] != output.shape[0] or input.shape[2] != output.shape[1]:
        raise ValueError("moe_sum expects input [T,k,H] and output [T,H]")
    if input.dtype != output.dtype or input.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("moe_sum supports bf16 and fp32 with matching input/output dtypes")
    if not input.is_contiguous() or not output.is_contiguous():
        raise ValueError("moe_sum needs contiguous tensors")
    T, k, H = input.shape
    scale = 1.0 if routed_scaling_factor is None else float(routed_scaling_factor)
    _C.check(_C.lib().fmoe_moe_sum_add(input.data_ptr(), _C.DTYPE_CODE[input.dtype], T, k, H, scale,
                                       _C.ptr(shared_output), output.data_ptr(), _C.stream_ptr(dev)))
    return output


__all__ = ["moe_sum"]
