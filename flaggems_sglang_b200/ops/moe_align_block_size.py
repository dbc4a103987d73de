"""moe_align_block_size: expert-sorted, block-padded token index buffers.

Takes over the routing-table construction the reference does with ~40 small torch
launches and host syncs (FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:119-146):
one CUDA kernel (histogram -> warp scan -> stable scatter), no host sync.
"""
from __future__ import annotations

import torch

from .. import _C


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Returns ``(sorted_token_ids, expert_ids, num_tokens_post_padded)``.

    ``sorted_token_ids`` (int32, ``numel + E*(block_size-1)``) lists, expert by
    expert, the flat indices ``t*k+j`` routed to that expert in ascending order,
    each expert padded to a multiple of ``block_size`` with the sentinel
    ``numel``; unused tail entries also hold the sentinel.  ``expert_ids`` gives
    the expert of every used block and -1 after them.  ``num_tokens_post_padded``
    is a one-element int32 tensor.  Ids outside ``[0, num_experts)`` are dropped.
    """
    dev = _C.require_cuda(topk_ids)
    ids = topk_ids
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    numel = ids.numel()
    cap = numel + num_experts * (block_size - 1)
    nblk = (cap + block_size - 1) // block_size
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(nblk, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    lib = _C.lib()
    ws_bytes = lib.fmoe_moe_align_workspace_bytes(numel, num_experts) if numel >= 8192 else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
    _C.check(lib.fmoe_moe_align_block_size_ws(ids.data_ptr(), numel, num_experts, block_size, sorted_ids.data_ptr(),
                                              cap, expert_ids.data_ptr(), nblk, num_post.data_ptr(), _C.ptr(ws),
                                              ws_bytes, _C.stream_ptr(dev)))
    return sorted_ids, expert_ids, num_post


__all__ = ["moe_align_block_size"]
