"""Router ops: softmax top-k and DeepSeek-V3 grouped, bias-corrected sigmoid top-k.

The reference leaves routing to its caller and only consumes
``topk_weights`` / ``topk_ids`` (FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:355-366);
its test builds them as softmax -> topk -> renormalise (tests/test_fused_moe.py:38-41).
Both routers here run as one CUDA kernel with one warp per token.
"""
from __future__ import annotations

import torch

from .. import _C


def _prep_logits(gating_output: torch.Tensor) -> torch.Tensor:
    _C.require_cuda(gating_output)
    if gating_output.dim() != 2:
        raise ValueError("gating_output must be [num_tokens, num_experts]")
    g = gating_output
    if g.dtype != torch.float32:
        g = g.float()
    return g.contiguous()


def fused_topk(hidden_states, gating_output: torch.Tensor, topk: int, renormalize: bool = True):
    """softmax over experts -> top-k -> optional renormalisation.

    Returns ``(topk_weights float32 [T,k], topk_ids int32 [T,k])`` ordered by
    descending weight; ties go to the lower expert index.  ``hidden_states`` is
    only checked for the token count (the serving-side signature carries it).
    """
    g = _prep_logits(gating_output)
    T, E = g.shape
    if hidden_states is not None and hidden_states.shape[0] != T:
        raise ValueError("Number of tokens mismatch")
    w = torch.empty(T, topk, dtype=torch.float32, device=g.device)
    ids = torch.empty(T, topk, dtype=torch.int32, device=g.device)
    _C.check(_C.lib().fmoe_topk_softmax(g.data_ptr(), T, E, topk, int(bool(renormalize)), w.data_ptr(),
                                        ids.data_ptr(), _C.stream_ptr(g.device)))
    return w, ids


def grouped_topk(
    hidden_states,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool,
    num_expert_group: int,
    topk_group: int,
    correction_bias: torch.Tensor | None = None,
    routed_scaling_factor: float | None = None,
):
    """Group-limited top-k on sigmoid scores with a per-expert selection bias.

    ``s = sigmoid(logits)``, ``c = s + bias``; a group's score is the sum of its two
    largest ``c``; the ``topk_group`` best groups stay; ids are the top-k of ``c``
    inside them; weights are ``s[ids]``, renormalised by ``sum + 1e-20`` and
    multiplied by ``routed_scaling_factor`` when given.
    """
    g = _prep_logits(gating_output)
    T, E = g.shape
    if hidden_states is not None and hidden_states.shape[0] != T:
        raise ValueError("Number of tokens mismatch")
    bias = None
    if correction_bias is not None:
        _C.require_cuda(correction_bias)
        bias = correction_bias.float().contiguous()
        if bias.numel() != E:
            raise ValueError("correction_bias must have num_experts entries")
    w = torch.empty(T, topk, dtype=torch.float32, device=g.device)
    ids = torch.empty(T, topk, dtype=torch.int32, device=g.device)
    scale = 1.0 if routed_scaling_factor is None else float(routed_scaling_factor)
    _C.check(_C.lib().fmoe_topk_grouped(g.data_ptr(), _C.ptr(bias), T, E, topk, num_expert_group, topk_group,
                                        int(bool(renormalize)), scale, w.data_ptr(), ids.data_ptr(),
                                        _C.stream_ptr(g.device)))
    return w, ids


def topk(hidden_states, gating_output, topk: int, renormalize: bool = True, use_grouped_topk: bool = False,
         num_expert_group: int | None = None, topk_group: int | None = None, correction_bias=None,
         routed_scaling_factor: float | None = None):
    """Single entry for both routers, selected by ``use_grouped_topk``."""
    if use_grouped_topk:
        if num_expert_group is None or topk_group is None:
            raise ValueError("grouped top-k needs num_expert_group and topk_group")
        return grouped_topk(hidden_states, gating_output, topk, renormalize, num_expert_group, topk_group,
                            correction_bias, routed_scaling_factor)
    return fused_topk(hidden_states, gating_output, topk, renormalize)


__all__ = ["fused_topk", "grouped_topk", "topk"]
