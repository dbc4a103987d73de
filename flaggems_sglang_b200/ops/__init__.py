"""Operators of the fused-MoE path (flat namespace, no vendor registry)."""
from .fused_moe import (  # noqa: F401
    GatherIndx,
    RoutingData,
    ScatterIndx,
    fused_experts,
    fused_moe,
    fused_moe_flagos,
    standard_topk_to_routing,
    triton_kernel_fused_experts,
    triton_kernel_fused_experts_with_bias,
)
from .moe_align_block_size import moe_align_block_size  # noqa: F401
from .moe_sum import moe_sum  # noqa: F401
from .quant import (  # noqa: F401
    per_token_group_quant_fp8, per_token_quant_fp8, quant_weight_block128, quant_weight_per_channel,
)
from .topk import fused_topk, grouped_topk, topk  # noqa: F401

__all__ = [
    "fused_experts", "fused_moe", "triton_kernel_fused_experts", "triton_kernel_fused_experts_with_bias",
    "fused_moe_flagos",
    "standard_topk_to_routing", "RoutingData", "GatherIndx", "ScatterIndx",
    "moe_align_block_size", "moe_sum", "per_token_group_quant_fp8", "quant_weight_block128",
    "per_token_quant_fp8", "quant_weight_per_channel",
    "fused_topk", "grouped_topk", "topk",
]
