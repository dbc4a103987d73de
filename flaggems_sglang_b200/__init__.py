"""B200-native (sm_100a) fused-MoE operators behind the FlagGems-sglang operator API.

    import flaggems_sglang_b200 as fg
    out = fg.fused_moe(hidden, w1, w2, router_logits, topk=2, renormalize=True)

Every op of `flaggems_sglang_b200.ops` is also available at package level, as the
reference exposes its ops (FlagGems-sglang src/flaggems_sglang/__init__.py:34-35).
The CUDA library must be built first (`python -m flaggems_sglang_b200.build`);
ops raise if it is missing or if they are given CPU tensors.
"""
from . import ops
from .ops import *  # noqa: F401,F403
from .ops import __all__ as _ops_all

device = "cuda"
vendor_name = "nvidia"


def all_registered_ops():
    return list(_ops_all)


def get_op(name: str):
    return getattr(ops, name)


__all__ = list(_ops_all) + ["ops", "all_registered_ops", "get_op", "device", "vendor_name"]
