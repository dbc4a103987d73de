"""Fused MoE expert computation on B200: align -> gate/up GEMM + silu*mul -> down GEMM * weight -> sum.

Host-side mirror of the reference operator
(FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py): the same entry points
(`triton_kernel_fused_experts`, `fused_moe_flagos`), argument meaning and error
behaviour, plus the serving-side `fused_experts` / `fused_moe` signatures on the
`w1 [E,2I,H]`, `w2 [E,H,I]` layouts.  All arithmetic runs in the hand-written
CUDA kernels behind the C ABI (include/fmoe_b200.h); nothing falls back to
torch or the CPU.

Kernel selection (per call, from shapes only, no host sync):
  rows per active expert <= 4    -> "stream": small-M weight-streaming kernel,
                                    moe_align block 8, x gathered on the fly
  larger                         -> "tcgen05": rows copied into expert-sorted order
                                    (block 128), TMA + tcgen05/TMEM persistent kernel
  fp32 inputs                    -> "simt"
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _C
from .moe_align_block_size import moe_align_block_size
from .topk import topk as _route

logger = logging.getLogger(__name__)

_UNSUPPORTED_FEATURE_MSG = "{name} is not supported"

# Optional per-stage timing for benchmarks: set to a list and every fused_experts call appends
# (stage name, start event, end event) recorded on the launching stream.  None = no events.
STAGE_EVENTS: Optional[list] = None


class _stage:
    """Context manager bracketing one kernel launch with CUDA events when STAGE_EVENTS is a list."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if STAGE_EVENTS is not None:
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t0.record()
        return self

    def __exit__(self, *exc):
        if STAGE_EVENTS is not None:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record()
            STAGE_EVENTS.append((self.name, self.t0, t1))
        return False


# --------------------------------------------------------------------------
# routing containers accepted by the reference-layout entry point
# --------------------------------------------------------------------------
@dataclass
class GatherIndx:
    src_indx: torch.Tensor  # sorted position -> flat slot
    dst_indx: torch.Tensor  # flat slot -> sorted position


@dataclass
class ScatterIndx:
    src_indx: torch.Tensor
    dst_indx: torch.Tensor


@dataclass
class RoutingData:
    gate_scal: torch.Tensor  # [T*k] weights in expert-sorted order
    expt_hist: torch.Tensor  # [E] rows per expert
    n_expts_tot: int
    n_expts_act: int
    expt_data: object = None


def standard_topk_to_routing(topk_weights: torch.Tensor, topk_ids: torch.Tensor, n_expts_tot: int):
    """(topk_weights, topk_ids) -> (RoutingData, GatherIndx, ScatterIndx).

    Same tables as the reference's `_standard_topk_to_triton_kernels`
    (src/flaggems_sglang/ops/fused_moe.py:119-146) without the per-block tile maps,
    which only the third-party grouped GEMM needs.  Torch ops; kept for callers that
    hold routing in this format — `fused_experts` does not go through it.
    """
    T, k = topk_weights.shape
    ids2, perm = torch.sort(topk_ids, dim=1)
    w2 = torch.gather(topk_weights, 1, perm)
    expt = ids2.reshape(-1).to(torch.int32)
    topk_indx = torch.argsort(expt, stable=True).to(torch.int32)
    gate_indx = torch.argsort(topk_indx, stable=True).to(torch.int32)
    gate_scal = w2.reshape(-1)[topk_indx.long()]
    hist = torch.bincount(expt.long(), minlength=n_expts_tot)[:n_expts_tot].to(torch.int32)
    rd = RoutingData(gate_scal, hist, n_expts_tot, k)
    return rd, GatherIndx(topk_indx, gate_indx), ScatterIndx(gate_indx, topk_indx)


# --------------------------------------------------------------------------
# kernel selection
# --------------------------------------------------------------------------
def _pick_variant(dtype, numel: int, E: int, I: int, H: int, forced: Optional[str]):
    """-> (kernel family name, moe_align block size); the choice is made by the library (fmoe_pick_variant)."""
    import ctypes

    forced = forced or os.environ.get("FMOE_VARIANT") or "auto"
    if forced not in _C.VARIANTS:
        raise ValueError(f"unknown variant {forced!r}")
    v, b = ctypes.c_int(0), ctypes.c_int(0)
    rc = _C.lib().fmoe_pick_variant(_C.DTYPE_CODE[dtype], numel, E, I, H, _C.VARIANTS[forced], ctypes.byref(v),
                                    ctypes.byref(b))
    if rc != _C.OK:
        raise ValueError(_C.lib().fmoe_last_error().decode())
    return _C.VARIANT_NAMES[v.value], b.value


def _gemm_args(**kw) -> _C.GemmArgs:
    a = _C.GemmArgs()
    for key, val in kw.items():
        setattr(a, key, val)
    return a


# --------------------------------------------------------------------------
# serving-side entry points
# --------------------------------------------------------------------------
def fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    per_channel_quant: bool = False,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
    no_combine: bool = False,
    routed_scaling_factor: Optional[float] = None,
    expert_map: Optional[torch.Tensor] = None,
    global_num_experts: int = -1,
    variant: Optional[str] = None,
    out_rows: Optional[torch.Tensor] = None,
    b1: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None,
    gemm1_alpha: Optional[float] = None,
    gemm1_clamp_limit: Optional[float] = None,
    weights_n_major: bool = False,
) -> torch.Tensor:
    """Expert computation for already-routed tokens.

    hidden_states [T,H]; w1 [E,2I,H] (rows [0,I) gate, [I,2I) up); w2 [E,H,I];
    topk_weights [T,k] float; topk_ids [T,k] int.  bf16 (or fp32) weights, or
    e4m3 weights with `use_fp8_w8a8=True`, `block_shape=[128,128]` and fp32
    block scales `w1_scale [E,2I/128,H/128]`, `w2_scale [E,H/128,I/128]`
    (activations are quantised per token per 128 channels on the fly), or with
    `per_channel_quant=True` (no `block_shape`): `w1_scale [E,2I]`, `w2_scale [E,H]`, one scale per output
    channel, activations quantised with one dynamic scale per token (tensor-core kernels only).
    Returns [T,H] (or [T,k,H] with `no_combine`).  `expert_map` maps global to
    local expert ids (-1 = not on this rank; such slots contribute zeros).
    `out_rows` (with `no_combine`): int64 [T*k] device addresses; the result row of every slot is stored
    there by the down-projection kernel instead of into a [T,k,H] tensor (0 = skip), and None is returned.
    Used by the expert-parallel path, whose addresses are slot rows in the source ranks' memory.
    `b1 [E,2I]` (gate entries then up entries) / `b2 [E,H]`: optional biases of the two projections;
    `activation="swiglu_oai"` with `gemm1_alpha` (default 1.702) and `gemm1_clamp_limit` (None = no clamp) is
    the gated unit of the reference's bias variant (src/flaggems_sglang/ops/fused_moe.py:235-325): bias, then
    activation, then top-k weight.  bf16 / fp32 weights only.
    `weights_n_major=True`: w1 is [E,H,2I] and w2 [E,I,H] (the layout the reference operator takes,
    src/flaggems_sglang/ops/fused_moe.py:192-199), read in place by the bf16 tensor-core kernels as an N-major
    operand; see `n_major_supported` for the shapes this covers.
    """
    logger.debug("FLAGGEMS_SGLANG_B200 FUSED_EXPERTS")
    assert inplace is False, "Inplace is not supported"
    assert a1_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a1_scale")
    assert a2_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a2_scale")
    if activation not in _C.ACTIVATIONS:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    dev = _C.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, expert_map)
    assert hidden_states.ndim == 2, "hidden_states must be 2D"
    T, H = hidden_states.shape
    if weights_n_major:
        E, Hw, twoI = w1.shape
        assert tuple(w2.shape) == (E, twoI // 2, H), "intermediate size mismatch"
        assert n_major_supported(w1, w2, activation) and b1 is None and b2 is None and not use_fp8_w8a8, \
            "weights_n_major needs contiguous bf16 weights with H % 32 == 0 and I % 32 == 0, silu or gelu, no bias"
        assert STAGE_EVENTS is None, "the per-stage profiling path takes [E,2I,H] / [E,H,I] weights only"
        w2 = w2.transpose(1, 2)  # shape bookkeeping below; the memory is never touched in this order
    else:
        E, twoI, Hw = w1.shape
    I = twoI // 2
    assert Hw == H, "hidden size mismatch"
    assert w2.shape[0] == E and w2.shape[1] == H and w2.shape[2] == I, "intermediate size mismatch"
    assert topk_ids.shape == topk_weights.shape and topk_ids.shape[0] == T, "topk shape mismatch"
    k = topk_ids.shape[1]
    numel = T * k

    if per_channel_quant:
        # one scale per output channel of the weights, one dynamic scale per activation row
        assert use_fp8_w8a8, "per_channel_quant needs use_fp8_w8a8=True"
        assert block_shape is None, "per_channel_quant and block_shape are mutually exclusive"
        assert w1.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn, "fp8 weights must be e4m3"
        assert w1_scale is not None and w2_scale is not None, "fp8 needs w1_scale and w2_scale"
        assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
        assert H % 32 == 0 and I % 32 == 0, "per-channel fp8 needs H and I to be multiples of 32"
        assert w1_scale.numel() == E * twoI and w2_scale.numel() == E * H, "w1_scale must be [E,2I], w2_scale [E,H]"
        assert b1 is None and b2 is None and activation != "swiglu_oai", "bias / swiglu_oai are not available with fp8"
        w1_scale = w1_scale.float().reshape(E, twoI).contiguous()
        w2_scale = w2_scale.float().reshape(E, H).contiguous()
    elif use_fp8_w8a8:
        assert block_shape is not None and list(block_shape) == [128, 128], "fp8 needs block_shape=[128, 128]"
        assert w1.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn, "fp8 weights must be e4m3"
        assert w1_scale is not None and w2_scale is not None, "fp8 needs w1_scale and w2_scale"
        assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
        assert H % 128 == 0 and I % 128 == 0, "fp8 block quantisation needs H and I to be multiples of 128"
        assert tuple(w1_scale.shape) == (E, twoI // 128, H // 128), "w1_scale shape"
        assert tuple(w2_scale.shape) == (E, H // 128, I // 128), "w2_scale shape"
        w1_scale = w1_scale.float().contiguous()
        w2_scale = w2_scale.float().contiguous()
    else:
        assert w1_scale is None and w2_scale is None and block_shape is None, "scales given without use_fp8_w8a8"
        assert hidden_states.dtype in (torch.bfloat16, torch.float32), "hidden_states must be bfloat16 or float32"
        assert w1.dtype == hidden_states.dtype and w2.dtype == hidden_states.dtype, "w1/w2 dtype must match hidden_states"
    out_dtype = hidden_states.dtype
    x = hidden_states.contiguous()
    if not weights_n_major:
        w1 = w1.contiguous()
        w2 = w2.contiguous()
    wts = topk_weights.float().contiguous()
    ids = topk_ids
    if expert_map is not None:
        ids = expert_map.to(torch.int32)[topk_ids.long()]
    ids = ids.to(torch.int32).contiguous()

    if b1 is not None or b2 is not None or activation == "swiglu_oai":
        assert not use_fp8_w8a8, "bias / swiglu_oai are not available with fp8 weights"
        assert b1 is None or tuple(b1.shape) == (E, twoI), "b1 must be [E, 2I]"
        assert b2 is None or tuple(b2.shape) == (E, H), "b2 must be [E, H]"
        if b1 is not None or b2 is not None:
            _C.require_cuda(hidden_states, b1, b2)
        b1 = None if b1 is None else b1.float().contiguous()
        b2 = None if b2 is None else b2.float().contiguous()
    act_alpha = 1.702 if gemm1_alpha is None else float(gemm1_alpha)
    act_limit = 0.0 if gemm1_clamp_limit is None else float(gemm1_clamp_limit)
    if out_rows is not None:
        assert no_combine and expert_map is None, "out_rows needs no_combine and no expert_map"
        assert out_rows.dtype == torch.int64 and out_rows.numel() >= numel and out_rows.is_contiguous()
    if T == 0:
        return None if out_rows is not None else x.new_empty((0, k, H) if no_combine else (0, H))

    lib = _C.lib()
    st = _C.stream_ptr(dev)
    if STAGE_EVENTS is None:
        # production path: one library call, intermediates in one workspace tensor
        forced = variant or os.environ.get("FMOE_VARIANT") or "auto"
        if forced not in _C.VARIANTS:
            raise ValueError(f"unknown variant {forced!r}")
        out = None if out_rows is not None else torch.empty((T, k, H) if no_combine else (T, H), dtype=out_dtype,
                                                            device=dev)
        fa = _C.FusedArgs(
            w_layout=_C.W_N_MAJOR if weights_n_major else _C.W_K_MAJOR,
            scale_mode=_C.SCALE_CHANNEL if per_channel_quant else _C.SCALE_BLOCK128,
            dtype=_C.E4M3 if use_fp8_w8a8 else _C.DTYPE_CODE[out_dtype], variant=_C.VARIANTS[forced], num_experts=E,
            top_k=k, apply_router_weight_on_input=int(apply_router_weight_on_input), no_combine=int(no_combine),
            zero_dropped=int(expert_map is not None), activation=_C.ACTIVATIONS[activation], T=T, H=H, I=I,
            routed_scaling_factor=1.0 if routed_scaling_factor is None else float(routed_scaling_factor),
            hidden=x.data_ptr(), w1=w1.data_ptr(), w2=w2.data_ptr(), w1_scale=_C.ptr(w1_scale),
            w2_scale=_C.ptr(w2_scale), topk_weights=wts.data_ptr(), topk_ids=ids.data_ptr(), out=_C.ptr(out),
            out_rows=_C.ptr(out_rows), b1=_C.ptr(b1), b2=_C.ptr(b2), act_alpha=act_alpha, act_limit=act_limit)
        need = lib.fmoe_fused_experts_workspace_bytes(fa)
        if need < 0:
            _C.check(_C.ERR_INVALID_ARG)
        ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=dev)
        fa.workspace, fa.workspace_bytes = ws.data_ptr(), ws.numel()
        _C.check(lib.fmoe_fused_experts(fa, st))
        return out

    # profiling path (STAGE_EVENTS set): the same kernels launched one by one with events around each launch
    if per_channel_quant:
        name, block = "tcgen05", 128  # the one kernel family of this format
    else:
        name, block = _pick_variant(w1.dtype if not use_fp8_w8a8 else torch.float8_e4m3fn, numel, E, I, H, variant)
    vcode = _C.VARIANTS[name]

    with _stage("align"):
        sorted_ids, expert_ids, num_post = moe_align_block_size(ids, block, E)
    cap = sorted_ids.numel()
    max_blocks = min(cap // block, numel)
    row_w = wts.data_ptr()
    code = _C.DTYPE_CODE[out_dtype]
    common = dict(variant=vcode, activation=_C.ACTIVATIONS[activation], num_experts=E, top_k=k, block_size=block, numel=numel, sorted_cap=cap,
                  max_blocks=max_blocks, sorted_token_ids=sorted_ids.data_ptr(), expert_ids=expert_ids.data_ptr(),
                  num_tokens_post_padded=num_post.data_ptr())
    if name == "tcgen05" and (not use_fp8_w8a8 or per_channel_quant):
        # the scratch that lets the kernel cut the tiles of a part-filled last round along K, as the one-call path has
        split_ws = torch.empty(int(lib.fmoe_gemm_split_workspace_bytes()), dtype=torch.uint8, device=dev)
        common.update(split_ws=split_ws.data_ptr(), split_ws_bytes=split_ws.numel())

    # Z holds one output row per flat slot; slots that no kernel writes (dropped ids) must read as zero
    z_alloc = torch.zeros if expert_map is not None else torch.empty
    z = None if out_rows is not None else z_alloc((numel, H), dtype=out_dtype, device=dev)
    z_args = dict(out=_C.ptr(z), out_rows=_C.ptr(out_rows))

    if not use_fp8_w8a8:
        if name == "tcgen05" and not os.environ.get("FMOE_TC_GATHER4"):
            # sorted copy of the input rows (FMOE_TC_GATHER4=1: the single-CTA kernel gathers them by TMA instead)
            xs = torch.empty((cap, H), dtype=out_dtype, device=dev)
            with _stage("gather_rows"):
                _C.check(lib.fmoe_gather_rows(x.data_ptr(), x.element_size(), cap, H, sorted_ids.data_ptr(), k, numel,
                                              num_post.data_ptr(), xs.data_ptr(), st))
            a_ptr, a_rows, gather = xs.data_ptr(), cap, 0
        else:
            a_ptr, a_rows, gather = x.data_ptr(), T, 1
        act = torch.empty((cap, I), dtype=out_dtype, device=dev)
        g1 = _gemm_args(dtype=code, out_dtype=code, a_gather=gather, n=I, k=H, a_rows=a_rows, a=a_ptr,
                        w=w1.data_ptr(), row_scale=row_w if apply_router_weight_on_input else None,
                        out=act.data_ptr(), bias=_C.ptr(b1), act_alpha=act_alpha, act_limit=act_limit, **common)
        with _stage("gemm1_" + name):
            _C.check(lib.fmoe_gemm1_silu(g1, st))
        g2 = _gemm_args(dtype=code, out_dtype=code, a_gather=0, n=H, k=I, a_rows=cap, a=act.data_ptr(),
                        w=w2.data_ptr(), row_scale=None if apply_router_weight_on_input else row_w,
                        bias=_C.ptr(b2), **z_args, **common)
        with _stage("gemm2_" + name):
            _C.check(lib.fmoe_gemm2(g2, st))
    elif per_channel_quant:
        common["scale_mode"] = _C.SCALE_CHANNEL
        xq = torch.empty((cap, H), dtype=torch.float8_e4m3fn, device=dev)
        xsc = torch.empty(cap, dtype=torch.float32, device=dev)
        with _stage("quant_input"):  # every sorted row with its own scale
            _C.check(lib.fmoe_quant_fp8_per_token(x.data_ptr(), _C.BF16, cap, H, sorted_ids.data_ptr(), k, numel,
                                                  num_post.data_ptr(), xq.data_ptr(), xsc.data_ptr(), st))
        act = torch.empty((cap, I), dtype=torch.bfloat16, device=dev)
        g1 = _gemm_args(dtype=_C.E4M3, out_dtype=_C.BF16, a_gather=0, n=I, k=H, a_rows=cap, a=xq.data_ptr(),
                        a_scale=xsc.data_ptr(), w=w1.data_ptr(), w_scale=w1_scale.data_ptr(),
                        row_scale=row_w if apply_router_weight_on_input else None, out=act.data_ptr(), **common)
        with _stage("gemm1_fp8_" + name):
            _C.check(lib.fmoe_gemm1_silu(g1, st))
        aq = torch.empty((cap, I), dtype=torch.float8_e4m3fn, device=dev)
        asc = torch.empty(cap, dtype=torch.float32, device=dev)
        with _stage("quant_act"):
            _C.check(lib.fmoe_quant_fp8_per_token(act.data_ptr(), _C.BF16, cap, I, sorted_ids.data_ptr(), 0, numel,
                                                  num_post.data_ptr(), aq.data_ptr(), asc.data_ptr(), st))
        g2 = _gemm_args(dtype=_C.E4M3, out_dtype=_C.BF16, a_gather=0, n=H, k=I, a_rows=cap, a=aq.data_ptr(),
                        a_scale=asc.data_ptr(), w=w2.data_ptr(), w_scale=w2_scale.data_ptr(),
                        row_scale=None if apply_router_weight_on_input else row_w, **z_args, **common)
        with _stage("gemm2_fp8_" + name):
            _C.check(lib.fmoe_gemm2(g2, st))
    else:
        if name == "tcgen05":
            # rows quantised straight into the padded expert-sorted order (gather fused into the quantiser)
            xq = torch.empty((cap, H), dtype=torch.float8_e4m3fn, device=dev)
            xsc = torch.empty((cap, H // 128), dtype=torch.float32, device=dev)
            if k >= 2 and H % 512 == 0:
                # each token row quantised once, then bytes and scales copied into the sorted order
                xt = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
                xtsc = torch.empty((T, H // 128), dtype=torch.float32, device=dev)
                with _stage("quant_input"):
                    _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, T, H, None, 1, 0, None, xt.data_ptr(),
                                                         xtsc.data_ptr(), st))
                with _stage("gather_rows"):
                    for src, dst, eb, cols in ((xt, xq, 1, H), (xtsc, xsc, 4, H // 128)):
                        _C.check(lib.fmoe_gather_rows(src.data_ptr(), eb, cap, cols, sorted_ids.data_ptr(), k, numel,
                                                      num_post.data_ptr(), dst.data_ptr(), st))
            else:
                with _stage("quant_input"):
                    _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, cap, H, sorted_ids.data_ptr(), k, numel,
                                                         num_post.data_ptr(), xq.data_ptr(), xsc.data_ptr(), st))
            a_rows, gather, act_dtype, act_code = cap, 0, torch.bfloat16, _C.BF16
        else:
            xq = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
            xsc = torch.empty((T, H // 128), dtype=torch.float32, device=dev)
            with _stage("quant_input"):
                _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, T, H, None, 1, 0, None, xq.data_ptr(),
                                                     xsc.data_ptr(), st))
            a_rows, gather, act_dtype, act_code = T, 1, torch.float32, _C.F32
        act = torch.empty((cap, I), dtype=act_dtype, device=dev)
        g1 = _gemm_args(dtype=_C.E4M3, out_dtype=act_code, a_gather=gather, n=I, k=H, a_rows=a_rows, a=xq.data_ptr(),
                        a_scale=xsc.data_ptr(), w=w1.data_ptr(), w_scale=w1_scale.data_ptr(),
                        row_scale=row_w if apply_router_weight_on_input else None, out=act.data_ptr(), **common)
        with _stage("gemm1_fp8_" + name):
            _C.check(lib.fmoe_gemm1_silu(g1, st))
        aq = torch.empty((cap, I), dtype=torch.float8_e4m3fn, device=dev)
        asc = torch.empty((cap, I // 128), dtype=torch.float32, device=dev)
        with _stage("quant_act"):
            _C.check(lib.fmoe_quant_fp8_group128(act.data_ptr(), act_code, cap, I, sorted_ids.data_ptr(), 0, numel, num_post.data_ptr(),
                                                 aq.data_ptr(), asc.data_ptr(), st))
        g2 = _gemm_args(dtype=_C.E4M3, out_dtype=_C.BF16, a_gather=0, n=H, k=I, a_rows=cap, a=aq.data_ptr(),
                        a_scale=asc.data_ptr(), w=w2.data_ptr(), w_scale=w2_scale.data_ptr(),
                        row_scale=None if apply_router_weight_on_input else row_w, **z_args, **common)
        with _stage("gemm2_fp8_" + name):
            _C.check(lib.fmoe_gemm2(g2, st))

    if out_rows is not None:
        return None
    if no_combine:
        return z.view(T, k, H)
    out = torch.empty((T, H), dtype=out_dtype, device=dev)
    scale = 1.0 if routed_scaling_factor is None else float(routed_scaling_factor)
    with _stage("moe_sum"):
        _C.check(lib.fmoe_moe_sum(z.data_ptr(), _C.DTYPE_CODE[out_dtype], T, k, H, scale, out.data_ptr(), st))
    return out


def fused_moe(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool = True,
    use_grouped_topk: bool = False,
    num_expert_group: Optional[int] = None,
    topk_group: Optional[int] = None,
    correction_bias: Optional[torch.Tensor] = None,
    routed_scaling_factor: Optional[float] = None,
    **kwargs,
) -> torch.Tensor:
    """Router (softmax top-k, or grouped biased-sigmoid top-k) followed by `fused_experts`.

    `routed_scaling_factor` is applied exactly once, after the combine
    (as the reference hook does, src/flaggems_sglang/ops/fused_moe.py:415-420).
    """
    w, ids = _route(hidden_states, gating_output, topk, renormalize, use_grouped_topk, num_expert_group,
                    topk_group, correction_bias, None)
    return fused_experts(hidden_states, w1, w2, w, ids, routed_scaling_factor=routed_scaling_factor, **kwargs)


# --------------------------------------------------------------------------
# reference-layout entry points
# --------------------------------------------------------------------------
def n_major_supported(w1: torch.Tensor, w2: torch.Tensor, activation: str = "silu") -> bool:
    """True when w1 [E,H,2I] / w2 [E,I,H] can be read in place (no transposed copy): contiguous bf16 tensors whose
    H and I are multiples of 32 (the tensor-core kernels' column pieces), silu or gelu."""
    if w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16 or w1.ndim != 3 or w2.ndim != 3:
        return False
    if not (w1.is_contiguous() and w2.is_contiguous()) or activation not in ("silu", "gelu"):
        return False
    H, twoI = w1.shape[1], w1.shape[2]
    return H % 32 == 0 and twoI % 64 == 0 and w1.data_ptr() % 16 == 0 and w2.data_ptr() % 16 == 0


def _k_major(w: torch.Tensor) -> torch.Tensor:
    """[E, K, N] (reference layout) -> [E, N, K] contiguous.  Free when the caller passes
    the transposed view of a serving-side weight, a copy otherwise."""
    wt = w.transpose(-1, -2)
    return wt if wt.is_contiguous() else wt.contiguous()


def triton_kernel_fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    routing_data,
    gather_indx,
    scatter_indx,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    use_fp8_w8a8: bool = False,
    per_channel_quant: bool = False,
    global_num_experts: int = -1,
    expert_map: Optional[torch.Tensor] = None,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[list[int]] = None,
) -> torch.Tensor:
    """Drop-in for the reference op of the same name (src/flaggems_sglang/ops/fused_moe.py:149-232).

    Same signature, layouts (w1 [E,H,2I], w2 [E,I,H], routing triple) and assertions.
    `scatter_indx=None` returns the un-combined rows in expert-sorted order, as the
    reference does.  Weights given as transposed views of [E,2I,H]/[E,H,I] tensors are
    used in place; truly [E,H,2I]-contiguous weights are transposed once per call.
    """
    logger.debug("FLAGGEMS_SGLANG FUSED_MOE")
    assert use_fp8_w8a8 is False, _UNSUPPORTED_FEATURE_MSG.format(name="use_fp8_w8a8")
    assert per_channel_quant is False, _UNSUPPORTED_FEATURE_MSG.format(name="per_channel_quant")
    assert expert_map is None, _UNSUPPORTED_FEATURE_MSG.format(name="expert_map")
    assert w1_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="w1_scale")
    assert w2_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="w2_scale")
    assert a1_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a1_scale")
    assert a2_scale is None, _UNSUPPORTED_FEATURE_MSG.format(name="a2_scale")
    assert block_shape is None, _UNSUPPORTED_FEATURE_MSG.format(name="block_shape")
    assert inplace is False, "Inplace is not supported"
    assert hidden_states.ndim == 2, "hidden_states must be 2D"
    assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
    assert w1.dtype == torch.bfloat16, "w1 must be bfloat16"
    assert w2.dtype == torch.bfloat16, "w2 must be bfloat16"
    assert hidden_states.shape[-1] == w1.shape[-2], "hidden size mismatch"
    assert w2.shape[-1] == w1.shape[1], "intermediate size mismatch"
    if activation not in _C.ACTIVATIONS:
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")

    T, H = hidden_states.shape
    k = routing_data.n_expts_act
    E = w1.shape[0]
    M = T * k
    dev = hidden_states.device
    topk_indx = gather_indx.src_indx.long()          # sorted position -> flat slot
    hist = routing_data.expt_hist.long()
    expert_of_pos = torch.repeat_interleave(torch.arange(E, device=dev), hist, output_size=M)
    ids_flat = torch.empty(M, dtype=torch.int32, device=dev)
    ids_flat[topk_indx] = expert_of_pos.to(torch.int32)
    w_flat = torch.empty(M, dtype=torch.float32, device=dev)
    w_flat[topk_indx] = routing_data.gate_scal.float()
    # contiguous reference-layout weights (what the reference's own tests and benchmarks pass) are read in place;
    # transposed views of serving-side weights are used as they are; anything else costs a transposed copy
    in_place = n_major_supported(w1, w2, activation) and os.environ.get("FMOE_N_MAJOR", "1") != "0"
    z_or_out = fused_experts(
        hidden_states, w1 if in_place else _k_major(w1), w2 if in_place else _k_major(w2), w_flat.view(T, k),
        ids_flat.view(T, k), weights_n_major=in_place,
        activation=activation, apply_router_weight_on_input=apply_router_weight_on_input,
        no_combine=scatter_indx is None,
    )
    if scatter_indx is None:
        # reference returns rows in sorted order p; ours are by flat slot
        return z_or_out.view(M, H)[topk_indx]
    return z_or_out.view(T, H)


def _split_interleaved(w13_rows: torch.Tensor, b13: Optional[torch.Tensor]):
    """[E,2I,H] with gate and linear rows interleaved (even = gate), b13 [E,2I] likewise -> the same tensors with
    the I gate rows first, the layout of this package's gate/up kernels.  One copy of w13."""
    w = torch.cat((w13_rows[:, 0::2], w13_rows[:, 1::2]), dim=1).contiguous()
    b = None if b13 is None else torch.cat((b13[:, 0::2], b13[:, 1::2]), dim=1)
    return w, b


def triton_kernel_fused_experts_with_bias(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w1_pcg,
    b1: torch.Tensor,
    w2: torch.Tensor,
    w2_pcg,
    b2: torch.Tensor,
    routing_data,
    gather_indx,
    scatter_indx,
    inplace: bool = False,
    activation: str = "silu",
    apply_router_weight_on_input: bool = False,
    global_num_experts: int = -1,
    gemm1_alpha: Optional[float] = None,
    gemm1_clamp_limit: Optional[float] = None,
) -> torch.Tensor:
    """The reference's bias variant (src/flaggems_sglang/ops/fused_moe.py:235-325), same signature.

    The reference hands the work to the third-party `matmul_ogs` with a fused swiglu; its call does not match
    any released signature of that library, so the contract here is the published algorithm of
    `triton_kernels.swiglu` and of the `matmul_ogs` epilogue (bias, activation, gammas):

        y[p,c] = swiglu(x[tok(p)] . w1[e][:, 2c] + b1[e][2c],  x[tok(p)] . w1[e][:, 2c+1] + b1[e][2c+1]) * g_in[p]
        swiglu(g, u) = s*u + s,  s = g'/(1 + exp(-alpha*g')),  g' = min(g, limit),  u clamped to +-limit
        z[p,:] = (y[p,:] . w2[e] + b2[e]) * g_out[p],      out[t] = sum over the k rows of token t

    w1 [E,H,2I] holds gate and linear columns interleaved (even = gate), b1 [E,2I] likewise, as that library
    expects; they are split into the [gate rows; up rows] layout of this package's kernels once per call.
    `activation="silu"` names this swiglu, as in the reference; alpha defaults to 1.702.  The precision
    configs are accepted for signature compatibility and must be None (bf16 only).
    """
    logger.debug("FLAGGEMS_SGLANG FUSED_MOE_WITH_BIAS")
    assert inplace is False, "Inplace is not supported"
    assert hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16"
    assert w1_pcg is None and w2_pcg is None, _UNSUPPORTED_FEATURE_MSG.format(name="precision configs")
    if activation != "silu":
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    assert w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16, "w1/w2 must be bfloat16"
    assert hidden_states.shape[-1] == w1.shape[-2], "hidden size mismatch"
    T, H = hidden_states.shape
    k = routing_data.n_expts_act
    E = w1.shape[0]
    M = T * k
    dev = hidden_states.device
    topk_indx = gather_indx.src_indx.long()          # sorted position -> flat slot
    hist = routing_data.expt_hist.long()
    expert_of_pos = torch.repeat_interleave(torch.arange(E, device=dev), hist, output_size=M)
    ids_flat = torch.empty(M, dtype=torch.int32, device=dev)
    ids_flat[topk_indx] = expert_of_pos.to(torch.int32)
    w_flat = torch.empty(M, dtype=torch.float32, device=dev)
    w_flat[topk_indx] = routing_data.gate_scal.float()
    w1_split, b1_split = _split_interleaved(w1.transpose(1, 2), b1)
    z_or_out = fused_experts(
        hidden_states, w1_split, _k_major(w2), w_flat.view(T, k), ids_flat.view(T, k), activation="swiglu_oai",
        apply_router_weight_on_input=apply_router_weight_on_input, no_combine=scatter_indx is None,
        b1=b1_split, b2=b2, gemm1_alpha=gemm1_alpha, gemm1_clamp_limit=gemm1_clamp_limit,
    )
    if scatter_indx is None:
        return z_or_out.view(M, H)[topk_indx]
    return z_or_out.view(T, H)


@dataclass
class StandardCombineInput:
    hidden_states: torch.Tensor


def _split_interleaved_cached(layer, b13):
    """`_split_interleaved` of the layer's w13 / bias, kept on the layer until either tensor is replaced or
    modified in place (data pointer and version counter), so that the copy is not repeated on every call."""
    w = layer.w13_weight
    key = (w.data_ptr(), w._version, tuple(w.shape), b13.data_ptr(), b13._version)
    cached = getattr(layer, "_fmoe_split_w13", None)
    if cached is None or cached[0] != key:
        cached = (key, _split_interleaved(w, b13))
        try:
            layer._fmoe_split_w13 = cached
        except Exception:  # noqa: BLE001  (a layer object that refuses new attributes: split per call)
            pass
    return cached[1]


def _standard_output_type():
    """The combine-input container of the serving stack when it is importable (the reference imports it at
    src/flaggems_sglang/ops/fused_moe.py:337-339), this module's stand-in with the same field otherwise."""
    try:
        from sglang.srt.layers.moe.token_dispatcher.standard import StandardCombineInput as _Sgl

        return _Sgl
    except Exception:  # noqa: BLE001
        return StandardCombineInput


def fused_moe_flagos(obj, layer: torch.nn.Module, dispatch_output):
    """Serving-side hook with the reference's signature (src/flaggems_sglang/ops/fused_moe.py:328-422).

    Reads `layer.w13_weight [E,2I,H]` / `layer.w2_weight [E,H,I]` in place (the reference
    transposes and copies both on every call, :342-343), accepts either the standard
    `(topk_weights, topk_ids)` output or a routing triple, honours `no_combine`,
    `apply_router_weight_on_input` and `routed_scaling_factor` of `obj.runner.config`,
    and returns SGLang's `StandardCombineInput` (or, without SGLang, an object with the same `.hidden_states`).

    `no_combine`: as in the reference (:355-366, 408-413), a standard top-k output is first converted to the
    routing triple, and the un-combined rows come back in EXPERT-SORTED order viewed as [T, k, H] — for both
    routing formats.  (`fused_experts(no_combine=True)` on the serving-side layouts returns rows by flat slot.)
    """
    cfg = obj.runner.config
    b13, b2 = getattr(layer, "w13_weight_bias", None), getattr(layer, "w2_weight_bias", None)
    hidden_states = dispatch_output.hidden_states
    topk_output = dispatch_output.topk_output
    if cfg.no_combine and hasattr(topk_output, "topk_weights"):
        topk_output = standard_topk_to_routing(topk_output.topk_weights, topk_output.topk_ids, layer.w13_weight.shape[0])
    Out = _standard_output_type()
    if b13 is not None or b2 is not None:
        # bias variant (src/flaggems_sglang/ops/fused_moe.py:380-398): interleaved gate/linear rows, swiglu
        assert b13 is not None and b2 is not None, "Bias execution requires both w13_bias and w2_bias"
        alpha, limit = getattr(cfg, "gemm1_alpha", None), getattr(cfg, "gemm1_clamp_limit", None)
        if hasattr(topk_output, "topk_weights"):
            w13, b13s = _split_interleaved_cached(layer, b13)
            out = fused_experts(
                hidden_states, w13, layer.w2_weight, topk_output.topk_weights, topk_output.topk_ids,
                activation="swiglu_oai", apply_router_weight_on_input=cfg.apply_router_weight_on_input,
                routed_scaling_factor=cfg.routed_scaling_factor,
                b1=b13s, b2=b2, gemm1_alpha=alpha, gemm1_clamp_limit=limit,
            )
        else:
            routing_data, gather_indx, scatter_indx = topk_output
            out = triton_kernel_fused_experts_with_bias(
                hidden_states, layer.w13_weight.transpose(-1, -2), None, b13, layer.w2_weight.transpose(-1, -2), None, b2,
                routing_data, gather_indx, None if cfg.no_combine else scatter_indx, activation=cfg.activation,
                apply_router_weight_on_input=cfg.apply_router_weight_on_input, gemm1_alpha=alpha,
                gemm1_clamp_limit=limit,
            )
            if cfg.no_combine:
                out = out.view(hidden_states.shape[0], -1, hidden_states.shape[-1])
            elif cfg.routed_scaling_factor is not None and cfg.routed_scaling_factor != 1.0:
                out.mul_(cfg.routed_scaling_factor)
        return Out(hidden_states=out)
    if hasattr(topk_output, "topk_weights"):
        tw, ti = topk_output.topk_weights, topk_output.topk_ids
        out = fused_experts(
            hidden_states, layer.w13_weight, layer.w2_weight, tw, ti, activation=cfg.activation,
            apply_router_weight_on_input=cfg.apply_router_weight_on_input,
            routed_scaling_factor=cfg.routed_scaling_factor,
        )
    else:
        routing_data, gather_indx, scatter_indx = topk_output
        out = triton_kernel_fused_experts(
            hidden_states, layer.w13_weight.transpose(-1, -2), layer.w2_weight.transpose(-1, -2), routing_data,
            gather_indx, None if cfg.no_combine else scatter_indx, activation=cfg.activation,
            apply_router_weight_on_input=cfg.apply_router_weight_on_input,
        )
        if cfg.no_combine:
            out = out.view(hidden_states.shape[0], -1, hidden_states.shape[-1])
        elif cfg.routed_scaling_factor is not None and cfg.routed_scaling_factor != 1.0:
            out.mul_(cfg.routed_scaling_factor)
    return Out(hidden_states=out)


__all__ = [
    "fused_experts",
    "fused_moe",
    "triton_kernel_fused_experts",
    "triton_kernel_fused_experts_with_bias",
    "fused_moe_flagos",
    "standard_topk_to_routing",
    "RoutingData",
    "GatherIndx",
    "ScatterIndx",
]
