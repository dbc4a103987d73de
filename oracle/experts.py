"""Oracle (test infrastructure): expert computation of the fused-MoE path on CPU.

All GEMMs are fp32 ``torch.matmul`` on up-cast operands; values are rounded to
the activation dtype at exactly the points where the reference materialises a
tensor.  Nothing here is imported by the product path.
"""
from __future__ import annotations

import numpy as np
import torch

from . import quant as Q
from . import routing as R


def _rb(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round to ``dtype`` (round-to-nearest-even) and come back to fp32."""
    if dtype == torch.float32:
        return x
    return x.to(dtype).to(torch.float32)


def silu_and_mul(y1: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    """out[r,c] = (g / (1 + exp(-g))) * u, g = y1[r,c], u = y1[r,I+c], fp32 math.

    Restates ref:src/flaggems_sglang/ops/fused_moe.py:58-62 (gate = first half,
    up = second half; the result is stored in the input dtype, :63).
    """
    dtype = y1.dtype if dtype is None else dtype
    f = y1.to(torch.float32)
    half = f.shape[-1] // 2
    g, u = f[..., :half], f[..., half:]
    return ((g / (1.0 + torch.exp(-g))) * u).to(dtype)


def gelu_and_mul(y1: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    """out[r,c] = gelu(y1[r,c]) * y1[r,I+c] with the erf form of gelu, fp32 math: the reference's second
    activation (ref:src/flaggems_sglang/ops/fused_moe.py:219-220 delegates it to an external kernel)."""
    dtype = y1.dtype if dtype is None else dtype
    f = y1.to(torch.float32)
    half = f.shape[-1] // 2
    return (torch.nn.functional.gelu(f[..., :half]) * f[..., half:]).to(dtype)


def _act(name: str):
    if name == "silu":
        return silu_and_mul
    if name == "gelu":
        return gelu_and_mul
    raise ValueError(f"Unsupported FusedMoe activation: {name}")


def _expert_segments(hist):
    offs = np.concatenate(([0], np.cumsum(hist)))
    return [(e, int(offs[e]), int(offs[e + 1])) for e in range(len(hist)) if hist[e] > 0]


def reference_fused_experts(
    x: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    routing: dict,
    apply_router_weight_on_input: bool = False,
    no_combine: bool = False,
    activation: str = "silu",
) -> torch.Tensor:
    """The reference op on its own layouts: w1 [E,H,2I], w2 [E,I,H], routing tables.

    Restates ref:src/flaggems_sglang/ops/fused_moe.py:197-232 together with the
    behaviour of the two grouped-GEMM calls it makes:
      GEMM1 (:205-212)  Y1[p] = rb((x[topk_indx[p]//k] @ w1[e(p)]) * gamma_in[p])
                        gather by ``//k`` TK:matmul_ogs_details/_matmul_ogs.py:198,
                        fp32 accumulate :354, epilogue acc -> *gamma -> round :384-429
      act   (:214-218)  A = rb(silu(Y1[:, :I]) * Y1[:, I:])
      GEMM2 (:224-231)  Z[p] = rb((A[p] @ w2[e(p)]) * gamma_out[p]) into a scratch
                        in the activation dtype (TK:matmul_ogs.py:168-170)
      combine           out[t] = rb(sum_j f32(Z[gate_indx[t*k+j]])), j ascending,
                        sequential fp32 adds (TK:matmul_ogs_details/_reduce_grouped.py:51-71)
    ``no_combine`` (scatter_indx=None, ref:...:371,408-413) returns Z in sorted order.
    """
    dtype = x.dtype
    k = routing["n_expts_act"]
    T, H = x.shape
    M = T * k
    xf = x.detach().cpu().to(torch.float32)
    topk_indx = torch.from_numpy(routing["topk_indx"].astype(np.int64))
    gate_indx = torch.from_numpy(routing["gate_indx"].astype(np.int64))
    gate_scal = torch.from_numpy(np.asarray(routing["gate_scal"], dtype=np.float32))
    tok = topk_indx // k
    Z = torch.zeros(M, H, dtype=torch.float32)
    for e, lo, hi in _expert_segments(routing["hist"]):
        rows = tok[lo:hi]
        acc1 = xf[rows] @ w1[e].detach().cpu().to(torch.float32)
        if apply_router_weight_on_input:
            acc1 = acc1 * gate_scal[lo:hi, None]
        y1 = _rb(acc1, dtype)
        a = _act(activation)(y1, dtype).to(torch.float32)
        acc2 = a @ w2[e].detach().cpu().to(torch.float32)
        if not apply_router_weight_on_input:
            acc2 = acc2 * gate_scal[lo:hi, None]
        Z[lo:hi] = _rb(acc2, dtype)
    if no_combine:
        return Z.to(dtype)
    out = torch.zeros(T, H, dtype=torch.float32)
    zs = Z[gate_indx].view(T, k, H)
    for j in range(k):
        out = out + zs[:, j]
    return out.to(dtype)


def fused_experts(
    x: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    apply_router_weight_on_input: bool = False,
    no_combine: bool = False,
    routed_scaling_factor: float | None = None,
    activation: str = "silu",
) -> torch.Tensor:
    """Same computation on the serving-side layouts: w1 [E,2I,H], w2 [E,H,I].

    These layouts are the per-expert transposes of the reference op's
    (ref:src/flaggems_sglang/ops/fused_moe.py:342-343); rows [0,I) of w1 are the
    gate projection and [I,2I) the up projection, consistent with :58-62.
    Slots keep the order of ``topk_ids``; Z is indexed by flat slot t*k+j and
    the combine sums j = 0..k-1 in fp32 (``no_combine`` returns Z as [T,k,H]).
    ``routed_scaling_factor`` multiplies the combined output afterwards
    (ref:...:415-420).  Ids outside [0,E) contribute nothing.
    """
    dtype = x.dtype
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w1.shape[0]
    xf = x.detach().cpu().to(torch.float32)
    ids = topk_ids.detach().cpu().to(torch.int64).reshape(-1)
    wts = topk_weights.detach().cpu().to(torch.float32).reshape(-1)
    Z = torch.zeros(T * k, H, dtype=torch.float32)
    for e in range(E):
        slots = torch.nonzero(ids == e).reshape(-1)
        if slots.numel() == 0:
            continue
        acc1 = xf[slots // k] @ w1[e].detach().cpu().to(torch.float32).t()
        if apply_router_weight_on_input:
            acc1 = acc1 * wts[slots, None]
        y1 = _rb(acc1, dtype)
        a = _act(activation)(y1, dtype).to(torch.float32)
        acc2 = a @ w2[e].detach().cpu().to(torch.float32).t()
        if not apply_router_weight_on_input:
            acc2 = acc2 * wts[slots, None]
        Z[slots] = _rb(acc2, dtype)
    if no_combine:
        return Z.view(T, k, H).to(dtype)
    out = moe_sum(Z.view(T, k, H))
    if routed_scaling_factor is not None and routed_scaling_factor != 1.0:
        out = _rb(out, dtype) * routed_scaling_factor
    return out.to(dtype)


def swiglu_oai(y1: torch.Tensor, alpha: float = 1.702, limit: float | None = None) -> torch.Tensor:
    """The gated unit of the reference's bias variant, on INTERLEAVED columns (even = gate, odd = linear), fp32:

        g = y1[..., 0::2] clamped to (-inf, limit], u = y1[..., 1::2] clamped to [-limit, limit],
        s = g / (1 + exp(-alpha*g)),  out = s*u + s.

    The reference only names the function (`swiglu_fn`, ref:src/flaggems_sglang/ops/fused_moe.py:261, 276); the
    arithmetic lives in the third-party dependency `triton_kernels` (not pinned by the reference): this restates
    its published `swiglu_torch` / `compute_swiglu` (triton_kernels/swiglu.py, swiglu_details/_swiglu.py).
    """
    f = y1.to(torch.float32)
    g, u = f[..., 0::2], f[..., 1::2]
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    sgl = g / (1.0 + torch.exp(-alpha * g))
    return sgl * u + sgl


def reference_fused_experts_with_bias(
    x: torch.Tensor,
    w1: torch.Tensor,
    b1: torch.Tensor | None,
    w2: torch.Tensor,
    b2: torch.Tensor | None,
    routing: dict,
    apply_router_weight_on_input: bool = False,
    alpha: float | None = None,
    limit: float | None = None,
    no_combine: bool = False,
) -> torch.Tensor:
    """The bias variant on the reference's layouts (ref:src/flaggems_sglang/ops/fused_moe.py:235-325):
    w1 [E,H,2I] with interleaved gate/linear columns, b1 [E,2I] likewise, w2 [E,I,H], b2 [E,H], routing tables as
    in `reference_fused_experts`.  Both `matmul_ogs` calls apply bias, then the fused activation, then the gammas
    and round once to the activation dtype (third-party epilogue order; :303-324 pass `bias`, `fused_activation`,
    `gammas` to it):

        y[p] = rb( swiglu(x[tok(p)] @ w1[e] + b1[e]) * g_in[p] )
        z[p] = rb( (y[p] @ w2[e] + b2[e]) * g_out[p] ),    out[t] = rb( sum_j z[gate_indx[t*k + j]] )

    Parity of this function is unpinned against the reference itself (its call does not run against any released
    `triton_kernels`); `swiglu_oai` is pinned against that library's torch reference in the tests.
    """
    dtype = x.dtype
    k = routing["n_expts_act"]
    alpha = 1.702 if alpha is None else alpha
    xf = x.detach().cpu().to(torch.float32)
    topk_indx = torch.from_numpy(routing["topk_indx"].astype(np.int64))
    gate_indx = torch.from_numpy(routing["gate_indx"].astype(np.int64))
    gs = torch.from_numpy(np.asarray(routing["gate_scal"], dtype=np.float32))
    M = topk_indx.numel()
    H = w2.shape[-1]
    tok = topk_indx // k
    Z = torch.zeros(M, H, dtype=torch.float32)
    for e, lo, hi in _expert_segments(routing["hist"]):
        acc1 = xf[tok[lo:hi]] @ w1[e].detach().cpu().to(torch.float32)
        if b1 is not None:
            acc1 = acc1 + b1[e].detach().cpu().to(torch.float32)
        y = swiglu_oai(acc1, alpha, limit)
        if apply_router_weight_on_input:
            y = y * gs[lo:hi, None]
        y = _rb(y, dtype)
        acc2 = y @ w2[e].detach().cpu().to(torch.float32)
        if b2 is not None:
            acc2 = acc2 + b2[e].detach().cpu().to(torch.float32)
        if not apply_router_weight_on_input:
            acc2 = acc2 * gs[lo:hi, None]
        Z[lo:hi] = _rb(acc2, dtype)
    if no_combine:
        return Z.to(dtype)
    T = M // k
    return moe_sum(Z[gate_indx].view(T, k, H)).to(dtype)


def fused_experts_with_bias(x, w1, b1, w2, b2, topk_weights, topk_ids, apply_router_weight_on_input=False,
                            alpha=None, limit=None, no_combine=False) -> torch.Tensor:
    """Same computation on the serving-side layouts: w1 [E,2I,H] with the gate rows first ([0,I) gate, [I,2I)
    linear), b1 [E,2I] likewise, w2 [E,H,I], b2 [E,H]; slots in `topk_ids` order."""
    dtype = x.dtype
    T, H = x.shape
    k = topk_ids.shape[1]
    E, twoI, _ = w1.shape
    I = twoI // 2
    alpha = 1.702 if alpha is None else alpha
    xf = x.detach().cpu().to(torch.float32)
    ids = topk_ids.detach().cpu().to(torch.int64).reshape(-1)
    wts = topk_weights.detach().cpu().to(torch.float32).reshape(-1)
    Z = torch.zeros(T * k, H, dtype=torch.float32)
    for e in range(E):
        slots = torch.nonzero(ids == e).reshape(-1)
        if slots.numel() == 0:
            continue
        acc1 = xf[slots // k] @ w1[e].detach().cpu().to(torch.float32).t()
        if b1 is not None:
            acc1 = acc1 + b1[e].detach().cpu().to(torch.float32)
        inter = torch.stack((acc1[:, :I], acc1[:, I:]), dim=-1).reshape(-1, twoI)  # back to interleaved columns
        y = swiglu_oai(inter, alpha, limit)
        if apply_router_weight_on_input:
            y = y * wts[slots, None]
        y = _rb(y, dtype)
        acc2 = y @ w2[e].detach().cpu().to(torch.float32).t()
        if b2 is not None:
            acc2 = acc2 + b2[e].detach().cpu().to(torch.float32)
        if not apply_router_weight_on_input:
            acc2 = acc2 * wts[slots, None]
        Z[slots] = _rb(acc2, dtype)
    if no_combine:
        return Z.view(T, k, H).to(dtype)
    return moe_sum(Z.view(T, k, H)).to(dtype)


def moe_sum(z: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_j z[t,j], sequential fp32 adds in ascending j; returns fp32."""
    zf = z.detach().cpu().to(torch.float32)
    out = torch.zeros(zf.shape[0], zf.shape[2], dtype=torch.float32)
    for j in range(zf.shape[1]):
        out = out + zf[:, j]
    return out


def fused_experts_fp8(
    x: torch.Tensor,
    w1_q: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_q: torch.Tensor,
    w2_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    no_combine: bool = False,
    routed_scaling_factor: float | None = None,
) -> torch.Tensor:
    """w8a8 block-quant experts: e4m3 weights with 128x128 scales, activations
    quantised per token per 128 channels before each GEMM.

    Builder-defined contract (the reference rejects fp8): quantise x ->
    GEMM1 on de-quantised operands in fp32 -> silu*mul in fp32 -> quantise ->
    GEMM2 -> * top-k weight -> round to bf16 -> combine as in ``fused_experts``.
    """
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w1_q.shape[0]
    xq, xs = Q.quant_act_group128(x)
    xf = Q.dequant_act_group128(xq, xs)
    ids = topk_ids.detach().cpu().to(torch.int64).reshape(-1)
    wts = topk_weights.detach().cpu().to(torch.float32).reshape(-1)
    Z = torch.zeros(T * k, H, dtype=torch.float32)
    for e in range(E):
        slots = torch.nonzero(ids == e).reshape(-1)
        if slots.numel() == 0:
            continue
        w1f = Q.dequant_weight_block128(w1_q[e], w1_scale[e])
        w2f = Q.dequant_weight_block128(w2_q[e], w2_scale[e])
        acc1 = xf[slots // k] @ w1f.t()
        a = silu_and_mul(acc1, torch.float32)
        aq, as_ = Q.quant_act_group128(a)
        af = Q.dequant_act_group128(aq, as_)
        acc2 = (af @ w2f.t()) * wts[slots, None]
        Z[slots] = _rb(acc2, torch.bfloat16)
    if no_combine:
        return Z.view(T, k, H).to(torch.bfloat16)
    out = moe_sum(Z.view(T, k, H))
    if routed_scaling_factor is not None and routed_scaling_factor != 1.0:
        out = _rb(out, torch.bfloat16) * routed_scaling_factor
    return out.to(torch.bfloat16)


def fused_experts_fp8_per_channel(x, w1_q, w1_scale, w2_q, w2_scale, topk_weights, topk_ids,
                                  no_combine: bool = False, routed_scaling_factor: float | None = None) -> torch.Tensor:
    """w8a8 with per-output-channel weight scales (w1_scale [E,2I], w2_scale [E,H]) and one dynamic scale per
    activation row.  Builder-defined contract (the reference asserts `per_channel_quant` off,
    ref:src/flaggems_sglang/ops/fused_moe.py:173-175), the one vLLM's fp8 MoE follows: quantise each token row ->
    GEMM1 on the e4m3 values in fp32 -> (acc * row scale) * channel scale -> silu*mul in fp32 -> round to bf16 ->
    quantise each row -> GEMM2 -> (acc * row scale) * channel scale * top-k weight -> bf16 -> combine."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w1_q.shape[0]
    xq, xs = Q.quant_act_per_token(x)
    xf = xq.to(torch.float32)
    ids = topk_ids.detach().cpu().to(torch.int64).reshape(-1)
    wts = topk_weights.detach().cpu().to(torch.float32).reshape(-1)
    Z = torch.zeros(T * k, H, dtype=torch.float32)
    for e in range(E):
        slots = torch.nonzero(ids == e).reshape(-1)
        if slots.numel() == 0:
            continue
        tok = slots // k
        acc1 = (xf[tok] @ w1_q[e].detach().cpu().to(torch.float32).t()) * xs[tok, None] * w1_scale[e].cpu()[None, :]
        a = _rb(silu_and_mul(acc1, torch.float32), torch.bfloat16)
        aq, as_ = Q.quant_act_per_token(a)
        acc2 = (aq.to(torch.float32) @ w2_q[e].detach().cpu().to(torch.float32).t()) * as_[:, None] * w2_scale[e].cpu()[None, :]
        Z[slots] = _rb(acc2 * wts[slots, None], torch.bfloat16)
    if no_combine:
        return Z.view(T, k, H).to(torch.bfloat16)
    out = moe_sum(Z.view(T, k, H))
    if routed_scaling_factor is not None and routed_scaling_factor != 1.0:
        out = _rb(out, torch.bfloat16) * routed_scaling_factor
    return out.to(torch.bfloat16)


def dense_moe(x, w1, w2, topk_weights, topk_ids) -> torch.Tensor:
    """Independent per-token formulation in fp32 with no intermediate rounding;
    used only to cross-check the restatements above (w1 [E,2I,H], w2 [E,H,I])."""
    xf = x.detach().cpu().to(torch.float32)
    T, H = xf.shape
    k = topk_ids.shape[1]
    out = torch.zeros(T, H, dtype=torch.float32)
    for t in range(T):
        for j in range(k):
            e = int(topk_ids[t, j])
            y = w1[e].detach().cpu().to(torch.float32) @ xf[t]
            half = y.shape[0] // 2
            a = torch.nn.functional.silu(y[:half]) * y[half:]
            out[t] += float(topk_weights[t, j]) * (w2[e].detach().cpu().to(torch.float32) @ a)
    return out


def fused_moe(x, w1, w2, gating_output, topk: int, renormalize: bool = True, **kw):
    """router (softmax top-k) -> fused_experts."""
    w, ids = R.softmax_topk(gating_output, topk, renormalize)
    return fused_experts(x, w1, w2, w, ids, **kw)
