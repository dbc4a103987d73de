"""Oracle (test infrastructure): routing stages of the fused-MoE path on CPU.

Integer work is numpy; floating point follows the order of operations of the
code it restates.  Nothing here is imported by the product path.
"""
from __future__ import annotations

import numpy as np
import torch

BLOCK_MS = (16, 32, 64, 128)


# ----------------------------------------------------------------------------
# Router: softmax top-k
# ----------------------------------------------------------------------------
def softmax_topk(logits: torch.Tensor, k: int, renormalize: bool = True):
    """softmax -> top-k -> optional renormalise.

    Follows ref:tests/test_fused_moe.py:38-41 (softmax over experts in fp32,
    top-k, divide by the sum of the k winners).  Tie rule, fixed so that ids
    are well defined: the lower expert index wins, as in the third-party torch
    routing reference (TK:routing.py:351-360, stable argsort of the negated
    key).  Ranking is done on the raw logits; softmax is monotone, so this
    selects the same experts unless two distinct logits collapse to one fp32
    probability.

    Returns (weights float32 [T,k] sorted by descending weight, ids int32 [T,k]).
    """
    logits = logits.detach().to(torch.float32).cpu()
    T, E = logits.shape
    # NaN contract (builder-defined): NaN ranks as -inf; a row with nothing above -inf counts as all-equal logits
    logits = torch.where(torch.isnan(logits), torch.full_like(logits, float("-inf")), logits)
    dead = (logits == float("-inf")).all(dim=1, keepdim=True)
    logits = torch.where(dead, torch.zeros_like(logits), logits)
    order = torch.argsort(-logits, dim=1, stable=True)[:, :k]
    probs = torch.softmax(logits, dim=-1)
    w = torch.take_along_dim(probs, order, dim=1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.contiguous(), order.to(torch.int32).contiguous()


# ----------------------------------------------------------------------------
# Router: DeepSeek-V3 grouped, bias-corrected sigmoid top-k
# ----------------------------------------------------------------------------
def sigmoid_f32(logits: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 sigmoid (evaluated in fp64, rounded once).

    The expert ids chosen by the grouped router depend on the last bit of the
    score, so the contract fixes the score as the correctly rounded value; the
    CUDA router evaluates it in fp64 as well.
    """
    return torch.sigmoid(logits.detach().cpu().to(torch.float64)).to(torch.float32)


def grouped_topk(
    logits: torch.Tensor,
    correction_bias: torch.Tensor | None,
    k: int,
    num_expert_group: int,
    topk_group: int,
    renormalize: bool = True,
    routed_scaling_factor: float | None = None,
):
    """Group-limited top-k with sigmoid scores and a per-expert selection bias.

    Contract (the reference delegates routing to its caller,
    ref:src/flaggems_sglang/ops/fused_moe.py:340,355-366, so this stage has no
    reference code; parity unpinned):
      s = sigmoid(logits); c = s + bias
      group score = sum of the two largest c in each group of E/num_expert_group
      keep the topk_group best groups (ties -> lower group index)
      ids = top-k of c restricted to kept groups (ties -> lower expert index)
      w = s[ids] (un-biased); renormalise: w /= (sum_j w_j + 1e-20) summed j=0..k-1
      w *= routed_scaling_factor when given.
    """
    logits = logits.detach().cpu().to(torch.float32)
    # NaN contract (builder-defined): a NaN logit counts as -inf, a NaN biased score or group score as -inf
    s = sigmoid_f32(torch.where(torch.isnan(logits), torch.full_like(logits, float("-inf")), logits))
    T, E = s.shape
    bias = (
        torch.zeros(E, dtype=torch.float32)
        if correction_bias is None
        else correction_bias.detach().cpu().to(torch.float32)
    )
    c = s + bias[None, :]
    c = torch.where(torch.isnan(c), torch.full_like(c, float("-inf")), c)
    gsz = E // num_expert_group
    cg = c.view(T, num_expert_group, gsz)
    if gsz >= 2:
        top2 = torch.sort(cg, dim=-1, descending=True).values[..., :2]
        gscore = top2[..., 0] + top2[..., 1]
    else:
        gscore = cg[..., 0]
    gscore = torch.where(torch.isnan(gscore), torch.full_like(gscore, float("-inf")), gscore)
    gorder = torch.argsort(-gscore, dim=1, stable=True)[:, :topk_group]
    gmask = torch.zeros(T, num_expert_group, dtype=torch.bool)
    gmask.scatter_(1, gorder, True)
    emask = gmask[:, :, None].expand(T, num_expert_group, gsz).reshape(T, E)
    masked = torch.where(emask, c, torch.full_like(c, float("-inf")))
    ids = torch.argsort(-masked, dim=1, stable=True)[:, :k]
    w = torch.take_along_dim(s, ids, dim=1)
    if renormalize:
        acc = torch.zeros(T, dtype=torch.float32)
        for j in range(k):  # sequential fp32 sum, j ascending
            acc = acc + w[:, j]
        w = w / (acc + torch.tensor(1e-20, dtype=torch.float32))[:, None]
    if routed_scaling_factor is not None:
        w = w * torch.tensor(routed_scaling_factor, dtype=torch.float32)
    return w.contiguous(), ids.to(torch.int32).contiguous()


# ----------------------------------------------------------------------------
# moe_align_block_size
# ----------------------------------------------------------------------------
def moe_align_block_size(topk_ids, block_size: int, num_experts: int):
    """Sort flat (token, slot) indices by expert and pad each expert to a block multiple.

    Contract (absent from the reference; the nearest analogue is the tile map of
    TK:routing.py:311-348; parity unpinned):
      n = topk_ids.numel(); flat slot s = t*k + j
      sorted_token_ids: int32 [n + E*(block-1)], filled with the sentinel n; for
        each expert ascending its slots in ascending s, then sentinel padding up
        to a multiple of block.
      expert_ids: int32 [ceil(len(sorted)/block)], expert of each used block,
        -1 beyond the used blocks.
      num_tokens_post_padded: int32 [1] = sum_e ceil(cnt_e/block)*block.
    Ids outside [0, E) (e.g. -1 for "not on this rank") are dropped.
    """
    ids = np.asarray(
        topk_ids.detach().cpu().numpy() if isinstance(topk_ids, torch.Tensor) else topk_ids
    ).astype(np.int64).reshape(-1)
    n = ids.size
    cap = n + num_experts * (block_size - 1)
    sorted_ids = np.full(cap, n, dtype=np.int32)
    nblk_cap = (cap + block_size - 1) // block_size
    expert_ids = np.full(nblk_cap, -1, dtype=np.int32)
    pos = 0
    for e in range(num_experts):
        slots = np.nonzero(ids == e)[0]
        cnt = slots.size
        if cnt == 0:
            continue
        sorted_ids[pos : pos + cnt] = slots
        nb = (cnt + block_size - 1) // block_size
        expert_ids[pos // block_size : pos // block_size + nb] = e
        pos += nb * block_size
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)


# ----------------------------------------------------------------------------
# Reference routing format
# ----------------------------------------------------------------------------
def standard_topk_to_routing(topk_weights, topk_ids, n_expts_tot: int):
    """(topk_weights, topk_ids) -> the routing tables the reference op consumes.

    Restates ref:src/flaggems_sglang/ops/fused_moe.py:128-146 and
    TK:routing.py:311-348 (compute_expt_data_torch).  Returns a dict:
      gate_scal  f32 [M]   weights in expert-sorted order
      hist       i32 [E]
      topk_indx  i32 [M]   sorted position p -> flat slot (per-token slots are
                           numbered after sorting the token's ids ascending)
      gate_indx  i32 [M]   flat slot -> sorted position
      token_offs_raw i32 [E+1]
      token_offs_pad {bm: i32 [E+1]}  exclusive cumsum of ceil(hist/bm), in tiles
      block_pid_map  {bm: i32 [max_tiles]}  (tile_in_expert << 16) | expert, else -1
    """
    w = np.asarray(topk_weights.detach().cpu().numpy(), dtype=np.float32)
    ids = np.asarray(topk_ids.detach().cpu().numpy()).astype(np.int64)
    T, k = w.shape
    M = T * k
    # ref:...fused_moe.py:130-133 : per-token ascending sort of the expert ids
    perm = np.argsort(ids, axis=1, kind="stable")
    ids2 = np.take_along_axis(ids, perm, axis=1)
    w2 = np.take_along_axis(w, perm, axis=1)
    expt = ids2.reshape(-1)
    wflat = w2.reshape(-1)
    # ref:...:134-136
    topk_indx = np.argsort(expt, kind="stable").astype(np.int32)
    gate_indx = np.argsort(topk_indx, kind="stable").astype(np.int32)
    gate_scal = wflat[topk_indx]
    # ref:...:137-139
    hist = np.bincount(expt, minlength=n_expts_tot)[:n_expts_tot].astype(np.int32)
    # TK:routing.py:311-348
    token_offs_raw = np.concatenate(([0], np.cumsum(hist))).astype(np.int32)
    if M <= n_expts_tot:
        max_tiles = M
    else:
        max_tiles = n_expts_tot - 1 - ((n_expts_tot - M - 1) // min(BLOCK_MS))
    token_offs_pad, block_pid_map = {}, {}
    for bm in BLOCK_MS:
        tiles = (hist + bm - 1) // bm
        offs = np.concatenate(([0], np.cumsum(tiles))).astype(np.int32)
        token_offs_pad[bm] = offs
        pm = np.full(max_tiles, -1, dtype=np.int32)
        for e in range(n_expts_tot):
            for b in range(int(tiles[e])):
                pm[offs[e] + b] = (b << 16) + e
        block_pid_map[bm] = pm
    return dict(
        gate_scal=gate_scal,
        hist=hist,
        topk_indx=topk_indx,
        gate_indx=gate_indx,
        token_offs_raw=token_offs_raw,
        token_offs_pad=token_offs_pad,
        block_pid_map=block_pid_map,
        n_expts_tot=n_expts_tot,
        n_expts_act=k,
    )
