"""Expert-parallel fused MoE on one NVLink/NVSwitch box: experts sharded E/N per GPU, tokens exchanged
with NCCL all-to-all (torch.distributed), one process per GPU.

The reference has no expert parallelism (`expert_map` is asserted None,
FlagGems-sglang src/flaggems_sglang/ops/fused_moe.py:176-178); the contract here is "same numbers
as the single-GPU op on the same global batch".

Per layer call, every rank
  1. routes its own tokens (global expert ids);
  2. sorts its T*k (token, slot) pairs by destination rank (stable) and exchanges the counts;
  3. dispatch: all-to-all of the hidden rows plus (local expert id, top-k weight) per row;
  4. runs the grouped GEMMs over the rows it received, with top_k = 1 and the weight applied in
     the down-projection epilogue exactly as on one GPU;
  5. combine: all-to-all of the result rows back, un-permute to slot order, sum the k slots.
Payloads land in local HBM through NCCL before any kernel reads them; no kernel touches peer memory.

The data movement is written against a small backend interface so that the exchange logic runs
unchanged on CPU ranks (gloo) in the tests, where the backend is the CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    """Host-side split sizes of one exchange."""
    send_counts: list  # rows this rank sends to each rank
    recv_counts: list  # rows this rank receives from each rank

    @property
    def total_recv(self) -> int:
        return int(sum(self.recv_counts))


def plan_from_count_matrix(counts: torch.Tensor, rank: int) -> DispatchPlan:
    """counts[i, j] = rows rank i sends to rank j (host tensor)."""
    n = counts.shape[0]
    if counts.shape != (n, n) or (counts < 0).any():
        raise ValueError("count matrix must be square and non-negative")
    return DispatchPlan(send_counts=[int(c) for c in counts[rank]], recv_counts=[int(c) for c in counts[:, rank]])


class CudaBackend:
    """Device work of the EP path on this rank's GPU (the package's CUDA kernels)."""

    def __init__(self, **expert_kwargs):
        self.expert_kwargs = expert_kwargs

    def sort_by_rank(self, dest: torch.Tensor, world: int):
        """dest int32 [numel] -> (perm int32 [numel]: positions sorted by destination, stable; counts int64 [world])."""
        from .ops.moe_align_block_size import moe_align_block_size

        perm, _, _ = moe_align_block_size(dest, 1, world)
        counts = torch.bincount(dest.long(), minlength=world)
        return perm, counts

    def gather_rows(self, x: torch.Tensor, perm: torch.Tensor, top_k: int) -> torch.Tensor:
        from . import _C

        numel = perm.numel()
        out = torch.empty(numel, x.shape[1], dtype=x.dtype, device=x.device)
        _C.check(_C.lib().fmoe_gather_rows(x.data_ptr(), x.element_size(), numel, x.shape[1], perm.data_ptr(), top_k,
                                           numel, None, out.data_ptr(), _C.stream_ptr(x.device)))
        return out

    def local_experts(self, rows, w1, w2, weights, ids, **kw):
        from .ops.fused_moe import fused_experts

        return fused_experts(rows, w1, w2, weights.view(-1, 1), ids.view(-1, 1), no_combine=True,
                             **self.expert_kwargs, **kw).view(rows.shape[0], -1)

    def combine(self, z: torch.Tensor, scale: Optional[float]) -> torch.Tensor:
        from .ops.moe_sum import moe_sum

        out = torch.empty(z.shape[0], z.shape[2], dtype=z.dtype, device=z.device)
        return moe_sum(z, out, scale)


# Optional phase timing for benchmarks: set to a list and every ep_fused_experts call on CUDA tensors appends
# (phase name, start event, end event) recorded on the current stream.
PHASE_EVENTS: Optional[list] = None


class _phase:
    def __init__(self, name: str, enabled: bool):
        self.name, self.enabled = name, enabled and PHASE_EVENTS is not None

    def __enter__(self):
        if self.enabled:
            self.t0 = torch.cuda.Event(enable_timing=True)
            self.t0.record()
        return self

    def __exit__(self, *exc):
        if self.enabled:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record()
            PHASE_EVENTS.append((self.name, self.t0, t1))
        return False


def _all_to_all_rows(send: torch.Tensor, plan: DispatchPlan, group, reverse: bool = False) -> torch.Tensor:
    s, r = (plan.recv_counts, plan.send_counts) if reverse else (plan.send_counts, plan.recv_counts)
    out = send.new_empty((int(sum(r)),) + tuple(send.shape[1:]))
    dist.all_to_all_single(out, send.contiguous(), output_split_sizes=list(r), input_split_sizes=list(s), group=group)
    return out


def ep_fused_experts(
    hidden_states: torch.Tensor,
    w1_local: torch.Tensor,
    w2_local: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    num_global_experts: int,
    group=None,
    backend=None,
    routed_scaling_factor: Optional[float] = None,
    **expert_kwargs,
) -> torch.Tensor:
    """Expert-parallel `fused_experts`: `w1_local`/`w2_local` hold experts
    [rank*E/N, (rank+1)*E/N) of the global layer; `topk_ids` are global ids of this rank's tokens."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if num_global_experts % world:
        raise ValueError(f"{num_global_experts} experts do not divide over {world} ranks")
    e_local = num_global_experts // world
    if w1_local.shape[0] != e_local:
        raise ValueError(f"this rank holds {w1_local.shape[0]} experts, expected {e_local}")
    T, H = hidden_states.shape
    k = topk_ids.shape[1]
    timed = hidden_states.is_cuda
    with _phase("plan", timed):
        ids = topk_ids.to(torch.int32).reshape(-1)
        dest = torch.div(ids, e_local, rounding_mode="floor").to(torch.int32)
        perm, counts = backend.sort_by_rank(dest, world)
        # count exchange: one [N,N] matrix, one host read per layer call
        matrix = torch.empty(world * world, dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(matrix, counts.contiguous(), group=group)
        plan = plan_from_count_matrix(matrix.view(world, world).cpu(), rank)
    if sum(plan.send_counts) != T * k:
        raise RuntimeError("dispatch counts do not add up to T*k (expert id out of range?)")

    with _phase("pack", timed):
        lperm = perm.long()
        send_rows = backend.gather_rows(hidden_states.contiguous(), perm, k)
        meta = torch.stack(((ids - dest * e_local)[lperm].to(torch.int32),
                            topk_weights.reshape(-1).float()[lperm].view(torch.int32)), dim=1)
    with _phase("dispatch", timed):
        recv_rows = _all_to_all_rows(send_rows, plan, group)
        recv_meta = _all_to_all_rows(meta, plan, group)

    with _phase("experts", timed):
        local_ids = recv_meta[:, 0].contiguous()
        local_w = recv_meta[:, 1].contiguous().view(torch.float32)
        if plan.total_recv > 0:
            z_recv = backend.local_experts(recv_rows, w1_local, w2_local, local_w, local_ids, **expert_kwargs)
        else:
            z_recv = recv_rows.new_empty((0, H))
    with _phase("combine_a2a", timed):
        back = _all_to_all_rows(z_recv, plan, group, reverse=True)
    with _phase("unpermute_sum", timed):
        z = torch.empty(T * k, H, dtype=back.dtype, device=back.device)
        z.index_copy_(0, lperm, back)
        out = backend.combine(z.view(T, k, H), routed_scaling_factor)
    return out


def ep_fused_moe(hidden_states, w1_local, w2_local, gating_output, topk: int, num_global_experts: int,
                 renormalize: bool = True, use_grouped_topk: bool = False, num_expert_group=None, topk_group=None,
                 correction_bias=None, routed_scaling_factor=None, group=None, backend=None, router=None,
                 **expert_kwargs):
    """Router on this rank's tokens, then `ep_fused_experts`."""
    if router is None:
        from .ops.topk import topk as router
    tw, ti = router(hidden_states, gating_output, topk, renormalize, use_grouped_topk, num_expert_group, topk_group,
                    correction_bias, None)
    return ep_fused_experts(hidden_states, w1_local, w2_local, tw, ti, num_global_experts, group=group,
                            backend=backend, routed_scaling_factor=routed_scaling_factor, **expert_kwargs)


__all__ = ["ep_fused_experts", "ep_fused_moe", "plan_from_count_matrix", "DispatchPlan", "CudaBackend"]
