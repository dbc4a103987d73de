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
Two exchanges are built.  The default one is NCCL all-to-all (steps 3 and 5 as library calls; it needs the split
sizes on the host, i.e. one device-to-host read per call).  With a `PeerExchange` (receive areas that the peers
map through CUDA IPC) steps 2-5 run without any host read: this package's kernels store the rows straight into
the destination rank's receive area and the expert outputs straight into the source rank's slot buffer over
NVLink, and the only library calls left are a tiny count all-gather and two barriers that order the phases.
Those kernels never wait on a peer and never read peer memory.

The data movement is written against a small backend interface so that the exchange logic runs
unchanged on CPU ranks (gloo) in the tests, where the backend is the CPU oracle.
"""
from __future__ import annotations

import contextlib
import os
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


# --------------------------------------------------------------------------
# exchange over peer memory
# --------------------------------------------------------------------------
class _DeviceBytes:
    """Exposes a raw device allocation to torch (zero copy) through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _up256(n: int) -> int:
    return (n + 255) & ~255


class PeerExchange:
    """Receive areas of one process group for the P2P exchange (see fmoe_ep_* in include/fmoe_b200.h).

    Created collectively (every rank of `group`, same arguments).  `capacity` = rows this rank can receive per
    call; the default world * max_tokens * top_k can never overflow, a smaller value saves memory and an
    overflow is then reported by `_C.check_device_status` (rows beyond it are dropped, nothing is overwritten).
    One instance serves one layer call at a time (calls on it must be stream-ordered).
    """

    def __init__(self, group, max_tokens: int, top_k: int, hidden_size: int, dtype=torch.bfloat16,
                 capacity: Optional[int] = None, device=None, _lib=None):
        """`_lib`: stand-in for the C library (tests inject allocation / mapping failures on chosen ranks)."""
        import ctypes

        from . import _C

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._layout(max_tokens, top_k, hidden_size, dtype, capacity)
        lib = self._lib = _lib if _lib is not None else _C.lib()
        base = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        self._own_base, self._opened = None, []

        def agree(problem: Optional[str], what: str):
            # a step that failed on one rank must fail on all of them, or the others would wait in the next collective
            flag = torch.tensor([0 if problem is None else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
            if int(flag.item()):
                self._release()
                raise RuntimeError(f"PeerExchange: {what} failed on " +
                                   (f"this rank: {problem}" if problem else "another rank"))

        on_device = torch.cuda.device(self.device) if self.device.type == "cuda" else contextlib.nullcontext()
        with on_device:
            problem = None
            try:
                _C.check(lib.fmoe_ep_buffer_create(self.nbytes, ctypes.byref(base), handle))
                self._own_base = base.value
            except Exception as e:  # noqa: BLE001
                problem = str(e)
            agree(problem, "allocating the receive area")
            mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
            every = torch.empty(self.world * 64, dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(every, mine, group=group)
            every = every.cpu().view(self.world, 64)
            bases = []
            try:
                for j in range(self.world):
                    if j == self.rank:
                        bases.append(base.value)
                        continue
                    peer = ctypes.c_void_p()
                    raw = (ctypes.c_ubyte * 64)(*every[j].tolist())
                    _C.check(lib.fmoe_ep_buffer_open(raw, ctypes.byref(peer)))
                    self._opened.append(peer.value)
                    bases.append(peer.value)
            except Exception as e:  # noqa: BLE001
                problem = str(e)
            agree(problem, "mapping the peers' receive areas (CUDA IPC)")
        self._bind(bases, torch.as_tensor(_DeviceBytes(base.value, self.nbytes), device=self.device))
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.ids.fill_(-1)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # -- shared with the single-process emulation used by the tests -------------------------------------
    def _layout(self, max_tokens, top_k, hidden_size, dtype, capacity):
        self.max_tokens, self.top_k, self.H, self.dtype = int(max_tokens), int(top_k), int(hidden_size), dtype
        # Result rows go back either from inside the down-projection kernel (its epilogue stores to the peer) or by a
        # separate copy kernel.  None = by kernel family: the bf16 tcgen05 kernel has dedicated epilogue warps, so the
        # slower peer stores overlap the next tile (measured 2.50 against 2.55 ms, Mixtral, 2 GPUs); in the fp8
        # kernel the fold warps do the epilogue and the stores sit on the critical path (4.58 against 4.22 ms,
        # DeepSeek-V3, 2 GPUs).  FMOE_EP_FUSE_RETURN=0/1 forces one way.
        env = os.environ.get("FMOE_EP_FUSE_RETURN")
        self.fuse_return = None if env is None else env != "0"
        eb = torch.empty(0, dtype=dtype).element_size()
        if (self.H * eb) % 16:
            raise ValueError("hidden rows must be a multiple of 16 bytes")
        self.z_slots = self.max_tokens * self.top_k
        self.capacity = int(capacity) if capacity is not None else self.world * self.z_slots
        off = 0
        self._off = {}
        for name, nbytes in (("rows", self.capacity * self.H * eb), ("ids", self.capacity * 4),
                             ("weights", self.capacity * 4), ("src", self.capacity * 8),
                             ("z", self.z_slots * self.H * eb)):
            self._off[name] = (off, nbytes)
            off += _up256(nbytes)
        self.nbytes = max(off, 256)

    def _bind(self, bases, own_bytes: torch.Tensor):
        self._bytes = own_bytes

        def own(name, dt, shape):
            o, n = self._off[name]
            return own_bytes[o:o + n].view(dt).view(shape)

        self.rows = own("rows", self.dtype, (self.capacity, self.H))
        self.ids = own("ids", torch.int32, (self.capacity,))
        self.weights = own("weights", torch.float32, (self.capacity,))
        self.src = own("src", torch.int32, (self.capacity, 2))
        self.z = own("z", self.dtype, (self.z_slots, self.H))
        self.ptrs = {name: torch.tensor([b + self._off[name][0] for b in bases], dtype=torch.int64, device=self.device)
                     for name in self._off}

    @classmethod
    def emulated(cls, world: int, max_tokens: int, top_k: int, hidden_size: int, dtype=torch.bfloat16,
                 capacity: Optional[int] = None, device="cuda"):
        """`world` exchanges living in ONE process and on one GPU, the "peers" being plain local tensors: the
        same kernels and pointer tables without IPC.  The caller runs every phase for all ranks before the next
        phase (there are no barriers to wait on)."""
        out, stores = [], []
        for r in range(world):
            xc = cls.__new__(cls)
            xc.group, xc.world, xc.rank, xc.device = None, world, r, torch.device(device)
            xc._layout(max_tokens, top_k, hidden_size, dtype, capacity)
            stores.append(torch.zeros(xc.nbytes, dtype=torch.uint8, device=xc.device))
            out.append(xc)
        bases = [st.data_ptr() for st in stores]
        for xc, st in zip(out, stores):
            xc._bind(bases, st)
            xc.ids.fill_(-1)
            xc._opened, xc._own_base, xc._flag, xc._lib = [], None, None, None
        return out

    def barrier(self):
        """Stream-ordered barrier over the group: every kernel a rank enqueued before it has completed (its
        peer stores included) before any rank's later kernels start."""
        dist.all_reduce(self._flag, group=self.group)

    def _release(self):
        lib = self._lib
        for p in self._opened:
            lib.fmoe_ep_buffer_close(p)
        self._opened = []
        if self._own_base:
            lib.fmoe_ep_buffer_destroy(self._own_base)
            self._own_base = None

    def close(self):
        """Collective: unmaps the peers' areas, then frees the own one once every rank has unmapped it."""
        from . import _C

        if not self._own_base:  # emulated instance, or closed already
            return
        lib = self._lib
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._opened:
            _C.check(lib.fmoe_ep_buffer_close(p))
        self._opened = []
        dist.barrier(group=self.group)
        _C.check(lib.fmoe_ep_buffer_destroy(self._own_base))
        self._own_base = None


def p2p_route(xc: PeerExchange, hidden_states, topk_weights, topk_ids, experts_per_rank: int) -> dict:
    """Phase 1 (local): destination rank per (token, slot), rows per destination, destination-sorted order."""
    from . import _C
    from .ops.moe_align_block_size import moe_align_block_size

    T, H = hidden_states.shape
    k = topk_ids.shape[1]
    if T > xc.max_tokens or k != xc.top_k or H != xc.H or hidden_states.dtype != xc.dtype:
        raise ValueError(f"this PeerExchange was sized for <= {xc.max_tokens} tokens, top_k {xc.top_k}, H {xc.H}, {xc.dtype}")
    dev = hidden_states.device
    x = hidden_states.contiguous()
    ids = topk_ids.to(torch.int32).contiguous().view(-1)
    wts = topk_weights.to(torch.float32).contiguous().view(-1)
    dest = torch.empty(T * k, dtype=torch.int32, device=dev)
    counts = torch.empty(xc.world, dtype=torch.int32, device=dev)
    _C.check(_C.lib().fmoe_ep_route(ids.data_ptr(), T * k, experts_per_rank, xc.world, dest.data_ptr(),
                                    counts.data_ptr(), _C.stream_ptr(dev)))
    perm, _, _ = moe_align_block_size(dest, 1, xc.world) if T > 0 else (dest, None, None)
    return dict(x=x, ids=ids, wts=wts, perm=perm, counts=counts, T=T, k=k, e_local=experts_per_rank)


def p2p_send(xc: PeerExchange, state: dict, matrix: torch.Tensor) -> None:
    """Phase 2: store this rank's rows and their metadata into the destination ranks' receive areas."""
    from . import _C

    state["matrix"] = matrix
    x = state["x"]
    _C.check(_C.lib().fmoe_ep_dispatch(
        x.data_ptr(), x.element_size(), state["T"], xc.H, state["k"], state["ids"].data_ptr(), state["wts"].data_ptr(),
        state["perm"].data_ptr(), matrix.data_ptr(), xc.rank, xc.world, state["e_local"], xc.ptrs["rows"].data_ptr(),
        xc.ptrs["ids"].data_ptr(), xc.ptrs["weights"].data_ptr(), xc.ptrs["src"].data_ptr(), xc.capacity,
        _C.stream_ptr(x.device)))


def p2p_experts(xc: PeerExchange, state: dict, w1_local, w2_local, fuse_return: Optional[bool] = None,
                **expert_kwargs) -> Optional[torch.Tensor]:
    """Phase 3 (after the barrier): grouped GEMMs over the receive area; rows past the received count carry
    id -1 and are skipped by moe_align_block_size.  With `fuse_return` (and a kernel family that takes row
    addresses) the down-projection epilogue stores every result row straight into the slot buffer of the
    rank the row came from, and None is returned; otherwise the rows come back for `p2p_return`.
    `fuse_return=None` decides by kernel family (bf16: fused, fp8: separate)."""
    from . import _C
    from .ops.fused_moe import _pick_variant, fused_experts

    dev = xc.rows.device
    fp8 = expert_kwargs.get("use_fp8_w8a8", False)
    # kernel family for the rows a balanced routing would bring (this rank's own count), not for the capacity
    name, _ = _pick_variant(torch.float8_e4m3fn if fp8 else w1_local.dtype, max(state["T"] * state["k"], 1),
                            w1_local.shape[0], w2_local.shape[2], xc.H, expert_kwargs.get("variant"))
    expert_kwargs = dict(expert_kwargs, variant=name)
    if fuse_return is None:
        fuse_return = not fp8
    fuse_return = fuse_return and name in ("stream", "tcgen05")
    out_rows = torch.empty(xc.capacity, dtype=torch.int64, device=dev) if fuse_return else None
    _C.check(_C.lib().fmoe_ep_mask_tail(xc.ids.data_ptr(), state["matrix"].data_ptr(), xc.rank, xc.world, xc.capacity,
                                        xc.src.data_ptr(), xc.z_slots, xc.ptrs["z"].data_ptr(),
                                        xc.H * xc.rows.element_size(), _C.ptr(out_rows), _C.stream_ptr(dev)))
    z = fused_experts(xc.rows, w1_local, w2_local, xc.weights.view(-1, 1), xc.ids.view(-1, 1), no_combine=True,
                      out_rows=out_rows, **expert_kwargs)
    return None if fuse_return else z.view(xc.capacity, xc.H)


def p2p_return(xc: PeerExchange, state: dict, z_rows: Optional[torch.Tensor]) -> None:
    """Phase 4: store every expert output row into the slot buffer of the rank it came from (nothing to do
    when the down projection already did)."""
    from . import _C

    if z_rows is None:
        return

    _C.check(_C.lib().fmoe_ep_combine(z_rows.data_ptr(), z_rows.element_size(), xc.H, xc.src.data_ptr(),
                                      state["matrix"].data_ptr(), xc.rank, xc.world, xc.capacity, xc.z_slots,
                                      xc.ptrs["z"].data_ptr(), _C.stream_ptr(z_rows.device)))


def p2p_finish(xc: PeerExchange, state: dict, routed_scaling_factor: Optional[float]) -> torch.Tensor:
    """Phase 5 (after the barrier): sum the top_k slots of every token."""
    from .ops.moe_sum import moe_sum

    T, k = state["T"], state["k"]
    out = torch.empty(T, xc.H, dtype=xc.dtype, device=xc.rows.device)
    if T == 0:
        return out
    return moe_sum(xc.z[:T * k].view(T, k, xc.H), out, routed_scaling_factor)


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
    exchange: Optional["PeerExchange"] = None,
    **expert_kwargs,
) -> torch.Tensor:
    """Expert-parallel `fused_experts`: `w1_local`/`w2_local` hold experts
    [rank*E/N, (rank+1)*E/N) of the global layer; `topk_ids` are global ids of this rank's tokens.
    `exchange`: a PeerExchange of the same group -> rows travel by P2P stores of this package's kernels
    instead of NCCL all-to-all, with no host read on the way."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if num_global_experts % world:
        raise ValueError(f"{num_global_experts} experts do not divide over {world} ranks")
    e_local = num_global_experts // world
    if w1_local.shape[0] != e_local:
        raise ValueError(f"this rank holds {w1_local.shape[0]} experts, expected {e_local}")
    if exchange is not None:
        if exchange.world != world or exchange.rank != rank:
            raise ValueError("the PeerExchange belongs to another group")
        with _phase("route", True):
            state = p2p_route(exchange, hidden_states, topk_weights, topk_ids, e_local)
        with _phase("counts", True):
            matrix = torch.empty(world * world, dtype=torch.int32, device=hidden_states.device)
            dist.all_gather_into_tensor(matrix, state["counts"], group=group)
        with _phase("dispatch", True):
            p2p_send(exchange, state, matrix)
            exchange.barrier()
        with _phase("experts", True):
            z_rows = p2p_experts(exchange, state, w1_local, w2_local, fuse_return=exchange.fuse_return,
                                 **expert_kwargs)
        with _phase("combine", True):
            p2p_return(exchange, state, z_rows)
            exchange.barrier()
        with _phase("sum", True):
            return p2p_finish(exchange, state, routed_scaling_factor)
    T, H = hidden_states.shape
    k = topk_ids.shape[1]
    timed = hidden_states.is_cuda
    with _phase("plan", timed):
        ids = topk_ids.to(torch.int32).reshape(-1)
        dest = torch.div(ids, e_local, rounding_mode="floor").to(torch.int32)
        dest = torch.where((ids >= 0) & (ids < num_global_experts), dest, torch.full_like(dest, world))  # world = nowhere
        perm, counts = backend.sort_by_rank(dest, world)
        # count exchange: one [N, N+1] matrix (last column = the slots the rank had to place), one host read per
        # layer call.  Every rank checks every row, so a rank whose counts do not add up (an expert id out of
        # range) makes ALL ranks raise here instead of leaving the others waiting in the all-to-all.
        mine = torch.cat((counts.to(torch.int64)[:world], counts.new_tensor([T * k], dtype=torch.int64)))
        matrix = torch.empty(world * (world + 1), dtype=torch.int64, device=counts.device)
        dist.all_gather_into_tensor(matrix, mine.contiguous(), group=group)
        matrix = matrix.view(world, world + 1).cpu()
        bad = [i for i in range(world) if int(matrix[i, :world].sum()) != int(matrix[i, world])]
        if bad:
            raise RuntimeError(f"dispatch counts of rank(s) {bad} do not add up to their T*k (expert id out of range?)")
        plan = plan_from_count_matrix(matrix[:, :world], rank)

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
                 exchange=None, **expert_kwargs):
    """Router on this rank's tokens, then `ep_fused_experts`."""
    if router is None:
        from .ops.topk import topk as router
    tw, ti = router(hidden_states, gating_output, topk, renormalize, use_grouped_topk, num_expert_group, topk_group,
                    correction_bias, None)
    return ep_fused_experts(hidden_states, w1_local, w2_local, tw, ti, num_global_experts, group=group,
                            backend=backend, routed_scaling_factor=routed_scaling_factor, exchange=exchange,
                            **expert_kwargs)


__all__ = ["ep_fused_experts", "ep_fused_moe", "plan_from_count_matrix", "DispatchPlan", "CudaBackend", "PeerExchange"]
