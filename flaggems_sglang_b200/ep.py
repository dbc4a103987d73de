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
map through CUDA IPC) steps 2-5 run without any host read: the ranks all-gather their per-expert row counts, and
this package's kernels store every row straight into the owner's receive area AT ITS PLACE IN THE PADDED
EXPERT-SORTED ORDER the grouped GEMMs read (for e4m3 layers as e4m3 bytes + scales, quantised once by the
sender), so the receiver runs neither moe_align, nor a row copy, nor a quantisation pass; the expert outputs go
straight into the source rank's slot buffer over NVLink, and the only library calls left are the count
all-gather and two barriers that order the phases.  Those kernels never wait on a peer and never read peer memory.

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

    Created collectively (every rank of `group`, same arguments) for one layer shape: `num_local_experts` experts
    per rank with intermediate size `intermediate_size`; `fp8=True` for e4m3 weights (token rows then travel as
    e4m3 bytes + 128-channel scales, quantised once by the sender).  Rows arrive in the padded expert-sorted order
    of the grouped GEMMs, so the kernel family and its row block are fixed here, from `max_tokens * top_k` slots
    per rank (`variant=` overrides the choice).

    `capacity` = rows this rank can receive per call; the default world * max_tokens * top_k (+ block padding per
    expert) can never overflow, a smaller value saves memory and an overflow is then reported by
    `_C.check_device_status` (rows beyond it are dropped, their result rows read as zero, nothing is overwritten).
    One instance serves one layer call at a time (calls on it must be stream-ordered).
    """

    def __init__(self, group, max_tokens: int, top_k: int, hidden_size: int, dtype=torch.bfloat16,
                 capacity: Optional[int] = None, device=None, _lib=None, num_local_experts: int = 1,
                 intermediate_size: int = 128, fp8: bool = False, variant: Optional[str] = None):
        """`_lib`: stand-in for the C library (tests inject allocation / mapping failures on chosen ranks)."""
        import ctypes

        from . import _C

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._layout(max_tokens, top_k, hidden_size, dtype, capacity, num_local_experts, intermediate_size, fp8, variant)
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
        self._bytes.zero_()  # padding rows of the area are read by the GEMMs (and ignored): keep them finite
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    # -- shared with the single-process emulation used by the tests -------------------------------------
    def _layout(self, max_tokens, top_k, hidden_size, dtype, capacity, num_local_experts, intermediate_size, fp8,
                variant):
        from .ops.fused_moe import _pick_variant

        self.max_tokens, self.top_k, self.H, self.dtype = int(max_tokens), int(top_k), int(hidden_size), dtype
        self.e_local, self.I, self.fp8 = int(num_local_experts), int(intermediate_size), bool(fp8)
        self.total_experts = self.e_local * self.world
        # kernel family and row block of the expert computation, the same on every rank (the senders lay the rows out)
        wdt = torch.float8_e4m3fn if fp8 else dtype
        self.variant, self.block = _pick_variant(wdt, max(self.max_tokens * self.top_k, 1), self.e_local, self.I,
                                                 self.H, variant)
        # Result rows go back either from inside the down-projection kernel (its epilogue stores to the peer:
        # fmoe_gemm_args.out_rows) or by a separate copy kernel.  The copy kernel is the default: measured on Mixtral,
        # fused against separate, 2.60-2.63 / 2.60-2.62 ms on 2 GPUs (a tie: the bf16 kernel's dedicated epilogue warps
        # hide the peer stores of half of the rows), 2.83 / 2.74 ms on 4 and 3.09 / 2.77 ms on 8 (with three quarters
        # or more of the rows remote the stores hold the GEMM up: down GEMM 1.27 against 0.79 ms); in the fp8 kernel
        # the fold warps do the epilogue and the stores sit on the critical path (4.58 against 4.22 ms, DeepSeek-V3,
        # 2 GPUs).  FMOE_EP_FUSE_RETURN=1 selects the fused return.
        env = os.environ.get("FMOE_EP_FUSE_RETURN")
        self.fuse_return = None if env is None else env != "0"
        eb = torch.empty(0, dtype=dtype).element_size()
        if (self.H * eb) % 16 or (fp8 and self.H % 128):
            raise ValueError("hidden rows must be a multiple of 16 bytes (128 channels for e4m3)")
        self.row_bytes = self.H if fp8 else self.H * eb
        self.z_slots = self.max_tokens * self.top_k
        worst = self.world * self.z_slots + self.e_local * (self.block - 1)
        cap = int(capacity) if capacity is not None else worst
        self.capacity = (cap + self.block - 1) // self.block * self.block
        off = 0
        self._off = {}
        for name, nbytes in (("rows", self.capacity * self.row_bytes),
                             ("scales", self.capacity * (self.H // 128) * 4 if fp8 else 0),
                             ("weights", self.capacity * 4), ("src", self.capacity * 8),
                             ("z", self.z_slots * self.H * eb)):
            self._off[name] = (off, nbytes)
            off += _up256(nbytes)
        self.nbytes = max(off, 256)

    def _bind(self, bases, own_bytes: torch.Tensor):
        self._bytes = own_bytes
        dev = self.device

        def own(name, dt, shape):
            o, n = self._off[name]
            return own_bytes[o:o + n].view(dt).view(shape)

        self.rows = own("rows", torch.float8_e4m3fn if self.fp8 else self.dtype, (self.capacity, self.H))
        self.scales = own("scales", torch.float32, (self.capacity, self.H // 128)) if self.fp8 else None
        self.weights = own("weights", torch.float32, (self.capacity,))
        self.src = own("src", torch.int32, (self.capacity, 2))
        self.z = own("z", self.dtype, (self.z_slots, self.H))
        self.ptrs = {name: torch.tensor([b + self._off[name][0] for b in bases], dtype=torch.int64, device=dev)
                     for name in self._off}
        # local tables and intermediates of the expert computation (never written by a peer)
        cap, blk = self.capacity, self.block
        self.sorted_ids = torch.empty(cap, dtype=torch.int32, device=dev)
        self.expert_ids = torch.empty(cap // blk, dtype=torch.int32, device=dev)
        self.npp = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out_rows = torch.zeros(cap, dtype=torch.int64, device=dev)
        tc = self.variant.startswith("tcgen05")
        if self.fp8:
            self.act = torch.empty(cap, self.I, dtype=torch.bfloat16 if tc else torch.float32, device=dev)
            self.actq = torch.empty(cap, self.I, dtype=torch.float8_e4m3fn, device=dev)
            self.act_scale = torch.empty(cap, self.I // 128, dtype=torch.float32, device=dev)
        else:
            self.act = torch.empty(cap, self.I, dtype=self.dtype, device=dev)
        self._z_local = None  # [capacity, H], allocated on first use of the separate return
        self._split_ws = None  # tail-split scratch of the bf16 tcgen05 GEMMs, allocated on first use

    @classmethod
    def emulated(cls, world: int, max_tokens: int, top_k: int, hidden_size: int, dtype=torch.bfloat16,
                 capacity: Optional[int] = None, device="cuda", num_local_experts: int = 1,
                 intermediate_size: int = 128, fp8: bool = False, variant: Optional[str] = None):
        """`world` exchanges living in ONE process and on one GPU, the "peers" being plain local tensors: the
        same kernels and pointer tables without IPC.  The caller runs every phase for all ranks before the next
        phase (there are no barriers to wait on)."""
        out, stores = [], []
        for r in range(world):
            xc = cls.__new__(cls)
            xc.group, xc.world, xc.rank, xc.device = None, world, r, torch.device(device)
            xc._layout(max_tokens, top_k, hidden_size, dtype, capacity, num_local_experts, intermediate_size, fp8, variant)
            stores.append(torch.zeros(xc.nbytes, dtype=torch.uint8, device=xc.device))
            out.append(xc)
        bases = [st.data_ptr() for st in stores]
        for xc, st in zip(out, stores):
            xc._bind(bases, st)
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
    """Phase 1 (local): rows per global expert, the expert-sorted order of this rank's (token, slot) pairs and,
    for e4m3 layers, the token rows quantised once."""
    from . import _C
    from .ops.moe_align_block_size import moe_align_block_size

    T, H = hidden_states.shape
    k = topk_ids.shape[1]
    if T > xc.max_tokens or k != xc.top_k or H != xc.H or hidden_states.dtype != xc.dtype or experts_per_rank != xc.e_local:
        raise ValueError(f"this PeerExchange was sized for <= {xc.max_tokens} tokens, top_k {xc.top_k}, H {xc.H}, "
                         f"{xc.dtype}, {xc.e_local} experts per rank")
    dev = hidden_states.device
    lib, st = _C.lib(), _C.stream_ptr(dev)
    x = hidden_states.contiguous()
    ids = topk_ids.to(torch.int32).contiguous().view(-1)
    wts = topk_weights.to(torch.float32).contiguous().view(-1)
    counts = torch.empty(xc.total_experts, dtype=torch.int32, device=dev)
    _C.check(lib.fmoe_ep_expert_counts(ids.data_ptr(), T * k, xc.total_experts, counts.data_ptr(), st))
    perm, _, _ = moe_align_block_size(ids, 1, xc.total_experts) if T > 0 else (ids, None, None)
    state = dict(x=x, ids=ids, wts=wts, perm=perm, counts=counts, T=T, k=k, scales=None)
    if xc.fp8 and T > 0:
        xq = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=dev)
        xs = torch.empty(T, H // 128, dtype=torch.float32, device=dev)
        _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, T, H, None, 1, 0, None, xq.data_ptr(), xs.data_ptr(), st))
        state.update(x=xq, scales=xs)
    return state


def p2p_send(xc: PeerExchange, state: dict, matrix: torch.Tensor) -> None:
    """Phase 2: store this rank's rows and their metadata into the owners' receive areas, at the positions the
    count matrix [world * total_experts] assigns."""
    from . import _C

    state["matrix"] = matrix
    x, sc = state["x"], state["scales"]
    _C.check(_C.lib().fmoe_ep_dispatch_sorted(
        x.data_ptr(), xc.row_bytes, _C.ptr(sc), xc.H // 128 if sc is not None else 0, state["T"], state["k"],
        state["ids"].data_ptr(), state["wts"].data_ptr(), state["perm"].data_ptr(), matrix.data_ptr(), xc.rank,
        xc.world, xc.total_experts, xc.e_local, xc.block, xc.ptrs["rows"].data_ptr(),
        xc.ptrs["scales"].data_ptr() if sc is not None else None, xc.ptrs["weights"].data_ptr(),
        xc.ptrs["src"].data_ptr(), xc.capacity, xc.z.data_ptr(), xc.H * xc.z.element_size(), _C.stream_ptr(x.device)))


def p2p_experts(xc: PeerExchange, state: dict, w1_local, w2_local, fuse_return: Optional[bool] = None,
                activation: str = "silu", apply_router_weight_on_input: bool = False, use_fp8_w8a8: bool = False,
                w1_scale=None, w2_scale=None, block_shape=None, variant=None) -> Optional[torch.Tensor]:
    """Phase 3 (after the barrier): the grouped GEMMs straight over the receive area, whose rows already stand in
    the padded expert-sorted order.  With `fuse_return` (and a kernel family that takes row addresses) the
    down-projection epilogue stores every result row straight into the slot buffer of the rank the row came
    from, and None is returned; otherwise the rows come back for `p2p_return`.
    `fuse_return=None` means separate (measured faster or equal everywhere, see PeerExchange)."""
    from . import _C

    assert use_fp8_w8a8 == xc.fp8, "this PeerExchange was created for the other weight type"
    assert variant in (None, xc.variant), "the kernel family is fixed when the PeerExchange is created"
    if xc.fp8:
        assert block_shape is not None and list(block_shape) == [128, 128] and w1_scale is not None and w2_scale is not None
    E, twoI, H = w1_local.shape
    assert E == xc.e_local and twoI == 2 * xc.I and H == xc.H, "local weights do not match the PeerExchange's layer shape"
    dev = xc.rows.device
    lib, st = _C.lib(), _C.stream_ptr(dev)
    if fuse_return is None:
        fuse_return = False
    fuse_return = fuse_return and xc.variant in ("stream", "tcgen05")
    cap, blk = xc.capacity, xc.block
    _C.check(lib.fmoe_ep_recv_tables(state["matrix"].data_ptr(), xc.rank, xc.world, xc.total_experts, xc.e_local, blk, cap,
                                     xc.src.data_ptr(), xc.z_slots, xc.ptrs["z"].data_ptr(), xc.H * xc.z.element_size(),
                                     xc.sorted_ids.data_ptr(), xc.expert_ids.data_ptr(), xc.expert_ids.numel(),
                                     xc.npp.data_ptr(), xc.out_rows.data_ptr(), st))
    w1c, w2c = w1_local.contiguous(), w2_local.contiguous()
    code = _C.E4M3 if xc.fp8 else _C.DTYPE_CODE[xc.dtype]
    common = dict(variant=_C.VARIANTS[xc.variant], activation=_C.ACTIVATIONS[activation], num_experts=xc.e_local, top_k=1,
                  block_size=blk, numel=cap, sorted_cap=cap, max_blocks=cap // blk, a_gather=0, a_rows=cap,
                  sorted_token_ids=xc.sorted_ids.data_ptr(), expert_ids=xc.expert_ids.data_ptr(),
                  num_tokens_post_padded=xc.npp.data_ptr())
    if xc.variant == "tcgen05" and not xc.fp8:
        if xc._split_ws is None:
            xc._split_ws = torch.empty(int(lib.fmoe_gemm_split_workspace_bytes()), dtype=torch.uint8, device=xc.device)
        common.update(split_ws=xc._split_ws.data_ptr(), split_ws_bytes=xc._split_ws.numel())
    row_w = xc.weights.data_ptr()
    act_code = _C.DTYPE_CODE[xc.act.dtype]
    g1 = _C.GemmArgs(dtype=code, out_dtype=act_code, n=xc.I, k=xc.H, a=xc.rows.data_ptr(), a_scale=_C.ptr(xc.scales),
                     w=w1c.data_ptr(), w_scale=_C.ptr(w1_scale.float().contiguous()) if xc.fp8 else None,
                     row_scale=row_w if apply_router_weight_on_input else None, out=xc.act.data_ptr(), **common)
    with _phase("gemm1", True):
        _C.check(lib.fmoe_gemm1_silu(g1, st))
    a2, a2_scale = xc.act, None
    if xc.fp8:
        _C.check(lib.fmoe_quant_fp8_group128(xc.act.data_ptr(), act_code, cap, xc.I, xc.sorted_ids.data_ptr(), 0, cap,
                                             xc.npp.data_ptr(), xc.actq.data_ptr(), xc.act_scale.data_ptr(), st))
        a2, a2_scale = xc.actq, xc.act_scale
    z_local = None
    if not fuse_return:
        if xc._z_local is None:
            xc._z_local = torch.empty(cap, xc.H, dtype=xc.dtype, device=dev)
        z_local = xc._z_local
    g2 = _C.GemmArgs(dtype=code, out_dtype=_C.DTYPE_CODE[xc.dtype], n=xc.H, k=xc.I, a=a2.data_ptr(), a_scale=_C.ptr(a2_scale),
                     w=w2c.data_ptr(), w_scale=_C.ptr(w2_scale.float().contiguous()) if xc.fp8 else None,
                     row_scale=None if apply_router_weight_on_input else row_w, out=_C.ptr(z_local),
                     out_rows=xc.out_rows.data_ptr() if fuse_return else None, **common)
    with _phase("gemm2", True):
        _C.check(lib.fmoe_gemm2(g2, st))
    return z_local


def p2p_return(xc: PeerExchange, state: dict, z_rows: Optional[torch.Tensor]) -> None:
    """Phase 4: store every expert output row into the slot buffer of the rank it came from (nothing to do
    when the down projection already did)."""
    from . import _C

    if z_rows is None:
        return
    _C.check(_C.lib().fmoe_ep_scatter_rows(z_rows.data_ptr(), xc.H * z_rows.element_size(), xc.out_rows.data_ptr(),
                                           xc.npp.data_ptr(), xc.capacity, _C.stream_ptr(z_rows.device)))


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
            matrix = torch.empty(world * exchange.total_experts, dtype=torch.int32, device=hidden_states.device)
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
