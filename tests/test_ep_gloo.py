"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2 and 4).

The device work is replaced by a backend built on the CPU oracle, so what runs here is exactly the
host logic of flaggems_sglang_b200.ep: destination sort, count exchange, split sizes, the three
all-to-alls, un-permute and combine.  Each rank's result must equal the single-process oracle on the
same tokens with the full (unsharded) weights.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import experts as OE
from oracle import routing as OR


class OracleBackend:
    def sort_by_rank(self, dest, world):
        perm = torch.argsort(dest.long(), stable=True).to(torch.int32)
        return perm, torch.bincount(dest.long(), minlength=world)

    def gather_rows(self, x, perm, top_k):
        return x[(perm.long() // top_k)]

    def local_experts(self, rows, w1, w2, weights, ids, **kw):
        return OE.fused_experts(rows, w1, w2, weights.view(-1, 1), ids.view(-1, 1), no_combine=True).view(rows.shape[0], -1)

    def combine(self, z, scale):
        out = OE.moe_sum(z).to(z.dtype)
        if scale is not None and scale != 1.0:
            out = (out.float() * scale).to(z.dtype)
        return out


def _oracle_router(hidden, logits, topk, renorm, grouped, ng, tg, bias, scale):
    if grouped:
        return OR.grouped_topk(logits, bias, topk, ng, tg, renorm, scale)
    return OR.softmax_topk(logits, topk, renorm)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _layer(E, H, I, seed=0):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16()
    return w1, w2


class _FailingLib:
    """Stand-in for the C library: the receive-area allocation fails on `bad_rank`, succeeds elsewhere."""

    def __init__(self, rank, bad_rank, fail_open=False):
        self.rank, self.bad_rank, self.fail_open = rank, bad_rank, fail_open
        self.destroyed, self.closed = [], []

    def fmoe_ep_buffer_create(self, nbytes, ptr_ref, handle):
        if self.rank == self.bad_rank and not self.fail_open:
            return 2
        ptr_ref._obj.value = 0x1000 * (self.rank + 1)
        return 0

    def fmoe_ep_buffer_open(self, raw, ptr_ref):
        if self.rank == self.bad_rank and self.fail_open:
            return 2
        ptr_ref._obj.value = 0x900000
        return 0

    def fmoe_ep_buffer_close(self, p):
        self.closed.append(p)
        return 0

    def fmoe_ep_buffer_destroy(self, p):
        self.destroyed.append(p)
        return 0


def _worker(rank, world, port, case, q):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20 if case == "early_exit" else 240))
    try:
        from flaggems_sglang_b200 import ep

        if case in ("alloc_fails", "map_fails"):
            # one rank cannot allocate (or map) its receive area: every rank must raise, none may be left waiting
            fake = _FailingLib(rank, bad_rank=1, fail_open=case == "map_fails")
            try:
                ep.PeerExchange(None, 8, 2, 64, torch.bfloat16, device="cpu", _lib=fake)
                q.put((rank, "no error"))
            except RuntimeError as e:
                released = (case == "alloc_fails" and rank == 1) or len(fake.destroyed) == 1
                q.put((rank, ("raised: " if released else "raised without releasing: ") + str(e)[:80]))
            return
        if case == "early_exit" and rank == 1:
            q.put((rank, "left"))
            return  # leaves between steps: never joins the layer call the others make

        E, H, I, k = 16, 64, 96, 4
        w1, w2 = _layer(E, H, I)
        el = E // world
        g = torch.Generator().manual_seed(100 + rank)
        T = [5, 0, 9, 3][rank] if case == "ragged" else 7
        x = torch.randn(T, H, generator=g).bfloat16()
        logits = torch.randn(T, E, generator=g)
        if case == "skew":
            logits[:, :el] += 6.0  # nearly everything goes to rank 0
        grouped = case == "grouped"
        bias = torch.randn(E, generator=torch.Generator().manual_seed(3)) * 0.1 if grouped else None
        if case in ("bad_ids", "bad_ids_one_rank", "early_exit"):
            tw = torch.full((T, k), 0.25)
            ti = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
            if case == "bad_ids":
                ti[:] = E + 5      # out of range on every rank
            elif case == "bad_ids_one_rank" and rank == 1:
                ti[2, 1] = -3      # one bad slot on one rank: its counts no longer add up to T*k
            try:
                ep.ep_fused_experts(x, w1[rank * el:(rank + 1) * el], w2[rank * el:(rank + 1) * el], tw, ti, E,
                                    backend=OracleBackend())
                q.put((rank, "no error"))
            except (RuntimeError, ValueError) as e:
                q.put((rank, "raised: " + str(e)[:60]))
            except Exception as e:  # noqa: BLE001  (gloo reports a lost peer with its own exception types)
                q.put((rank, "raised: " + type(e).__name__))
            return
        out = ep.ep_fused_moe(x, w1[rank * el:(rank + 1) * el], w2[rank * el:(rank + 1) * el], logits, k, E,
                              use_grouped_topk=grouped, num_expert_group=4, topk_group=2, correction_bias=bias,
                              routed_scaling_factor=2.5 if grouped else None, backend=OracleBackend(),
                              router=_oracle_router)
        tw, ti = _oracle_router(x, logits, k, True, grouped, 4, 2, bias, None)
        ref = OE.fused_experts(x, w1, w2, tw, ti, routed_scaling_factor=2.5 if grouped else None)
        # the CPU GEMM blocks differently for different row counts, so allow bf16 rounding noise
        ok = out.shape == ref.shape and (T == 0 or bool(
            (out.float() - ref.float()).norm() <= 2e-3 * ref.float().norm()
            and (out.float() - ref.float()).abs().max() <= 2.0 ** -7 * ref.float().abs().max()))
        q.put((rank, ok, float((out.float() - ref.float()).abs().max()) if T else 0.0))
    finally:
        dist.destroy_process_group()


def _run(world, case):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(res)


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", ["uniform", "skew", "ragged", "grouped"])
def test_ep_matches_single_process_oracle(world, case):
    for rank, equal, err in _run(world, case):
        assert equal, f"rank {rank}: EP result differs from the oracle (max abs {err})"


def test_ep_rejects_out_of_range_ids():
    for rank, msg in _run(2, "bad_ids"):
        assert msg.startswith("raised"), f"rank {rank}: {msg}"


def test_one_rank_with_bad_counts_makes_every_rank_raise():
    """A rank whose count vector does not add up to its T*k (one expert id out of range) is seen by all ranks in
    the count exchange: all raise before the all-to-all, nobody hangs."""
    for rank, msg in _run(2, "bad_ids_one_rank"):
        assert msg.startswith("raised") and "rank(s) [1]" in msg, f"rank {rank}: {msg}"


def test_rank_that_leaves_before_dispatch_is_detected():
    """A rank that exits between steps: the others' next collective ends with an error (connection lost or the
    process-group time-out) instead of blocking for ever."""
    res = dict(_run(2, "early_exit"))
    assert res[1] == "left"
    assert res[0].startswith("raised"), res[0]


@pytest.mark.parametrize("case", ["alloc_fails", "map_fails"])
def test_peer_exchange_setup_failure_is_collective(case):
    """PeerExchange set-up: a failure on one rank (allocation of the receive area / mapping a peer's area) raises
    on every rank, and a rank that had allocated its area gives it back."""
    res = dict(_run(2, case))
    assert res[0].startswith("raised: ") and "another rank" in res[0], res[0]
    assert res[1].startswith("raised: ") and "this rank" in res[1], res[1]


def test_plan_from_count_matrix():
    from flaggems_sglang_b200.ep import plan_from_count_matrix

    m = torch.tensor([[1, 2, 3], [4, 5, 6], [7, 8, 9]])
    p = plan_from_count_matrix(m, 1)
    assert p.send_counts == [4, 5, 6] and p.recv_counts == [2, 5, 8] and p.total_recv == 15
    with pytest.raises(ValueError):
        plan_from_count_matrix(torch.tensor([[1, -2], [0, 1]]), 0)
    with pytest.raises(ValueError):
        plan_from_count_matrix(torch.zeros(2, 3, dtype=torch.long), 0)
