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


def _worker(rank, world, port, case, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flaggems_sglang_b200 import ep

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
        if case == "bad_ids":
            tw = torch.full((T, k), 0.25)
            ti = torch.full((T, k), E + 5, dtype=torch.int32)  # out of range on every rank
            try:
                ep.ep_fused_experts(x, w1[rank * el:(rank + 1) * el], w2[rank * el:(rank + 1) * el], tw, ti, E,
                                    backend=OracleBackend())
                q.put((rank, "no error"))
            except (RuntimeError, ValueError) as e:
                q.put((rank, "raised: " + str(e)[:60]))
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


def test_plan_from_count_matrix():
    from flaggems_sglang_b200.ep import plan_from_count_matrix

    m = torch.tensor([[1, 2, 3], [4, 5, 6], [7, 8, 9]])
    p = plan_from_count_matrix(m, 1)
    assert p.send_counts == [4, 5, 6] and p.recv_counts == [2, 5, 8] and p.total_recv == 15
    with pytest.raises(ValueError):
        plan_from_count_matrix(torch.tensor([[1, -2], [0, 1]]), 0)
    with pytest.raises(ValueError):
        plan_from_count_matrix(torch.zeros(2, 3, dtype=torch.long), 0)
