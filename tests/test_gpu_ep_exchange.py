"""Expert-parallel exchange over peer memory, exercised on ONE GPU: `PeerExchange.emulated` makes the "peers"
plain local tensors, so the count / dispatch / table / return kernels and their pointer tables run exactly as
between processes, phase by phase for all ranks (there is nothing to wait on).  Every emulated rank's output
must match the single-GPU op on that rank's tokens with the full weights.  The IPC mapping itself is covered
by test_gpu_ep.py on two GPUs."""
import pytest
import torch

from oracle import routing as OR

pytestmark = pytest.mark.gpu


def _layer(E, H, I, seed):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16().cuda()
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16().cuda()
    return w1, w2


def _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, kw_of_rank, capacity=None, rsf=None, bad_id=False,
                  fuse=None, variant=None):
    el = E // world
    fp8 = bool(kw_of_rank(0).get("use_fp8_w8a8"))
    xcs = ep.PeerExchange.emulated(world, max(max(tokens), 1), k, H, torch.bfloat16, capacity=capacity,
                                   num_local_experts=el, intermediate_size=w2.shape[2], fp8=fp8, variant=variant)
    xs, states = [], []
    for r in range(world):
        g = torch.Generator().manual_seed(100 + r)
        x = torch.randn(tokens[r], H, generator=g).bfloat16()
        tw, ti = OR.softmax_topk(torch.randn(tokens[r], E, generator=g), k, True)
        if bad_id and r == 1:
            ti[0, 0] = E + 3
        xs.append((x.cuda(), tw.cuda(), ti.cuda()))
        states.append(ep.p2p_route(xcs[r], xs[r][0], xs[r][1], xs[r][2], el))
    matrix = torch.cat([s["counts"] for s in states])
    for r in range(world):
        ep.p2p_send(xcs[r], states[r], matrix)
    zs = [ep.p2p_experts(xcs[r], states[r], w1[r * el:(r + 1) * el].contiguous(), w2[r * el:(r + 1) * el].contiguous(),
                         fuse_return=fuse, **kw_of_rank(r)) for r in range(world)]
    if fuse is not None:
        assert all((z is None) == fuse for z in zs)
    for r in range(world):
        ep.p2p_return(xcs[r], states[r], zs[r])
    outs = [ep.p2p_finish(xcs[r], states[r], rsf) for r in range(world)]
    torch.cuda.synchronize()
    return xs, outs, matrix, xcs


@pytest.mark.parametrize("fuse", [True, False], ids=["gemm2_stores_to_peer", "separate_combine"])
@pytest.mark.parametrize("world,tokens", [(4, [300, 77, 1, 0]), (2, [64, 64]), (8, [40, 3, 0, 129, 7, 1, 55, 20])])
def test_emulated_ranks_match_single_gpu_bf16(world, tokens, fuse):
    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import _C, ep

    E, H, I, k = 16, 512, 256, 4
    w1, w2 = _layer(E, H, I, 0)
    xs, outs, matrix, xcs = _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {}, rsf=1.5, fuse=fuse)
    _C.check_device_status()
    m = matrix.view(world, E).cpu()  # rows per (rank, global expert)
    assert m.sum(1).tolist() == [t * k for t in tokens]
    for r in range(world):
        x, tw, ti = xs[r]
        if tokens[r] == 0:
            assert outs[r].shape == (0, H)
            continue
        ref = fg.fused_experts(x, w1, w2, tw, ti, routed_scaling_factor=1.5)
        err = float((outs[r].float() - ref.float()).norm() / ref.float().norm())
        assert err < 5e-3, f"rank {r}: rel-L2 {err}"
        # the receive area's tables describe exactly the announced rows: per local expert a block-aligned
        # segment holding the rows of all ranks, padding marked by the sentinel
        el, blk, cap = E // world, xcs[r].block, xcs[r].capacity
        per_expert = m[:, r * el:(r + 1) * el].sum(0)
        sid = xcs[r].sorted_ids.cpu()
        assert int((sid < cap).sum()) == int(per_expert.sum())
        assert int(xcs[r].npp.item()) == int(((per_expert + blk - 1) // blk * blk).sum())
        eid = xcs[r].expert_ids.cpu()
        used_blocks = int(xcs[r].npp.item()) // blk
        assert eid[:used_blocks].tolist() == [e for e in range(el) for _ in range(int((per_expert[e] + blk - 1) // blk))]
        assert (eid[used_blocks:] == -1).all()


def test_emulated_ranks_forced_same_kernel_family_is_bit_exact(monkeypatch):
    """With the kernel family pinned on both sides, dispatching the rows to the expert ranks and back changes
    nothing in the arithmetic of a row: the result equals the single-GPU op bit for bit.  (The single-GPU op runs
    without its tail split here: cutting a tile along K over several CTAs changes the fp32 summation order, and
    which tiles are cut depends on how many rows a launch holds.)"""
    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import _C, ep

    monkeypatch.setenv("FMOE_TC_SPLIT_TAIL", "0")

    world, tokens, E, H, I, k = 4, [200, 130, 90, 256], 8, 256, 128, 2
    w1, w2 = _layer(E, H, I, 1)
    xs, outs, _, _ = _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {}, variant="tcgen05")
    _C.check_device_status()
    for r in range(world):
        x, tw, ti = xs[r]
        ref = fg.fused_experts(x, w1, w2, tw, ti, variant="tcgen05")
        assert torch.equal(outs[r], ref)


@pytest.mark.parametrize("fuse", [True, False], ids=["gemm2_stores_to_peer", "separate_combine"])
def test_emulated_ranks_fp8(fuse):
    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import _C, ep

    world, tokens, E, H, I, k = 2, [150, 33], 8, 512, 256, 2
    w1, w2 = _layer(E, H, I, 2)
    w1q, s1 = fg.quant_weight_block128(w1)
    w2q, s2 = fg.quant_weight_block128(w2)
    el = E // world

    def kw(r):
        return dict(use_fp8_w8a8=True, w1_scale=s1[r * el:(r + 1) * el].contiguous(),
                    w2_scale=s2[r * el:(r + 1) * el].contiguous(), block_shape=[128, 128])

    xs, outs, _, _ = _run_emulated(fg, ep, world, tokens, E, H, k, w1q, w2q, kw, fuse=fuse)
    _C.check_device_status()
    for r in range(world):
        x, tw, ti = xs[r]
        ref = fg.fused_experts(x, w1q, w2q, tw, ti, use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, block_shape=[128, 128])
        err = float((outs[r].float() - ref.float()).norm() / ref.float().norm())
        assert err < 3e-2, f"rank {r}: rel-L2 {err}"


def test_capacity_overflow_and_bad_id_are_reported_not_fatal():
    import flaggems_sglang_b200 as fg
    from flaggems_sglang_b200 import _C, ep

    world, tokens, E, H, I, k = 2, [64, 64], 8, 256, 128, 2
    w1, w2 = _layer(E, H, I, 3)
    _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {}, capacity=16)
    with pytest.raises(_C.FmoeError) as ei:
        _C.check_device_status()
    assert ei.value.code == _C.ERR_INVALID_ARG and "site code 0xa01" in str(ei.value).lower()
    _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {}, bad_id=True)
    with pytest.raises(_C.FmoeError) as ei:
        _C.check_device_status()
    assert "site code 0xa00" in str(ei.value).lower()
    # a dropped slot (bad id) contributes zeros, not the previous call's values
    xs_b, outs_b, _, xcs_b = _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {}, bad_id=True)
    with pytest.raises(_C.FmoeError):
        _C.check_device_status()
    assert (xcs_b[1].z[0] == 0).all()
    # the context is still usable and the status is clear again
    xs, outs, _, _ = _run_emulated(fg, ep, world, tokens, E, H, k, w1, w2, lambda r: {})
    _C.check_device_status()
    ref = fg.fused_experts(*xs[0][:1], w1, w2, xs[0][1], xs[0][2])
    assert float((outs[0].float() - ref.float()).norm() / ref.float().norm()) < 5e-3
