"""GPU parity: router kernels and moe_align_block_size against the CPU oracle (bit-exact ids / buffers)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import routing as OR

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROUTING = sorted(glob.glob(os.path.join(GOLDEN, "routing_*.npz")))


@pytest.fixture(scope="module")
def fg():
    import flaggems_sglang_b200 as fg

    assert torch.cuda.is_available()
    return fg


def _zipf_logits(T, E, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    ranks = torch.randperm(E, generator=g).float() + 1
    pmf = ranks.pow(-1.2)
    return logits + (pmf / pmf.sum()).log()[None, :]


# ---------------------------------------------------------------- softmax top-k
@pytest.mark.parametrize("path", ROUTING, ids=[os.path.basename(p)[8:-4] for p in ROUTING])
def test_softmax_topk_golden_logits(fg, path):
    """Same logits as the fixtures made with the reference's test router: ids equal the
    reference's torch.topk ids, weights within fp32 rounding."""
    g = np.load(path)
    logits = torch.from_numpy(g["logits"])
    k = g["topk_ids"].shape[1]
    w, ids = fg.fused_topk(None, logits.cuda(), k, True)
    np.testing.assert_array_equal(ids.cpu().numpy(), g["topk_ids"])
    np.testing.assert_allclose(w.cpu().numpy(), g["topk_weights"], rtol=2e-6, atol=1e-9)


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (16, 8, 2), (1, 128, 8), (32, 128, 8), (512, 128, 8), (8192, 128, 8),
                                    (33, 60, 6), (5, 256, 8), (7, 1000, 32), (3, 4, 4)])
@pytest.mark.parametrize("renorm", [True, False])
def test_softmax_topk_vs_oracle(fg, T, E, k, renorm):
    torch.manual_seed(T * 131 + E + k)
    logits = torch.randn(T, E)
    w, ids = fg.fused_topk(None, logits.cuda(), k, renorm)
    ow, oids = OR.softmax_topk(logits, k, renorm)
    assert torch.equal(ids.cpu(), oids)
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-9)


def test_softmax_topk_ties_go_to_lower_index(fg):
    logits = torch.zeros(6, 40)
    logits[1, 7] = logits[1, 33] = 2.0
    logits[2, :] = torch.arange(40).float().flip(0).div(8).floor()  # runs of equal values
    w, ids = fg.fused_topk(None, logits.cuda(), 4, True)
    ow, oids = OR.softmax_topk(logits, 4, True)
    assert torch.equal(ids.cpu(), oids)
    assert ids[0].tolist() == [0, 1, 2, 3] and ids[1].tolist()[:2] == [7, 33]


def test_softmax_topk_skewed(fg):
    logits = _zipf_logits(512, 128, 3)
    w, ids = fg.fused_topk(None, logits.cuda(), 8, True)
    ow, oids = OR.softmax_topk(logits, 8, True)
    assert torch.equal(ids.cpu(), oids)
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-9)


# ---------------------------------------------------------------- grouped top-k
@pytest.mark.parametrize("T,E,k,ng,tg", [(1, 256, 8, 8, 4), (64, 256, 8, 8, 4), (1024, 256, 8, 8, 4),
                                          (37, 16, 4, 4, 2), (9, 64, 6, 8, 3), (5, 32, 8, 1, 1), (4, 32, 2, 32, 4)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_grouped_topk_vs_oracle(fg, T, E, k, ng, tg, with_bias):
    torch.manual_seed(T + E * 7 + k)
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.1 if with_bias else None
    w, ids = fg.grouped_topk(None, logits.cuda(), k, True, ng, tg, None if bias is None else bias.cuda(), 2.5)
    ow, oids = OR.grouped_topk(logits, bias, k, ng, tg, True, 2.5)
    assert torch.equal(ids.cpu(), oids)
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-6, atol=1e-12)
    w2, ids2 = fg.grouped_topk(None, logits.cuda(), k, False, ng, tg, None if bias is None else bias.cuda(), None)
    ow2, oids2 = OR.grouped_topk(logits, bias, k, ng, tg, False, None)
    assert torch.equal(ids2.cpu(), oids2)
    torch.testing.assert_close(w2.cpu(), ow2, rtol=1e-6, atol=1e-12)


def test_grouped_topk_large_and_deterministic(fg):
    torch.manual_seed(5)
    logits = torch.randn(16384, 256)
    bias = torch.randn(256) * 0.1
    a = fg.grouped_topk(None, logits.cuda(), 8, True, 8, 4, bias.cuda(), 2.5)
    b = fg.grouped_topk(None, logits.cuda(), 8, True, 8, 4, bias.cuda(), 2.5)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    ow, oids = OR.grouped_topk(logits, bias, 8, 8, 4, True, 2.5)
    assert torch.equal(a[1].cpu(), oids)
    # every token stays inside 4 of the 8 groups
    groups = (a[1] // 32).cpu()
    assert max(len(set(r.tolist())) for r in groups[:2048]) <= 4


def test_router_argument_errors(fg):
    from flaggems_sglang_b200._C import FmoeError

    with pytest.raises(FmoeError, match="k"):
        fg.fused_topk(None, torch.randn(4, 8).cuda(), 9, True)
    with pytest.raises(FmoeError, match="n_group"):
        fg.grouped_topk(None, torch.randn(4, 30).cuda(), 2, True, 4, 2)


# ---------------------------------------------------------------- moe_align_block_size
def _check_align(fg, ids_cpu, block, E):
    s, e, n = fg.moe_align_block_size(ids_cpu.cuda(), block, E)
    os_, oe, on = OR.moe_align_block_size(ids_cpu, block, E)
    np.testing.assert_array_equal(n.cpu().numpy(), on)
    np.testing.assert_array_equal(s.cpu().numpy(), os_)
    np.testing.assert_array_equal(e.cpu().numpy(), oe)


@pytest.mark.parametrize("block", [8, 16, 32, 64, 128])
@pytest.mark.parametrize("T,E,k,skew", [(1, 128, 8, False), (32, 128, 8, False), (512, 128, 8, True), (8192, 128, 8, True),
                                         (8192, 128, 8, False), (33, 128, 8, False), (1, 8, 2, False), (4096, 8, 2, False),
                                         (16384, 256, 8, False), (3, 256, 8, False)])
def test_align_vs_oracle(fg, block, T, E, k, skew):
    logits = _zipf_logits(T, E, T + E) if skew else torch.randn(T, E, generator=torch.Generator().manual_seed(T + E))
    _, ids = OR.softmax_topk(logits, k, True)
    _check_align(fg, ids, block, E)


@pytest.mark.parametrize("T,E", [(16, 8), (4, 32), (32, 16), (8, 64), (128, 4)])
def test_align_reference_benchmark_shapes(fg, T, E):
    """(T,E) list of the reference's MoeAlignBlockSize benchmark entry (benchmark/core_shapes.yaml:310-316)."""
    g = torch.Generator().manual_seed(T * E)
    ids = torch.randint(0, E, (T, 2), generator=g, dtype=torch.int32)
    for block in (16, 64):
        _check_align(fg, ids, block, E)


def test_align_edge_cases(fg):
    # all tokens on one expert; ids outside the range are dropped; empty input
    _check_align(fg, torch.full((100, 2), 5, dtype=torch.int32), 16, 8)
    ids = torch.tensor([[0, -1], [7, 3], [-1, -1], [3, 9]], dtype=torch.int32)
    _check_align(fg, ids, 4, 8)
    _check_align(fg, torch.zeros(0, 2, dtype=torch.int32), 16, 8)
    # block size 1: plain stable sort by expert
    g = torch.Generator().manual_seed(1)
    _check_align(fg, torch.randint(0, 1024, (777, 3), generator=g, dtype=torch.int32), 1, 1024)


@pytest.mark.parametrize("path", ROUTING, ids=[os.path.basename(p)[8:-4] for p in ROUTING])
def test_align_agrees_with_reference_tile_maps(fg, path):
    g = np.load(path)
    ids = torch.from_numpy(g["topk_ids"])
    E = g["hist"].shape[0]
    k = ids.shape[1]
    for bm in (16, 32, 64, 128):
        s, e, n = fg.moe_align_block_size(ids.cuda(), bm, E)
        tiles = int(g[f"token_offs_pad_{bm}"][E])
        assert int(n.item()) == tiles * bm
        np.testing.assert_array_equal(e.cpu().numpy()[:tiles], g[f"block_pid_map_{bm}"][:tiles] & 0xFFFF)
        used = s.cpu().numpy()[: tiles * bm]
        np.testing.assert_array_equal(used[used < ids.numel()] // k, g["topk_indx"] // k)


# ---------------------------------------------------------------- NaN / -inf rows stay in bounds
def _poisoned_logits(T, E, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    logits[0] = float("nan")                 # a whole NaN row (a diverged model)
    logits[1] = float("-inf")                # nothing selectable
    logits[2, ::3] = float("nan")            # scattered NaNs
    logits[3, : E - 2] = float("-inf")       # fewer finite logits than k
    return logits


@pytest.mark.parametrize("E,k", [(8, 2), (128, 8), (256, 8)])
def test_softmax_topk_nan_rows_in_bounds(fg, E, k):
    logits = _poisoned_logits(6, E, 3)
    w, ids = fg.fused_topk(None, logits.cuda(), k, True)
    ow, oids = OR.softmax_topk(logits, k, True)
    assert int(ids.min()) >= 0 and int(ids.max()) < E
    assert torch.equal(ids.cpu(), oids)
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-9, equal_nan=True)
    assert torch.isfinite(w[:3]).all()       # NaN and all -inf rows give finite weights


@pytest.mark.parametrize("with_bias", [True, False])
def test_grouped_topk_nan_rows_in_bounds(fg, with_bias):
    E, k, ng, tg = 256, 8, 8, 4
    logits = _poisoned_logits(6, E, 4)
    bias = torch.randn(E) * 0.1 if with_bias else None
    if with_bias:
        bias[5] = float("nan")
    w, ids = fg.grouped_topk(None, logits.cuda(), k, True, ng, tg, None if bias is None else bias.cuda(), 2.5)
    ow, oids = OR.grouped_topk(logits, bias, k, ng, tg, True, 2.5)
    assert int(ids.min()) >= 0 and int(ids.max()) < E
    assert torch.equal(ids.cpu(), oids)
    torch.testing.assert_close(w.cpu(), ow, rtol=1e-5, atol=1e-9, equal_nan=True)
