"""Property tests of the oracle's routing stages (CPU, hypothesis): invariants that hold for every input."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from oracle import routing as OR


@settings(max_examples=60, deadline=None)
@given(T=st.integers(0, 70), k=st.integers(1, 4), E=st.integers(1, 40), block=st.sampled_from([1, 4, 16, 32, 64, 128]),
       seed=st.integers(0, 10_000), hot=st.booleans())
def test_align_invariants(T, k, E, block, seed, hot):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, E, size=(T, k)).astype(np.int32)
    if hot and T:
        ids[: T // 2] = ids[0, 0]  # a hot expert, many empty ones
    ids[rng.random((T, k)) < 0.05] = -1  # dropped slots
    n = ids.size
    s, e, npp = OR.moe_align_block_size(ids, block, E)
    total = int(npp[0])
    assert s.shape[0] == n + E * (block - 1) and total % block == 0 and total <= s.shape[0]
    used = s[:total]
    real = used[used < n]
    flat = ids.reshape(-1)
    assert sorted(real.tolist()) == np.nonzero((flat >= 0) & (flat < E))[0].tolist()  # every kept slot exactly once
    assert (s[total:] == n).all() and (e[total // block:] == -1).all()
    for b in range(total // block):
        blk = used[b * block:(b + 1) * block]
        valid = blk[blk < n]
        assert valid.size >= 1 and (flat[valid] == e[b]).all()       # one expert per block, no empty block
        assert (np.diff(valid) > 0).all()                             # ascending slots
        assert (blk[valid.size:] == n).all()                          # padding only at the end of the block
    assert (np.diff(e[: total // block]) >= 0).all()                  # experts ascending


@settings(max_examples=60, deadline=None)
@given(T=st.integers(1, 40), E=st.integers(2, 64), seed=st.integers(0, 10_000), ties=st.booleans())
def test_softmax_topk_invariants(T, E, seed, ties):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if ties:
        logits = (logits * 2).round() / 2
    k = min(4, E)
    w, ids = OR.softmax_topk(logits, k, True)
    assert torch.allclose(w.sum(-1), torch.ones(T), atol=1e-5)
    assert (w[:, :-1] >= w[:, 1:] - 1e-7).all()
    for t in range(T):
        row = logits[t]
        chosen = ids[t].tolist()
        assert len(set(chosen)) == k
        worst = min(row[c].item() for c in chosen)
        rest = [row[i].item() for i in range(E) if i not in chosen]
        assert not rest or max(rest) <= worst
        # among equal logits the lower index is taken first
        for a, b in zip(chosen, chosen[1:]):
            assert row[a] > row[b] or (row[a] == row[b] and a < b)


@settings(max_examples=40, deadline=None)
@given(T=st.integers(1, 30), seed=st.integers(0, 10_000), ng=st.sampled_from([1, 2, 4, 8]), tg=st.integers(1, 8))
def test_grouped_topk_invariants(T, seed, ng, tg):
    E, k = 64, 4
    tg = min(tg, ng)
    if tg * (E // ng) < k:
        tg = ng
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1
    w, ids = OR.grouped_topk(logits, bias, k, ng, tg, True, 2.5)
    assert torch.allclose(w.sum(-1), torch.full((T,), 2.5), atol=1e-4)
    groups = ids // (E // ng)
    assert all(len(set(r.tolist())) <= tg for r in groups)
    assert all(len(set(r.tolist())) == k for r in ids)


@settings(max_examples=30, deadline=None)
@given(T=st.integers(1, 50), k=st.integers(1, 4), E=st.integers(4, 32), seed=st.integers(0, 10_000))
def test_reference_routing_tables_are_inverse_permutations(T, k, E, seed):
    g = torch.Generator().manual_seed(seed)
    k = min(k, E)
    logits = torch.randn(T, E, generator=g)
    w, ids = OR.softmax_topk(logits, k, True)
    r = OR.standard_topk_to_routing(w, ids, E)
    M = T * k
    assert sorted(r["topk_indx"].tolist()) == list(range(M))
    assert (r["gate_indx"][r["topk_indx"]] == np.arange(M)).all()
    assert r["hist"].sum() == M and r["token_offs_raw"][-1] == M
    for bm in OR.BLOCK_MS:
        pm = r["block_pid_map"][bm]
        tiles = int(r["token_offs_pad"][bm][-1])
        assert (pm[:tiles] >= 0).all() and (pm[tiles:] == -1).all()


def test_routers_keep_ids_in_range_on_nan_and_inf_rows():
    """NaN contract of both routers: NaN ranks as -inf, ids always inside [0, E), NaN / all -inf rows of the
    softmax router get finite weights."""
    E, k = 64, 6
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(5, E, generator=g)
    logits[0] = float("nan")
    logits[1] = float("-inf")
    logits[2, 1::2] = float("nan")
    w, ids = OR.softmax_topk(logits, k, True)
    assert ids.min() >= 0 and ids.max() < E and torch.isfinite(w).all()
    assert ids[0].tolist() == list(range(k)) and ids[1].tolist() == list(range(k))
    assert not set(ids[2].tolist()) & set(range(1, E, 2))   # NaN entries lose to every finite logit
    torch.testing.assert_close(w[0], torch.full((k,), 1.0 / k))
    bias = torch.randn(E, generator=g) * 0.1
    bias[3] = float("nan")
    gw, gids = OR.grouped_topk(logits, bias, k, 8, 4, True, 2.5)
    assert gids.min() >= 0 and gids.max() < E
    assert 3 not in gids[3:].reshape(-1).tolist()           # the NaN-biased expert is never chosen over finite ones


def test_per_channel_fp8_oracle_tracks_the_unquantised_layer():
    """Per-channel / per-token w8a8 restatement against the fp32 dense formulation on the same (unquantised) weights:
    the quantisation noise of e4m3 with row / channel scales stays inside the fp8 bar."""
    import torch

    from oracle import experts as OE
    from oracle import quant as OQ
    from oracle import routing as OR

    g = torch.Generator().manual_seed(3)
    T, H, I, E, k = 24, 256, 128, 4, 2
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16()
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g), k, True)
    w1q, w1s = OQ.quant_weight_per_channel(w1)
    w2q, w2s = OQ.quant_weight_per_channel(w2)
    assert w1s.shape == (E, 2 * I) and w2s.shape == (E, H)
    # de-quantised weights are within half an e4m3 step of the originals
    assert float(((w1q.float() * w1s[..., None]) - w1.float()).abs().max()) <= float(w1.float().abs().max()) / 16
    xq, xs = OQ.quant_act_per_token(x)
    assert xs.shape == (T,) and float((xq.float() * xs[:, None] - x.float()).abs().max()) <= float(x.float().abs().max()) / 16
    zero_q, zero_s = OQ.quant_act_per_token(torch.zeros(2, 64))
    assert float(zero_s[0]) == float(torch.tensor(OQ.MIN_TOKEN_SCALE, dtype=torch.float32)) and not zero_q.float().any()
    out = OE.fused_experts_fp8_per_channel(x, w1q, w1s, w2q, w2s, tw, ti).float()
    ref = OE.dense_moe(x, w1, w2, tw, ti)
    assert float((out - ref).norm() / ref.norm()) <= 8e-2  # e4m3 noise of three quantisation points
