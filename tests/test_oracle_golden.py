"""The oracle against fixtures produced by the real reference (tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import experts as OE
from oracle import routing as OR

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ROUTING = sorted(glob.glob(os.path.join(GOLDEN, "routing_*.npz")))
SILU = sorted(glob.glob(os.path.join(GOLDEN, "silu_*.npz")))


def test_fixtures_present():
    assert len(ROUTING) >= 10 and len(SILU) >= 2


@pytest.mark.parametrize("path", ROUTING, ids=[os.path.basename(p)[8:-4] for p in ROUTING])
def test_routing_tables_match_reference(path):
    g = np.load(path)
    E = g["hist"].shape[0]
    r = OR.standard_topk_to_routing(
        torch.from_numpy(g["topk_weights"]), torch.from_numpy(g["topk_ids"]), E
    )
    np.testing.assert_array_equal(r["hist"], g["hist"])
    np.testing.assert_array_equal(r["topk_indx"], g["topk_indx"])
    np.testing.assert_array_equal(r["gate_indx"], g["gate_indx"])
    # ScatterIndx is the GatherIndx pair swapped (ref fused_moe.py:144-145)
    np.testing.assert_array_equal(r["gate_indx"], g["scatter_src"])
    np.testing.assert_array_equal(r["topk_indx"], g["scatter_dst"])
    np.testing.assert_array_equal(r["gate_scal"], g["gate_scal"])  # a pure gather: exact
    np.testing.assert_array_equal(r["token_offs_raw"], g["token_offs_raw"])
    for bm in OR.BLOCK_MS:
        np.testing.assert_array_equal(r["token_offs_pad"][bm], g[f"token_offs_pad_{bm}"])
        np.testing.assert_array_equal(r["block_pid_map"][bm], g[f"block_pid_map_{bm}"])


@pytest.mark.parametrize("path", ROUTING, ids=[os.path.basename(p)[8:-4] for p in ROUTING])
def test_softmax_topk_matches_reference_test_router(path):
    """ids and weights of the oracle router vs softmax->torch.topk->renormalise as the
    reference's test builds them (ref tests/test_fused_moe.py:38-41)."""
    g = np.load(path)
    logits = torch.from_numpy(g["logits"])
    k = g["topk_ids"].shape[1]
    w, ids = OR.softmax_topk(logits, k, renormalize=True)
    np.testing.assert_array_equal(ids.numpy(), g["topk_ids"])
    np.testing.assert_allclose(w.numpy(), g["topk_weights"], rtol=1e-6, atol=0)


@pytest.mark.parametrize("path", ROUTING, ids=[os.path.basename(p)[8:-4] for p in ROUTING])
def test_align_consistent_with_reference_tile_maps(path):
    """moe_align_block_size has no reference code; its block->expert map and padded
    length must agree with the reference's tile maps for every block size."""
    g = np.load(path)
    ids = g["topk_ids"]
    E = g["hist"].shape[0]
    k = ids.shape[1]
    n = ids.size
    for bm in OR.BLOCK_MS:
        sorted_ids, expert_ids, npp = OR.moe_align_block_size(ids, bm, E)
        tiles = int(g[f"token_offs_pad_{bm}"][E])
        assert npp[0] == tiles * bm
        pm = g[f"block_pid_map_{bm}"]
        np.testing.assert_array_equal(expert_ids[:tiles], pm[:tiles] & 0xFFFF)
        assert (expert_ids[tiles:] == -1).all()
        used = sorted_ids[: npp[0]]
        real = used[used < n]
        # same tokens in the same order as the reference's gather index
        np.testing.assert_array_equal(real // k, g["topk_indx"] // k)
        assert (sorted_ids[npp[0]:] == n).all()


@pytest.mark.parametrize("path", SILU, ids=[os.path.basename(p)[5:-4] for p in SILU])
def test_silu_and_mul_matches_reference_kernel(path):
    g = np.load(path)
    y1 = torch.from_numpy(g["y1_bits"]).view(torch.bfloat16)
    got = OE.silu_and_mul(y1, torch.float32).numpy()
    # both sides evaluate g/(1+exp(-g))*u in fp32; exp may differ in the last ulp
    np.testing.assert_allclose(got, g["out_f32"], rtol=2e-6, atol=1e-30)


SWIGLU = sorted(glob.glob(os.path.join(GOLDEN, "swiglu_*.npz")))


@pytest.mark.parametrize("path", SWIGLU, ids=[os.path.basename(p)[7:-4] for p in SWIGLU])
def test_swiglu_matches_third_party_torch_reference(path):
    g = np.load(path)
    limit = float(g["limit"])
    got = OE.swiglu_oai(torch.from_numpy(g["a_f32"]), float(g["alpha"]), None if limit < 0 else limit).numpy()
    # a/(1+exp(-alpha a)) against a*sigmoid(alpha a): the same value up to fp32 rounding of exp and the division
    np.testing.assert_allclose(got, g["out_f32"], rtol=3e-6, atol=1e-6)


def test_bias_variant_layouts_agree():
    """The bias variant on the reference's layouts (interleaved gate/linear columns, routing tables) and on the
    serving-side layouts (gate rows first, topk ids) is one computation."""
    torch.manual_seed(5)
    T, H, I, E, k = 19, 64, 48, 6, 3
    x = torch.randn(T, H).bfloat16()
    w1_ref = (torch.randn(E, H, 2 * I) / H ** 0.5).bfloat16()   # interleaved columns
    w2_ref = (torch.randn(E, I, H) / I ** 0.5).bfloat16()
    b1_ref = torch.randn(E, 2 * I) * 0.2
    b2 = torch.randn(E, H) * 0.2
    w, ids = OR.softmax_topk(torch.randn(T, E), k, True)
    r = OR.standard_topk_to_routing(w, ids, E)
    for on_input in (False, True):
        ref = OE.reference_fused_experts_with_bias(x, w1_ref, b1_ref, w2_ref, b2, r, on_input, 1.702, 7.0)
        rows = w1_ref.transpose(1, 2)
        w1_split = torch.cat((rows[:, 0::2], rows[:, 1::2]), dim=1).contiguous()
        b1_split = torch.cat((b1_ref[:, 0::2], b1_ref[:, 1::2]), dim=1)
        # slots in the reference are ordered by ascending expert per token: give the serving-side form the same order
        ids2, perm = torch.sort(ids, dim=1)
        w2d = torch.gather(w, 1, perm)
        got = OE.fused_experts_with_bias(x, w1_split, b1_split, w2_ref.transpose(1, 2).contiguous(), b2, w2d, ids2,
                                         on_input, 1.702, 7.0)
        assert torch.equal(ref, got)


def test_restatements_agree_with_dense_formulation():
    """Config 1 of the benchmark set (T=16,H=256,I=512,E=8,k=2, fp32, seed 0): the
    sorted/grouped restatements equal the naive per-token MoE."""
    torch.manual_seed(0)
    T, H, I, E, k = 16, 256, 512, 8, 2
    x = torch.randn(T, H)
    w1 = torch.randn(E, 2 * I, H) / H ** 0.5
    w2 = torch.randn(E, H, I) / I ** 0.5
    logits = torch.randn(T, E)
    w, ids = OR.softmax_topk(logits, k, True)
    dense = OE.dense_moe(x, w1, w2, w, ids)
    a = OE.fused_experts(x, w1, w2, w, ids)
    r = OR.standard_topk_to_routing(w, ids, E)
    b = OE.reference_fused_experts(
        x, w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous(), r
    )
    assert (a - dense).abs().max() < 1e-5
    assert (b - dense).abs().max() < 1e-5
    # no_combine returns rows in sorted order for the reference layout
    z = OE.reference_fused_experts(
        x, w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous(), r, no_combine=True
    )
    z2 = OE.fused_experts(x, w1, w2, w, ids, no_combine=True).reshape(T * k, H)
    # slot numbering differs (per-token ascending-expert order vs given order): compare by (token, expert)
    ids_sorted, perm = torch.sort(ids.long(), dim=1)
    slot_of = (torch.arange(T)[:, None] * k + perm).reshape(-1)  # sorted-slot -> original slot
    for p in range(T * k):
        s_sorted = int(r["topk_indx"][p])
        assert torch.allclose(z[p], z2[slot_of[s_sorted]], atol=1e-5)
