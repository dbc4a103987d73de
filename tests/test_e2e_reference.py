"""End-to-end parity with the REAL reference operator.

tests/golden/e2e_*.npz hold what `flaggems_sglang.triton_kernel_fused_experts`
(src/flaggems_sglang/ops/fused_moe.py:149-232) returned on a B200 for the reference's own test shapes and
seeds (generator: tests/golden/make_golden_e2e.py).  The CPU test holds the oracle to them, the GPU test
holds this package's drop-in of the same name to them, both at the bf16 bar of tests/util.py.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import experts as OE
from oracle import routing as OR
from tests.util import BF16_MAX_ABS_FRAC_E2E as BF16_MAX_ABS_FRAC, BF16_REL_L2, checksum, e2e_inputs, max_abs_frac, rel_l2

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
E2E = sorted(glob.glob(os.path.join(GOLDEN, "e2e_*.npz")))
IDS = [os.path.basename(p)[4:-4] for p in E2E]
VARIANTS = [("out", False, True), ("out_on_input", True, True)]


def test_e2e_fixtures_present():
    assert len(E2E) >= 8, "run tests/golden/make_golden_e2e.py on a GPU box to create the e2e fixtures"


def _load(path, device="cpu"):
    """Fixture + regenerated inputs (on the CPU only the weights of the experts the case routes to)."""
    g = np.load(path)
    shape = tuple(int(v) for v in g["shape"])
    used = sorted(set(g["topk_ids"].reshape(-1).tolist()))
    hidden, w1, w2, logits = e2e_inputs(*shape, device=device, experts=used if device == "cpu" else None)
    for name, t in (("hidden", hidden), ("logits", logits)):
        np.testing.assert_array_equal(checksum(t), g["sum_" + name], err_msg=f"regenerated {name} differs from the fixture's inputs")
    for name, t in (("w1", w1), ("w2", w2)):
        np.testing.assert_array_equal(checksum(t)[used], g["sum_" + name][used],
                                      err_msg=f"regenerated {name} differs from the fixture's inputs")
    return g, shape, hidden, w1, w2, logits


def _compare(got, g, key, what):
    ref = torch.from_numpy(g[key + "_bits"]).view(torch.bfloat16).float()
    assert got.shape[0] == int(g[key + "_n"]), f"{what}: {got.shape[0]} rows, the reference returned {int(g[key + '_n'])}"
    got = got.float().cpu()[torch.from_numpy(g[key + "_rows"])]
    l2, ma = rel_l2(got, ref), max_abs_frac(got, ref)
    assert l2 <= BF16_REL_L2 and ma <= BF16_MAX_ABS_FRAC, (
        f"{what}: rel-L2 {l2:.3e} (<= {BF16_REL_L2}), max-abs/max {ma:.3e} (<= {BF16_MAX_ABS_FRAC:.3e})")
    return l2, ma


@pytest.mark.parametrize("path", [p for p in E2E if "_K1280_" not in p or "_M1_" in p],
                         ids=[i for i in IDS if "_K1280_" not in i or i.startswith("M1_")])
def test_oracle_matches_reference_operator(path):
    g, (M, K, N, E, topk), hidden, w1, w2, logits = _load(path)
    tw, ti = OR.softmax_topk(logits, topk, True)
    np.testing.assert_array_equal(ti.numpy(), g["topk_ids"])  # same routing as the reference test's router
    routing = OR.standard_topk_to_routing(torch.from_numpy(g["topk_weights"]), torch.from_numpy(g["topk_ids"]), E)
    for key, on_input, combine in VARIANTS:
        if key + "_bits" not in g:
            continue
        got = OE.reference_fused_experts(hidden, w1, w2, routing, apply_router_weight_on_input=on_input,
                                         no_combine=not combine)
        l2, ma = _compare(got.reshape(-1, K), g, key, f"oracle {key}")
        print(f"oracle vs reference op {os.path.basename(path)} {key}: rel-L2 {l2:.2e} max-abs/max {ma:.2e}")


@pytest.mark.gpu
@pytest.mark.parametrize("path", E2E, ids=IDS)
def test_drop_in_matches_reference_operator(path):
    import flaggems_sglang_b200 as fg

    dev = torch.device("cuda", 0)
    g, (M, K, N, E, topk), xd, w1d, w2d, logits = _load(path, dev)
    tw = torch.from_numpy(g["topk_weights"]).to(dev)
    ti = torch.from_numpy(g["topk_ids"]).to(dev)
    rd, gi, si = fg.standard_topk_to_routing(tw, ti, E)
    for key, on_input, combine in VARIANTS:
        if key + "_bits" not in g:
            continue
        got = fg.triton_kernel_fused_experts(xd, w1d, w2d, rd, gi, si if combine else None,
                                             apply_router_weight_on_input=on_input)
        l2, ma = _compare(got.reshape(-1, K), g, key, f"drop-in {key}")
        print(f"drop-in vs reference op {os.path.basename(path)} {key}: rel-L2 {l2:.2e} max-abs/max {ma:.2e}")
