"""GPU parity of the CTA-pair (cta_group::2) bf16 kernel against the CPU oracle and the single-CTA kernel."""
import pytest
import torch

from oracle import experts as OE
from oracle import routing as OR
from tests.util import assert_close_moe, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _device_status():
    yield
    from flaggems_sglang_b200 import _C

    _C.check_device_status()


def _layer(T, H, I, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16()
    logits = torch.randn(T, E, generator=g)
    return x, w1, w2, logits


@pytest.mark.parametrize("T,H,I,E,k", [(7, 128, 256, 8, 2), (300, 256, 512, 8, 2), (1024, 1280, 3072, 64, 8),
                                        (2000, 512, 384, 4, 2)])
def test_pair_kernel_vs_oracle(T, H, I, E, k):
    import flaggems_sglang_b200 as fg

    x, w1, w2, logits = _layer(T, H, I, E, k, T + H)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), variant="tcgen05_pair")
    ref = OE.fused_experts(x, w1, w2, tw, ti)
    assert_close_moe(out, ref, "bf16", f"pair T={T}")
    again = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), variant="tcgen05_pair")
    assert torch.equal(out, again)
    single = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), variant="tcgen05")
    assert rel_l2(out, single) < 2e-3


def test_pair_kernel_options():
    import flaggems_sglang_b200 as fg

    x, w1, w2, logits = _layer(500, 256, 384, 8, 2, 9)
    tw, ti = OR.softmax_topk(logits, 2, True)
    out = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), variant="tcgen05_pair",
                           apply_router_weight_on_input=True, routed_scaling_factor=2.5)
    ref = OE.fused_experts(x, w1, w2, tw, ti, apply_router_weight_on_input=True, routed_scaling_factor=2.5)
    assert_close_moe(out, ref, "bf16", "pair options")
