"""GPU parity of the bias + swiglu variant (the reference's `triton_kernel_fused_experts_with_bias`,
src/flaggems_sglang/ops/fused_moe.py:235-325) against the CPU oracle, through every kernel family that takes it."""
import pytest
import torch

from oracle import experts as OE
from oracle import routing as OR
from tests.util import assert_close_moe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fg():
    import flaggems_sglang_b200 as fg

    return fg


@pytest.fixture(autouse=True)
def _device_status():
    yield
    from flaggems_sglang_b200 import _C

    _C.check_device_status()


def _layer(T, H, I, E, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(dtype)
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(dtype)  # gate rows, then linear rows
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(dtype)
    b1 = torch.randn(E, 2 * I, generator=g) * 0.3
    b2 = torch.randn(E, H, generator=g) * 0.3
    logits = torch.randn(T, E, generator=g)
    return x, w1, w2, b1, b2, logits


@pytest.mark.parametrize("variant", ["simt", "stream", "tcgen05"])
@pytest.mark.parametrize("T,H,I,E,k", [(40, 256, 384, 8, 2), (1, 128, 128, 4, 2), (300, 512, 256, 16, 4),
                                       (150, 352, 160, 8, 2)])  # last: sizes that are not multiples of 128
@pytest.mark.parametrize("limit", [None, 1.25])
def test_bias_and_swiglu_serving_layouts(fg, variant, T, H, I, E, k, limit):
    x, w1, w2, b1, b2, logits = _layer(T, H, I, E, 31 + T)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), activation="swiglu_oai", b1=b1.cuda(),
                           b2=b2.cuda(), gemm1_alpha=1.702, gemm1_clamp_limit=limit, variant=variant)
    ref = OE.fused_experts_with_bias(x, w1, b1, w2, b2, tw, ti, alpha=1.702, limit=limit)
    assert_close_moe(out, ref, "bf16", f"bias variant {variant} T={T} limit={limit}")


@pytest.mark.parametrize("variant", ["stream", "tcgen05"])
def test_bias_variant_options(fg, variant):
    """Weight on the input side (applied after the activation, as that path's GEMM epilogue does), no_combine,
    bias on one projection only, and bias with the plain silu unit."""
    T, H, I, E, k = 70, 256, 128, 8, 1
    x, w1, w2, b1, b2, logits = _layer(T, H, I, E, 9)
    tw, ti = OR.softmax_topk(logits, k, False)
    run = lambda **kw: fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), variant=variant, **kw)  # noqa: E731
    out = run(activation="swiglu_oai", b1=b1.cuda(), b2=b2.cuda(), apply_router_weight_on_input=True)
    assert_close_moe(out, OE.fused_experts_with_bias(x, w1, b1, w2, b2, tw, ti, True), "bf16", "on input")
    out = run(activation="swiglu_oai", b2=b2.cuda(), no_combine=True, gemm1_alpha=1.0)
    assert_close_moe(out, OE.fused_experts_with_bias(x, w1, None, w2, b2, tw, ti, alpha=1.0, no_combine=True), "bf16", "b2 only")
    out = run(activation="swiglu_oai")
    assert_close_moe(out, OE.fused_experts_with_bias(x, w1, None, w2, None, tw, ti), "bf16", "no bias")


def test_fp32_bias_variant_on_the_simt_kernels(fg):
    x, w1, w2, b1, b2, logits = _layer(16, 256, 512, 8, 0, torch.float32)
    tw, ti = OR.softmax_topk(logits, 2, True)
    out = fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), activation="swiglu_oai", b1=b1.cuda(),
                           b2=b2.cuda(), gemm1_clamp_limit=7.0)
    ref = OE.fused_experts_with_bias(x, w1, b1, w2, b2, tw, ti, limit=7.0)
    assert_close_moe(out, ref, "fp32", "fp32 bias variant")


@pytest.mark.parametrize("scatter", [True, False])
def test_reference_entry_point_with_bias(fg, scatter):
    """`triton_kernel_fused_experts_with_bias` on the reference's layouts: w1 [E,H,2I] with interleaved gate/linear
    columns, routing triple; `scatter_indx=None` returns rows in sorted order."""
    T, H, I, E, k = 33, 256, 128, 16, 4
    g = torch.Generator().manual_seed(77)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = (torch.randn(E, H, 2 * I, generator=g) / H ** 0.5).bfloat16()
    w2 = (torch.randn(E, I, H, generator=g) / I ** 0.5).bfloat16()
    b1 = torch.randn(E, 2 * I, generator=g) * 0.3
    b2 = torch.randn(E, H, generator=g) * 0.3
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g), k, True)
    r = OR.standard_topk_to_routing(tw, ti, E)
    rd, gi, si = fg.standard_topk_to_routing(tw.cuda(), ti.cuda(), E)
    out = fg.triton_kernel_fused_experts_with_bias(x.cuda(), w1.cuda(), None, b1.cuda(), w2.cuda(), None, b2.cuda(), rd, gi,
                                                   si if scatter else None, gemm1_alpha=1.702, gemm1_clamp_limit=7.0)
    ref = OE.reference_fused_experts_with_bias(x, w1, b1, w2, b2, r, False, 1.702, 7.0, no_combine=not scatter)
    assert out.shape == ref.shape
    assert_close_moe(out, ref, "bf16", f"reference entry point, scatter={scatter}")


def test_bias_variant_is_refused_with_fp8_weights(fg):
    from oracle import quant as OQ

    x, w1, w2, b1, b2, logits = _layer(8, 256, 128, 4, 1)
    tw, ti = OR.softmax_topk(logits, 2, True)
    w1q, s1 = OQ.quant_weight_block128(w1)
    w2q, s2 = OQ.quant_weight_block128(w2)
    with pytest.raises(AssertionError, match="fp8"):
        fg.fused_experts(x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True, w1_scale=s1.cuda(),
                         w2_scale=s2.cuda(), block_shape=[128, 128], b1=b1.cuda())


def test_hook_routes_biased_layers_to_the_bias_variant(fg):
    """`fused_moe_flagos` with `w13_weight_bias` / `w2_weight_bias` on the layer (reference hook :380-398): the
    serving-side w13 [E,2I,H] holds gate and linear rows interleaved."""
    from types import SimpleNamespace as NS

    T, H, I, E, k = 21, 256, 128, 8, 2
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16()     # interleaved rows
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16()
    b13 = torch.randn(E, 2 * I, generator=g) * 0.3
    b2 = torch.randn(E, H, generator=g) * 0.3
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g), k, True)
    r = OR.standard_topk_to_routing(tw, ti, E)
    ref = OE.reference_fused_experts_with_bias(x, w13.transpose(1, 2), b13, w2.transpose(1, 2), b2, r, False, 1.702, 7.0)
    layer = NS(w13_weight=w13.cuda(), w2_weight=w2.cuda(), w13_weight_bias=b13.cuda(), w2_weight_bias=b2.cuda())
    cfg = NS(num_experts=E, activation="silu", apply_router_weight_on_input=False, no_combine=False,
             routed_scaling_factor=None, gemm1_alpha=1.702, gemm1_clamp_limit=7.0)
    disp = NS(hidden_states=x.cuda(), topk_output=NS(topk_weights=tw.cuda(), topk_ids=ti.cuda()))
    out = fg.fused_moe_flagos(NS(runner=NS(config=cfg)), layer, disp).hidden_states
    assert_close_moe(out, ref, "bf16", "hook, (weights, ids) routing")
    disp2 = NS(hidden_states=x.cuda(), topk_output=fg.standard_topk_to_routing(tw.cuda(), ti.cuda(), E))
    out2 = fg.fused_moe_flagos(NS(runner=NS(config=cfg)), layer, disp2).hidden_states
    assert_close_moe(out2, ref, "bf16", "hook, routing triple")
    with pytest.raises(AssertionError, match="both w13_bias and w2_bias"):
        fg.fused_moe_flagos(NS(runner=NS(config=cfg)), NS(w13_weight=w13.cuda(), w2_weight=w2.cuda(),
                                                          w13_weight_bias=b13.cuda(), w2_weight_bias=None), disp)
