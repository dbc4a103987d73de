"""GPU parity: the expert computation (all three kernel families, bf16 / fp32 / fp8) through the
public ops against the CPU oracle, on the reference's own test shapes, reduced benchmark shapes,
and — by sampled tokens and variant cross-checks — at full benchmark sizes."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import experts as OE
from oracle import quant as OQ
from oracle import routing as OR
from tests.util import assert_close_moe, rel_l2

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def fg():
    import flaggems_sglang_b200 as fg

    return fg


@pytest.fixture(autouse=True)
def _device_status():
    yield
    from flaggems_sglang_b200 import _C

    _C.check_device_status()  # a bounded wait that gave up fails the test that ran the kernel


def _layer(T, H, I, E, k, dtype, seed, wscale=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(dtype)
    s1 = wscale if wscale is not None else H ** -0.5
    s2 = wscale if wscale is not None else I ** -0.5
    w1 = (torch.randn(E, 2 * I, H, generator=g) * s1).to(dtype)
    w2 = (torch.randn(E, H, I, generator=g) * s2).to(dtype)
    logits = torch.randn(T, E, generator=g)
    return x, w1, w2, logits


def _run(fg, x, w1, w2, tw, ti, **kw):
    return fg.fused_experts(x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda(), **kw)


# ------------------------------------------------------------------ fp32 (tiny benchmark config)
def test_tiny_fp32_config(fg):
    """T=16,H=256,I=512,E=8,k=2, fp32, seed 0, softmax top-2 renormalised, through fused_moe."""
    torch.manual_seed(0)
    T, H, I, E, k = 16, 256, 512, 8, 2
    x = torch.randn(T, H)
    w1 = torch.randn(E, 2 * I, H) / H ** 0.5
    w2 = torch.randn(E, H, I) / I ** 0.5
    logits = torch.randn(T, E)
    out = fg.fused_moe(x.cuda(), w1.cuda(), w2.cuda(), logits.cuda(), k, True)
    ref = OE.fused_moe(x, w1, w2, logits, k, True)
    assert_close_moe(out, ref, "fp32", "tiny fp32")
    dense = OE.dense_moe(x, w1, w2, *OR.softmax_topk(logits, k, True))
    assert_close_moe(out, dense, "fp32", "tiny fp32 vs dense")


# ------------------------------------------------------------------ bf16, every kernel family
SMALL = [(1, 128, 256, 8, 2), (7, 128, 256, 8, 2), (33, 256, 512, 16, 4)]  # reference small shapes (M,K,N,E,topk)
MID = [(1, 1280, 3072, 64, 8), (4, 1280, 3072, 64, 8), (17, 1280, 3072, 64, 8), (64, 1280, 3072, 64, 8)]


@pytest.mark.parametrize("shape", SMALL + MID, ids=lambda s: "M%d_K%d_N%d_E%d_k%d" % s)
@pytest.mark.parametrize("variant", ["simt", "stream", "tcgen05"])
def test_bf16_reference_shapes(fg, shape, variant):
    """Shapes, seeds and value distribution of the reference test (tests/test_fused_moe.py:64-72)."""
    M, K, N, E, topk = shape
    if variant == "simt" and M * topk * K * N > 2e10:
        pytest.skip("simt cross-check kept to small problems")
    x, w1, w2, logits = _layer(M, K, N, E, topk, torch.bfloat16, M + K + N + E + topk, wscale=0.1)
    tw, ti = OR.softmax_topk(logits, topk, True)
    out = _run(fg, x, w1, w2, tw, ti, variant=variant)
    ref = OE.fused_experts(x, w1, w2, tw, ti)
    assert_close_moe(out, ref, "bf16", f"{variant} {shape}")
    again = _run(fg, x, w1, w2, tw, ti, variant=variant)
    assert torch.equal(out, again), "run-to-run results differ"


@pytest.mark.parametrize("variant", ["stream", "tcgen05"])
def test_bf16_large_reference_shape(fg, variant):
    M, K, N, E, topk = 1024, 1280, 3072, 64, 8
    x, w1, w2, logits = _layer(M, K, N, E, topk, torch.bfloat16, M + K + N + E + topk, wscale=0.1)
    tw, ti = OR.softmax_topk(logits, topk, True)
    out = _run(fg, x, w1, w2, tw, ti, variant=variant)
    ref = OE.fused_experts(x, w1, w2, tw, ti)
    assert_close_moe(out, ref, "bf16", f"{variant} M1024")


@pytest.mark.parametrize("T", [1, 5, 16, 40, 130, 700])
def test_bf16_auto_variant_ragged(fg, T):
    """Automatic kernel choice over ragged token counts with a skewed router (hot and empty experts)."""
    H, I, E, k = 512, 256, 32, 4
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 100 + T)
    logits[:, :8] -= 20.0  # never selected
    logits[:, 9] += 3.0    # hot
    tw, ti = OR.softmax_topk(logits, k, True)
    out = _run(fg, x, w1, w2, tw, ti)
    ref = OE.fused_experts(x, w1, w2, tw, ti)
    assert_close_moe(out, ref, "bf16", f"auto T={T}")


@pytest.mark.parametrize("variant", ["stream", "tcgen05"])
def test_options(fg, variant):
    """apply_router_weight_on_input, no_combine, routed_scaling_factor, expert_map."""
    T, H, I, E, k = 50, 256, 384, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 77)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = _run(fg, x, w1, w2, tw, ti, variant=variant, apply_router_weight_on_input=True)
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti, apply_router_weight_on_input=True), "bf16", "w-on-input")
    out = _run(fg, x, w1, w2, tw, ti, variant=variant, no_combine=True)
    assert out.shape == (T, k, H)
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti, no_combine=True), "bf16", "no_combine")
    out = _run(fg, x, w1, w2, tw, ti, variant=variant, routed_scaling_factor=2.5)
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti, routed_scaling_factor=2.5), "bf16", "scaling")
    # expert_map: this "rank" owns experts 4..7 only
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[4:] = torch.arange(4, dtype=torch.int32)
    out = fg.fused_experts(x.cuda(), w1[4:].cuda(), w2[4:].cuda(), tw.cuda(), ti.cuda(), expert_map=emap.cuda(),
                           variant=variant)
    ti_local = emap[ti.long()]
    ref = OE.fused_experts(x, w1[4:], w2[4:], tw, ti_local)
    assert_close_moe(out, ref, "bf16", "expert_map")


@pytest.mark.parametrize("variant", ["stream", "tcgen05"])
@pytest.mark.parametrize("fp8", [False, True])
def test_one_call_entry_equals_kernel_by_kernel_path(fg, variant, fp8):
    """fused_experts goes through the single C entry (fmoe_fused_experts); with stage events switched on it
    launches the same kernels one by one.  Both must give bit-identical results."""
    import importlib

    FM = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")
    T, H, I, E, k = 70, 512, 256, 16, 4
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 11)
    tw, ti = OR.softmax_topk(logits, k, True)
    kw = dict(variant=variant)
    if fp8:
        w1, s1 = OQ.quant_weight_block128(w1)
        w2, s2 = OQ.quant_weight_block128(w2)
        kw.update(use_fp8_w8a8=True, w1_scale=s1.cuda(), w2_scale=s2.cuda(), block_shape=[128, 128])
    a = _run(fg, x, w1, w2, tw, ti, **kw)
    FM.STAGE_EVENTS = []
    try:
        b = _run(fg, x, w1, w2, tw, ti, **kw)
        assert sum(name.startswith("gemm") for name, _, _ in FM.STAGE_EVENTS) == 2
    finally:
        FM.STAGE_EVENTS = None
    assert torch.equal(a, b)


@pytest.mark.parametrize("T,H,I,E,k", [(70, 512, 256, 16, 4), (1, 128, 128, 4, 2), (300, 1032, 384, 8, 2),
                                       (2048, 2048, 768, 32, 8)])
@pytest.mark.parametrize("on_input", [False, True])
def test_tcgen05_gate_up_row_gather_equals_sorted_copy(fg, T, H, I, E, k, on_input):
    """The tcgen05 gate/up kernel either reads a sorted copy of the input rows (a_gather = 0) or fetches
    row slot/top_k of the [T,H] input itself with TMA gather (a_gather = 1); padding rows read as zeros in
    both.  The two must agree bit for bit, and rows past num_tokens_post_padded stay untouched."""
    import importlib

    from flaggems_sglang_b200 import _C

    FM = importlib.import_module("flaggems_sglang_b200.ops.fused_moe")
    kk = 1 if on_input else k
    x, w1, _, logits = _layer(T, H, I, E, kk, torch.bfloat16, 23)
    tw, ti = OR.softmax_topk(logits, kk, True)
    x, w1, tw, ti = x.cuda(), w1.cuda(), tw.cuda().float().contiguous(), ti.cuda().int().contiguous()
    lib, st = _C.lib(), _C.stream_ptr(x.device)
    numel = T * kk
    sorted_ids, expert_ids, num_post = fg.moe_align_block_size(ti, 128, E)
    cap = sorted_ids.numel()
    common = dict(variant=_C.VARIANTS["tcgen05"], activation=_C.ACTIVATIONS["silu"], num_experts=E, top_k=kk,
                  block_size=128, numel=numel, sorted_cap=cap, max_blocks=min(cap // 128, numel),
                  sorted_token_ids=sorted_ids.data_ptr(), expert_ids=expert_ids.data_ptr(),
                  num_tokens_post_padded=num_post.data_ptr(), dtype=_C.BF16, out_dtype=_C.BF16, n=I, k=H,
                  w=w1.data_ptr(), row_scale=tw.data_ptr() if on_input else None)
    xs = torch.empty((cap, H), dtype=torch.bfloat16, device="cuda")
    _C.check(lib.fmoe_gather_rows(x.data_ptr(), 2, cap, H, sorted_ids.data_ptr(), kk, numel, num_post.data_ptr(),
                                  xs.data_ptr(), st))
    outs = []
    for gather in (0, 1):
        act = torch.full((cap, I), -7.0, dtype=torch.bfloat16, device="cuda")
        a, rows = (x, T) if gather else (xs, cap)
        g1 = FM._gemm_args(a_gather=gather, a_rows=rows, a=a.data_ptr(), out=act.data_ptr(), **common)
        _C.check(lib.fmoe_gemm1_silu(g1, st))
        outs.append(act)
    torch.cuda.synchronize()
    _C.check_device_status()
    used = int(num_post.item())
    assert torch.equal(outs[0], outs[1])
    assert (outs[1][used:] == -7.0).all()
    pad = (sorted_ids[:used] >= numel)
    assert (outs[1][:used][pad] == 0).all()


@pytest.mark.parametrize("variant", ["simt", "stream", "tcgen05"])
def test_gelu_activation(fg, variant):
    """The reference's second activation (gelu-and-mul, ref fused_moe.py:219-220)."""
    T, H, I, E, k = 40, 256, 384, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 21)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = _run(fg, x, w1, w2, tw, ti, variant=variant, activation="gelu")
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti, activation="gelu"), "bf16", f"gelu {variant}")
    with pytest.raises(ValueError, match="Unsupported FusedMoe activation"):
        _run(fg, x, w1, w2, tw, ti, activation="relu")


def test_bounded_wait_reports_and_context_survives(fg):
    """A wait that can never be satisfied gives up after its cycle limit, the status word reports it, and
    the same context keeps computing (no trap, no hang)."""
    from flaggems_sglang_b200 import _C

    lib = _C.lib()
    _C.check(lib.fmoe_selftest_bounded_wait(2_000_000, _C.stream_ptr()))  # ~1 ms
    with pytest.raises(_C.FmoeError) as ei:
        _C.check_device_status()
    assert ei.value.code == _C.ERR_DEVICE_TIMEOUT and "0xe00" in str(ei.value)
    _C.check_device_status()  # cleared by the read above
    x, w1, w2, logits = _layer(9, 128, 128, 4, 2, torch.bfloat16, 3)
    tw, ti = OR.softmax_topk(logits, 2, True)
    out = _run(fg, x, w1, w2, tw, ti, variant="tcgen05")
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti), "bf16", "after time-out")


def test_empty_batch(fg):
    x, w1, w2, logits = _layer(4, 128, 128, 4, 2, torch.bfloat16, 1)
    out = fg.fused_experts(x[:0].cuda(), w1.cuda(), w2.cuda(), torch.zeros(0, 2).cuda(),
                           torch.zeros(0, 2, dtype=torch.int32).cuda())
    assert out.shape == (0, 128)


# ------------------------------------------------------------------ reference-layout entry point
@pytest.mark.parametrize("name", ["M7_E8_k2", "M33_E16_k4", "M17_E64_k8"])
@pytest.mark.parametrize("on_input", [False, True])
def test_reference_entry_point_with_golden_routing(fg, name, on_input):
    """triton_kernel_fused_experts on the reference layouts, fed with routing tables produced by the
    reference's own conversion (golden fixtures), against the restatement of the reference op."""
    g = np.load(os.path.join(GOLDEN, f"routing_{name}.npz"))
    T, k = g["topk_ids"].shape
    E = g["hist"].shape[0]
    H, I = 256, 384
    gen = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=gen).bfloat16()
    w1r = (torch.randn(E, H, 2 * I, generator=gen) * 0.1).bfloat16()   # reference layout [E,H,2I]
    w2r = (torch.randn(E, I, H, generator=gen) * 0.1).bfloat16()       # [E,I,H]
    rd = fg.RoutingData(torch.from_numpy(g["gate_scal"]).cuda(), torch.from_numpy(g["hist"]).cuda(), E, k)
    gi = fg.GatherIndx(torch.from_numpy(g["topk_indx"]).cuda(), torch.from_numpy(g["gate_indx"]).cuda())
    si = fg.ScatterIndx(torch.from_numpy(g["scatter_src"]).cuda(), torch.from_numpy(g["scatter_dst"]).cuda())
    out = fg.triton_kernel_fused_experts(x.cuda(), w1r.cuda(), w2r.cuda(), rd, gi, si,
                                         apply_router_weight_on_input=on_input)
    routing = OR.standard_topk_to_routing(torch.from_numpy(g["topk_weights"]), torch.from_numpy(g["topk_ids"]), E)
    ref = OE.reference_fused_experts(x, w1r, w2r, routing, apply_router_weight_on_input=on_input)
    assert out.shape == (T, H)
    assert_close_moe(out, ref, "bf16", f"reference entry {name}")
    # scatter_indx=None: un-combined rows in expert-sorted order
    z = fg.triton_kernel_fused_experts(x.cuda(), w1r.cuda(), w2r.cuda(), rd, gi, None,
                                       apply_router_weight_on_input=on_input)
    zref = OE.reference_fused_experts(x, w1r, w2r, routing, apply_router_weight_on_input=on_input, no_combine=True)
    assert_close_moe(z, zref, "bf16", f"reference entry no-combine {name}")
    # own conversion produces the same tables as the reference's
    rd2, gi2, si2 = fg.standard_topk_to_routing(torch.from_numpy(g["topk_weights"]).cuda(),
                                                torch.from_numpy(g["topk_ids"]).cuda(), E)
    np.testing.assert_array_equal(gi2.src_indx.cpu().numpy(), g["topk_indx"])
    np.testing.assert_array_equal(gi2.dst_indx.cpu().numpy(), g["gate_indx"])
    np.testing.assert_array_equal(rd2.expt_hist.cpu().numpy(), g["hist"])
    np.testing.assert_array_equal(rd2.gate_scal.cpu().numpy(), g["gate_scal"])


def test_hook(fg):
    """fused_moe_flagos with the reference's calling convention (objects with the same attributes)."""
    from types import SimpleNamespace as NS

    T, H, I, E, k = 20, 256, 256, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 5)
    tw, ti = OR.softmax_topk(logits, k, True)
    layer = NS(w13_weight=w1.cuda(), w2_weight=w2.cuda())
    cfg = NS(num_experts=E, activation="silu", apply_router_weight_on_input=False, no_combine=False,
             routed_scaling_factor=2.5, gemm1_alpha=None, gemm1_clamp_limit=None)
    disp = NS(hidden_states=x.cuda(), topk_output=NS(topk_weights=tw.cuda(), topk_ids=ti.cuda()))
    out = fg.fused_moe_flagos(NS(runner=NS(config=cfg)), layer, disp).hidden_states
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti, routed_scaling_factor=2.5), "bf16", "hook")
    triple = fg.standard_topk_to_routing(tw.cuda(), ti.cuda(), E)
    disp2 = NS(hidden_states=x.cuda(), topk_output=triple)
    out2 = fg.fused_moe_flagos(NS(runner=NS(config=cfg)), layer, disp2).hidden_states
    assert_close_moe(out2, OE.fused_experts(x, w1, w2, tw, ti, routed_scaling_factor=2.5), "bf16", "hook triple")
    # no_combine: both routing formats return the rows in expert-sorted order viewed [T,k,H], as the reference
    # hook does (src/flaggems_sglang/ops/fused_moe.py:355-366, 408-413), without the scaling factor
    cfg_nc = NS(**{**vars(cfg), "no_combine": True})
    routing = OR.standard_topk_to_routing(tw, ti, E)
    w1r, w2r = w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous()
    zref = OE.reference_fused_experts(x, w1r, w2r, routing, no_combine=True).view(T, k, H)
    z_std = fg.fused_moe_flagos(NS(runner=NS(config=cfg_nc)), layer, disp).hidden_states
    z_tri = fg.fused_moe_flagos(NS(runner=NS(config=cfg_nc)), layer, disp2).hidden_states
    assert z_std.shape == (T, k, H) and torch.equal(z_std, z_tri)
    assert_close_moe(z_std, zref, "bf16", "hook no_combine")


# ------------------------------------------------------------------ fp8 w8a8 block quant
@pytest.mark.parametrize("T,variant", [(1, "stream"), (9, "stream"), (64, "stream"), (9, "simt"), (200, "stream"),
                                       (9, "tcgen05"), (200, "tcgen05"), (1000, "tcgen05")])
def test_fp8_block_quant(fg, T, variant):
    H, I, E, k = 512, 256, 16, 4
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 300 + T)
    w1q, w1s = OQ.quant_weight_block128(w1)
    w2q, w2s = OQ.quant_weight_block128(w2)
    bias = torch.randn(E) * 0.1
    tw, ti = OR.grouped_topk(logits, bias, k, 4, 2, True, None)
    out = fg.fused_experts(x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                           w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128],
                           routed_scaling_factor=2.5, variant=variant)
    ref = OE.fused_experts_fp8(x, w1q, w1s, w2q, w2s, tw, ti, routed_scaling_factor=2.5)
    assert_close_moe(out, ref, "fp8", f"fp8 T={T} {variant}")


@pytest.mark.parametrize("H", [512, 640])
def test_fp8_tcgen05_both_input_quant_routes(fg, H):
    """H % 512 == 0: token rows are quantised once and copied into the sorted order; otherwise every sorted
    row is quantised.  Both feed the same GEMM and must match the oracle."""
    T, I, E, k = 300, 256, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 77)
    w1q, w1s = OQ.quant_weight_block128(w1)
    w2q, w2s = OQ.quant_weight_block128(w2)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = fg.fused_experts(x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                           w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128], variant="tcgen05")
    ref = OE.fused_experts_fp8(x, w1q, w1s, w2q, w2s, tw, ti)
    assert_close_moe(out, ref, "fp8", f"fp8 H={H}")


@pytest.mark.parametrize("H,I", [(512, 256), (7168, 256)])
def test_fp8_tcgen05_ring_depths_agree(fg, monkeypatch, H, I):
    """The e4m3 tensor-core kernel runs a four-stage ring when the staged scales fit beside it (two scale buffers
    for short reductions, one for long ones such as H = 7168) and a three-stage ring otherwise; the depth changes the
    timing only, so the results are the same bits."""
    T, E, k = 300, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 78)
    w1q, w1s = OQ.quant_weight_block128(w1)
    w2q, w2s = OQ.quant_weight_block128(w2)
    tw, ti = OR.softmax_topk(logits, k, True)
    args = (x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda())
    kw = dict(use_fp8_w8a8=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), block_shape=[128, 128], variant="tcgen05")
    out4 = fg.fused_experts(*args, **kw)
    monkeypatch.setenv("FMOE_FP8_STAGES", "3")
    out3 = fg.fused_experts(*args, **kw)
    assert torch.equal(out4, out3)
    if H <= 512:
        assert_close_moe(out4, OE.fused_experts_fp8(x, w1q, w1s, w2q, w2s, tw, ti), "fp8", f"fp8 ring depth H={H}")


def test_fp8_quantise_once_then_copy_equals_quantising_sorted_rows(fg):
    from flaggems_sglang_b200 import _C

    T, H, E, k = 130, 1024, 8, 4
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    ti = torch.randint(0, E, (T, k), generator=g).int().cuda()
    sorted_ids, _, num_post = fg.moe_align_block_size(ti, 128, E)
    cap, numel, used = sorted_ids.numel(), T * k, int(num_post.item())
    lib, st = _C.lib(), _C.stream_ptr(x.device)
    qa = torch.empty((cap, H), dtype=torch.uint8, device="cuda")
    sa = torch.empty((cap, H // 128), dtype=torch.float32, device="cuda")
    _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, cap, H, sorted_ids.data_ptr(), k, numel,
                                         num_post.data_ptr(), qa.data_ptr(), sa.data_ptr(), st))
    qt = torch.empty((T, H), dtype=torch.uint8, device="cuda")
    stt = torch.empty((T, H // 128), dtype=torch.float32, device="cuda")
    _C.check(lib.fmoe_quant_fp8_group128(x.data_ptr(), _C.BF16, T, H, None, 1, 0, None, qt.data_ptr(), stt.data_ptr(), st))
    qb, sb = torch.empty_like(qa), torch.empty_like(sa)
    for src, dst, eb, cols in ((qt, qb, 1, H), (stt, sb, 4, H // 128)):
        _C.check(lib.fmoe_gather_rows(src.data_ptr(), eb, cap, cols, sorted_ids.data_ptr(), k, numel,
                                      num_post.data_ptr(), dst.data_ptr(), st))
    torch.cuda.synchronize()
    real = sorted_ids[:used] < numel
    assert torch.equal(qa[:used][real], qb[:used][real])
    assert torch.equal(sa[:used][real], sb[:used][real])
    assert (qb[:used][~real] == 0).all() and (qa[:used][~real] == 0).all()


# ------------------------------------------------------------------ full benchmark sizes
def _sampled_oracle_check(fg, cfg_name, T, sample, kind, variant=None, skew=False):
    """Run the layer at its full size on the GPU and check `sample` evenly spaced tokens against the CPU oracle
    evaluated on the same weights (the oracle walks the experts those tokens route to, one expert at a time)."""
    from flaggems_sglang_b200 import workloads as W

    cfg = W.CONFIGS[cfg_name]
    wts = W.make_weights(cfg, "cuda", seed=0)
    tok = W.make_tokens(cfg, T, "cuda", seed=0, skew=skew)
    tw, ti = W.route(cfg, tok)
    kw = {}
    channel = cfg.dtype == "fp8" and cfg.fp8_scales == "channel"
    if channel:
        kw = dict(use_fp8_w8a8=True, per_channel_quant=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"])
    elif cfg.dtype == "fp8":
        kw = dict(use_fp8_w8a8=True, w1_scale=wts["w1_scale"], w2_scale=wts["w2_scale"], block_shape=[128, 128])
    out = fg.fused_experts(tok["hidden"], wts["w1"], wts["w2"], tw, ti, variant=variant, **kw)
    idx = torch.linspace(0, T - 1, min(sample, T)).long().unique().cuda()
    x_s, tw_s, ti_s = tok["hidden"][idx].cpu(), tw[idx].cpu(), ti[idx].cpu()
    if channel:
        ref = OE.fused_experts_fp8_per_channel(x_s, wts["w1"], wts["w1_scale"], wts["w2"], wts["w2_scale"], tw_s, ti_s)
    elif cfg.dtype == "fp8":
        ref = OE.fused_experts_fp8(x_s, wts["w1"], wts["w1_scale"], wts["w2"], wts["w2_scale"], tw_s, ti_s)
    else:
        ref = OE.fused_experts(x_s, wts["w1"], wts["w2"], tw_s, ti_s)
    l2, ma = assert_close_moe(out[idx], ref, kind, f"{cfg_name} T={T}{' zipf' if skew else ''} {idx.numel()} tokens")
    print(f"{cfg_name} T={T} skew={skew}: {idx.numel()} tokens vs oracle rel-L2 {l2:.2e} max-abs/max {ma:.2e}")
    return out


@pytest.mark.parametrize("T", [1, 64, 1024, 4096])
def test_mixtral_full_size_sampled(fg, T):
    out = _sampled_oracle_check(fg, "mixtral", T, 64, "bf16")
    if T == 64:  # the two tensor-core families agree at full size
        other = _sampled_oracle_check(fg, "mixtral", T, 8, "bf16", variant="tcgen05")
        assert rel_l2(out, other) < 5e-3


@pytest.mark.parametrize("T,skew", [(1, False), (512, False), (8192, False), (512, True), (8192, True)])
def test_qwen3_full_size_sampled(fg, T, skew):
    """Uniform and Zipf(1.2)-skewed routing (hot and empty experts) at the configuration's sizes."""
    _sampled_oracle_check(fg, "qwen3", T, 64, "bf16", skew=skew)


@pytest.mark.parametrize("T", [1, 64, 1024, 4096, 16384])
def test_dsv3_fp8_full_size_sampled(fg, T):
    _sampled_oracle_check(fg, "dsv3", T, 24, "fp8")


@pytest.mark.parametrize("T", [64, 4096])
def test_dsv3_fp8_per_channel_full_size_sampled(fg, T):
    _sampled_oracle_check(fg, "dsv3_channel", T, 24, "fp8")


def test_two_devices_in_one_process(fg):
    """Kernels that opt in to large dynamic shared memory are configured per device: a second GPU driven from the
    same process runs the tcgen05 kernels too."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    from flaggems_sglang_b200 import _C

    T, H, I, E, k = 300, 256, 256, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 31)
    tw, ti = OR.softmax_topk(logits, k, True)
    ref = OE.fused_experts(x, w1, w2, tw, ti)
    q1, s1 = OQ.quant_weight_block128(w1.float())
    q2, s2 = OQ.quant_weight_block128(w2.float())
    ref8 = OE.fused_experts_fp8(x, q1, s1, q2, s2, tw, ti)
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            out = fg.fused_experts(x.to(dev), w1.to(dev), w2.to(dev), tw.to(dev), ti.to(dev), variant="tcgen05")
            out8 = fg.fused_experts(x.to(dev), q1.to(dev), q2.to(dev), tw.to(dev), ti.to(dev), variant="tcgen05",
                                    use_fp8_w8a8=True, w1_scale=s1.to(dev), w2_scale=s2.to(dev), block_shape=[128, 128])
            _C.check_device_status(dev)
        assert_close_moe(out, ref, "bf16", f"tcgen05 on cuda:{d}")
        assert_close_moe(out8, ref8, "fp8", f"tcgen05 fp8 on cuda:{d}")


def test_integration_stub_runs(fg):
    """The ctypes stub of INTEGRATION.md, executed as printed, computes the bf16 layer through the raw C ABI."""
    import re

    from flaggems_sglang_b200 import _C

    text = open(os.path.join(os.path.dirname(os.path.dirname(GOLDEN)), "INTEGRATION.md")).read()
    stub = [b for b in re.findall(r"```python\n(.*?)```", text, flags=re.S) if "class GemmArgs" in b]
    assert len(stub) == 1
    ns = {"LIBFMOE_PATH": _C.LIB_PATH}
    exec(compile(stub[0], "INTEGRATION.md", "exec"), ns)
    T, H, I, E, k = 50, 256, 384, 8, 2
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 77)
    tw, ti = OR.softmax_topk(logits, k, True)
    out = ns["fused_experts_bf16"](x.cuda(), w1.cuda(), w2.cuda(), tw.cuda(), ti.cuda().to(torch.int32))
    _C.check_device_status()
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti), "bf16", "INTEGRATION.md stub")


# ------------------------------------------------------------------ sizes that are not multiples of 128
@pytest.mark.parametrize("variant", ["stream", "tcgen05", None])
@pytest.mark.parametrize("T,H,I,E,k", [(40, 320, 192, 8, 2), (9, 96, 160, 4, 2), (300, 352, 96, 8, 2)])
def test_bf16_sizes_not_multiple_of_128(fg, variant, T, H, I, E, k):
    """Hidden / intermediate sizes such as GPT-OSS's 2880: the tensor-core kernels cut their last column tile and
    zero-fill the last K step, the streaming kernel masks its last 128-k chunk; none falls back to the plain kernel."""
    from flaggems_sglang_b200.ops.fused_moe import _pick_variant

    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, T + H + I)
    tw, ti = OR.softmax_topk(logits, k, True)
    name, _ = _pick_variant(torch.bfloat16, T * k, E, I, H, variant)
    assert name in ("stream", "tcgen05")
    out = _run(fg, x, w1, w2, tw, ti, variant=variant)
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti), "bf16", f"{name} T={T} H={H} I={I}")


@pytest.mark.parametrize("T", [4, 64, 600])
def test_gpt_oss_layer_shape(fg, T):
    """H = I = 2880, 32 experts, top-4 (the model the reference's bias variant exists for), plain silu layer."""
    H, I, E, k = 2880, 2880, 32, 4
    g = torch.Generator(device="cuda").manual_seed(T)
    x = torch.randn(T, H, generator=g, device="cuda").bfloat16()
    w1 = (torch.randn(E, 2 * I, H, generator=g, device="cuda") / H ** 0.5).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g, device="cuda") / I ** 0.5).bfloat16()
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g, device="cuda").cpu(), k, True)
    out = fg.fused_experts(x, w1, w2, tw.cuda(), ti.cuda())
    idx = torch.linspace(0, T - 1, min(T, 16)).long().unique()
    ref = OE.fused_experts(x[idx.cuda()].cpu(), w1, w2, tw[idx], ti[idx])
    assert_close_moe(out[idx.cuda()], ref, "bf16", f"gpt-oss shape T={T}")


# ------------------------------------------------------------------ weights in the reference operator's own layout
@pytest.mark.parametrize("on_input", [False, True])
@pytest.mark.parametrize("T,H,I,E,k", [(1, 256, 128, 8, 2), (40, 320, 192, 8, 2), (300, 352, 96, 8, 2),
                                       (700, 512, 384, 16, 4), (64, 1280, 3072, 64, 8)])
def test_reference_layout_weights_read_in_place(fg, T, H, I, E, k, on_input):
    """w1 [E,H,2I] / w2 [E,I,H] (what the reference's tests and benchmarks pass, ref tests/test_fused_moe.py:64-72)
    are read in place as an N-major tensor-core operand: same bits as the [E,2I,H] / [E,H,I] kernels, since the
    products and the accumulation order are the same."""
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, T + H + I + 1)
    tw, ti = OR.softmax_topk(logits, k, True)
    w1n, w2n = w1.cuda().transpose(1, 2).contiguous(), w2.cuda().transpose(1, 2).contiguous()
    got = fg.fused_experts(x.cuda(), w1n, w2n, tw.cuda(), ti.cuda(), weights_n_major=True,
                           apply_router_weight_on_input=on_input)
    same = _run(fg, x, w1, w2, tw, ti, variant="tcgen05", apply_router_weight_on_input=on_input)
    assert torch.equal(got, same)
    if T * k * H * I <= 3e9:
        assert_close_moe(got, OE.fused_experts(x, w1, w2, tw, ti, apply_router_weight_on_input=on_input), "bf16",
                         f"n-major T={T} H={H} I={I}")


def test_reference_entry_point_makes_no_transposed_copy(fg):
    """`triton_kernel_fused_experts` with contiguous [E,H,2I] / [E,I,H] weights: the peak of device memory during the
    call stays below the size of one weight tensor (a transposed copy would need both)."""
    T, H, I, E, k = 128, 1024, 2048, 16, 4
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 5)
    tw, ti = OR.softmax_topk(logits, k, True)
    xd, w1n, w2n = x.cuda(), w1.cuda().transpose(1, 2).contiguous(), w2.cuda().transpose(1, 2).contiguous()
    rd, gi, si = fg.standard_topk_to_routing(tw.cuda(), ti.cuda(), E)
    fg.triton_kernel_fused_experts(xd, w1n, w2n, rd, gi, si)  # first call: lazy initialisation
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    out = fg.triton_kernel_fused_experts(xd, w1n, w2n, rd, gi, si)
    torch.cuda.synchronize()
    assert torch.cuda.max_memory_allocated() - base < w2n.numel() * 2
    assert_close_moe(out, OE.fused_experts(x, w1, w2, tw, ti), "bf16", "reference entry, weights in place")
    # a transposed VIEW of serving-side weights keeps taking the [E,2I,H] kernels, also without a copy
    torch.cuda.reset_peak_memory_stats()
    out2 = fg.triton_kernel_fused_experts(xd, w1.cuda().transpose(1, 2), w2.cuda().transpose(1, 2), rd, gi, si)
    assert_close_moe(out2, OE.fused_experts(x, w1, w2, tw, ti), "bf16", "reference entry, transposed views")


# ------------------------------------------------------------------ fp8 w8a8 with per-channel / per-token scales
@pytest.mark.parametrize("T,H,I,E,k", [(9, 512, 256, 16, 4), (200, 512, 256, 16, 4), (1000, 512, 256, 16, 4),
                                       (300, 352, 96, 8, 2), (64, 2880, 2880, 8, 2)])
def test_fp8_per_channel_quant(fg, T, H, I, E, k):
    """`per_channel_quant=True` (ref src/flaggems_sglang/ops/fused_moe.py:160, asserted off there): e4m3 weights with
    one scale per output channel, activations with one dynamic scale per token; the tensor-core kernel applies both to
    the finished accumulator."""
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 500 + T)
    w1q, w1s = OQ.quant_weight_per_channel(w1)
    w2q, w2s = OQ.quant_weight_per_channel(w2)
    gq, gs = fg.quant_weight_per_channel(w1.cuda())
    assert torch.equal(gs.cpu(), w1s) and torch.equal(gq.cpu().view(torch.uint8), w1q.view(torch.uint8))
    tw, ti = OR.softmax_topk(logits, k, True)
    out = fg.fused_experts(x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                           per_channel_quant=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), routed_scaling_factor=2.5)
    again = fg.fused_experts(x.cuda(), w1q.cuda(), w2q.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                             per_channel_quant=True, w1_scale=w1s.cuda(), w2_scale=w2s.cuda(), routed_scaling_factor=2.5)
    assert torch.equal(out, again), "run-to-run results differ"
    idx = torch.linspace(0, T - 1, min(T, 64)).long().unique()
    ref = OE.fused_experts_fp8_per_channel(x[idx], w1q, w1s, w2q, w2s, tw[idx], ti[idx], routed_scaling_factor=2.5)
    assert_close_moe(out[idx.cuda()], ref, "fp8", f"fp8 per-channel T={T} H={H} I={I}")


# ------------------------------------------------------------------ tail split of the tensor-core GEMMs
@pytest.mark.parametrize("T,H,I,E,k", [(700, 1024, 768, 8, 2), (1024, 4096, 1024, 4, 2)])
def test_tail_split_on_and_off(fg, monkeypatch, T, H, I, E, k):
    """A last round of tiles that fills at most half of the CTAs is cut along K over the idle CTAs (fp32 partials summed
    strip-wise in a fixed order).  On and off are both deterministic, both match the oracle, and differ from each other
    by summation order only."""
    x, w1, w2, logits = _layer(T, H, I, E, k, torch.bfloat16, 900 + T)
    tw, ti = OR.softmax_topk(logits, k, True)
    on = _run(fg, x, w1, w2, tw, ti, variant="tcgen05")
    assert torch.equal(on, _run(fg, x, w1, w2, tw, ti, variant="tcgen05")), "run-to-run results differ"
    monkeypatch.setenv("FMOE_TC_SPLIT_TAIL", "0")
    off = _run(fg, x, w1, w2, tw, ti, variant="tcgen05")
    assert rel_l2(on, off) < 1e-3
    idx = torch.linspace(0, T - 1, 64).long().unique()
    ref = OE.fused_experts(x[idx], w1, w2, tw[idx], ti[idx])
    assert_close_moe(on[idx.cuda()], ref, "bf16", f"tail split on T={T}")
    assert_close_moe(off[idx.cuda()], ref, "bf16", f"tail split off T={T}")
