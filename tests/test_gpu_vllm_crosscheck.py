"""Independent sanity cross-check of the oracle's builder-defined stages against another implementation.

The reference has no grouped router, no moe_align_block_size, no per-token-group fp8 quantiser and no fp8
expert computation (src/flaggems_sglang/ops/fused_moe.py:170-185 rejects fp8), so the oracle's contracts for
them are stated by this project.  vLLM ships CUDA / Triton implementations of the same serving-side ops; where
it is installed, the oracle (and the kernels of this package) are compared with it.  vLLM is not the reference:
a case is skipped when vLLM or one of its ops cannot be loaded, and only the used prefix of its buffers is
compared (its tail conventions are its own).
"""
import os

import numpy as np
import pytest
import torch

# vLLM's Blackwell default rounds fp8 block scales to powers of two (UE8M0) on its DeepGEMM path; the contract
# checked here keeps fp32 scales, so that path is switched off before vLLM reads its environment
os.environ.setdefault("VLLM_USE_DEEP_GEMM", "0")
os.environ.setdefault("VLLM_USE_DEEP_GEMM_E8M0", "0")

from oracle import experts as OE
from oracle import quant as OQ
from oracle import routing as OR
from tests.util import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    try:
        from vllm import _custom_ops as ops

        ops.moe_align_block_size  # noqa: B018
        torch.ops._moe_C.moe_align_block_size  # noqa: B018
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM custom ops unavailable: {e}")
    return ops


@pytest.mark.parametrize("T,E,k,block", [(16, 8, 2, 16), (300, 128, 8, 64), (1000, 256, 8, 128), (5, 64, 8, 16)])
def test_moe_align_block_size_used_prefix(vops, T, E, k, block):
    import flaggems_sglang_b200 as fg

    g = torch.Generator().manual_seed(T + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    numel = T * k
    cap = numel + E * (block - 1)
    sorted_v = torch.empty(cap, dtype=torch.int32, device="cuda")
    experts_v = torch.empty((cap + block - 1) // block, dtype=torch.int32, device="cuda")
    npp_v = torch.empty(1, dtype=torch.int32, device="cuda")
    try:
        vops.moe_align_block_size(ids.cuda(), E, block, sorted_v, experts_v, npp_v)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM moe_align_block_size did not run: {e}")
    so, eo, no = OR.moe_align_block_size(ids.numpy(), block, E)
    used = int(no[0])
    assert int(npp_v.item()) == used
    np.testing.assert_array_equal(experts_v.cpu().numpy()[: used // block], eo[: used // block])
    sv = sorted_v.cpu().numpy()[:used]
    # same slots in every block (vLLM does not promise an order inside an expert; padding = numel in both)
    np.testing.assert_array_equal(np.sort(sv.reshape(-1, block), axis=1), np.sort(so[:used].reshape(-1, block), axis=1))
    # and this package's kernel agrees with the oracle bit for bit (stable order)
    sk, ek, nk = fg.moe_align_block_size(ids.cuda(), block, E)
    np.testing.assert_array_equal(sk.cpu().numpy(), so)
    np.testing.assert_array_equal(ek.cpu().numpy(), eo)


@pytest.mark.parametrize("T,E,k,ng,tg", [(64, 256, 8, 8, 4), (7, 64, 6, 8, 3), (500, 256, 8, 8, 4)])
def test_grouped_topk(vops, T, E, k, ng, tg):
    g = torch.Generator().manual_seed(T * 3 + E)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.1
    w_o, i_o = OR.grouped_topk(logits, bias, k, ng, tg, True, 2.5)
    try:
        w_v, i_v = vops.grouped_topk(logits.cuda(), ng, tg, k, True, 2.5, bias.cuda(), 1)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM grouped_topk did not run: {e}")
    i_v = i_v.cpu().long()
    w_v = w_v.cpu().float()
    order_o = torch.argsort(i_o.long(), dim=1)
    order_v = torch.argsort(i_v, dim=1)
    ids_o = torch.gather(i_o.long(), 1, order_o)
    ids_v = torch.gather(i_v, 1, order_v)
    same = (ids_o == ids_v).all(dim=1)
    # random fp32 logits: a different expert set can only come from a near-tie decided by rounding
    assert same.float().mean() >= 0.99, f"only {same.float().mean():.3f} of the tokens got the same expert set"
    wo = torch.gather(w_o, 1, order_o)[same]
    wv = torch.gather(w_v, 1, order_v)[same]
    torch.testing.assert_close(wv, wo, rtol=2e-5, atol=1e-6)


def test_per_token_group_quant(vops):
    try:
        from vllm.model_executor.layers.quantization.utils.fp8_utils import per_token_group_quant_fp8
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM quantiser unavailable: {e}")
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(37, 1024, generator=g) * 3).bfloat16()
    try:
        q_v, s_v = per_token_group_quant_fp8(x.cuda(), 128, use_ue8m0=False)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM quantiser did not run: {e}")
    q_o, s_o = OQ.quant_act_group128(x)
    torch.testing.assert_close(s_v.cpu().float(), s_o, rtol=1e-6, atol=0)
    # bytes may differ by one e4m3 step where x/scale sits on a rounding boundary (division against reciprocal)
    diff = (q_v.cpu().float() - q_o.float()).abs()
    step = q_o.float().abs().clamp_min(2.0 ** -6) * 0.125
    assert (diff <= step).all() and (diff > 0).float().mean() < 0.01


def test_fp8_block_quant_experts(vops):
    """Oracle fp8 w8a8 128x128 expert computation against vLLM's (its Triton block-quant kernels)."""
    try:
        from vllm.model_executor.layers.fused_moe.config import fp8_w8a8_moe_quant_config
        from vllm.model_executor.layers.fused_moe.fused_moe import fused_experts as vllm_fused_experts
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM fused_experts unavailable: {e}")
    import flaggems_sglang_b200 as fg

    T, H, I, E, k = 48, 512, 256, 8, 2
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = torch.randn(E, 2 * I, H, generator=g) / H ** 0.5
    w2 = torch.randn(E, H, I, generator=g) / I ** 0.5
    q1, s1 = OQ.quant_weight_block128(w1)
    q2, s2 = OQ.quant_weight_block128(w2)
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g), k, True)
    ref = OE.fused_experts_fp8(x, q1, s1, q2, s2, tw, ti)
    ours = fg.fused_experts(x.cuda(), q1.cuda(), q2.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True, w1_scale=s1.cuda(),
                            w2_scale=s2.cuda(), block_shape=[128, 128])
    assert rel_l2(ours, ref) <= 3e-2
    try:
        from vllm.utils.deep_gemm import is_deep_gemm_e8m0_used

        if is_deep_gemm_e8m0_used():
            pytest.skip("this vLLM build rounds block scales to powers of two (UE8M0): not the fp32-scale contract")
    except ImportError:
        pass
    try:
        qc = fp8_w8a8_moe_quant_config(w1_scale=s1.cuda(), w2_scale=s2.cuda(), block_shape=[128, 128])
        out_v = vllm_fused_experts(x.cuda(), q1.cuda(), q2.cuda(), tw.cuda(), ti.cuda().to(torch.int32), quant_config=qc)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM fp8 fused_experts did not run here: {type(e).__name__}: {e}")
    l2_oracle, l2_ours = rel_l2(out_v, ref), rel_l2(ours, out_v)
    print(f"vLLM fp8 experts vs oracle rel-L2 {l2_oracle:.2e}; this package vs vLLM {l2_ours:.2e}")
    assert l2_oracle <= 3e-2 and l2_ours <= 3e-2


def test_per_token_quant(vops):
    """One dynamic scale per row: this package's kernel and the oracle against vLLM's dynamic per-token quantiser."""
    import flaggems_sglang_b200 as fg

    g = torch.Generator().manual_seed(9)
    x = (torch.randn(77, 2048, generator=g) * torch.rand(77, 1, generator=g) * 4).bfloat16()
    x[3] = 0
    try:
        qv, sv = vops.scaled_fp8_quant(x.cuda(), None, use_per_token_if_dynamic=True)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM per-token quantiser did not run here: {type(e).__name__}: {e}")
    oq, os_ = OQ.quant_act_per_token(x)
    q, s = fg.per_token_quant_fp8(x.cuda())
    assert torch.equal(s.cpu(), os_) and torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    torch.testing.assert_close(sv.reshape(-1).cpu(), os_, rtol=1e-6, atol=0)
    # vLLM multiplies by a reciprocal where the oracle divides: bytes may differ by one step on exact ties only
    diff = (qv.cpu().float() - oq.float()).abs()
    assert float((diff > 0).float().mean()) <= 2e-3, "more than 0.2 % of the bytes differ from vLLM's quantiser"


def test_fp8_per_channel_experts(vops):
    """Per-channel w8a8 experts (`per_channel_quant`): oracle and this package against vLLM's fused experts with
    per-token activation scales and per-output-channel weight scales."""
    try:
        from vllm.model_executor.layers.fused_moe.config import fp8_w8a8_moe_quant_config
        from vllm.model_executor.layers.fused_moe.fused_moe import fused_experts as vllm_fused_experts
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM fused_experts unavailable: {e}")
    import flaggems_sglang_b200 as fg

    T, H, I, E, k = 48, 512, 256, 8, 2
    g = torch.Generator().manual_seed(12)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = torch.randn(E, 2 * I, H, generator=g) / H ** 0.5
    w2 = torch.randn(E, H, I, generator=g) / I ** 0.5
    q1, s1 = OQ.quant_weight_per_channel(w1)
    q2, s2 = OQ.quant_weight_per_channel(w2)
    tw, ti = OR.softmax_topk(torch.randn(T, E, generator=g), k, True)
    ref = OE.fused_experts_fp8_per_channel(x, q1, s1, q2, s2, tw, ti)
    ours = fg.fused_experts(x.cuda(), q1.cuda(), q2.cuda(), tw.cuda(), ti.cuda(), use_fp8_w8a8=True,
                            per_channel_quant=True, w1_scale=s1.cuda(), w2_scale=s2.cuda())
    assert rel_l2(ours, ref) <= 3e-2
    try:
        qc = fp8_w8a8_moe_quant_config(w1_scale=s1.cuda().unsqueeze(-1), w2_scale=s2.cuda().unsqueeze(-1),
                                       per_act_token_quant=True, per_out_ch_quant=True)
        out_v = vllm_fused_experts(x.cuda(), q1.cuda(), q2.cuda(), tw.cuda(), ti.cuda().to(torch.int32), quant_config=qc)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"vLLM per-channel fp8 fused_experts did not run here: {type(e).__name__}: {e}")
    l2_oracle, l2_ours = rel_l2(out_v, ref), rel_l2(ours, out_v)
    print(f"vLLM per-channel fp8 experts vs oracle rel-L2 {l2_oracle:.2e}; this package vs vLLM {l2_ours:.2e}")
    assert l2_oracle <= 3e-2 and l2_ours <= 3e-2
