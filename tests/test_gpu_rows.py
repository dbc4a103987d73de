"""GPU parity: fp8 group quantisation, row gather and moe_sum against the CPU oracle (bit-exact)."""
import pytest
import torch

from oracle import experts as OE
from oracle import quant as OQ

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fg():
    import flaggems_sglang_b200 as fg

    return fg


@pytest.mark.parametrize("rows,K", [(1, 128), (7, 512), (64, 7168), (300, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant_group128_bit_exact(fg, rows, K, dtype):
    torch.manual_seed(rows + K)
    x = (torch.randn(rows, K) * torch.rand(rows, 1) * 4).to(dtype)
    x[0, :128] = 0  # an all-zero group
    q, s = fg.per_token_group_quant_fp8(x.cuda())
    oq, os_ = OQ.quant_act_group128(x)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quant_group128_division_bit_exact_over_wide_range(fg, dtype):
    """The kernel divides by the group scale through a shared reciprocal with two exact-residual corrections;
    8M quotients with group magnitudes from 2^-60 to 2^60 and exact ties must give the bits of the oracle's
    IEEE division."""
    g = torch.Generator().manual_seed(99)
    rows, K = 4096, 2048
    x = torch.randn(rows, K, generator=g)
    expo = torch.randint(-60, 61, (rows, K // 128), generator=g).float()
    x = (x.view(rows, K // 128, 128) * torch.exp2(expo).unsqueeze(-1)).view(rows, K)
    # exact e4m3 grid points and midpoints relative to a group maximum of 448 * 2^e
    grid = torch.tensor([448.0, 13.0, 13.5, 14.0, 0.001953125, 0.0009765625, 240.0, 232.0, -17.0, -18.0])
    x[5, :10] = grid
    x[6, 128:138] = grid * 2.0 ** -20
    x = x.to(dtype)
    q, s = fg.per_token_group_quant_fp8(x.cuda())
    oq, os_ = OQ.quant_act_group128(x)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


def test_quant_in_place_rows_with_padding_marks(fg):
    """map_div = 0: output row p reads input row p, and the map only says which positions are padding."""
    from flaggems_sglang_b200 import _C

    torch.manual_seed(3)
    T, k, K, E, block = 21, 2, 256, 8, 16
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    s, _, n = fg.moe_align_block_size(ids.cuda(), block, E)
    cap, used = s.numel(), int(n.item())
    x = torch.randn(cap, K).bfloat16()
    q = torch.full((cap, K), 0x55, dtype=torch.uint8, device="cuda")
    qs = torch.full((cap, K // 128), -1.0, dtype=torch.float32, device="cuda")
    _C.check(_C.lib().fmoe_quant_fp8_group128(x.cuda().data_ptr(), _C.BF16, cap, K, s.data_ptr(), 0, T * k,
                                              n.data_ptr(), q.data_ptr(), qs.data_ptr(), _C.stream_ptr()))
    oq, os_ = OQ.quant_act_group128(x)
    real = torch.zeros(cap, dtype=torch.bool)
    real[:used] = s.cpu()[:used] < T * k
    pad = ~real
    pad[used:] = False
    assert torch.equal(q.cpu()[real], oq.view(torch.uint8)[real]) and torch.equal(qs.cpu()[real], os_[real])
    assert (q.cpu()[pad] == 0).all() and (qs.cpu()[pad] == 1.0).all()
    assert (q.cpu()[used:] == 0x55).all() and (qs.cpu()[used:] == -1.0).all()


def test_weight_quant_matches_oracle(fg):
    torch.manual_seed(0)
    w = (torch.randn(3, 256, 384) / 16).bfloat16()
    q, s = fg.quant_weight_block128(w.cuda())
    oq, os_ = OQ.quant_weight_block128(w)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))


@pytest.mark.parametrize("T,k,H", [(1, 2, 256), (16, 2, 4096), (33, 8, 2048), (512, 8, 7168)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("scale", [None, 2.5])
def test_moe_sum_bit_exact(fg, T, k, H, dtype, scale):
    torch.manual_seed(T + k + H)
    z = torch.randn(T, k, H).to(dtype)
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    fg.moe_sum(z.cuda(), out, scale)
    ref = OE.moe_sum(z).to(dtype)
    if scale is not None:
        ref = (ref.float() * scale).to(dtype)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("scale", [None, 2.5])
def test_moe_sum_with_shared_expert_addend_bit_exact(fg, dtype, scale):
    """out = round(round(round(sum_j z) * scale) + shared): the post-scale (ref fused_moe.py:415-420) and the
    shared expert's `+=` folded into the combine pass, with the roundings of the separate ops."""
    torch.manual_seed(11)
    T, k, H = 37, 8, 1024
    z = torch.randn(T, k, H).to(dtype)
    shared = torch.randn(T, H).to(dtype)
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    fg.moe_sum(z.cuda(), out, scale, shared_output=shared.cuda())
    ref = OE.moe_sum(z).to(dtype)
    if scale is not None:
        ref = (ref.float() * scale).to(dtype)
    ref = (ref.float() + shared.float()).to(dtype)
    assert torch.equal(out.cpu(), ref)
    with pytest.raises(ValueError, match="shared_output"):
        fg.moe_sum(z.cuda(), out, scale, shared_output=shared[:, :512].cuda())


def test_gather_rows_and_fused_gather_quant(fg):
    from flaggems_sglang_b200 import _C

    torch.manual_seed(1)
    T, k, H, E, block = 37, 4, 512, 16, 16
    x = torch.randn(T, H).bfloat16()
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    s, e, n = fg.moe_align_block_size(ids.cuda(), block, E)
    cap = s.numel()
    out = torch.full((cap, H), 7.0, dtype=torch.bfloat16, device="cuda")
    st = _C.stream_ptr()
    _C.check(_C.lib().fmoe_gather_rows(x.cuda().data_ptr(), 2, cap, H, s.data_ptr(), k, T * k, n.data_ptr(),
                                       out.data_ptr(), st))
    sc = s.cpu().long()
    used = int(n.item())
    exp = torch.zeros(cap, H, dtype=torch.bfloat16)
    valid = sc[:used] < T * k
    exp[:used][valid] = x[sc[:used][valid] // k]
    assert torch.equal(out.cpu()[:used], exp[:used])
    assert (out.cpu()[used:] == 7.0).all()  # rows past the padded length are not touched
    q = torch.empty(cap, H, dtype=torch.float8_e4m3fn, device="cuda")
    qs = torch.empty(cap, H // 128, dtype=torch.float32, device="cuda")
    _C.check(_C.lib().fmoe_quant_fp8_group128(x.cuda().data_ptr(), _C.BF16, cap, H, s.data_ptr(), k, T * k,
                                              n.data_ptr(), q.data_ptr(), qs.data_ptr(), st))
    oq, os_ = OQ.quant_act_group128(exp[:used])
    vq = q.cpu().view(torch.uint8)[:used]
    assert torch.equal(vq[valid], oq.view(torch.uint8)[valid])
    assert torch.equal(qs.cpu()[:used][valid], os_[valid])
    assert (vq[~valid] == 0).all() and (qs.cpu()[:used][~valid] == 1.0).all()


@pytest.mark.parametrize("rows,K", [(1, 32), (7, 512), (64, 7168), (300, 2880), (5, 16384)])
def test_quant_per_token_bit_exact(fg, rows, K):
    """One dynamic scale per row (the activation side of per-channel w8a8): scales and bytes of the oracle."""
    torch.manual_seed(rows + K)
    x = (torch.randn(rows, K) * torch.rand(rows, 1) * 4).bfloat16()
    if rows > 2:
        x[1] = 0  # an all-zero row: the scale floor
        x[2] = x[2] * 1e-9  # tiny row: scale floor again
    q, s = fg.per_token_quant_fp8(x.cuda())
    oq, os_ = OQ.quant_act_per_token(x)
    assert torch.equal(s.cpu(), os_)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
