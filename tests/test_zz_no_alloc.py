"""The allocation-free entry point (fmoe_fused_experts_static) against the workspace-taking one.

Collected last on purpose (file name): a failure here cannot hide the other GPU tests from a run that
stops at the first failure.

The entry point is for callers that may not allocate device memory where they run the layer (a thread
that must not touch the allocator, a host that owns all GPU memory); it keeps
its intermediates in an array inside the library image.  The test drives both entry points through the
C ABI with ctypes, twice in a row with different inputs, because the array keeps the previous call's
contents and the second call must not be affected by them.
"""
import pytest
import torch

from tests.util import assert_close_moe

pytestmark = pytest.mark.gpu


def _case(seed, T, H, I, E, k):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).bfloat16().cuda()
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).bfloat16().cuda()
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).bfloat16().cuda()
    w = torch.rand(T, k, generator=g).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
    return x, w1, w2, w, ids


def _args(_C, x, w1, w2, w, ids, out, variant):
    T, H = x.shape
    E, twoI, _ = w1.shape
    return _C.FusedArgs(dtype=_C.BF16, variant=_C.VARIANTS[variant], num_experts=E, top_k=ids.shape[1], T=T, H=H,
                        I=twoI // 2, routed_scaling_factor=1.0, hidden=x.data_ptr(), w1=w1.data_ptr(),
                        w2=w2.data_ptr(), topk_weights=w.data_ptr(), topk_ids=ids.data_ptr(), out=out.data_ptr())


@pytest.mark.parametrize("variant", ["stream", "tcgen05"])
def test_static_scratch_entry_matches_workspace_entry(variant):
    from flaggems_sglang_b200 import _C

    lib = _C.lib()
    st = _C.stream_ptr()
    assert lib.fmoe_static_scratch_bytes() == 64 << 20
    # two calls in a row; the second has fewer tokens and other routing, so stale scratch would show
    for seed, T in [(1, 96), (2, 41)]:
        x, w1, w2, w, ids = _case(seed, T, 512, 384, 16, 4)
        ref = torch.empty(T, 512, dtype=torch.bfloat16, device="cuda")
        a = _args(_C, x, w1, w2, w, ids, ref, variant)
        need = lib.fmoe_fused_experts_workspace_bytes(a)
        assert 0 < need <= lib.fmoe_static_scratch_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        _C.check(lib.fmoe_fused_experts(a, st))

        out = torch.full((T, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        b = _args(_C, x, w1, w2, w, ids, out, variant)  # no workspace given
        if seed == 2:
            # second call (every one-time set-up is behind us): the device's free memory must not move across
            # it -- the property the entry point exists for.  Nothing else in this process allocates meanwhile.
            torch.cuda.synchronize()
            free_before, _ = torch.cuda.mem_get_info()
        _C.check(lib.fmoe_fused_experts_static(b, st))
        torch.cuda.synchronize()
        if seed == 2:
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes"
        _C.check_device_status()
        assert_close_moe(out, ref, "bf16", f"static vs workspace entry, {variant}, T={T}")
        assert torch.equal(out, ref)  # same kernels on the same inputs


def test_static_scratch_entry_rejects_oversized_problems():
    from flaggems_sglang_b200 import _C

    lib = _C.lib()
    # sizes only: the plan is refused before any pointer is read
    a = _C.FusedArgs(dtype=_C.BF16, variant=_C.VARIANT_AUTO, num_experts=8, top_k=2, T=1 << 16, H=4096, I=14336,
                     routed_scaling_factor=1.0)
    assert lib.fmoe_fused_experts_workspace_bytes(a) > lib.fmoe_static_scratch_bytes()
    rc = lib.fmoe_fused_experts_static(a, None)
    assert rc == _C.ERR_UNSUPPORTED
    msg = lib.fmoe_last_error().decode()
    assert "scratch" in msg and "fmoe_fused_experts" in msg
