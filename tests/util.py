"""Shared helpers for the parity tests."""
import torch

# Tolerances of the floating-point parity tests (the kernels fuse silu*mul into the first
# GEMM's epilogue and accumulate in a different order than the oracle's fp32 matmul, so
# outputs differ from it by rounding noise of the storage type):
BF16_REL_L2 = 1e-2          # relative L2 error, bf16 path
BF16_MAX_ABS_FRAC = 2.0 ** -6  # max |diff| <= this * max|ref|
FP8_REL_L2 = 3e-2
FP8_MAX_ABS_FRAC = 2.0 ** -3
FP32_REL_L2 = 1e-5


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs_frac(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def assert_close_moe(got, ref, kind: str, what: str = ""):
    lim_l2, lim_abs = {
        "bf16": (BF16_REL_L2, BF16_MAX_ABS_FRAC),
        "fp8": (FP8_REL_L2, FP8_MAX_ABS_FRAC),
        "fp32": (FP32_REL_L2, 1e-4),
    }[kind]
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite output"
    l2, ma = rel_l2(got, ref), max_abs_frac(got, ref)
    assert l2 <= lim_l2 and ma <= lim_abs, f"{what}: rel-L2 {l2:.3e} (<= {lim_l2}), max-abs/max {ma:.3e} (<= {lim_abs})"
    return l2, ma


def has_gpu() -> bool:
    return torch.cuda.is_available()
