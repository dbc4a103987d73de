"""Shared helpers for the parity tests."""
import numpy as np
import torch

# Tolerances of the floating-point parity tests (the kernels fuse silu*mul into the first
# GEMM's epilogue and accumulate in a different order than the oracle's fp32 matmul, so
# outputs differ from it by rounding noise of the storage type):
BF16_REL_L2 = 1e-2          # relative L2 error, bf16 path (worst seen on B200: 5.1e-3)
# max |diff| <= this * max|ref|.  One bf16 ulp at the largest magnitude is between 2^-8 and 2^-7 of it, and the two
# sides round intermediates at different points, so a 2-ulp difference on the largest element (2^-6) is the bar
# for arbitrary cases (worst seen: 9.9e-3); the end-to-end comparison with the real reference operator
# (tests/test_e2e_reference.py) holds the tighter 2^-7 (worst seen: 6.8e-3).
BF16_MAX_ABS_FRAC = 2.0 ** -6
BF16_MAX_ABS_FRAC_E2E = 2.0 ** -7
FP8_REL_L2 = 3e-2           # worst seen: 1.2e-2
FP8_MAX_ABS_FRAC = 2.0 ** -5   # worst seen: 1.9e-2
FP32_REL_L2 = 1e-5


# (kind, case, rel-L2, max-abs/max) of every comparison made through assert_close_moe in this process; the
# terminal summary (tests/conftest.py) prints the worst values per kind, so the margin to the bars is visible
ACHIEVED: list = []


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
    ACHIEVED.append((kind, what, l2, ma))
    assert l2 <= lim_l2 and ma <= lim_abs, f"{what}: rel-L2 {l2:.3e} (<= {lim_l2}), max-abs/max {ma:.3e} (<= {lim_abs})"
    return l2, ma


def has_gpu() -> bool:
    return torch.cuda.is_available()


# ---- inputs of the end-to-end fixtures (tests/golden/make_golden_e2e.py and the tests that read them) ----
MAX_STORED_ROWS = 192  # larger outputs are stored as an evenly spaced sample of their rows


_M53 = (1 << 53) - 1


def _i64(v: int) -> int:
    """Two's-complement int64 value of an unsigned 64-bit constant."""
    return v - (1 << 64) if v >= (1 << 63) else v


def _mix64(z: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on int64 tensors (wrap-around multiplies, logical shifts by masking)."""
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _i64(0xBF58476D1CE4E5B9)
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _i64(0x94D049BB133111EB)
    return z ^ ((z >> 31) & ((1 << 33) - 1))


def hash_normal(seed: int, stream: int, n: int, device="cpu") -> torch.Tensor:
    """n standard-normal float64 values that depend only on (seed, stream, index): a counter-based generator
    (splitmix64 of the index, Box-Muller in float64) built from integer and float64 tensor ops, so the CPU and a
    GPU produce the same values once rounded to a 16- or 32-bit type (checksums in the fixtures guard this)."""
    i = torch.arange(n, dtype=torch.int64, device=device)
    base = _i64((seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D) & ((1 << 64) - 1))
    h1 = _mix64(i * 2 + base)
    h2 = _mix64(i * 2 + 1 + base)
    u1 = (((h1 >> 11) & _M53) + 1).to(torch.float64) * (2.0 ** -53)  # (0, 1]
    u2 = ((h2 >> 11) & _M53).to(torch.float64) * (2.0 ** -53)        # [0, 1)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * 3.141592653589793) * u2)


def e2e_inputs(M, K, N, E, topk, device="cpu", experts=None):
    """Seeded inputs of one case in the reference's layouts and distributions (tests/test_fused_moe.py:64-72;
    seed M+K+N+E+topk): hidden [M,K] bf16 ~ N(0,1), w1 [E,K,2N] and w2 [E,N,K] bf16 ~ 0.1 N(0,1), logits [M,E] f32.
    `experts`: generate only these experts' weights (the rest stay zero; the operator never reads the weights of
    an expert no token routes to)."""
    seed = M + K + N + E + topk
    hidden = hash_normal(seed, 1, M * K, device).view(M, K).to(torch.bfloat16)
    logits = hash_normal(seed, 2, M * E, device).view(M, E).to(torch.float32)
    w1 = torch.zeros(E, K, 2 * N, dtype=torch.bfloat16, device=device)
    w2 = torch.zeros(E, N, K, dtype=torch.bfloat16, device=device)
    for e in (range(E) if experts is None else experts):
        w1[e] = (hash_normal(seed, 16 + 2 * e, K * 2 * N, device) * 0.1).view(K, 2 * N).to(torch.bfloat16)
        w2[e] = (hash_normal(seed, 17 + 2 * e, N * K, device) * 0.1).view(N, K).to(torch.bfloat16)
    return hidden, w1, w2, logits


def checksum(t: torch.Tensor) -> np.ndarray:
    """Per-slice (first dimension) 64-bit sums of the tensor's raw 16-bit (or 32-bit) words."""
    words = t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)
    return words.reshape(words.shape[0], -1).to(torch.int64).sum(dim=1).cpu().numpy()


def stored_rows(n_rows: int) -> np.ndarray:
    if n_rows <= MAX_STORED_ROWS:
        return np.arange(n_rows, dtype=np.int64)
    return np.unique(np.linspace(0, n_rows - 1, MAX_STORED_ROWS).astype(np.int64))
