import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def pytest_terminal_summary(terminalreporter):
    """Worst achieved parity figures per storage type, next to the bars they were held to."""
    from tests import util

    if not util.ACHIEVED:
        return
    bars = {"bf16": (util.BF16_REL_L2, util.BF16_MAX_ABS_FRAC), "fp8": (util.FP8_REL_L2, util.FP8_MAX_ABS_FRAC),
            "fp32": (util.FP32_REL_L2, 1e-4)}
    terminalreporter.write_sep("-", "parity margins (worst case per kind)")
    for kind, (b_l2, b_ma) in bars.items():
        rows = [r for r in util.ACHIEVED if r[0] == kind]
        if not rows:
            continue
        w_l2 = max(rows, key=lambda r: r[2])
        w_ma = max(rows, key=lambda r: r[3])
        terminalreporter.write_line(
            f"{kind}: {len(rows)} comparisons; worst rel-L2 {w_l2[2]:.3e} (bar {b_l2:.1e}) in '{w_l2[1]}'; "
            f"worst max-abs/max {w_ma[3]:.3e} (bar {b_ma:.3e}) in '{w_ma[1]}'")
