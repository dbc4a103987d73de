"""Work plan of the tensor-core grouped GEMMs (whole tiles dealt round-robin, a part-filled last round cut along K over
the idle CTAs), checked on the host through the C ABI: every (tile, K step) is computed exactly once, slices of a tile
are contiguous in K and numbered in order, and the partial-accumulator slots stay inside the scratch."""
import ctypes
import random

import pytest


@pytest.fixture(scope="module")
def lib():
    from flaggems_sglang_b200 import _C

    return _C.lib()


def _units(lib, total, k_steps, max_split, grid, cta):
    out = (ctypes.c_int64 * 5)()
    units, it = [], 0
    while True:
        rc = lib.fmoe_debug_tail_plan(total, k_steps, max_split, grid, cta, it, out)
        assert rc in (0, 1)
        if rc == 0:
            return units
        units.append(tuple(out))
        it += 1
        assert it < 10000


def test_every_k_step_of_every_tile_is_covered_once(lib):
    rng = random.Random(7)
    cases = [(1056, 224, 8, 148), (7392, 64, 4, 148), (320, 48, 8, 148), (2240, 64, 4, 148), (0, 10, 8, 148), (5, 3, 8, 148)]
    cases += [(rng.randint(0, 5 * g), rng.randint(1, 300), rng.choice([0, 1, 4, 8]), g)
              for g in (1, 2, 7, 64, 132, 148) for _ in range(40)]
    for total, k_steps, max_split, grid in cases:
        cover, split_tiles = {}, 0
        for cta in range(grid):
            units = _units(lib, total, k_steps, max_split, grid, cta)
            for i, (tile, ks0, ks1, sl, ns) in enumerate(units):
                assert 0 <= tile < total and 0 <= ks0 < ks1 <= k_steps and 0 <= sl < ns
                assert ns == 1 or i == len(units) - 1, "only a CTA's last unit may be a slice"
                assert ns & (ns - 1) == 0 and ns <= max(max_split, 1), "slice counts are powers of two within the cap"
                cover.setdefault(tile, []).append((ks0, ks1, sl, ns, cta))
        assert len(cover) == total
        for tile, parts in cover.items():
            parts.sort()
            assert parts[0][0] == 0 and parts[-1][1] == k_steps
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:])), "slices are contiguous in K"
            assert [p[2] for p in parts] == list(range(len(parts))) and all(p[3] == len(parts) for p in parts)
            if len(parts) > 1:
                split_tiles += 1
                ctas = [p[4] for p in parts]
                assert ctas == list(range(ctas[0], ctas[0] + len(parts))) and ctas[0] % len(parts) == 0
                assert ctas[0] // len(parts) * len(parts) + len(parts) <= grid, "partial slots stay inside the scratch"
                assert all(p[1] - p[0] >= 8 for p in parts), "a slice keeps at least 8 K steps"
        if max_split < 2:
            assert split_tiles == 0


def test_mixtral_down_gemm_tail(lib):
    """1056 tiles of 224 K steps on 148 CTAs: 7 whole rounds, the 20 tiles of the eighth are cut into 4 slices each
    (148 / 20 = 7 -> the power of two below), so 80 CTAs run 56 K steps instead of 20 CTAs running 224."""
    tail = [u for cta in range(148) for u in _units(lib, 1056, 224, 8, 148, cta) if u[4] > 1]
    assert len(tail) == 80 and {u[4] for u in tail} == {4} and {u[2] - u[1] for u in tail} == {56}
    assert len({u[0] for u in tail}) == 20
    assert lib.fmoe_debug_tail_plan(10, 8, 8, 148, 148, 0, (ctypes.c_int64 * 5)()) == -1  # CTA index outside the grid
