"""The kernel's scheduling arithmetic and fragment layout, modelled on CPU, against the oracle."""
import numpy as np
import pytest

import kernel_model as M
from oracle import oracle as O


@pytest.mark.parametrize("N,K,B,grid", [(40, 192, 3, 5), (33, 1104, 2, 7), (16, 2112, 8, 3), (160, 128, 1, 4)])
def test_model_matches_oracle_nvfp4(qg, N, K, B, grid):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K, ts=0.75)
    x = O.make_x(B, K, seed=B)
    y, info = M.model_gemv(qg.pack(qg.FMT_NVFP4, codes, scales, ts), x, grid)
    assert not np.isnan(y).any()
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < 1e-12


def test_model_matches_oracle_fp8(qg):
    codes, scales = O.make_fp8(40, 192, seed=9)
    x = O.make_x(2, 192, seed=9)
    y, _ = M.model_gemv(qg.pack(qg.FMT_FP8, codes, scales), x, 5)
    assert O.rel_l2(y, O.gemv_fp8_f64(codes, scales, x)) < 1e-6


SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096), (10240, 8192),
          (8192, 28672), (1536, 2048), (2048, 768), (1280, 8192), (8192, 3584), (48, 64)]


@pytest.mark.parametrize("N,K", SHAPES)
@pytest.mark.parametrize("grid", [148, 132, 296, 1, 7])
def test_work_split_covers_everything_once(N, K, grid):
    """Every (panel, unit) block belongs to exactly one item; split panels have unique slots."""
    n_panels, units = (N + 15) // 16, (K + 63) // 64
    total = n_panels * units
    g = min(grid, total)
    pos = 0
    slots = set()
    parts = {}
    for cta in range(g):
        items = M.items_of_cta(cta, g, total, units, n_panels)
        assert items, "every participating CTA owns work"
        assert sum(it["partial"] for it in items) <= 2
        for it in items:
            assert it["start"] == pos
            assert 1 <= it["np"] <= M.PMAX and 0 <= it["u0"] < it["u1"] <= units
            if it["partial"]:
                assert it["np"] == 1
                s = M.part_slot(cta, it["vp"], units, total, g)
                assert s not in slots and s < 2 * g
                slots.add(s)
                parts.setdefault(it["vp"], []).append(cta)
            else:
                assert it["u0"] == 0 and it["u1"] == units
                assert it["vp"] // n_panels == (it["vp"] + it["np"] - 1) // n_panels
            pos += it["np"] * (it["u1"] - it["u0"])
    assert pos == total
    for vp, ctas in parts.items():
        c_lo, c_hi = M.cta_of(vp * units, total, g), M.cta_of((vp + 1) * units - 1, total, g)
        assert ctas == list(range(c_lo, c_hi + 1))
    # balance: no CTA gets more than one block above the mean
    sizes = [((c + 1) * total) // g - (c * total) // g for c in range(g)]
    assert max(sizes) - min(sizes) <= 1
