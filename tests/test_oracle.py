"""The CPU oracle against the committed golden vectors and independent codec implementations."""
import os

import ml_dtypes
import numpy as np
import pytest

from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qgemv_golden.npz"))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_e2m1_table_exhaustive():
    got = np.array([O.lib().orc_e2m1_decode(i) for i in range(16)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(G["e2m1"]))
    assert np.array_equal(bits(got), bits(O.np_e2m1_decode(np.arange(16))))
    assert sorted(set(np.abs(got).tolist())) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_e4m3_table_exhaustive():
    got = np.array([O.lib().orc_e4m3_decode(i) for i in range(256)], dtype=np.float32)
    ref = G["e4m3"]
    nan = np.isnan(ref)
    assert nan.sum() == 2 and nan[0x7F] and nan[0xFF]
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(ref)[~nan])
    assert np.array_equal(bits(O.np_e4m3_decode(np.arange(256)))[~nan], bits(ref)[~nan])
    assert got[0x7E] == 448.0 and got[0x01] == 2.0 ** -9


def test_e4m3_against_torch():
    torch = pytest.importorskip("torch")
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    got = np.array([O.lib().orc_e4m3_decode(i) for i in range(256)], dtype=np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(bits(got)[~nan], bits(ref)[~nan])


def test_e4m3_encode_known_answers():
    assert np.array_equal(O.e4m3_encode(G["e4m3_enc_in"]), G["e4m3_enc_out"])
    # every finite code survives decode -> encode
    codes = np.array([c for c in range(256) if c not in (0x7F, 0xFF)], dtype=np.uint8)
    assert np.array_equal(O.e4m3_encode(G["e4m3"][codes]), codes)
    # saturation and NaN
    assert O.lib().orc_e4m3_encode(1e9) == 0x7E and O.lib().orc_e4m3_encode(-1e9) == 0xFE
    assert O.lib().orc_e4m3_encode(float("nan")) & 0x7F == 0x7F


def test_bf16_known_answers():
    assert np.array_equal(O.bf16_encode(G["bf16_kat_in"]), G["bf16_kat_out"])
    x = np.random.default_rng(5).standard_normal(50000).astype(np.float32) * 37
    assert np.array_equal(O.bf16_encode(x), x.astype(ml_dtypes.bfloat16).view(np.uint16))
    assert np.array_equal(bits(O.bf16_decode(O.bf16_encode(x))),
                          bits(x.astype(ml_dtypes.bfloat16).astype(np.float32)))


def test_nvfp4_products_exhaustive():
    """All 16 x 256 (code, scale) pairs: the dequantised weight is bit-exact."""
    codes = np.repeat(np.arange(16, dtype=np.uint8), 16)  # 256 codes per row -> K = 256... build [256][?]
    # matrix with N = 256 rows (one scale value per row), K = 16 (one block holding all 16 codes)
    N = 256
    nib = np.tile(np.arange(16, dtype=np.uint8), (N, 1))
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    scales = np.arange(256, dtype=np.uint8).reshape(N, 1)
    w = O.dequant_nvfp4(packed, scales, 1.0)
    ref = G["nvfp4_prod"].T  # [scale][code]
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(w), nan)
    assert np.array_equal(bits(w)[~nan], bits(ref)[~nan])
    del codes


def test_seeded_gemv_matches_golden():
    w = O.dequant_nvfp4(G["codes"], G["scales"], float(G["ts"]))
    assert np.array_equal(bits(w), bits(G["w"]))
    y = O.gemv_nvfp4_f64(G["codes"], G["scales"], float(G["ts"]), G["x"])
    assert O.rel_l2(y, G["y"]) < 1e-14
    yf, _ = O.gemv_nvfp4_fast(G["codes"], G["scales"], float(G["ts"]), G["x"])
    assert O.rel_l2(yf, G["y"]) < 1e-5


def test_seeded_fp8_matches_golden():
    w = O.dequant_fp8(G["fp8_codes"], G["fp8_scales"])
    assert np.array_equal(bits(w), bits(G["fp8_w"]))
    y = O.gemv_fp8_f64(G["fp8_codes"], G["fp8_scales"], G["fp8_x"])
    assert O.rel_l2(y, G["fp8_y"]) < 1e-14
    yf, _ = O.gemv_fp8_fast(G["fp8_codes"], G["fp8_scales"], G["fp8_x"])
    assert O.rel_l2(yf, G["fp8_y"]) < 1e-5


def test_config0_runs_on_cpu():
    """BASELINE configs[0]: one 4096 x 4096 NVFP4 GEMV, host reference only."""
    codes, scales, ts = O.make_nvfp4(4096, 4096, seed=1)
    x = O.make_x(1, 4096, seed=1)
    # the stated scale distribution: about a fifth of the scales are E4M3 subnormals, some exactly zero
    sub = (((scales >> 3) & 15) == 0).mean()
    assert 0.15 < sub < 0.3 and (scales == 0).mean() > 0.005
    y64 = O.gemv_nvfp4_f64(codes, scales, ts, x)
    y32, threads = O.gemv_nvfp4_fast(codes, scales, ts, x)
    assert threads >= 1
    assert O.rel_l2(y32, y64) < 1e-5
    # bf16 output rounding alone stays inside the 2e-3 budget
    assert O.rel_l2(O.bf16_decode(O.bf16_encode(y32)), y64) < 2e-3


def test_moe_oracle_consistent():
    E, N, K, T, topk = 6, 32, 64, 3, 2
    cs = [O.make_nvfp4(N, K, 100 + e, ts=1.0 + e / 8) for e in range(E)]
    codes = np.stack([c[0] for c in cs])
    scales = np.stack([c[1] for c in cs])
    ts = np.array([c[2] for c in cs], dtype=np.float32)
    ids = np.array([[0, 3], [5, 1], [3, 3]], dtype=np.int32)
    x = O.make_x(T, K, 7)
    out = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=False)
    for t in range(T):
        for j in range(topk):
            e = ids[t, j]
            ref = O.gemv_nvfp4_f64(codes[e], scales[e], float(ts[e]), x[t:t + 1])
            assert np.array_equal(out[t * topk + j], ref[0])


def test_oracle_matches_skinny_golden():
    """Several token rows against vectors made from the third-party codecs (tests/golden/make_golden.py)."""
    import os
    S = np.load(os.path.join(os.path.dirname(__file__), "golden", "skinny_golden.npz"))
    for t in "ab":
        y = O.gemv_nvfp4_f64(S[f"{t}_codes"], S[f"{t}_scales"], float(S[f"{t}_ts"]), S[f"{t}_x"])
        assert O.rel_l2(y, S[f"{t}_y"]) < 1e-12
    assert O.rel_l2(O.gemv_fp8_f64(S["f_codes"], S["f_scales"], S["f_x"]), S["f_y"]) < 1e-12
