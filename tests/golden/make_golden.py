"""Generates the committed golden vectors for the quantized GEMV path.

    python tests/golden/make_golden.py

The reference project ships no vectors for this arithmetic, so the tables are produced from
independent third-party implementations of the public formats that are importable here
(`ml_dtypes.float4_e2m1fn`, `ml_dtypes.float8_e4m3fn`, `ml_dtypes.bfloat16`) -- NOT from the
oracle under test.  The seeded GEMV case is produced with plain numpy float64 from those
tables.  Everything is stored as one small .npz.
"""
import os

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    e2m1 = np.arange(16, dtype=np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32)
    e4m3 = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    # exhaustive NVFP4 products: [code][scale] = fp32(e2m1 * e4m3), exact in fp32
    prod = (e2m1.astype(np.float64)[:, None] * e4m3.astype(np.float64)[None, :]).astype(np.float32)
    # bf16 round-to-nearest-even known answers: ties, subnormals, signed zero, overflow to inf
    kat_in = np.array([1.0, 1.00390625, 1.01171875, 1.005859375, -1.005859375, 3.3895314e38, 1e-40, -0.0,
                       65504.0, 0.1, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, 2.0 ** -133], dtype=np.float32)
    kat_out = kat_in.astype(ml_dtypes.bfloat16).view(np.uint16)
    # E4M3 encode known answers inside the finite range
    rng = np.random.Generator(np.random.Philox(20240611))
    enc_in = np.concatenate([
        (rng.standard_normal(4096) * 0.05).astype(np.float32),
        (rng.standard_normal(1024) * 30).astype(np.float32),
        np.array([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -11,
                  0.0009765625 * 3, 17.0, 18.0, 19.0, 0.9375, 0.96875], dtype=np.float32)])
    enc_in = enc_in[np.abs(enc_in) <= 448]
    enc_out = enc_in.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    # seeded 64 x 256 NVFP4 case with fp64 result, built from the tables above only
    N, K, B = 64, 256, 3
    codes = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sc = np.abs(rng.standard_normal((N, K // 16)).astype(np.float32)) * np.float32(0.05)
    scales = sc.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    ts = np.float32(0.8125)
    x = rng.standard_normal((B, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
    nib = np.empty((N, K), dtype=np.uint8)
    nib[:, 0::2] = codes & 15
    nib[:, 1::2] = codes >> 4
    w = (prod[nib, np.repeat(scales, 16, axis=1)] * ts).astype(np.float32)
    y = x.astype(np.float64) @ w.astype(np.float64).T
    # FP8 case
    fcodes = rng.integers(0, 254, size=(32, 128), dtype=np.uint8)
    fcodes = np.where(fcodes >= 127, fcodes + 1, fcodes).astype(np.uint8)
    fs = (np.abs(rng.standard_normal(32)) * 0.02).astype(np.float32)
    fx = rng.standard_normal((2, 128)).astype(np.float32).astype(ml_dtypes.bfloat16)
    fw = (e4m3[fcodes] * fs[:, None]).astype(np.float32)
    fy = fx.astype(np.float64) @ fw.astype(np.float64).T
    np.savez_compressed(
        os.path.join(HERE, "qgemv_golden.npz"),
        e2m1=e2m1, e4m3=e4m3, nvfp4_prod=prod, bf16_kat_in=kat_in, bf16_kat_out=kat_out,
        e4m3_enc_in=enc_in, e4m3_enc_out=enc_out,
        codes=codes, scales=scales, ts=ts, x=x.view(np.uint16), w=w, y=y,
        fp8_codes=fcodes, fp8_scales=fs, fp8_x=fx.view(np.uint16), fp8_w=fw, fp8_y=fy)
    print("wrote", os.path.join(HERE, "qgemv_golden.npz"))


def main_skinny() -> None:
    """Seeded skinny-GEMM cases (several token rows, N a multiple of 128) with fp64 results, from the
    third-party codecs only; a file of its own so that the GEMV vectors above stay byte-identical."""
    e2m1 = np.arange(16, dtype=np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float64)
    e4m3 = np.arange(256, dtype=np.uint8).view(ml_dtypes.float8_e4m3fn).astype(np.float64)
    rng = np.random.Generator(np.random.Philox(20250319))
    out = {}
    for tag, (N, K, M) in {"a": (128, 192, 16), "b": (256, 256, 32)}.items():
        codes = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        sc = np.abs(rng.standard_normal((N, K // 16)).astype(np.float32)) * np.float32(0.05)
        scales = sc.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
        ts = np.float32(1.375)
        x = (rng.standard_normal((M, K)) * rng.choice([0.01, 1.0, 300.0], size=(M, 1))).astype(np.float32).astype(ml_dtypes.bfloat16)
        nib = np.empty((N, K), dtype=np.uint8)
        nib[:, 0::2] = codes & 15
        nib[:, 1::2] = codes >> 4
        w = (e2m1[nib] * e4m3[np.repeat(scales, 16, axis=1)]).astype(np.float32) * ts  # the dequantisation rule
        out.update({f"{tag}_codes": codes, f"{tag}_scales": scales, f"{tag}_ts": ts, f"{tag}_x": x.view(np.uint16),
                    f"{tag}_y": x.astype(np.float64) @ w.astype(np.float64).T})
    N, K, M = 128, 128, 16
    fcodes = rng.integers(0, 254, size=(N, K), dtype=np.uint8)
    fcodes = np.where(fcodes >= 127, fcodes + 1, fcodes).astype(np.uint8)
    fs = (np.abs(rng.standard_normal(N)) * 0.02).astype(np.float32)
    fx = rng.standard_normal((M, K)).astype(np.float32).astype(ml_dtypes.bfloat16)
    fw = (e4m3[fcodes].astype(np.float32) * fs[:, None]).astype(np.float32)
    out.update({"f_codes": fcodes, "f_scales": fs, "f_x": fx.view(np.uint16), "f_y": fx.astype(np.float64) @ fw.astype(np.float64).T})
    np.savez_compressed(os.path.join(HERE, "skinny_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "skinny_golden.npz"))


if __name__ == "__main__":
    main()
    main_skinny()
