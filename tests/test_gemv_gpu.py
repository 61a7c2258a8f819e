"""GPU parity tests proper: every call goes through the C ABI to the sm_100a kernels and is
compared with the CPU oracle on the same seeded inputs."""
import os

import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qgemv_golden.npz"))

TOL_F32 = 5e-5   # fp32 accumulation on the tensor cores vs the fp64 oracle (relative L2)
TOL_BF16 = 2e-3  # the stated bound for bf16 outputs (relative L2)


# ---- dequantisation: bit exact ----------------------------------------------------------------
def test_dequant_nvfp4_exhaustive(qg, handle):
    """All 16 codes x all 256 scale bytes, through the kernel's cvt + f16x2 multiply."""
    N = 256
    nib = np.tile(np.arange(16, dtype=np.uint8), (N, 1))
    codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    scales = np.arange(256, dtype=np.uint8).reshape(N, 1)
    for ts in (1.0, 0.3):
        w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
        U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_nvfp4(codes, scales, ts))
        w.unload()
    U.assert_bits_equal(O.dequant_nvfp4(codes, scales, 1.0), G["nvfp4_prod"].T)


@pytest.mark.parametrize("N,K", [(64, 256), (100, 448), (4096, 4096), (17, 1040)])
def test_dequant_nvfp4_random(qg, handle, N, K):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K, ts=0.8125)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_nvfp4(codes, scales, ts))
    w.unload()


def test_dequant_fp8_exhaustive(qg, handle):
    codes = np.tile(np.arange(256, dtype=np.uint8), (32, 1))
    scales = (np.abs(np.random.default_rng(3).standard_normal(32)) * 0.02).astype(np.float32)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, scales))
    U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_fp8(codes, scales))
    w.unload()


def test_dequant_golden_fixture(qg, handle):
    w = handle.load(qg.pack(qg.FMT_NVFP4, G["codes"], G["scales"], float(G["ts"])))
    U.assert_bits_equal(U.dequant(qg, handle, w), G["w"])
    w.unload()
    w = handle.load(qg.pack(qg.FMT_FP8, G["fp8_codes"], G["fp8_scales"]))
    U.assert_bits_equal(U.dequant(qg, handle, w), G["fp8_w"])
    w.unload()


# ---- GEMV parity --------------------------------------------------------------------------------
def test_golden_gemv(qg, handle):
    w = handle.load(qg.pack(qg.FMT_NVFP4, G["codes"], G["scales"], float(G["ts"])))
    y = U.run_gemv(qg, handle, w, G["x"])
    U.status_ok(handle)
    assert O.rel_l2(y, G["y"]) < TOL_F32
    w.unload()
    w = handle.load(qg.pack(qg.FMT_FP8, G["fp8_codes"], G["fp8_scales"]))
    y = U.run_gemv(qg, handle, w, G["fp8_x"])
    U.status_ok(handle)
    assert O.rel_l2(y, G["fp8_y"]) < TOL_F32
    w.unload()


def test_config0(qg, handle):
    """BASELINE configs[0]: 4096 x 4096 NVFP4, batch 1, bf16 output, tensor scale 1."""
    codes, scales, ts = O.make_nvfp4(4096, 4096, seed=1)
    x = O.make_x(1, 4096, seed=1)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y32 = U.run_gemv(qg, handle, w, x, out_f32=True)
    y16 = U.run_gemv(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    assert O.rel_l2(y32, ref) < TOL_F32
    assert O.rel_l2(O.bf16_decode(y16), ref) < TOL_BF16
    # the bf16 output is the fp32 result rounded once
    assert np.array_equal(y16, O.bf16_encode(y32))
    w.unload()


@pytest.mark.parametrize("N,K", [(16, 64), (48, 1024), (100, 448), (33, 1104), (1000, 2112), (6144, 4096),
                                 (4096, 14336), (272, 16)])
@pytest.mark.parametrize("B", [1, 2, 3, 8])
def test_gemv_nvfp4_shapes(qg, handle, N, K, B):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N * 3 + K, ts=1.25)
    x = O.make_x(B, K, seed=B + K)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    assert not np.isnan(y).any()
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    w.unload()


@pytest.mark.parametrize("N,K,B", [(4096, 14336, 8), (4096, 14336, 3), (8192, 8192, 5), (8192, 28672, 8),
                                   (3000, 9280, 7), (2400, 4160, 8)])
def test_gemv_k_chunked(qg, handle, N, K, B):
    """Activations too large to stage at once: the call becomes several launches over K chunks whose
    panel sums run through an fp32 scratch; bf16 output is rounded once, at the last chunk."""
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K + B, ts=0.9)
    x = O.make_x(B, K, seed=B * 7 + 1)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y32 = U.run_gemv(qg, handle, w, x)
    y16 = U.run_gemv(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    assert O.rel_l2(y32, ref) < TOL_F32
    assert np.array_equal(y16, O.bf16_encode(y32))
    assert np.array_equal(U.bits(y32), U.bits(U.run_gemv(qg, handle, w, x)))  # deterministic
    w.unload()


# Ragged K where units * B <= 512 but ceil(K / 1024) * B exceeds the 32 (phase, row) pairs the
# activation staging of the streaming kernels holds, and the nearest shapes on the other side of
# that edge.  Default schedule, the always-split streaming kernel (bit 9) and both formats.
_EDGE = [(512, 4608, 7), (512, 4160, 7), (512, 5184, 6), (512, 5376, 6), (512, 6208, 5), (512, 6400, 5),
         (256, 10304, 3), (256, 10752, 3),
         (512, 4096, 7), (512, 4096, 8), (512, 5120, 6), (512, 6144, 5), (256, 10240, 3), (4096, 4608, 7)]


@pytest.mark.parametrize("N,K,B", _EDGE)
@pytest.mark.parametrize("bits", [0, 512])
def test_gemv_activation_staging_edge(qg, handle, N, K, B, bits):
    h = handle if bits == 0 else qg.QGemv(debug_bits=bits, debug=True)
    x = O.make_x(B, K, seed=K + B)
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K + B, ts=0.75)
    w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    for b in range(B):  # per row: an unstaged row would hide in a whole-matrix norm
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, (b, N, K, B)
    w.unload()
    codes8, scales8 = O.make_fp8(N, K, seed=N + K + B)
    w = h.load(qg.pack(qg.FMT_FP8, codes8, scales8))
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    ref = O.gemv_fp8_f64(codes8, scales8, x)
    for b in range(B):
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, (b, N, K, B)
    w.unload()
    if bits:
        h.close()


def test_gemv_k_chunked_fp8(qg, handle):
    N, K, B = 4096, 8192, 8
    codes, scales = O.make_fp8(N, K, seed=5)
    x = O.make_x(B, K, seed=6)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, scales))
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    assert O.rel_l2(y, O.gemv_fp8_f64(codes, scales, x)) < TOL_F32
    w.unload()


@pytest.mark.parametrize("bits", [256, 512])
@pytest.mark.parametrize("fmt", ["nvfp4", "fp8"])
def test_gemv_schedule_overrides(qg, bits, fmt):
    """The general ring kernel (bit 8) and the always-split streaming kernel (bit 9) on shapes the
    default schedule would give to the whole-panel kernel: same oracle, same tolerance."""
    h = qg.QGemv(debug_bits=bits, debug=True)
    for (N, K, B) in [(4096, 4096, 1), (6144, 2048, 3), (1000, 2112, 8)]:
        x = O.make_x(B, K, seed=N + B)
        if fmt == "nvfp4":
            codes, scales, ts = O.make_nvfp4(N, K, seed=N + K, ts=0.5)
            w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
            ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
        else:
            codes, scales = O.make_fp8(N, K, seed=N + K)
            w = h.load(qg.pack(qg.FMT_FP8, codes, scales))
            ref = O.gemv_fp8_f64(codes, scales, x)
        y = U.run_gemv(qg, h, w, x, h=h)
        U.status_ok(h)
        assert O.rel_l2(y, ref) < TOL_F32, (N, K, B)
        w.unload()
    h.close()


@pytest.mark.parametrize("N,K,B", [(64, 128, 1), (4096, 4096, 4), (500, 1344, 8), (28672, 4096, 1)])
def test_gemv_fp8_shapes(qg, handle, N, K, B):
    codes, scales = O.make_fp8(N, K, seed=N + K)
    x = O.make_x(B, K, seed=B)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, scales))
    y32 = U.run_gemv(qg, handle, w, x)
    y16 = U.run_gemv(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    ref = O.gemv_fp8_f64(codes, scales, x)
    assert O.rel_l2(y32, ref) < TOL_F32
    assert O.rel_l2(O.bf16_decode(y16), ref) < TOL_BF16
    w.unload()


def test_column_invariance_and_determinism(qg, handle):
    """Row b of the result has the same bits whatever the batch is, and from run to run."""
    N, K = 1024, 4096
    codes, scales, ts = O.make_nvfp4(N, K, seed=11)
    x = O.make_x(8, K, seed=12)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y8 = U.run_gemv(qg, handle, w, x)
    assert np.array_equal(U.bits(y8), U.bits(U.run_gemv(qg, handle, w, x)))
    for B in (1, 2, 5):
        yb = U.run_gemv(qg, handle, w, x[:B])
        assert np.array_equal(U.bits(yb), U.bits(y8[:B]))
    # a single row placed anywhere gives the same bits
    y1 = U.run_gemv(qg, handle, w, x[3:4])
    assert np.array_equal(U.bits(y1[0]), U.bits(y8[3]))
    U.status_ok(handle)
    w.unload()


@pytest.mark.parametrize("grid", [1, 3, 37, 148, 296])
def test_k_split_across_ctas(qg, grid):
    """Different CTA counts move the K split; every split sums its parts in a fixed order."""
    h = qg.QGemv(device=0, grid_override=grid, debug=True)
    N, K = 160, 4288
    codes, scales, ts = O.make_nvfp4(N, K, seed=grid)
    x = O.make_x(4, K, seed=grid + 1)
    w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    assert O.rel_l2(y, ref) < TOL_F32
    # the workspace counters are back to zero: a second launch gives the same bits
    assert np.array_equal(U.bits(y), U.bits(U.run_gemv(qg, h, w, x, h=h)))
    w.unload()
    h.close()


def test_activation_ranges(qg, handle):
    """Huge, tiny, zero and mixed-magnitude activation rows: the per-row power-of-two scaling of
    the f16 fragments is exact, so the tolerance does not move."""
    N, K = 256, 2048
    codes, scales, ts = O.make_nvfp4(N, K, seed=21)
    rng = np.random.default_rng(22)
    base = rng.standard_normal((6, K)).astype(np.float32)
    base[0] *= 1e30
    base[1] *= 1e-30
    base[2] = 0.0
    base[3, : K // 2] *= 1e4      # phases with very different maxima
    base[3, K // 2:] *= 1e-4
    base[4, 5] = 1e37
    base[5] *= 70000.0            # beyond the f16 range before scaling
    x = O.bf16_encode(base)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    assert np.isfinite(y).all()
    for b in range(6):
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, b
    assert not y[2].any()
    w.unload()


def test_lm_head_batch_16(qg, handle):
    """Rows 9..16 of one call run as a second launch: FP8 head with fp32 logits, 16 rows."""
    N, K, B = 4000, 1024, 16
    codes, scales = O.make_fp8(N, K, seed=8)
    x = O.make_x(B, K, seed=9)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, scales))
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    assert O.rel_l2(y, O.gemv_fp8_f64(codes, scales, x)) < TOL_F32
    y11 = U.run_gemv(qg, handle, w, x[:11])
    assert np.array_equal(U.bits(y[:11]), U.bits(y11))
    w.unload()


def test_bad_arguments(qg, handle):
    codes, scales, ts = O.make_nvfp4(16, 64, seed=1)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    import torch
    x = torch.zeros(17 * 64, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(17 * 16, dtype=torch.float32, device="cuda")
    for B in (0, 17, -1):
        with pytest.raises(qg.QgemvError) as e:
            handle.gemv(w, x.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
        assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    with pytest.raises(qg.QgemvError):
        handle.gemv(w, 0, 1, y.data_ptr(), qg.OUT_F32)
    with pytest.raises(qg.QgemvError):
        handle.gemv(w, x.data_ptr() + 2, 1, y.data_ptr(), qg.OUT_F32)  # misaligned activations
    bad = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    bad[400] ^= 1
    with pytest.raises(qg.QgemvError) as e:
        handle.load(bad)
    assert e.value.status == qg.ERR_BAD_BLOB
    w.unload()


def test_bounded_wait_reports_timeout(qg):
    """A wait on a barrier that nothing completes ends the kernel with a status word instead of
    hanging: the host-set injection makes the producer issue no copy, so the consumers' wait on
    the first stage runs out of its (small) poll budget."""
    h = qg.QGemv(device=0, spin_limit=2000, inject_drop_copies=True)
    codes, scales, ts = O.make_nvfp4(512, 4096, seed=5)
    w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = O.make_x(1, 4096, seed=5)
    U.run_gemv(qg, h, w, x, h=h)
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and st.where in (1, 3, 4, 5, 6, 7)
    assert h.device_status().code == 0  # reading clears it
    w.unload()
    h.close()
    # the context is still usable
    h2 = qg.QGemv(device=0)
    w2 = h2.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = U.run_gemv(qg, h2, w2, x, h=h2)
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    w2.unload()
    h2.close()


# ---- MoE ------------------------------------------------------------------------------------------
def _experts(E, N, K, seed):
    cs = [O.make_nvfp4(N, K, seed + e, ts=1.0 + (e % 5) / 8) for e in range(E)]
    return (np.stack([c[0] for c in cs]), np.stack([c[1] for c in cs]),
            np.array([c[2] for c in cs], dtype=np.float32))


def _route(T, E, topk, seed):
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    ids = np.argsort(-p, axis=1, kind="stable")[:, :topk].astype(np.int32)
    wts = np.take_along_axis(p, ids, axis=1)
    wts = (wts / wts.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, wts


@pytest.mark.parametrize("T", [1, 3, 8, 64])
@pytest.mark.parametrize("per_slot", [False, True])
@pytest.mark.parametrize("fmt_name", ["lane", "tc"])
def test_moe_gemv(qg, handle, T, per_slot, fmt_name):
    """Both layouts: the lane-order experts on the streaming kernel, the tensor-core layout as an expert list of
    the sequence kernel (T = 64 gives experts with more than eight rows, i.e. two problems)."""
    import torch
    E, topk = 32, 4
    N, K = (96, 256) if not per_slot else (128, 192)
    fmt = qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4
    codes, scales, ts = _experts(E, N, K, seed=300)
    blobs = np.stack([qg.pack(fmt, codes[e], scales[e], float(ts[e])) for e in range(E)])
    w = handle.load_stacked(blobs)
    ids, wts = _route(T, E, topk, seed=T)
    rows = T * topk if per_slot else T
    x = O.make_x(rows, K, seed=T + 1)
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=per_slot)
    xd = U.dev_u16(x)
    idd = torch.from_numpy(ids).cuda()
    out = torch.full((T * topk, N), float("nan"), dtype=torch.float32, device="cuda")
    handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, per_slot, out.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    assert O.rel_l2(got, ref) < TOL_F32
    # weighted combine, fixed slot order
    wd = torch.from_numpy(wts).cuda()
    y = torch.empty((T, N), dtype=torch.float32, device="cuda")
    handle.moe_combine(out.data_ptr(), qg.OUT_F32, wd.data_ptr(), T, topk, N, y.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    yref = np.einsum("tj,tjn->tn", wts.astype(np.float64), ref.reshape(T, topk, N))
    assert O.rel_l2(y.cpu().numpy(), yref) < TOL_F32
    w.unload()


@pytest.mark.parametrize("fmt_name,K", [("lane", 4352), ("tc", 4352), ("tc", 7168)])
def test_moe_gemv_long_k(qg, handle, fmt_name, K):
    """Experts with K > 2048: lane order runs as K chunks of the streaming kernel, added in chunk order; the
    tensor-core layout holds the digit planes of the whole K, for fewer rows at a time when K is very long
    (7168: four rows, so the experts with more entries make two problems)."""
    import torch
    E, topk, T, N = 16, 4, 8, 256
    fmt = qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4
    codes, scales, ts = _experts(E, N, K, seed=900)
    blobs = np.stack([qg.pack(fmt, codes[e], scales[e], float(ts[e])) for e in range(E)])
    w = handle.load_stacked(blobs)
    ids, _ = _route(T, E, topk, seed=5)
    x = O.make_x(T, K, seed=6)
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=False)
    xd = U.dev_u16(x)
    idd = torch.from_numpy(ids).cuda()
    for dt, tol in ((qg.OUT_F32, TOL_F32), (qg.OUT_BF16, TOL_BF16)):
        tdt = torch.float32 if dt == qg.OUT_F32 else torch.bfloat16
        out = torch.full((T * topk, N), float("nan"), dtype=tdt, device="cuda")
        handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), dt)
        torch.cuda.synchronize()
        U.status_ok(handle)
        got = out.float().cpu().numpy()
        assert not np.isnan(got).any()
        assert O.rel_l2(got, ref) < tol
    w.unload()


@pytest.mark.parametrize("fmt_name", ["lane", "tc"])
def test_moe_gemv_repeated_and_bad_ids(qg, handle, fmt_name):
    """A token that names the same expert twice gets two rows of that expert's problem; an id outside the stacked
    weight is reported in the status word (no result is written, nothing faults) and the next call is clean."""
    import torch
    E, topk, T, N, K = 8, 4, 2, 128, 128
    fmt = qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4
    codes, scales, ts = _experts(E, N, K, seed=77)
    w = handle.load_stacked(np.stack([qg.pack(fmt, codes[e], scales[e], float(ts[e])) for e in range(E)]))
    ids = np.array([[3, 3, 5, 3], [5, 0, 5, 7]], dtype=np.int32)      # three rows of expert 3 from ONE token: more rows than tokens
    x = O.make_x(T, K, seed=9)
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=False)
    xd, idd = U.dev_u16(x), torch.from_numpy(ids).cuda()
    out = torch.full((T * topk, N), float("nan"), dtype=torch.float32, device="cuda")
    handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    assert O.rel_l2(out.cpu().numpy(), ref) < TOL_F32
    bad = torch.from_numpy(np.array([[3, 1, 5, 2], [5, 0, E, 7]], dtype=np.int32)).cuda()
    handle.moe_gemv(w, bad.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    st = handle.device_status()
    assert st.code == qg.ERR_BOUNDS and st.where == 21
    out.fill_(float("nan"))
    handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    assert O.rel_l2(out.cpu().numpy(), ref) < TOL_F32
    w.unload()


@pytest.mark.parametrize("T", [1, 8, 64])
def test_moe_down_stage_with_silu_mul(qg, handle, T):
    """The experts' down stage fed with the gate/up stage's output rows: the launch multiplies bf16(silu(gate) * up) of
    rows that hold 2 K values (tensor-core layout); the lane-order layout refuses the option."""
    import torch
    E, topk, N, K = 32, 4, 256, 192
    codes, scales, ts = _experts(E, N, K, seed=611)
    w = handle.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, codes[e], scales[e], float(ts[e])) for e in range(E)]))
    ids, _ = _route(T, E, topk, seed=T + 9)
    gu = O.make_x(T * topk, 2 * K, seed=T + 10)           # per slot: K gate values, then K up values
    v = O.bf16_decode(gu).astype(np.float64)
    act = O.bf16_encode((v[:, :K] / (1.0 + np.exp(-v[:, :K])) * v[:, K:]).astype(np.float32))
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, act, per_slot_input=True)
    gd, idd = U.dev_u16(gu), torch.from_numpy(ids).cuda()
    out = torch.full((T * topk, N), float("nan"), dtype=torch.float32, device="cuda")
    handle.moe_gemv(w, idd.data_ptr(), gd.data_ptr(), T, topk, True, out.data_ptr(), qg.OUT_F32, x_act=qg.MOE_X_SILU_MUL)
    torch.cuda.synchronize()
    U.status_ok(handle)
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    assert O.rel_l2(got, ref) < 2e-4      # the device's fast exponential may round a bf16 product the other way
    w.unload()
    if T == 1:
        wl = handle.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4, codes[e], scales[e], float(ts[e])) for e in range(E)]))
        with pytest.raises(qg.QgemvError) as e:
            handle.moe_gemv(wl, idd.data_ptr(), gd.data_ptr(), T, topk, True, out.data_ptr(), qg.OUT_F32, x_act=qg.MOE_X_SILU_MUL)
        assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
        wl.unload()


@pytest.mark.parametrize("T", [1, 3, 8, 64])
def test_moe_mlp_one_launch(qg, handle, T):
    """Gate/up, silu(gate) * up and down of the routed experts as ONE launch: the same bits as the two launches it
    replaces (gate/up rows and results), and within the bound of the fp64 oracle fed with the device's gate/up rows."""
    import torch
    E, topk, H, I, N2 = 32, 4, 256, 128, 320
    cg, sg, tg = _experts(E, 2 * I, H, seed=801)
    cd, sd, td = _experts(E, N2, I, seed=802)
    wg = handle.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, cg[e], sg[e], float(tg[e])) for e in range(E)]))
    wd = handle.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, cd[e], sd[e], float(td[e])) for e in range(E)]))
    ids, _ = _route(T, E, topk, seed=T + 21)
    x = O.make_x(T, H, seed=T + 22)
    xd, idd = U.dev_u16(x), torch.from_numpy(ids).cuda()
    S = T * topk
    mid2 = torch.zeros((S, 2 * I), dtype=torch.bfloat16, device="cuda")
    out2 = torch.full((S, N2), float("nan"), dtype=torch.float32, device="cuda")
    handle.moe_gemv(wg, idd.data_ptr(), xd.data_ptr(), T, topk, False, mid2.data_ptr(), qg.OUT_BF16)
    handle.moe_gemv(wd, idd.data_ptr(), mid2.data_ptr(), T, topk, True, out2.data_ptr(), qg.OUT_F32, x_act=qg.MOE_X_SILU_MUL)
    torch.cuda.synchronize()
    U.status_ok(handle)
    for rep in range(2):      # twice: the stage counters are back at zero after a launch
        mid1 = torch.zeros((S, 2 * I), dtype=torch.bfloat16, device="cuda")
        out1 = torch.full((S, N2), float("nan"), dtype=torch.float32, device="cuda")
        handle.moe_mlp(wg, wd, idd.data_ptr(), xd.data_ptr(), T, topk, mid1.data_ptr(), out1.data_ptr(), qg.OUT_F32)
        torch.cuda.synchronize()
        U.status_ok(handle)
        assert torch.equal(mid1.view(torch.int16), mid2.view(torch.int16)), rep
        assert torch.equal(out1.view(torch.int32), out2.view(torch.int32)), rep
    v = mid2.float().cpu().numpy().astype(np.float64)
    act = O.bf16_encode((v[:, :I] / (1.0 + np.exp(-v[:, :I])) * v[:, I:]).astype(np.float32))
    ref = O.moe_gemv_nvfp4_f64(cd, sd, td, ids, act, per_slot_input=True)
    assert O.rel_l2(out1.cpu().numpy(), ref) < 5e-4
    refg = O.moe_gemv_nvfp4_f64(cg, sg, tg, ids, x, per_slot_input=False)
    assert O.rel_l2(v, refg) < TOL_BF16
    wg.unload()
    wd.unload()


def test_moe_mlp_bounded_waits(qg):
    """Host-set injection (no weight copy is ever issued): the waits of the one-launch expert MLP run out -- also the
    second stage's wait for the first stage's rows -- the status word says so, twice in a row (the counters of the
    abandoned launch are cleared with the status), and nothing hangs; a handle without the injection then computes."""
    import torch
    E, topk, T, H, I, N2 = 8, 2, 4, 128, 64, 128
    cg, sg, tg = _experts(E, 2 * I, H, seed=901)
    cd, sd, td = _experts(E, N2, I, seed=902)
    ids, _ = _route(T, E, topk, seed=31)
    x = O.make_x(T, H, seed=32)
    S = T * topk
    outs = []
    for inject in (True, False):
        h = qg.QGemv(device=0, spin_limit=2000, inject_drop_copies=inject)
        wg = h.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, cg[e], sg[e], float(tg[e])) for e in range(E)]))
        wd = h.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, cd[e], sd[e], float(td[e])) for e in range(E)]))
        xd, idd = U.dev_u16(x), torch.from_numpy(ids).cuda()
        mid = torch.zeros((S, 2 * I), dtype=torch.bfloat16, device="cuda")
        out = torch.zeros((S, N2), dtype=torch.float32, device="cuda")
        for _ in range(2):
            h.moe_mlp(wg, wd, idd.data_ptr(), xd.data_ptr(), T, topk, mid.data_ptr(), out.data_ptr(), qg.OUT_F32)
            torch.cuda.synchronize()
            st = h.device_status()
            if inject:
                assert st.code == qg.ERR_TIMEOUT and 71 <= st.where <= 86
            else:
                assert st.code == 0
        outs.append(out.cpu().numpy())
        wg.unload(), wd.unload()
        h.close()
    act_ref = O.moe_gemv_nvfp4_f64(cg, sg, tg, ids, x, per_slot_input=False)
    g = O.bf16_decode(O.bf16_encode(act_ref.astype(np.float32))).astype(np.float64)
    act = O.bf16_encode((g[:, :I] / (1.0 + np.exp(-g[:, :I])) * g[:, I:]).astype(np.float32))
    ref = O.moe_gemv_nvfp4_f64(cd, sd, td, ids, act, per_slot_input=True)
    assert O.rel_l2(outs[1], ref) < 5e-3    # (the oracle's own gate/up rows here: bf16 roundings may differ from the device's)


def test_moe_gemv_tc_many_experts_and_limits(qg, handle):
    """Tensor-core layout: 300 experts with top-1 routing (every problem a single row, most experts untouched), bf16
    output; a stacked weight of more than 512 experts is refused by the expert-list launch."""
    import torch
    E, topk, T, N, K = 300, 1, 40, 128, 64
    codes, scales, ts = _experts(E, N, K, seed=41)
    blob = [qg.pack(qg.FMT_NVFP4_TC, codes[e], scales[e], float(ts[e])) for e in range(E)]
    w = handle.load_stacked(np.stack(blob))
    rng = np.random.default_rng(3)
    ids = rng.integers(0, E, size=(T, topk)).astype(np.int32)
    x = O.make_x(T, K, seed=4)
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=False)
    xd, idd = U.dev_u16(x), torch.from_numpy(ids).cuda()
    out = torch.full((T * topk, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_BF16)
    torch.cuda.synchronize()
    U.status_ok(handle)
    got = out.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert O.rel_l2(got, ref) < TOL_BF16
    w.unload()
    big = handle.load_stacked(np.stack([blob[e % E] for e in range(513)]))
    with pytest.raises(qg.QgemvError) as e:
        handle.moe_gemv(big, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_BF16)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    big.unload()


# ---- tensor-parallel exchange ----------------------------------------------------------------------
def test_tp_allreduce_single_rank(qg):
    """World of one: the exchange degenerates to push-to-self, flag, reduce; replaying it checks
    the device-side epochs and the two parities."""
    import torch
    h = qg.QGemv(device=0)
    handle_bytes = h.tp_create(0, 1, 4096)
    h.tp_connect(handle_bytes.reshape(1, 64))
    y = torch.randn(1000, device="cuda", dtype=torch.float32)
    ref = y.clone()
    for _ in range(5):
        h.tp_allreduce(y.data_ptr(), qg.OUT_F32, y.numel())
    torch.cuda.synchronize()
    assert h.device_status().code == 0
    assert torch.equal(y, ref)
    yb = torch.randn(777, device="cuda").bfloat16()
    refb = yb.clone()
    h.tp_allreduce(yb.data_ptr(), qg.OUT_BF16, yb.numel())
    torch.cuda.synchronize()
    assert torch.equal(yb, refb)
    with pytest.raises(qg.QgemvError):
        h.tp_allreduce(y.data_ptr(), qg.OUT_F32, 5000)  # above max_elems
    h.close()


def _tp_worker(rank, world, port, q):
    import os
    import numpy as np
    import torch
    import torch.distributed as dist
    import crit_hub_b200 as qg
    from oracle import oracle as O
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, B = 512, 4096, 2
        codes, scales, ts = O.make_nvfp4(N, K, seed=9)
        x = O.make_x(B, K, seed=9)
        h = qg.QGemv(device=rank)
        mine = torch.from_numpy(h.tp_create(rank, world, B * N))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        h.tp_connect(torch.stack(gathered).numpy())
        dist.barrier()
        # row-parallel shard: this rank owns K/world input columns
        k0, k1 = rank * K // world, (rank + 1) * K // world
        w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=qg.Shard(0, N, k0, k1)))
        xd = torch.from_numpy(np.ascontiguousarray(x[:, k0:k1]).view(np.int16)).cuda()
        y = torch.empty((B, N), dtype=torch.float32, device="cuda")
        for _ in range(3):
            h.gemv(w, xd.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
            h.tp_allreduce(y.data_ptr(), qg.OUT_F32, y.numel())
        torch.cuda.synchronize()
        st = h.device_status()
        err = O.rel_l2(y.cpu().numpy(), O.gemv_nvfp4_f64(codes, scales, ts, x))
        q.put((rank, st.code, err, y.cpu().numpy().tobytes()))
        dist.barrier()  # leave only between steps, nothing in flight
    finally:
        dist.destroy_process_group()


def test_tp_allreduce_two_gpus(qg):
    """Row-parallel GEMV on two GPUs + peer-memory all-reduce equals the unsharded oracle, and
    both ranks hold the same bits."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, 29533, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    assert all(r[1] == 0 for r in res)
    assert all(r[2] < TOL_F32 for r in res)
    assert res[0][3] == res[1][3]
