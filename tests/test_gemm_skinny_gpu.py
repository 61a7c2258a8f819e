"""GPU parity of the tcgen05 skinny GEMM (Y[M][N] = X[M][K] dequant(W)^T, M = 16..256) against the
fp64 CPU oracle on the same seeded inputs; every call goes through the C ABI."""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 5e-5   # fp32 accumulation in tensor memory vs the fp64 oracle (relative L2)
TOL_BF16 = 2e-3  # stated bound for bf16 outputs (relative L2)


def run_skinny(qg, handle, w, x_bf16, out_f32=True):
    import torch
    M = x_bf16.shape[0]
    xd = U.dev_u16(x_bf16)
    dt = torch.float32 if out_f32 else torch.bfloat16
    yd = torch.full((M, w.N), float("nan"), dtype=dt, device="cuda")
    handle.gemm_skinny(w, xd.data_ptr(), M, yd.data_ptr(), qg.OUT_F32 if out_f32 else qg.OUT_BF16)
    torch.cuda.synchronize()
    if out_f32:
        return yd.cpu().numpy()
    return yd.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("N,K,M", [(128, 64, 16), (128, 256, 16), (256, 512, 64), (384, 1088, 48),
                                   (1024, 4096, 128), (256, 2048, 256), (2048, 8192, 32), (128, 36864, 16)])
def test_skinny_nvfp4(qg, handle, N, K, M):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K + M, ts=0.75)
    x = O.make_x(M, K, seed=M + K)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y32 = run_skinny(qg, handle, w, x)
    U.status_ok(handle)
    assert not np.isnan(y32).any()
    assert O.rel_l2(y32, ref) < TOL_F32
    y16 = run_skinny(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    assert O.rel_l2(O.bf16_decode(y16), ref) < TOL_BF16
    assert np.array_equal(y16, O.bf16_encode(y32))  # the bf16 output is the fp32 result rounded once
    w.unload()


def test_skinny_golden_fixture(qg, handle):
    """Against the committed vectors made from third-party codecs, not from the oracle."""
    import os
    S = np.load(os.path.join(os.path.dirname(__file__), "golden", "skinny_golden.npz"))
    for t in "ab":
        w = handle.load(qg.pack(qg.FMT_NVFP4, S[f"{t}_codes"], S[f"{t}_scales"], float(S[f"{t}_ts"])))
        y = run_skinny(qg, handle, w, S[f"{t}_x"])
        U.status_ok(handle)
        assert O.rel_l2(y, S[f"{t}_y"]) < TOL_F32
        w.unload()
    w = handle.load(qg.pack(qg.FMT_FP8, S["f_codes"], S["f_scales"]))
    y = run_skinny(qg, handle, w, S["f_x"])
    assert O.rel_l2(y, S["f_y"]) < TOL_F32
    w.unload()


@pytest.mark.parametrize("N,K,M", [(128, 128, 16), (512, 1024, 80), (256, 4096, 256)])
def test_skinny_fp8(qg, handle, N, K, M):
    codes, scales = O.make_fp8(N, K, seed=N + K)
    x = O.make_x(M, K, seed=M)
    ref = O.gemv_fp8_f64(codes, scales, x)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, scales))
    y32 = run_skinny(qg, handle, w, x)
    U.status_ok(handle)
    assert O.rel_l2(y32, ref) < TOL_F32
    w.unload()


def test_skinny_rows_independent_and_deterministic(qg, handle):
    """A token row's result depends on no other row (per-row scaling, one accumulator column per
    token), and a repeat gives the same bits."""
    N, K = 512, 2048
    codes, scales, ts = O.make_nvfp4(N, K, seed=9)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = O.make_x(64, K, seed=4)
    y = run_skinny(qg, handle, w, x)
    assert np.array_equal(U.bits(y), U.bits(run_skinny(qg, handle, w, x)))
    x2 = x.copy()
    x2[1::2] = O.make_x(32, K, seed=77)            # replace every other token
    y2 = run_skinny(qg, handle, w, x2)
    assert np.array_equal(U.bits(y[0::2]), U.bits(y2[0::2]))
    y3 = run_skinny(qg, handle, w, x[:16])          # fewer tokens: same bits for the ones kept
    assert np.array_equal(U.bits(y[:16]), U.bits(y3))
    U.status_ok(handle)
    w.unload()


def test_skinny_matches_gemv(qg, handle):
    """Same weights, same tokens: the tensor-memory path and the decode GEMV agree to fp32 rounding."""
    N, K = 1024, 4096
    codes, scales, ts = O.make_nvfp4(N, K, seed=5, ts=1.5)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = O.make_x(16, K, seed=6)
    ys = run_skinny(qg, handle, w, x)
    yg = U.run_gemv(qg, handle, w, x[:8])
    assert O.rel_l2(ys[:8], yg) < 2e-6
    w.unload()


def test_skinny_activation_ranges(qg, handle):
    """Rows of very different magnitude (per-row power-of-two scaling), a zero row, tiny values."""
    N, K, M = 256, 1024, 32
    codes, scales, ts = O.make_nvfp4(N, K, seed=12)
    xf = O.bf16_decode(O.make_x(M, K, seed=3)).astype(np.float64)
    mags = np.array([2.0 ** e for e in np.linspace(-60, 60, M)])
    xf *= mags[:, None]
    xf[5] = 0.0
    x = O.bf16_encode(xf.astype(np.float32))
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = run_skinny(qg, handle, w, x)
    U.status_ok(handle)
    assert np.all(y[5] == 0.0)
    for m in range(M):
        if m != 5:
            assert O.rel_l2(y[m:m + 1], ref[m:m + 1]) < TOL_F32, m
    w.unload()


def test_skinny_bad_args(qg, handle):
    import torch
    codes, scales, ts = O.make_nvfp4(128, 128, seed=1)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = torch.zeros((256, 128), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((256, 128), dtype=torch.float32, device="cuda")
    for M in (0, 8, 24, 272):
        with pytest.raises(qg.QgemvError):
            handle.gemm_skinny(w, x.data_ptr(), M, y.data_ptr(), qg.OUT_F32)
    with pytest.raises(qg.QgemvError):  # activation-quantising modes are a different operator
        handle.gemm_skinny(w, x.data_ptr(), 16, y.data_ptr(), qg.OUT_F32, act_mode=1)
    w.unload()
    codes, scales, ts = O.make_nvfp4(64, 128, seed=1)  # N not a multiple of 128
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    with pytest.raises(qg.QgemvError):
        handle.gemm_skinny(w, x.data_ptr(), 16, y.data_ptr(), qg.OUT_F32)
    w.unload()


def test_skinny_bounded_wait(qg):
    """With the producer told (from the host) to issue no copies, every role's wait runs out, the
    kernel records a timeout, releases its tensor memory and returns; the next call works."""
    import torch
    h = qg.QGemv(spin_limit=2000, inject_drop_copies=True)
    codes, scales, ts = O.make_nvfp4(256, 512, seed=2)
    w = h.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = O.make_x(32, 512, seed=2)
    xd = U.dev_u16(x)
    yd = torch.zeros((32, 256), dtype=torch.float32, device="cuda")
    h.gemm_skinny(w, xd.data_ptr(), 32, yd.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and st.where in (42, 44, 45, 46)
    w.unload()
    h.close()
    h2 = qg.QGemv()
    w = h2.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y = run_skinny(qg, h2, w, x)
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    U.status_ok(h2)
    w.unload()
    h2.close()
