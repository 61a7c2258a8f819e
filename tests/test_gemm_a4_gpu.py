"""The block-scaled prefill GEMM (activations quantised to NVFP4, both operands consumed as stored by
tcgen05.mma kind::mxf4nvf4), through the C ABI.

Parity has two parts.  The device quantiser is specified bit for bit and must reproduce the
oracle's codes, block scales and row scales EXACTLY.  The GEMM is then compared with an fp64 GEMM on
the same quantised activations (the stated bound is 2e-3; fp32 accumulation keeps it near 1e-6), and
the error against the unquantised oracle -- FP4's own quantisation error -- is checked to be what
that quantiser gives on the CPU too.
"""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_SAME_QUANTISER_F32 = 5e-5
TOL_BF16 = 2e-3


def _special_rows(M, K, seed):
    x = O.bf16_decode(O.make_x(M, K, seed=seed)).copy()
    x[0] = 0.0                                   # an all-zero row
    if M > 1:
        x[1, :64] = 0.0                          # zero blocks inside a row
        x[1, 64:80] *= 1e-4                      # a block far below the row maximum (its scale underflows)
    if M > 2:
        x[2] *= 3e4                              # large magnitudes
    if M > 3:
        x[3] *= 1e-20                            # tiny magnitudes
    if M > 4:
        x[4, 5] = -x[4].max() * 7.0              # one outlier sets the row scale
    return O.bf16_encode(x)


@pytest.mark.parametrize("M,K", [(16, 256), (48, 4096), (256, 8192), (5, 2112)])
def test_quantiser_matches_the_oracle_exactly(qg, handle, M, K):
    import torch
    x = _special_rows(M, K, seed=M + K)
    xd = U.dev_u16(x)
    codes = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda")
    scales = torch.zeros((M, K // 16), dtype=torch.uint8, device="cuda")
    g = torch.zeros((M,), dtype=torch.float32, device="cuda")
    handle.quantize_a4(xd.data_ptr(), M, K, codes.data_ptr(), scales.data_ptr(), g.data_ptr())
    torch.cuda.synchronize()
    rc, rs, rg = O.quantize_a4(x)
    assert np.array_equal(U.bits(g.cpu().numpy()), U.bits(rg))
    assert np.array_equal(scales.cpu().numpy(), rs)
    assert np.array_equal(codes.cpu().numpy(), rc)


def _run(qg, handle, w, x, out_f32=True):
    import torch
    M = x.shape[0]
    xd = U.dev_u16(x)
    y = torch.full((M, w.N), float("nan"), dtype=torch.float32 if out_f32 else torch.bfloat16, device="cuda")
    handle.gemm_skinny(w, xd.data_ptr(), M, y.data_ptr(), qg.OUT_F32 if out_f32 else qg.OUT_BF16, qg.ACT_A4_BLOCKSCALED)
    torch.cuda.synchronize()
    U.status_ok(handle)
    return y.float().cpu().numpy()


@pytest.mark.parametrize("N,K,M", [(128, 64, 16), (256, 1024, 32), (1000, 2112, 48), (4096, 4096, 128),
                                   (1024, 2048, 256), (512, 8192, 144), (8192, 1024, 256), (384, 14336, 64)])
def test_gemm_a4_against_the_same_quantiser(qg, handle, N, K, M):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K + M, ts=0.75)
    w = handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts))
    x = _special_rows(M, K, seed=M + N)
    xc, xs, g = O.quantize_a4(x)
    ref = O.gemm_nvfp4_a4_f64(codes, scales, ts, xc, xs, g)
    y = _run(qg, handle, w, x)
    assert not np.isnan(y).any()
    assert O.rel_l2(y, ref) < TOL_SAME_QUANTISER_F32
    yb = _run(qg, handle, w, x, out_f32=False)
    assert O.rel_l2(yb, ref) < TOL_BF16
    # against unquantised activations: FP4's quantisation error, the same as the CPU quantiser's
    exact = O.gemv_nvfp4_f64(codes, scales, ts, x)
    err_q = O.rel_l2(y, exact)
    assert abs(err_q - O.rel_l2(ref, exact)) < 1e-4 and err_q < 0.25
    # a second call gives the same bits (deterministic split)
    assert np.array_equal(U.bits(_run(qg, handle, w, x)), U.bits(y))
    w.unload()


def test_gemm_a4_refusals_and_timeout(qg, handle):
    import torch
    codes, scales, ts = O.make_nvfp4(256, 1024, seed=1)
    x = U.dev_u16(O.make_x(16, 1024, seed=1))
    y = torch.zeros((16, 256), dtype=torch.float32, device="cuda")
    w_lane = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    with pytest.raises(qg.QgemvError) as e:      # this mode consumes the tensor-core layout
        handle.gemm_skinny(w_lane, x.data_ptr(), 16, y.data_ptr(), qg.OUT_F32, qg.ACT_A4_BLOCKSCALED)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    w_tc = handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts))
    for bad in ((w_tc, 16, qg.ACT_A8), (w_tc, 24, qg.ACT_A4_BLOCKSCALED), (w_tc, 272, qg.ACT_A4_BLOCKSCALED)):
        with pytest.raises(qg.QgemvError) as e:
            handle.gemm_skinny(bad[0], x.data_ptr(), bad[1], y.data_ptr(), qg.OUT_F32, bad[2])
        assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    w_lane.unload()
    w_tc.unload()
    # host-set injection: no copy is ever issued, every wait runs out, the status word says where
    h = qg.QGemv(device=0, spin_limit=2000, inject_drop_copies=True)
    w = h.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts))
    h.gemm_skinny(w, x.data_ptr(), 16, y.data_ptr(), qg.OUT_F32, qg.ACT_A4_BLOCKSCALED)
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and 91 <= st.where <= 94, st
    h.close()
