"""The allocation-free GEMV entry point (collected last on purpose).

`qgemv_gemv_noalloc` is for callers that cannot allocate device memory at call time (code inside a
pool that owns the GPU, plugins restricted to the buffers they were given, latency-critical
paths).  It takes the caller's device copy of a packed blob and keeps its own scratch in a static
array inside the library.  The test calls it through the C ABI twice in a row and compares each
result with the regular entry point's, and with the oracle.
"""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 5e-5  # same bound as the other GPU parity tests (relative L2 against the fp64 oracle)


@pytest.mark.parametrize("N,K,B", [(1024, 4096, 1), (6144, 4096, 3), (272, 2112, 8)])
def test_noalloc_matches_regular_entry_point(qg, handle, N, K, B):
    import torch
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + B, ts=0.75)
    blob = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    x = O.make_x(B, K, seed=K + B)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    # regular entry point
    w = handle.load(blob)
    y_regular = U.run_gemv(qg, handle, w, x)
    # allocation-free entry point: the blob lives in a buffer owned by the caller (torch here)
    dev_blob = torch.from_numpy(blob).cuda()
    xd = U.dev_u16(x)
    for call in range(2):  # the static scratch keeps the previous call's contents
        y = torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda")
        qg.gemv_noalloc(dev_blob.data_ptr(), blob, xd.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert not np.isnan(got).any(), call
        assert O.rel_l2(got, ref) < TOL_F32, call
        assert O.rel_l2(got, y_regular) < TOL_F32, call
        if call == 0:
            first = got
        else:
            assert np.array_equal(U.bits(got), U.bits(first))
        st = qg.noalloc_last_status()
        assert st.code == 0, st
    w.unload()


@pytest.mark.parametrize("N,K,B", [(512, 4608, 7), (512, 4160, 7), (512, 5184, 6), (512, 6208, 5), (256, 10304, 3)])
def test_noalloc_ragged_k_edge(qg, N, K, B):
    """Shapes with units * B <= 512 but more than 32 (phase, row) pairs: beyond what the activation
    staging holds, so the entry point must refuse them instead of computing with unstaged rows."""
    import torch
    codes, scales, ts = O.make_nvfp4(N, K, seed=K + B)
    blob = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    dev_blob = torch.from_numpy(blob).cuda()
    x = torch.zeros(B * K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(B * N, dtype=torch.float32, device="cuda")
    with pytest.raises(qg.QgemvError) as e:
        qg.gemv_noalloc(dev_blob.data_ptr(), blob, x.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    # one row fewer fits: results match the oracle
    Bf = B - 1 if (K + 1023) // 1024 * (B - 1) <= 32 else 1
    xf = O.make_x(Bf, K, seed=3)
    yf = torch.full((Bf, N), float("nan"), dtype=torch.float32, device="cuda")
    qg.gemv_noalloc(dev_blob.data_ptr(), blob, U.dev_u16(xf).data_ptr(), Bf, yf.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    assert O.rel_l2(yf.cpu().numpy(), O.gemv_nvfp4_f64(codes, scales, ts, xf)) < TOL_F32


def test_noalloc_fp8_and_bf16_output(qg, handle):
    import torch
    codes, scales = O.make_fp8(512, 1024, seed=5)
    blob = qg.pack(qg.FMT_FP8, codes, scales)
    x = O.make_x(2, 1024, seed=6)
    ref = O.gemv_fp8_f64(codes, scales, x)
    dev_blob = torch.from_numpy(blob).cuda()
    xd = U.dev_u16(x)
    y = torch.zeros((2, 512), dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        qg.gemv_noalloc(dev_blob.data_ptr(), blob, xd.data_ptr(), 2, y.data_ptr(), qg.OUT_BF16)
    torch.cuda.synchronize()
    assert O.rel_l2(y.float().cpu().numpy(), ref) < 2e-3


def test_noalloc_rejects_sizes_beyond_its_scratch(qg):
    import torch
    codes, scales, ts = O.make_nvfp4(16, 8192, seed=1)
    blob = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    dev_blob = torch.from_numpy(blob).cuda()
    x = torch.zeros(8 * 8192, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(8 * 16, dtype=torch.float32, device="cuda")
    with pytest.raises(qg.QgemvError) as e:   # ceil(K / 1024) * B = 64 phases-times-rows, above 32
        qg.gemv_noalloc(dev_blob.data_ptr(), blob, x.data_ptr(), 8, y.data_ptr(), qg.OUT_F32)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    big = blob.copy()
    big[16:24] = np.frombuffer(np.int64(16 * 20000).tobytes(), dtype=np.uint8)       # N
    big[32:40] = np.frombuffer(np.int64(20000).tobytes(), dtype=np.uint8)            # n_panels > 16384
    with pytest.raises(qg.QgemvError) as e:
        qg.gemv_noalloc(dev_blob.data_ptr(), big, x.data_ptr(), 1, y.data_ptr(), qg.OUT_F32)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    bad = blob.copy()
    bad[0] ^= 1
    with pytest.raises(qg.QgemvError) as e:
        qg.gemv_noalloc(dev_blob.data_ptr(), bad, x.data_ptr(), 1, y.data_ptr(), qg.OUT_F32)
    assert e.value.status == qg.ERR_BAD_BLOB
    # a header whose aux / payload sizes do not follow from its format and shape is refused
    hd = np.frombuffer(blob[:256].tobytes(), dtype=np.uint8).copy()
    for off in (64, 72):   # aux_bytes, payload_bytes
        stale = blob.copy()
        stale[off:off + 8] = np.frombuffer(np.uint64(int(np.frombuffer(hd[off:off + 8].tobytes(), dtype=np.uint64)[0]) + 576).tobytes(), dtype=np.uint8)
        with pytest.raises(qg.QgemvError) as e:
            qg.gemv_noalloc(dev_blob.data_ptr(), stale, x.data_ptr(), 1, y.data_ptr(), qg.OUT_F32)
        assert e.value.status == qg.ERR_BAD_BLOB, off
