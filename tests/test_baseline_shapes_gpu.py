"""Parity at the full sizes the benchmark configurations name, through the C ABI.

The whole matrix is packed, loaded and multiplied on the GPU; the fp64 oracle is evaluated on a
sample of output rows (first rows, a middle stripe, the ragged end) so that the CPU time stays in
seconds, and a size-independent property (a row's bits do not depend on the batch it is in) is
checked on all rows.
"""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 5e-5
TOL_BF16 = 2e-3


def _rows(N, count=96):
    c = count // 3
    return np.unique(np.concatenate([np.arange(c), np.arange(N // 2 - c // 2, N // 2 + c // 2), np.arange(N - c, N)]))


@pytest.mark.parametrize("fmt_name", ["lane", "tc"])
def test_nvfp4_gate_up_28672x4096(qg, handle, fmt_name):
    N, K = 28672, 4096
    codes, scales, ts = O.make_nvfp4(N, K, seed=28672, ts=0.8125)
    w = handle.load(qg.pack(qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4, codes, scales, ts))
    idx = _rows(N)
    x8 = O.make_x(8, K, seed=8)
    y8 = U.run_gemv(qg, handle, w, x8)
    U.status_ok(handle)
    assert not np.isnan(y8).any()
    assert O.rel_l2(y8[:, idx], O.gemv_nvfp4_f64(codes[idx], scales[idx], ts, x8)) < TOL_F32
    y1 = U.run_gemv(qg, handle, w, x8[:1])
    assert O.rel_l2(y1[:, idx], O.gemv_nvfp4_f64(codes[idx], scales[idx], ts, x8[:1])) < TOL_F32
    U.assert_bits_equal(y1[0], y8[0])   # a row's bits do not depend on the batch it is in (either layout)
    yb = U.run_gemv(qg, handle, w, x8[:1], out_f32=False)
    assert O.rel_l2(O.bf16_decode(yb)[:, idx], O.gemv_nvfp4_f64(codes[idx], scales[idx], ts, x8[:1])) < TOL_BF16
    assert np.array_equal(yb, O.bf16_encode(y1))
    w.unload()


@pytest.mark.parametrize("B", [1, 16])
def test_fp8_lm_head_128256x4096(qg, handle, B):
    import torch
    N, K = 128256, 4096
    codes, ch = O.make_fp8(N, K, seed=128256)
    w = handle.load(qg.pack(qg.FMT_FP8, codes, ch))
    x = O.make_x(B, K, seed=B)
    xd = U.dev_u16(x)
    y = torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda")     # fp32 logits
    handle.gemv(w, xd.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    idx = _rows(N, 192)
    assert O.rel_l2(got[:, idx], O.gemv_fp8_f64(codes[idx], ch[idx], x)) < TOL_F32
    w.unload()


@pytest.mark.parametrize("T", [1, 8, 64])
@pytest.mark.parametrize("fmt_name", ["lane", "tc"])
def test_moe_128_experts_top8(qg, handle, T, fmt_name):
    """128 experts, top-8: gate/up 1536 x 2048 on the tokens' rows, down 2048 x 768 on the slots' own rows.
    All experts are loaded; the experts of a handful of (token, choice) slots are checked in fp64."""
    import torch
    E, topk = 128, 8
    rng = np.random.Generator(np.random.Philox(T))
    ids = np.stack([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.int32)
    for (N, K, per_slot) in ((1536, 2048, False), (2048, 768, True)):
        mats = [O.make_nvfp4(N, K, seed=5000 + e, ts=0.5 + e / 256.0) for e in range(E)]
        fmt = qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4
        w = handle.load_stacked(np.stack([qg.pack(fmt, c, s, t) for c, s, t in mats]))
        rows = T * topk if per_slot else T
        x = O.make_x(rows, K, seed=T + N)
        out = torch.full((T * topk, N), float("nan"), dtype=torch.float32, device="cuda")
        idd, xd = torch.from_numpy(ids).cuda(), U.dev_u16(x)      # kept alive until the kernel has run
        handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, per_slot, out.data_ptr(), qg.OUT_F32)
        torch.cuda.synchronize()
        U.status_ok(handle)
        got = out.cpu().numpy()
        assert not np.isnan(got).any()
        slots = sorted({0, T * topk - 1} | {int(s) for s in rng.integers(0, T * topk, size=6)})
        for s in slots:
            t, e = s // topk, int(ids[s // topk, s % topk])
            c, sc, ts = mats[e]
            xin = x[s:s + 1] if per_slot else x[t:t + 1]
            assert O.rel_l2(got[s], O.gemv_nvfp4_f64(c, sc, ts, xin)[0]) < TOL_F32, (N, s)
        w.unload()


@pytest.mark.parametrize("N,K,shard", [(1280, 8192, "rows"), (8192, 1024, "cols"), (7168, 8192, "rows"), (8192, 3584, "cols")])
@pytest.mark.parametrize("fmt_name", ["lane", "tc"])
def test_tp8_shard_shapes(qg, handle, N, K, shard, fmt_name):
    """The per-rank matrices of the 70B-shaped stack at 8 ranks, cut by the shard-aware packer from a
    canonical matrix twice their size (rank 1's share), batch 1."""
    fmt = qg.FMT_NVFP4_TC if fmt_name == "tc" else qg.FMT_NVFP4
    if shard == "rows":
        codes, scales, ts = O.make_nvfp4(2 * N, K, seed=N + K, ts=0.75)
        sh = qg.Shard(N, 2 * N, 0, K)
        cs, ss = codes[N:], scales[N:]
    else:
        codes, scales, ts = O.make_nvfp4(N, 2 * K, seed=N + K, ts=0.75)
        sh = qg.Shard(0, N, K, 2 * K)
        cs, ss = np.ascontiguousarray(codes[:, K // 2:]), np.ascontiguousarray(scales[:, K // 16:])
    w = handle.load(qg.pack(fmt, codes, scales, ts, shard=sh))
    assert (w.N, w.K) == (N, K)
    x = O.make_x(1, K, seed=K)
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    assert O.rel_l2(y, O.gemv_nvfp4_f64(cs, ss, ts, x)) < TOL_F32
    w.unload()


@pytest.mark.parametrize("N,K,M", [(10240, 8192, 128), (8192, 8192, 256)])
def test_skinny_gemm_70b_shapes(qg, handle, N, K, M):
    import torch
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + M, ts=0.625)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    x = O.make_x(M, K, seed=M)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    xd = U.dev_u16(x)
    handle.gemm_skinny(w, xd.data_ptr(), M, y.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    idx = _rows(N, 48)
    assert O.rel_l2(got[:, idx], O.gemv_nvfp4_f64(codes[idx], scales[idx], ts, x)) < TOL_F32
    w.unload()
