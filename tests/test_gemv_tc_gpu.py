"""GPU parity tests of the tensor-core NVFP4 GEMV (QGEMV_FMT_NVFP4_TC): weights consumed as stored by
the block-scaled tcgen05.mma, activations as eight E2M1 digit planes.  Every call goes through the
C ABI and is compared with the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

# fp32 outputs against the fp64 oracle (relative L2).  The digit planes round an activation to
# 2^-16 of its row's largest magnitude (exact within 2^-8 of it), which moves the result by a few
# 1e-6 on N(0,1) rows; the bound is the one the CUDA-core path is held to.
TOL_F32 = 5e-5
TOL_BF16 = 2e-3  # the stated bound for bf16 outputs


def _load(qg, h, codes, scales, ts):
    return h.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts))


def test_dequant_tc_exhaustive(qg, handle):
    """All 16 codes x all 256 scale bytes laid out in the tensor-core order, read back bit-exact."""
    N = 256
    nib = np.tile(np.arange(16, dtype=np.uint8), (N, 1))
    codes = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    scales = np.arange(256, dtype=np.uint8).reshape(N, 1)
    for ts in (1.0, 0.3):
        w = _load(qg, handle, codes, scales, ts)
        U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_nvfp4(codes, scales, ts))
        w.unload()


@pytest.mark.parametrize("N,K", [(64, 256), (100, 448), (1024, 4096), (17, 1040), (300, 80)])
def test_dequant_tc_random(qg, handle, N, K):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K, ts=0.8125)
    w = _load(qg, handle, codes, scales, ts)
    U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_nvfp4(codes, scales, ts))
    w.unload()


def test_tc_config0(qg, handle):
    """BASELINE configs[0]: 4096 x 4096 NVFP4, batch 1, bf16 output, tensor scale 1."""
    codes, scales, ts = O.make_nvfp4(4096, 4096, seed=1)
    x = O.make_x(1, 4096, seed=1)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = _load(qg, handle, codes, scales, ts)
    y32 = U.run_gemv(qg, handle, w, x, out_f32=True)
    y16 = U.run_gemv(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    assert O.rel_l2(y32, ref) < TOL_F32
    assert O.rel_l2(O.bf16_decode(y16), ref) < TOL_BF16
    assert np.array_equal(y16, O.bf16_encode(y32))  # the bf16 output is the fp32 result rounded once
    w.unload()


@pytest.mark.parametrize("N,K", [(128, 64), (16, 64), (48, 1024), (100, 448), (33, 1104), (1000, 2112), (6144, 4096),
                                 (4096, 14336), (272, 16), (130, 4096)])
@pytest.mark.parametrize("B", [1, 2, 3, 8])
def test_tc_gemv_shapes(qg, handle, N, K, B):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N * 3 + K, ts=1.25)
    x = O.make_x(B, K, seed=B + K)
    w = _load(qg, handle, codes, scales, ts)
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    assert not np.isnan(y).any()
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    for b in range(B):
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, (b, N, K, B)
    w.unload()


def test_tc_matches_cuda_core_path(qg, handle):
    """The same canonical matrix through both stored forms gives the same result to rounding."""
    N, K, B = 768, 2048, 4
    codes, scales, ts = O.make_nvfp4(N, K, seed=77, ts=0.6)
    x = O.make_x(B, K, seed=78)
    w_tc = _load(qg, handle, codes, scales, ts)
    w_cc = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    y_tc = U.run_gemv(qg, handle, w_tc, x)
    y_cc = U.run_gemv(qg, handle, w_cc, x)
    U.status_ok(handle)
    assert O.rel_l2(y_tc, y_cc) < TOL_F32
    w_tc.unload()
    w_cc.unload()


def test_tc_column_invariance_and_determinism(qg, handle):
    """Row b of the result has the same bits whatever the batch is, and from run to run."""
    N, K = 1024, 4096
    codes, scales, ts = O.make_nvfp4(N, K, seed=11)
    x = O.make_x(8, K, seed=12)
    w = _load(qg, handle, codes, scales, ts)
    y8 = U.run_gemv(qg, handle, w, x)
    assert np.array_equal(U.bits(y8), U.bits(U.run_gemv(qg, handle, w, x)))
    for B in (1, 2, 5):
        yb = U.run_gemv(qg, handle, w, x[:B])
        assert np.array_equal(U.bits(yb), U.bits(y8[:B]))
    y1 = U.run_gemv(qg, handle, w, x[3:4])
    assert np.array_equal(U.bits(y1[0]), U.bits(y8[3]))
    U.status_ok(handle)
    w.unload()


@pytest.mark.parametrize("grid", [1, 3, 37, 148, 296])
def test_tc_k_split_across_ctas(qg, grid):
    """Different CTA counts move the K split; every split sums its parts in a fixed order."""
    h = qg.QGemv(device=0, grid_override=grid, debug=True)
    N, K = 300, 4288
    codes, scales, ts = O.make_nvfp4(N, K, seed=grid)
    x = O.make_x(4, K, seed=grid + 1)
    w = _load(qg, h, codes, scales, ts)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    assert O.rel_l2(y, ref) < TOL_F32
    # the arrival counters are back to zero: a second launch gives the same bits
    assert np.array_equal(U.bits(y), U.bits(U.run_gemv(qg, h, w, x, h=h)))
    w.unload()
    h.close()


@pytest.mark.parametrize("N,K,B", [(128, 4096, 1), (4096, 4096, 1), (6144, 4096, 3), (1000, 2112, 8), (300, 128, 2)])
def test_tc_cluster_handover(qg, N, K, B):
    """Debug bit 5: a thread-block cluster per row tile, partial sums through distributed shared memory."""
    h = qg.QGemv(device=0, debug_bits=32)
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K)
    x = O.make_x(B, K, seed=B)
    w = _load(qg, h, codes, scales, ts)
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    for b in range(B):
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, b
    assert np.array_equal(U.bits(y), U.bits(U.run_gemv(qg, h, w, x, h=h)))
    w.unload()
    h.close()


@pytest.mark.parametrize("stage_items,smem_kb", [(1, 0), (2, 64), (8, 227), (4, 227)])
def test_tc_ring_shapes(qg, stage_items, smem_kb):
    """Ring geometry is a tuning knob, never a result: same bits for every stage size and depth."""
    N, K, B = 640, 4160, 2
    codes, scales, ts = O.make_nvfp4(N, K, seed=5)
    x = O.make_x(B, K, seed=6)
    h0 = qg.QGemv(device=0)
    w0 = _load(qg, h0, codes, scales, ts)
    y0 = U.run_gemv(qg, h0, w0, x, h=h0)
    h = qg.QGemv(device=0, tc_stage_items=stage_items, tc_smem_kb=smem_kb)
    w = _load(qg, h, codes, scales, ts)
    y = U.run_gemv(qg, h, w, x, h=h)
    U.status_ok(h)
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    assert np.array_equal(U.bits(y), U.bits(y0))
    w.unload(), w0.unload()
    h.close(), h0.close()


@pytest.mark.parametrize("N,K,B", [(8192, 8192, 8), (4096, 14336, 8), (1024, 28672, 8), (57344, 8192, 5)])
def test_tc_large_activations(qg, handle, N, K, B):
    """Digit planes that need most of an SM's shared memory, or several launches over K chunks whose
    fp32 results are added in chunk order; bf16 output is rounded once."""
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K + B, ts=0.9)
    x = O.make_x(B, K, seed=B * 7 + 1)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    w = _load(qg, handle, codes, scales, ts)
    y32 = U.run_gemv(qg, handle, w, x)
    y16 = U.run_gemv(qg, handle, w, x, out_f32=False)
    U.status_ok(handle)
    assert O.rel_l2(y32, ref) < TOL_F32
    assert np.array_equal(y16, O.bf16_encode(y32))
    assert np.array_equal(U.bits(y32), U.bits(U.run_gemv(qg, handle, w, x)))
    w.unload()


def test_tc_activation_ranges(qg, handle):
    """Huge, tiny, zero and mixed-magnitude rows.  Rows whose elements all lie within 2^-8 of the row
    maximum are exact; an element far below its row's maximum is rounded to 2^-16 of that maximum,
    so those rows are held to an absolute bound relative to the row maximum."""
    N, K = 256, 2048
    codes, scales, ts = O.make_nvfp4(N, K, seed=21)
    rng = np.random.default_rng(22)
    base = rng.standard_normal((6, K)).astype(np.float32)
    base[0] *= 1e30
    base[1] *= 1e-30
    base[2] = 0.0
    base[3, : K // 2] *= 1e4
    base[3, K // 2:] *= 1e-4      # below 2^-16 of the row maximum: rounded away
    base[4, 5] = 1e37
    base[5] *= 70000.0
    x = O.bf16_encode(base)
    w = _load(qg, handle, codes, scales, ts)
    y = U.run_gemv(qg, handle, w, x)
    U.status_ok(handle)
    ref = O.gemv_nvfp4_f64(codes, scales, ts, x)
    assert np.isfinite(y).all()
    for b in (0, 1, 5):
        assert O.rel_l2(y[b], ref[b]) < TOL_F32, b
    assert not y[2].any()
    # rows 3 and 4: error bounded by 2^-17 of the row maximum per element, against the weights' L1 mass
    W = np.abs(O.dequant_nvfp4(codes, scales, ts).astype(np.float64))
    xm = np.abs(O.bf16_decode(x).astype(np.float64)).max(axis=1)
    for b in (3, 4):
        bound = W.sum(axis=1) * xm[b] * 2.0 ** -16
        assert (np.abs(y[b] - ref[b]) <= bound + 1e-6 * np.abs(ref[b])).all(), b
    w.unload()


def test_tc_bounded_wait_reports_timeout(qg):
    """Host-set injection: the producer issues no copy, the MMA issuer's wait on the first stage runs
    out of its small poll budget, the kernel reports and returns, and the context stays usable."""
    h = qg.QGemv(device=0, spin_limit=2000, inject_drop_copies=True)
    codes, scales, ts = O.make_nvfp4(512, 4096, seed=5)
    w = _load(qg, h, codes, scales, ts)
    x = O.make_x(1, 4096, seed=5)
    U.run_gemv(qg, h, w, x, h=h)
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and st.where in (61, 62, 63, 64, 65)
    assert h.device_status().code == 0  # reading clears it
    w.unload()
    h.close()
    h2 = qg.QGemv(device=0)
    w2 = _load(qg, h2, codes, scales, ts)
    y = U.run_gemv(qg, h2, w2, x, h=h2)
    assert O.rel_l2(y, O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    w2.unload()
    h2.close()


def test_tc_refused_by_other_entry_points(qg, handle):
    import torch
    codes, scales, ts = O.make_nvfp4(128, 64, seed=1)
    w = _load(qg, handle, codes, scales, ts)
    x = torch.zeros(16 * 64, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(16 * 128, dtype=torch.float32, device="cuda")
    with pytest.raises(qg.QgemvError) as e:
        handle.gemm_skinny(w, x.data_ptr(), 16, y.data_ptr(), qg.OUT_F32)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    w.unload()
    # a stacked weight (the experts of an MoE layer) is no job of a list
    ws = handle.load_stacked(np.stack([qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)] * 2))
    with pytest.raises(qg.QgemvError) as e:
        handle.sequence([(ws, x.data_ptr(), y.data_ptr(), qg.OUT_F32)], 1)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    ws.unload()


# ---- a sequence of GEMVs as one persistent launch -------------------------------------------------
def _chain(qg, h, shapes, B, seed):
    """Weights W_i: N_i x K_i with K_{i+1} = N_i; device buffers; the job list x_{i+1} = y_i (bf16)."""
    import torch
    ws, mats = [], []
    for i, (N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=seed + i, ts=0.02)   # small scale keeps the chain finite
        mats.append((codes, scales, ts))
        ws.append(h.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)))
    x0 = O.make_x(B, shapes[0][1], seed=seed + 100)
    bufs = [U.dev_u16(x0)] + [torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda") for N, _ in shapes]
    jobs = [(ws[i], bufs[i].data_ptr(), bufs[i + 1].data_ptr(), qg.OUT_BF16) for i in range(len(shapes))]
    return ws, mats, x0, bufs, jobs


@pytest.mark.parametrize("B", [1, 3, 8])
def test_sequence_chain(qg, handle, B):
    """Each job reads what the one before it wrote: parity of every link against the oracle fed with
    the previous link's device result, bit-equality with one launch per GEMV, and a second run."""
    import torch
    shapes = [(2048, 1024), (512, 2048), (4096, 512), (144, 4096)]
    ws, mats, x0, bufs, jobs = _chain(qg, handle, shapes, B, seed=40)
    seq = handle.sequence(jobs, B)
    for rep in range(2):
        for b in bufs[1:]:
            b.fill_(float("nan"))
        seq.run()
        torch.cuda.synchronize()
        U.status_ok(handle)
        xin = x0
        for i, (codes, scales, ts) in enumerate(mats):
            got = bufs[i + 1].view(torch.int16).cpu().numpy().view(np.uint16)
            ref = O.gemv_nvfp4_f64(codes, scales, ts, xin)
            assert not np.isnan(O.bf16_decode(got)).any(), (rep, i)
            assert O.rel_l2(O.bf16_decode(got), ref) < TOL_BF16, (rep, i)
            xin = got
    # the same chain, one launch per GEMV: same split along K, same bits
    seq_out = [b.clone() for b in bufs[1:]]
    for i, (w, xp, yp, dt) in enumerate(jobs):
        bufs[i + 1].fill_(float("nan"))
        handle.gemv(w, xp, B, yp, dt)
    torch.cuda.synchronize()
    for a, b in zip(seq_out, bufs[1:]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    seq.destroy()
    for w in ws:
        w.unload()


def test_sequence_in_a_graph_and_small_jobs(qg, handle):
    """Jobs with fewer items than CTAs, fp32 outputs, replayed from a CUDA graph."""
    import torch
    B = 2
    shapes = [(128, 64), (16, 128), (300, 16)]
    codes_l, ws, xs, ys = [], [], [], []
    for i, (N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=60 + i)
        codes_l.append((codes, scales, ts))
        ws.append(handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)))
        xs.append(O.make_x(B, K, seed=70 + i))
        ys.append(torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda"))
    xd = [U.dev_u16(x) for x in xs]
    seq = handle.sequence([(ws[i], xd[i].data_ptr(), ys[i].data_ptr(), qg.OUT_F32) for i in range(len(shapes))], B)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        seq.run(st.cuda_stream)
    st.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        seq.run(torch.cuda.current_stream().cuda_stream)
    for y in ys:
        y.fill_(float("nan"))
    with torch.cuda.stream(st):
        g.replay()
        g.replay()
    st.synchronize()
    U.status_ok(handle)
    for (codes, scales, ts), x, y in zip(codes_l, xs, ys):
        assert O.rel_l2(y.cpu().numpy(), O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    seq.destroy()
    for w in ws:
        w.unload()


def test_sequence_bounded_wait_reports_timeout(qg):
    """Host-set injection (no weight copy is ever issued): every wait of the persistent kernel runs
    out, the CTAs leave together, the status word says why, and the handle works afterwards."""
    import torch
    h = qg.QGemv(device=0, spin_limit=2000, inject_drop_copies=True)
    ws, mats, x0, bufs, jobs = _chain(qg, h, [(1024, 1024), (512, 1024)], 1, seed=80)
    seq = h.sequence(jobs, 1)
    seq.run()
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and 71 <= st.where <= 85
    # the same list once more on the same handle: the abandoned launch's tagged words must not be taken for new ones
    seq.run()
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and 71 <= st.where <= 85
    seq.destroy()
    for w in ws:
        w.unload()
    h.close()
    h2 = qg.QGemv(device=0)
    ws, mats, x0, bufs, jobs = _chain(qg, h2, [(1024, 1024), (512, 1024)], 1, seed=80)
    seq = h2.sequence(jobs, 1)
    seq.run()
    torch.cuda.synchronize()
    assert h2.device_status().code == 0
    got = bufs[1].view(torch.int16).cpu().numpy().view(np.uint16)
    assert O.rel_l2(O.bf16_decode(got), O.gemv_nvfp4_f64(*mats[0], x0)) < TOL_BF16
    seq.destroy()
    for w in ws:
        w.unload()
    h2.close()


def test_sequence_independent_and_distant_dependencies(qg, handle):
    """Twelve jobs: most independent of one another (no barrier between them: their digit planes are
    made while the job before still multiplies, and the parts buffers wrap around), two that read
    the output of a job two and five places back."""
    import torch
    B = 2
    shapes = [(640, 1024), (4096, 512), (256, 4160), (1000, 640), (6144, 1024), (512, 256),
              (2048, 2048), (384, 4096), (128, 1024), (3000, 320), (768, 640), (130, 2048)]
    mats, ws, xh, xd, ys = [], [], [], [], []
    for i, (N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=200 + i, ts=0.03)
        mats.append((codes, scales, ts))
        ws.append(handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)))
        xh.append(O.make_x(B, K, seed=300 + i))
        xd.append(U.dev_u16(xh[-1]))
        ys.append(torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda"))
    # job 3 (K = 640) reads y of job 0 (N = 640); job 10 (K = 640) reads y of job 0 as well... and
    # job 8 (K = 1024) reads nothing new.  Job 5 (K = 256)'s input is y of job 2?  No: N of job 2 is 256.
    src = {3: 0, 10: 0, 5: 2}
    jobs = []
    for i in range(len(shapes)):
        xp = ys[src[i]].data_ptr() if i in src else xd[i].data_ptr()
        jobs.append((ws[i], xp, ys[i].data_ptr(), qg.OUT_BF16))
    seq = handle.sequence(jobs, B)
    for rep in range(3):
        for y in ys:
            y.fill_(float("nan"))
        seq.run()
        torch.cuda.synchronize()
        U.status_ok(handle)
        outs = [y.view(torch.int16).cpu().numpy().view(np.uint16) for y in ys]
        for i, (codes, scales, ts) in enumerate(mats):
            xin = outs[src[i]] if i in src else xh[i]
            ref = O.gemv_nvfp4_f64(codes, scales, ts, xin)
            assert not np.isnan(O.bf16_decode(outs[i])).any(), (rep, i)
            assert O.rel_l2(O.bf16_decode(outs[i]), ref) < TOL_BF16, (rep, i)
    # bit-equal to one launch per GEMV
    keep = [o.copy() for o in outs]
    for i, (w, xp, yp, dt) in enumerate(jobs):
        ys[i].fill_(float("nan"))
        handle.gemv(w, xp, B, yp, dt)
    torch.cuda.synchronize()
    for i, y in enumerate(ys):
        assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), keep[i]), i
    seq.destroy()
    for w in ws:
        w.unload()


def test_sequence_forced_order_flag(qg, handle):
    """QGEMV_JOB_AFTER_PREVIOUS: jobs whose buffers are unrelated run strictly one after the other;
    the results are the bits of the unordered list and of one launch per GEMV."""
    import torch
    B = 2
    shapes = [(640, 1024), (4096, 512), (256, 4160), (6144, 1024), (130, 2048)]
    ws, xd, ys, refs = [], [], [], []
    for i, (N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=500 + i, ts=0.5)
        ws.append(handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)))
        xh = O.make_x(B, K, seed=600 + i)
        xd.append(U.dev_u16(xh))
        ys.append(torch.full((B, N), float("nan"), dtype=torch.float32, device="cuda"))
        refs.append(O.gemv_nvfp4_f64(codes, scales, ts, xh))
    jobs = [(ws[i], xd[i].data_ptr(), ys[i].data_ptr(), qg.OUT_F32) for i in range(len(shapes))]
    outs = {}
    for chained in (False, True):
        seq = handle.sequence(jobs, B, chained=chained)
        for rep in range(2):
            for y in ys:
                y.fill_(float("nan"))
            seq.run()
            torch.cuda.synchronize()
            U.status_ok(handle)
        outs[chained] = [y.cpu().numpy().copy() for y in ys]
        seq.destroy()
    for i in range(len(shapes)):
        assert O.rel_l2(outs[True][i], refs[i]) < TOL_F32, i
        U.assert_bits_equal(outs[True][i], outs[False][i])
    for w in ws:
        w.unload()


@pytest.mark.parametrize("N,K,shard", [(128, 64, None), (272, 2112, None), (1000, 4112, None), (6144, 4096, None),
                                       (1024, 4096, (0, 1024, 2048, 4096)), (1000, 2112, (300, 811, 0, 2112)),
                                       (512, 1024, (128, 384, 16, 1008))])
def test_load_device_matches_host_pack(qg, handle, N, K, shard):
    """The device-side packer writes byte for byte what the host packer writes (header apart from the
    checksum, payload, zero padding), also for shards; and the GEMV on it matches the oracle."""
    import torch
    codes, scales, ts = O.make_nvfp4(N, K, seed=N + K, ts=0.625)
    sh = qg.Shard(*shard) if shard else None
    blob = qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts, shard=sh)
    cd, sd = torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda()
    w = handle.load_device(qg.FMT_NVFP4_TC, cd.data_ptr(), sd.data_ptr(), N, K, ts, shard=sh)
    got = w.read_blob()
    assert got.size == blob.size
    assert np.array_equal(got[256:], blob[256:])
    assert np.array_equal(got[:80], blob[:80]) and np.array_equal(got[88:256], blob[88:256])   # [80, 88): checksum
    n0, n1, k0, k1 = shard if shard else (0, N, 0, K)
    assert (w.N, w.K) == (n1 - n0, k1 - k0)
    cs, ss, t2 = qg.unpack(blob)
    x = O.make_x(2, k1 - k0, seed=7)
    assert O.rel_l2(U.run_gemv(qg, handle, w, x), O.gemv_nvfp4_f64(cs, ss, t2, x)) < TOL_F32
    w.unload()
    with pytest.raises(qg.QgemvError) as e:
        handle.load_device(qg.FMT_NVFP4, cd.data_ptr(), sd.data_ptr(), N, K, ts)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE


@pytest.mark.parametrize("B", [1, 4])
def test_sequence_column_range_chain(qg, handle, B):
    """Jobs that read a column range of the previous job's output (row stride = that job's N): the
    path that picks the producer's rows up as they are published.  Checked link by link against
    the oracle, run three times (the tags of one run must not satisfy the next), and compared with
    one launch per GEMV on copies of the ranges."""
    import torch
    shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (6144, 4096), (1024, 2048)]
    ws, mats = [], []
    for i, (N, K) in enumerate(shapes):
        codes, scales, _ = O.make_nvfp4(N, K, seed=700 + i)
        ts = 1.0 / (0.1463 * K ** 0.5)
        mats.append((codes, scales, ts))
        ws.append(handle.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)))
    x0 = O.make_x(B, shapes[0][1], seed=777)
    x0d = U.dev_u16(x0)
    ys = [torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda") for N, _ in shapes]
    jobs = [(ws[0], x0d.data_ptr(), ys[0].data_ptr(), qg.OUT_BF16)]
    for i in range(1, len(shapes)):
        jobs.append((ws[i], ys[i - 1].data_ptr(), ys[i].data_ptr(), qg.OUT_BF16, 0, shapes[i - 1][0]))
    seq = handle.sequence(jobs, B)
    first = None
    for rep in range(3):
        for y in ys:
            y.fill_(float("nan"))
        seq.run()
        torch.cuda.synchronize()
        U.status_ok(handle)
        outs = [y.view(torch.int16).cpu().numpy().view(np.uint16) for y in ys]
        xin = x0
        for i, (codes, scales, ts) in enumerate(mats):
            assert not np.isnan(O.bf16_decode(outs[i])).any(), (rep, i)
            assert O.rel_l2(O.bf16_decode(outs[i]), O.gemv_nvfp4_f64(codes, scales, ts, xin)) < TOL_BF16, (rep, i)
            if i + 1 < len(shapes):
                xin = np.ascontiguousarray(outs[i][:, :shapes[i + 1][1]])
        if first is None:
            first = [o.copy() for o in outs]
        else:
            for a, b in zip(first, outs):
                assert np.array_equal(a, b)
    # one launch per GEMV on contiguous copies of the column ranges: the same bits
    xin = x0d
    for i, (N, K) in enumerate(shapes):
        y = torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        handle.gemv(ws[i], xin.data_ptr(), B, y.data_ptr(), qg.OUT_BF16)
        torch.cuda.synchronize()
        assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), first[i]), i
        if i + 1 < len(shapes):
            xin = y[:, :shapes[i + 1][1]].contiguous()
    seq.destroy()
    for w in ws:
        w.unload()


def _silu_mul_bf16(gu_bits, K):
    """bf16(silu(gate) * up) from rows that hold K gate values and then K up values (fp64 inside)."""
    v = O.bf16_decode(gu_bits).astype(np.float64)
    g, u = v[:, :K], v[:, K:2 * K]
    return O.bf16_encode((g / (1.0 + np.exp(-g)) * u).astype(np.float32))


def _rms_parts(x_bits, w_bits, eps):
    """What a job with a norm multiplies, bf16(x * w), and the fp64 row factor rsqrt(mean(x^2) + eps)."""
    x = O.bf16_decode(x_bits)
    xs = O.bf16_encode((x * O.bf16_decode(w_bits)[None, :]).astype(np.float32))      # the fp32 product of two bf16 is exact
    r = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1) + eps)
    return xs, r


@pytest.mark.parametrize("B", [1, 3])
def test_sequence_fused_decoder_layer(qg, handle, B):
    """The element-wise work of a decoder layer folded into the jobs: o-projection + residual, RMS norm
    into gate/up, SiLU * up into down + residual, RMS norm into the next QKV -- four jobs, one launch,
    every link checked against the fp64 oracle fed with the device's previous output."""
    import torch
    H, I, Q = 1024, 2816, 1536
    eps = 1e-5
    mk = lambda N, K, seed: O.make_nvfp4(N, K, seed=seed, ts=1.0 / (0.1463 * K ** 0.5))
    m_o, m_gu, m_dn, m_qkv = mk(H, H, 901), mk(2 * I, H, 902), mk(H, I, 903), mk(Q, H, 904)
    ws = [handle.load(qg.pack(qg.FMT_NVFP4_TC, *m)) for m in (m_o, m_gu, m_dn, m_qkv)]
    attn, h0 = O.make_x(B, H, seed=905), O.make_x(B, H, seed=906)
    nw1 = O.bf16_encode(1.0 + 0.1 * O.bf16_decode(O.make_x(1, H, seed=907))[0])
    nw2 = O.bf16_encode(1.0 + 0.1 * O.bf16_decode(O.make_x(1, H, seed=908))[0])
    d = lambda a: U.dev_u16(a)
    attn_d, h0_d, nw1_d, nw2_d = d(attn), d(h0), d(nw1), d(nw2)
    y0 = torch.zeros((B, H), dtype=torch.bfloat16, device="cuda")
    y1 = torch.zeros((B, 2 * I), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((B, H), dtype=torch.bfloat16, device="cuda")
    y3 = torch.zeros((B, Q), dtype=torch.float32, device="cuda")
    jobs = [(ws[0], attn_d.data_ptr(), y0.data_ptr(), qg.OUT_BF16, 0, 0, {"residual": h0_d.data_ptr()}),
            (ws[1], y0.data_ptr(), y1.data_ptr(), qg.OUT_BF16, 0, 0, {"norm_weight": nw1_d.data_ptr(), "norm_eps": eps}),
            (ws[2], y1.data_ptr(), y2.data_ptr(), qg.OUT_BF16, qg.JOB_X_SILU_MUL, 0, {"residual": y0.data_ptr()}),
            (ws[3], y2.data_ptr(), y3.data_ptr(), qg.OUT_F32, 0, 0, {"norm_weight": nw2_d.data_ptr(), "norm_eps": eps})]
    seq = handle.sequence(jobs, B)
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    for rep in range(2):
        for y in (y0, y1, y2, y3):
            y.zero_()
        seq.run()
        torch.cuda.synchronize()
        U.status_ok(handle)
        g0, g1, g2 = bits(y0), bits(y1), bits(y2)
        ref0 = O.gemv_nvfp4_f64(*m_o, attn) + O.bf16_decode(h0)
        assert O.rel_l2(O.bf16_decode(g0), ref0) < TOL_BF16, rep
        xs, r = _rms_parts(g0, nw1, eps)
        ref1 = O.gemv_nvfp4_f64(*m_gu, xs) * r[:, None]
        assert O.rel_l2(O.bf16_decode(g1), ref1) < TOL_BF16, rep
        ref2 = O.gemv_nvfp4_f64(*m_dn, _silu_mul_bf16(g1, I)) + O.bf16_decode(g0)
        assert O.rel_l2(O.bf16_decode(g2), ref2) < TOL_BF16, rep
        xs, r = _rms_parts(g2, nw2, eps)
        ref3 = O.gemv_nvfp4_f64(*m_qkv, xs) * r[:, None]
        assert O.rel_l2(y3.cpu().numpy(), ref3) < 2e-4, rep      # fp32 output; silu's fast exp sits upstream only
    seq.destroy()
    # the same options on jobs whose inputs are plain buffers (no published rows), fp32 residual
    res32 = torch.randn((B, H), device="cuda")
    y4 = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    gu_in = d(O.make_x(B, 2 * I, seed=909))
    seq = handle.sequence([(ws[2], gu_in.data_ptr(), y4.data_ptr(), qg.OUT_F32, qg.JOB_X_SILU_MUL, 0, {"residual": res32.data_ptr()})], B)
    seq.run()
    torch.cuda.synchronize()
    U.status_ok(handle)
    ref4 = O.gemv_nvfp4_f64(*m_dn, _silu_mul_bf16(O.make_x(B, 2 * I, seed=909), I)) + res32.cpu().numpy().astype(np.float64)
    assert O.rel_l2(y4.cpu().numpy(), ref4) < 2e-4
    seq.destroy()
    for w in ws:
        w.unload()
