"""Tensor-parallel exchange on the GPU.

One-GPU tests stand in for the peers: the exchange is "push tagged pairs into every rank's buffer,
gather the ranks' pairs from my own", so a peer that has already pushed is a slot that the test
fills beforehand (value, tag) and a peer that never arrives is a slot nobody writes.  No second
kernel waits on the first, nothing faults.  The two-GPU tests (skipped on a one-GPU box) run real
ranks as child processes.
"""
import numpy as np
import pytest

import gpu_util as U
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_F32 = 5e-5
TOL_BF16 = 2e-3


class _Raw:
    """A device range owned by the library, seen by torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // 8,), "typestr": "<i8", "data": (ptr, False), "version": 2}


def _pairs_view(handle):
    import torch
    ptr, nbytes = handle.tp_buffer()
    return torch.as_tensor(_Raw(ptr, nbytes), device="cuda")


def _pair(values_f32: np.ndarray, tag: int):
    import torch
    v = np.ascontiguousarray(values_f32, dtype=np.float32).view(np.uint32).astype(np.int64)
    return torch.from_numpy(v | (np.int64(tag) << 32)).cuda()


def _emulated_rank0(qg, max_elems, spin_limit=0):
    """Handle as rank 0 of a world of two whose peer buffer is a scratch tensor of the same size."""
    import torch
    h = qg.QGemv(device=0, spin_limit=spin_limit)
    h.tp_create(0, 2, max_elems)
    ptr, nbytes = h.tp_buffer()
    peer = torch.zeros(nbytes // 8, dtype=torch.int64, device="cuda")
    h.tp_connect_ptrs([0, peer.data_ptr()])
    return h, _pairs_view(h), peer


def test_allreduce_with_a_prefilled_peer(qg):
    import torch
    M = 4096
    h, mine, peer = _emulated_rank0(qg, M)
    n = 3001
    rng = np.random.default_rng(3)
    for call in range(1, 4):                       # tags 1, 2, 3: parities 1, 0, 1
        other = rng.standard_normal(n).astype(np.float32)
        par = call & 1
        mine[(par * 2 + 1) * M:(par * 2 + 1) * M + n] = _pair(other, call)   # rank 1's slot of my buffer
        y = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
        own = y.cpu().numpy().copy()
        h.tp_allreduce(y.data_ptr(), qg.OUT_F32, n)
        torch.cuda.synchronize()
        assert h.device_status().code == 0
        U.assert_bits_equal(y.cpu().numpy(), own + other)           # fp32, rank order: own first
        pushed = peer[(par * 2 + 0) * M:(par * 2 + 0) * M + n].cpu().numpy()   # my slot of the peer's buffer
        assert np.array_equal(pushed >> 32, np.full(n, call))
        assert np.array_equal((pushed & 0xFFFFFFFF).astype(np.uint32), own.view(np.uint32))
    # bf16 vectors travel as fp32 pairs and are rounded once
    other = rng.standard_normal(n).astype(np.float32)
    mine[(0 * 2 + 1) * M:(0 * 2 + 1) * M + n] = _pair(other, 4)
    yb = torch.randn(n, device="cuda").bfloat16()
    own = yb.float().cpu().numpy()
    h.tp_allreduce(yb.data_ptr(), qg.OUT_BF16, n)
    torch.cuda.synchronize()
    want = torch.from_numpy(own + other).bfloat16()
    assert torch.equal(yb.cpu(), want)
    h.close()


def test_allgather_with_a_prefilled_peer(qg):
    import torch
    M = 2048
    h, mine, peer = _emulated_rank0(qg, M)
    n = 1000
    other = np.random.default_rng(5).standard_normal(n).astype(np.float32)
    mine[(1 * 2 + 1) * M:(1 * 2 + 1) * M + n] = _pair(other, 1)
    shard = torch.randn(n, device="cuda")
    y = torch.full((2 * n,), float("nan"), device="cuda")
    h.tp_allgather(shard.data_ptr(), y.data_ptr(), qg.OUT_F32, n)
    torch.cuda.synchronize()
    assert h.device_status().code == 0
    got = y.cpu().numpy()
    U.assert_bits_equal(got[:n], shard.cpu().numpy())
    U.assert_bits_equal(got[n:], other)
    with pytest.raises(qg.QgemvError):
        h.tp_allgather(y.data_ptr(), y.data_ptr(), qg.OUT_F32, n)   # in place is refused
    h.close()


def test_exchange_wait_runs_out(qg, handle):
    """The peer's slot is never written: the bounded wait gives up, the status word names the site
    (30), y keeps its contents and the device stays usable."""
    import torch
    h, mine, peer = _emulated_rank0(qg, 1024, spin_limit=2000)
    y = torch.arange(512, device="cuda", dtype=torch.float32)
    h.tp_allreduce(y.data_ptr(), qg.OUT_F32, 512)
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and st.where == 30 and st.extra == 1, st
    assert torch.equal(y.cpu(), torch.arange(512, dtype=torch.float32))
    assert h.device_status().code == 0          # reading the status clears it
    h.close()
    # the device still computes
    codes, scales, ts = O.make_nvfp4(256, 1024, seed=2)
    x = O.make_x(1, 1024, seed=2)
    w = handle.load(qg.pack(qg.FMT_NVFP4, codes, scales, ts))
    assert O.rel_l2(U.run_gemv(qg, handle, w, x), O.gemv_nvfp4_f64(codes, scales, ts, x)) < TOL_F32
    w.unload()


def _tc_shard(qg, h, codes, scales, ts, n0, n1, k0, k1):
    N, K = scales.shape[0], scales.shape[1] * 16
    return h.load(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts, shard=qg.Shard(n0, n1, k0, k1)))


@pytest.mark.parametrize("B", [1, 3])
def test_sequence_allreduce_with_prefilled_peers(qg, B):
    """A job list as rank 0 of two runs: row-parallel job (summed over the ranks inside the launch)
    -> local job reading its output -> second row-parallel job.  Rank 1's partial sums sit in its
    slots beforehand; what rank 0 pushes for rank 1 is read back from the stand-in buffer."""
    import torch
    N0, K0, N1, N2 = 512, 4096, 1024, 640
    total = B * N0 + B * N2
    M = (total + 8192 + 3) // 4 * 4
    h, mine, peer = _emulated_rank0(qg, M)
    c0, s0, t0 = O.make_nvfp4(N0, K0, seed=11)
    c1, s1, t1 = O.make_nvfp4(N1, N0, seed=12)
    c2, s2, t2 = O.make_nvfp4(N2, 2 * N1, seed=13)
    w0 = _tc_shard(qg, h, c0, s0, t0, 0, N0, 0, K0 // 2)          # this rank: the first half of K
    w1 = h.load(qg.pack(qg.FMT_NVFP4_TC, c1, s1, t1))
    w2 = _tc_shard(qg, h, c2, s2, t2, 0, N2, 0, N1)
    x_full = O.make_x(B, K0, seed=14)
    x0 = U.dev_u16(np.ascontiguousarray(x_full[:, :K0 // 2]))
    y0 = torch.zeros((B, N0), dtype=torch.bfloat16, device="cuda")
    y1 = torch.zeros((B, N1), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((B, N2), dtype=torch.float32, device="cuda")
    seq = h.sequence([(w0, x0.data_ptr(), y0.data_ptr(), qg.OUT_BF16, qg.JOB_ALLREDUCE),
                      (w1, y0.data_ptr(), y1.data_ptr(), qg.OUT_BF16),
                      (w2, y1.data_ptr(), y2.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], B)
    off0, off2 = M - total, M - total + B * N0     # blocks in job order from max_elems - (sum of B * N)
    # rank 1's partial of job 0: the second half of K, from the oracle; of job 2: any known vector
    cs, ss, tss = qg.unpack(qg.pack(qg.FMT_NVFP4, c0, s0, t0, shard=qg.Shard(0, N0, K0 // 2, K0)))
    p0 = O.gemv_nvfp4_f64(cs, ss, tss, np.ascontiguousarray(x_full[:, K0 // 2:])).astype(np.float32)
    p2 = np.random.default_rng(B).standard_normal((B, N2)).astype(np.float32)
    for run in (1, 2):                             # tags 1 and 2: both parities
        par = run & 1
        base = (par * 2 + 1) * M
        mine[base + off0:base + off0 + B * N0] = _pair(p0.ravel(), run)
        mine[base + off2:base + off2 + B * N2] = _pair(p2.ravel(), run)
        y0.zero_(), y1.zero_(), y2.zero_()
        seq.run()
        torch.cuda.synchronize()
        st = h.device_status()
        assert st.code == 0, st
        full0 = O.gemv_nvfp4_f64(c0, s0, t0, x_full)
        assert O.rel_l2(y0.float().cpu().numpy(), full0) < TOL_BF16
        y0_bits = y0.view(torch.int16).cpu().numpy().view(np.uint16)
        assert O.rel_l2(y1.float().cpu().numpy(), O.gemv_nvfp4_f64(c1, s1, t1, y0_bits)) < TOL_BF16
        # job 2: bit-exact against (what this rank pushed) + (what rank 1 "pushed"), fp32, rank order
        mybase = (par * 2 + 0) * M
        pushed = peer[mybase + off2:mybase + off2 + B * N2].cpu().numpy()
        assert np.array_equal(pushed >> 32, np.full(B * N2, run))
        own2 = (pushed & 0xFFFFFFFF).astype(np.uint32).view(np.float32).reshape(B, N2)
        U.assert_bits_equal(y2.cpu().numpy(), own2 + p2)
        y1_bits = y1.view(torch.int16).cpu().numpy().view(np.uint16)
        c2s, s2s, t2s = qg.unpack(qg.pack(qg.FMT_NVFP4, c2, s2, t2, shard=qg.Shard(0, N2, 0, N1)))
        assert O.rel_l2(own2, O.gemv_nvfp4_f64(c2s, s2s, t2s, y1_bits)) < TOL_F32
        # what it stored in its own buffer for itself is the same pair
        kept = mine[mybase + off2:mybase + off2 + B * N2].cpu().numpy()
        assert np.array_equal(kept, pushed)
    seq.destroy()
    # the blocks are free again: a stand-alone exchange may use the whole slot
    y = torch.zeros(M, device="cuda")
    mine[(1 * 2 + 1) * M:(1 * 2 + 2) * M] = _pair(np.ones(M, dtype=np.float32), 1)
    h.tp_allreduce(y.data_ptr(), qg.OUT_F32, M)
    torch.cuda.synchronize()
    assert h.device_status().code == 0 and float(y.sum()) == M
    h.close()


def test_sequence_allreduce_wait_runs_out(qg):
    import torch
    B, N, K = 1, 512, 2048
    h, mine, peer = _emulated_rank0(qg, 4096, spin_limit=20000)
    c, s, t = O.make_nvfp4(N, K, seed=21)
    w = h.load(qg.pack(qg.FMT_NVFP4_TC, c, s, t))
    x = U.dev_u16(O.make_x(B, K, seed=21))
    y = torch.zeros((B, N), dtype=torch.float32, device="cuda")
    seq = h.sequence([(w, x.data_ptr(), y.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], B)
    seq.run()
    torch.cuda.synchronize()
    st = h.device_status()
    assert st.code == qg.ERR_TIMEOUT and st.where == 83 and st.extra == 1, st
    # the same weights through the plain entry point afterwards
    h.gemv(w, x.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    assert h.device_status().code == 0
    assert O.rel_l2(y.cpu().numpy(), O.gemv_nvfp4_f64(c, s, t, O.make_x(B, K, seed=21))) < TOL_F32
    h.close()


def test_sequence_allreduce_refusals(qg):
    import torch
    h, mine, peer = _emulated_rank0(qg, 1024)
    c, s, t = O.make_nvfp4(512, 1024, seed=1)
    w = h.load(qg.pack(qg.FMT_NVFP4_TC, c, s, t))
    x = torch.zeros(1024, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(8 * 512, dtype=torch.float32, device="cuda")
    with pytest.raises(qg.QgemvError) as e:      # 4 * 512 elements do not fit 1024
        h.sequence([(w, x.data_ptr(), y.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], 4)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    with pytest.raises(qg.QgemvError) as e:
        h.sequence([(w, x.data_ptr(), y.data_ptr(), qg.OUT_F32, 8)], 1)   # unknown flag
    assert e.value.status == qg.ERR_INVALID_ARG
    h.close()
    # one CTA's share would hold a whole row tile (a grid of 2 CTAs for 4 tiles): refused
    h2 = qg.QGemv(device=0, grid_override=2)
    h2.tp_create(0, 2, 1024)
    peer2 = torch.zeros(h2.tp_buffer()[1] // 8, dtype=torch.int64, device="cuda")
    h2.tp_connect_ptrs([0, peer2.data_ptr()])
    w2 = h2.load(qg.pack(qg.FMT_NVFP4_TC, c, s, t))
    with pytest.raises(qg.QgemvError) as e:
        h2.sequence([(w2, x.data_ptr(), y.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], 1)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    h2.close()


# ---- real ranks ----------------------------------------------------------------------------------
def _layer_worker(rank, world, port, q):
    """One tensor-parallel decoder layer as ONE launch per rank: column-parallel qkv and gate/up,
    row-parallel o and down summed over the ranks inside the sequence kernel; then an all-gather."""
    import os
    import torch
    import torch.distributed as dist
    import crit_hub_b200 as qg
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, I, B = 1024, 2048, 2            # hidden, intermediate
        h = qg.QGemv(device=rank)
        mine = torch.from_numpy(h.tp_create(rank, world, 4 * B * H + 4096))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        h.tp_connect(torch.stack(gathered).numpy())
        dist.barrier()
        mats = {"o": O.make_nvfp4(H, H, seed=31), "gu": O.make_nvfp4(I, H, seed=32), "dn": O.make_nvfp4(H, I, seed=33)}

        def shard(name, n0, n1, k0, k1):
            c, s, t = mats[name]
            return h.load(qg.pack(qg.FMT_NVFP4_TC, c, s, t, shard=qg.Shard(n0, n1, k0, k1)))

        ks, ke = rank * H // world, (rank + 1) * H // world
        w_o = shard("o", 0, H, ks, ke)
        w_gu = shard("gu", rank * I // world, (rank + 1) * I // world, 0, H)
        w_dn = shard("dn", 0, H, rank * I // world, (rank + 1) * I // world)
        attn = O.make_x(B, H, seed=34)
        x_o = torch.from_numpy(np.ascontiguousarray(attn[:, ks:ke]).view(np.int16)).cuda()
        y_o = torch.zeros((B, H), dtype=torch.bfloat16, device="cuda")
        y_gu = torch.zeros((B, I // world), dtype=torch.bfloat16, device="cuda")
        y_dn = torch.zeros((B, H), dtype=torch.float32, device="cuda")
        seq = h.sequence([(w_o, x_o.data_ptr(), y_o.data_ptr(), qg.OUT_BF16, qg.JOB_ALLREDUCE),
                          (w_gu, y_o.data_ptr(), y_gu.data_ptr(), qg.OUT_BF16),
                          (w_dn, y_gu.data_ptr(), y_dn.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], B)
        for _ in range(4):
            seq.run()
        torch.cuda.synchronize()
        st = h.device_status()
        # oracle, unsharded
        full_o = O.gemv_nvfp4_f64(*mats["o"], attn)
        err_o = O.rel_l2(y_o.float().cpu().numpy(), full_o)
        yo_bits = y_o.view(torch.int16).cpu().numpy().view(np.uint16)
        full_gu = O.gemv_nvfp4_f64(*mats["gu"], yo_bits)
        # all-gather of the column-parallel output (2-D rows are gathered per batch row)
        gu_all = torch.zeros((world, B * (I // world)), dtype=torch.bfloat16, device="cuda")
        h.tp_allgather(y_gu.data_ptr(), gu_all.data_ptr(), qg.OUT_BF16, B * (I // world))
        torch.cuda.synchronize()
        gu_full = gu_all.view(world, B, I // world).permute(1, 0, 2).reshape(B, I).contiguous()
        err_gu = O.rel_l2(gu_full.float().cpu().numpy(), full_gu)
        gu_bits = gu_full.view(torch.int16).cpu().numpy().view(np.uint16)
        err_dn = O.rel_l2(y_dn.cpu().numpy(), O.gemv_nvfp4_f64(*mats["dn"], gu_bits))
        st2 = h.device_status()
        q.put((rank, st.code, st2.code, err_o, err_gu, err_dn, y_dn.cpu().numpy().tobytes(), y_o.cpu().view(torch.int16).numpy().tobytes()))
        dist.barrier()  # leave only between steps, nothing in flight
    finally:
        dist.destroy_process_group()


def test_tp_layer_two_gpus(qg):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_worker, args=(r, 2, 29537, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[1] == 0 and r[2] == 0, r[:3]
        assert r[3] < TOL_BF16 and r[4] < TOL_BF16 and r[5] < TOL_F32, r[3:6]
    assert res[0][6] == res[1][6] and res[0][7] == res[1][7]      # every rank holds the same bits
