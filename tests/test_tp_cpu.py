"""Tensor-parallel sharding logic on CPU: two gloo ranks, each holding the shard the packer cuts for
it, reproduce the unsharded oracle after the exchange step (no GPU involved)."""
import os

import numpy as np
import pytest

from oracle import oracle as O


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    import crit_hub_b200 as qg
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, B = 96, 512, 3
        codes, scales, ts = O.make_nvfp4(N, K, seed=4, ts=0.5)
        x = O.make_x(B, K, seed=4)
        full = O.gemv_nvfp4_f64(codes, scales, ts, x)
        # row-parallel (o / down): split K, partial outputs are summed over the ranks
        k0, k1 = rank * K // world, (rank + 1) * K // world
        c, s, t2 = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=qg.Shard(0, N, k0, k1)))
        part = torch.from_numpy(O.gemv_nvfp4_f64(c, s, t2, np.ascontiguousarray(x[:, k0:k1])))
        dist.all_reduce(part)
        err_row = O.rel_l2(part.numpy(), full)
        # column-parallel (QKV, gate/up): split N, outputs are concatenated (all-gather)
        n0, n1 = rank * N // world, (rank + 1) * N // world
        c, s, t2 = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=qg.Shard(n0, n1, 0, K)))
        mine = torch.from_numpy(O.gemv_nvfp4_f64(c, s, t2, x))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        err_col = O.rel_l2(torch.cat(parts, dim=1).numpy(), full)
        q.put((rank, err_row, err_col))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded_oracle():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29547, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    for _, err_row, err_col in res:
        assert err_row < 1e-12 and err_col < 1e-12
