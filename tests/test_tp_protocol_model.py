"""A host model of the peer-memory all-reduce protocol (csrc/tp_allreduce.cuh): every rank pushes
{value, epoch} pairs into its slot of every rank's buffer, then waits on its own buffer for the
call's epoch and adds the slots in rank order.  Ranks run as threads with random delays; the model
checks the two-parity argument (no pair of call k is overwritten before every rank has read it)
at world sizes up to 8.  It tests the protocol, not the CUDA code."""
import random
import threading
import time

import pytest


def _run(world, calls, n, seed):
    # buf[rank][parity][src][i] = (value, epoch)
    buf = [[[[(0.0, 0)] * n for _ in range(world)] for _ in range(2)] for _ in range(world)]
    results = [[None] * calls for _ in range(world)]
    errors = []

    def contribution(rank, call, i):
        return float((rank + 1) * 1000 + call * 7 + i)

    def rank_main(rank):
        rng = random.Random(seed * 100 + rank)
        try:
            for call in range(calls):
                epoch = call + 1
                par = epoch & 1
                for d in range(world):                      # push, starting with myself
                    peer = (rank + d) % world
                    if rng.random() < 0.2:
                        time.sleep(rng.random() * 1e-4)
                    for i in range(n):
                        buf[peer][par][rank][i] = (contribution(rank, call, i), epoch)
                acc = [0.0] * n
                for i in range(n):                          # wait on MY buffer, add in rank order
                    for src in range(world):
                        t0 = time.time()
                        while True:
                            v, e = buf[rank][par][src][i]
                            if e == epoch:
                                break
                            if e > epoch:
                                raise AssertionError(f"rank {rank} call {call}: slot of {src} already holds epoch {e}")
                            if time.time() - t0 > 20:
                                raise AssertionError("wait ran out")
                            time.sleep(0)
                        acc[i] = v if src == 0 else acc[i] + v
                results[rank][call] = acc
                if rng.random() < 0.1:
                    time.sleep(rng.random() * 2e-4)        # a slow rank
        except AssertionError as ex:
            errors.append(str(ex))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not errors, errors
    for call in range(calls):
        want = [sum(contribution(r, call, i) for r in range(world)) for i in range(n)]
        for r in range(world):
            assert results[r][call] == want, (r, call)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_two_parities_suffice(world):
    _run(world, calls=60, n=3, seed=world)
