"""The N > 1 bookkeeping (cubert_b200/replicas.py) with two real processes on the gloo backend."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cubert_b200 import replicas


def test_shard_range_partitions_exactly():
    for total in (0, 1, 7, 256, 511, 512):
        for world in (1, 2, 3, 8):
            spans = [replicas.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        replicas.shard_range(10, 2, 2)


def test_single_process_needs_no_process_group():
    assert replicas.max_over_ranks(3.5) == 3.5
    assert replicas.job_throughput(256, 0.5) == 512.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), LOCAL_RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert replicas.rank_info() == (rank, rank, world)
        begin, end = replicas.shard_range(513, rank, world)      # one batch split over the ranks (strong scaling)
        seconds = 0.25 * (rank + 1)                              # rank 1 is the slow one
        covered = replicas.sum_over_ranks(end - begin)
        slowest = replicas.max_over_ranks(seconds)
        rate = replicas.job_throughput(end - begin, seconds)
        dist.barrier()
        out.put((rank, begin, end, covered, slowest, rate, replicas.stream_seed(2, rank)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, b0, e0, c0, s0, t0, seed0), (r1, b1, e1, c1, s1, t1, seed1) = results
    assert (b0, e0, b1, e1) == (0, 257, 257, 513)           # disjoint, contiguous, complete
    assert c0 == c1 == 513.0 and s0 == s1 == 0.5            # both ranks agree on totals and on the slowest time
    assert t0 == t1 == 513.0 / 0.5
    assert seed0 != seed1
