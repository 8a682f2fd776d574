"""Host-side multi-rank logic on CPU: stream partition and max-over-ranks
timing, exercised with two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from litnicelm_b200.streams import aggregate_tokens_per_s, all_partitions, partition_streams


def test_partition_covers_every_stream_once():
    for total in (0, 1, 7, 64, 512):
        for world in (1, 2, 3, 4, 8):
            parts = all_partitions(total, world)
            covered = [i for first, n in parts for i in range(first, first + n)]
            assert covered == list(range(total))
            sizes = [n for _, n in parts]
            assert max(sizes) - min(sizes) <= 1
    assert partition_streams(512, 8, 3) == (192, 64)
    with pytest.raises(ValueError):
        partition_streams(4, 2, 2)


def test_aggregate_uses_slowest_rank():
    assert aggregate_tokens_per_s([100, 100], [1.0, 2.0]) == 100.0
    with pytest.raises(ValueError):
        aggregate_tokens_per_s([], [])


def _worker(rank, world, port, total, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    first, count = partition_streams(total, world, rank)
    # each rank "decodes" its streams: 10 tokens per stream, rank-dependent time
    tokens = torch.tensor([count * 10], dtype=torch.float64)
    seconds = torch.tensor([0.5 + rank], dtype=torch.float64)
    dist.barrier()
    dist.all_reduce(tokens, op=dist.ReduceOp.SUM)
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    owned = torch.zeros(total)
    owned[first:first + count] = 1
    dist.all_reduce(owned, op=dist.ReduceOp.SUM)
    if rank == 0:
        out.put((float(tokens), float(seconds), owned.tolist()))
    dist.destroy_process_group()


def test_two_gloo_ranks_partition_and_reduce():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 7, q)) for r in range(2)]
    for p in procs:
        p.start()
    tokens, seconds, owned = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tokens == 70.0 and seconds == 1.5
    assert owned == [1.0] * 7  # every stream owned by exactly one rank
    assert aggregate_tokens_per_s([40, 30], [0.5, 1.5]) == 70 / 1.5
