"""The N > 1 path without GPUs: two gloo ranks on CPU."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from latentserve_b200 import replicas


def test_partition_balances_outstanding_tokens_deterministically():
    lens = [32768, 1024, 9000, 2048, 16000, 4096, 1500, 30000]
    shards = replicas.partition_by_tokens(lens, 2)
    assert sorted(i for s in shards for i in s) == list(range(len(lens)))
    loads = [sum(lens[i] for i in s) for s in shards]
    assert abs(loads[0] - loads[1]) <= 2048
    assert shards == replicas.partition_by_tokens(lens, 2)
    assert replicas.partition_by_tokens(lens, 1) == [list(range(len(lens)))]
    many = replicas.partition_by_tokens([5] * 3, 8)
    assert sum(len(s) for s in many) == 3 and len(many) == 8


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = [700, 300, 61, 17, 1, 4096]
        mine = replicas.partition_by_tokens(lens, world)[rank]
        ms = 10.0 + 5.0 * rank                       # rank 1 is the slow one
        slowest = replicas.max_over_ranks(ms, dist)
        units = torch.tensor([float(sum(lens[i] for i in mine))])
        dist.all_reduce(units)                        # every token is owned exactly once
        dist.barrier()
        out[rank] = (slowest, float(units.item()), mine)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_slowest_time_and_cover_the_batch():
    world, port = 2, 29581
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert out[0][0] == out[1][0] == 15.0
        assert out[0][1] == out[1][1] == 700 + 300 + 61 + 17 + 1 + 4096
        assert sorted(out[0][2] + out[1][2]) == list(range(6))
    assert replicas.aggregate_throughput(100.0, 0.5, 2) == 400.0
