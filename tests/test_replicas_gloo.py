"""The multi-GPU path is N independent replicas: the only cross-rank step is the timing reduction (maximum over
ranks) that turns per-replica times into whole-job throughput.  Checked here with two gloo ranks on CPU, together
with the dispatcher that spreads requests over the replicas."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    # rank 1 is the slow replica: its times must define the job on every rank
    mine = [10.0 + 5.0 * rank, 100.0 - 20.0 * rank]
    reduced = bench.max_over_ranks(mine, torch.device("cpu"), world)
    dist.barrier()
    results[rank] = (reduced, bench.aggregate_throughput(128 * 4, world, reduced[0]))
    dist.destroy_process_group()


def test_two_replicas_report_the_slowest_time_and_the_summed_throughput():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    for rank in range(world):
        reduced, throughput = results[rank]
        assert reduced == [15.0, 100.0]
        assert throughput == pytest.approx(128 * 4 * 2 / 15e-3)


def test_single_replica_needs_no_process_group():
    import bench
    assert bench.max_over_ranks([3.0, 4.0], torch.device("cpu"), 1) == [3.0, 4.0]
    assert bench.aggregate_throughput(64, 1, 2.0) == pytest.approx(32000.0)
