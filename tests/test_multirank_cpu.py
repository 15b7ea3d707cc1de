"""The N > 1 path of bench.py on CPU: two gloo ranks, no data-path collective, only the max-over-ranks timing
reduction, the aggregate over ranks and the split of the workload's batch rows."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    local_ms = 10.0 + 5.0 * rank                 # rank 1 is the slow one
    per_s, ms = bench.aggregate_throughput(1000.0, local_ms, world)
    dist.barrier()
    out[rank] = (per_s, ms, bench.max_over_ranks(float(rank)))
    dist.destroy_process_group()


def test_two_ranks_report_the_slowest_time_and_total_work():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, 29631, out), nprocs=world, join=True)
    for rank in range(world):
        per_s, ms, mx = out[rank]
        assert ms == 15.0 and mx == 1.0
        assert abs(per_s - world * 1000.0 / 15e-3) < 1e-6


def test_single_process_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.max_over_ranks(3.5) == 3.5
    assert bench.aggregate_throughput(10.0, 2.0, 1) == (5000.0, 2.0)


def test_workload_is_split_by_batch_rows_under_strong_scaling():
    sys.path.insert(0, ROOT)
    import pytest
    import bench
    assert [bench.shard_batch(8, n, "strong") for n in (1, 2, 4, 8)] == [8, 4, 2, 1]
    assert [bench.shard_batch(8, n, "weak") for n in (1, 2, 4, 8)] == [8, 8, 8, 8]
    with pytest.raises(SystemExit):
        bench.shard_batch(8, 3, "strong")
    # the job's figure: every rank's share of the FLOPs over the slowest rank's time = whole workload / that time
    total = 3.5 * bench.flops_fwd(8, 32, 8192, 128)
    share = 3.5 * bench.flops_fwd(bench.shard_batch(8, 4, "strong"), 32, 8192, 128)
    per_s, ms = bench.aggregate_throughput(share, 5.0, 1)
    assert abs(4 * share - total) < 1e-3 * total and ms == 5.0
