"""World-size-2 checks of the multi-process host logic, on CPU with the gloo backend."""
import os
import socket
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, results) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bench._barrier_fn(world)()
        # the slowest rank defines the step time
        slowest = bench._max_over_ranks(0.010 * (rank + 1), world)
        results[rank] = slowest
    finally:
        dist.destroy_process_group()


def test_step_time_is_the_maximum_over_ranks():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert results[0] == pytest.approx(0.020) and results[1] == pytest.approx(0.020)


def test_single_rank_helpers_need_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    bench._barrier_fn(1)()
    assert bench._max_over_ranks(1.5, 1) == 1.5
