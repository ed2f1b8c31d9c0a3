"""World-size-2 gloo test of the multi-GPU host logic (sharding, gather, max-over-ranks) on CPU processes."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fast_vision_models_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        g = torch.Generator().manual_seed(0)
        full = torch.randn(7, 5, generator=g)            # 7 images: uneven shards (4 + 3)
        local = parallel.shard_batch(full)
        gathered = parallel.gather_batch(local * 2, 7)    # "the forward" doubles each row
        ok = torch.equal(gathered, full * 2)
        tmax = parallel.max_over_ranks([1.0 + rank, 5.0 - rank])
        ok = ok and tmax == [float(world_size), 5.0]
        out[rank] = bool(ok) and local.shape[0] == (4 if rank == 0 else 3)
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_gather_and_max():
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    assert out[0] and out[1]


def _window_worker(rank, world_size, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        import bench
        first = 20.0 + 7.0 * rank                # the ranks time their first window differently
        alone = bench.window_count(first, 2.0, 10, 200)
        shared = bench.window_count(first, 2.0, 10, 200, agree=lambda v: parallel.max_over_ranks([float(v)])[0])
        out[rank] = (alone, shared)
    finally:
        dist.destroy_process_group()


def test_all_ranks_run_the_same_number_of_timed_windows():
    # bench.py brackets every timed window with a barrier: a window count taken from each rank's own first window would
    # differ between ranks (100 against 74 here) and leave them in different collectives
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_window_worker, args=(2, port, out), nprocs=2, join=True)
    assert out[0][0] != out[1][0]
    assert out[0][1] == out[1][1] == 74


def test_shard_ranges_cover_everything_once():
    for n in (0, 1, 7, 64, 65):
        for ws in (1, 2, 3, 8):
            spans = [parallel.shard_range(n, r, ws) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, b0), (a1, b1) in zip(spans, spans[1:]):
                assert b0 == a1 and 0 <= (b0 - a0) - (b1 - a1) <= 1


def test_single_process_is_a_no_op():
    x = torch.arange(6.0).view(3, 2)
    assert parallel.world() == (0, 1)
    assert torch.equal(parallel.shard_batch(x), x)
    assert torch.equal(parallel.gather_batch(x, 3), x)
    assert parallel.max_over_ranks([1.0, 2.0]) == [1.0, 2.0]
