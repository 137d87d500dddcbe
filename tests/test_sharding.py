"""Batch sharding host logic on CPU: shard arithmetic, and a world-size-2 gloo run in which each rank works on
its slice with the CPU oracle and the gathered result equals the unsharded one."""
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ngraph_b200 import sharding


def test_shard_bounds_cover_everything():
    for n in (0, 1, 5, 128, 1001):
        for world in (1, 2, 3, 8):
            counts, offsets = sharding.shard_bounds(n, world)
            assert sum(counts) == n and len(counts) == world
            assert max(counts) - min(counts) <= 1
            assert offsets == [sum(counts[:r]) for r in range(world)]
            covered = []
            for r in range(world):
                s = sharding.local_slice(n, r, world)
                covered += list(range(n))[s]
            assert covered == list(range(n))
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 0)


def test_gather_rows_single_process():
    x = torch.arange(12).reshape(4, 3)
    assert sharding.gather_rows(x, [4]) is x
    with pytest.raises(ValueError):
        sharding.gather_rows(x, [3])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_items, result_queue):
    from oracle import ref
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)
        x = rng.standard_normal((n_items, 3, 5, 7)).astype(np.float32) * 3
        counts, _ = sharding.shard_bounds(n_items, world)
        mine = x[sharding.local_slice(n_items, rank, world)]
        # the per-shard work: Quantize then Dequantize with the reference arithmetic
        q = ref.quantize(mine, np.float32(0.05), np.uint8(128)) if mine.shape[0] else np.empty((0, 3, 5, 7), np.uint8)
        got = sharding.gather_rows(torch.from_numpy(q), counts)
        full = ref.quantize(x, np.float32(0.05), np.uint8(128))
        result_queue.put((rank, bool(np.array_equal(got.numpy(), full)), tuple(got.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_items", [8, 5, 1])
def test_two_rank_gather_matches_unsharded(n_items):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_items, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, shape in results:
        assert same, "rank %d gathered a different tensor" % rank
        assert shape == (n_items, 3, 5, 7)
