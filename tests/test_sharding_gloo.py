"""Host-side logic of the multi-GPU path on CPU: shard arithmetic, and a world_size-2 gloo run
of the bench's aggregation (sum of units over the slowest rank's time, no data-path collective)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from VAR_Q.sharding import aggregate_throughput, cfg_rows, shard_images


def test_shards_cover_the_batch_without_splitting_cfg_pairs():
    for n in (1, 7, 32, 64, 65):
        for world in (1, 2, 4, 8):
            seen = []
            for r in range(world):
                b, e = shard_images(n, world, r)
                assert 0 <= b <= e <= n and (e - b) in (n // world, n // world + 1)
                rows = cfg_rows(b, e, n)
                assert len(rows) == 2 * (e - b)
                assert all(rows[i] + n == rows[i + (e - b)] for i in range(e - b))   # cond / uncond of one image together
                seen += list(range(b, e))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        shard_images(8, 2, 2)
    with pytest.raises(ValueError):
        aggregate_throughput([1.0], [0.0])


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, n_images, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    b, e = shard_images(n_images, world, rank)
    units = float(e - b)
    seconds = 0.5 * (rank + 1)                       # rank 1 is the slow one
    dist.barrier()
    t = torch.tensor([seconds], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)         # timing only: the data path has no collective
    u = torch.tensor([units], dtype=torch.float64)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    if rank == 0:
        out.put((u.item(), t.item()))
    dist.destroy_process_group()


def test_world_size_2_aggregation_over_gloo():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 65, out)) for r in range(2)]
    for p in procs:
        p.start()
    units, slowest = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert units == 65.0 and slowest == 1.0
    assert aggregate_throughput([33.0, 32.0], [0.5, 1.0]) == units / slowest
