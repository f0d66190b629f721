"""The N>1 path on CPU: two gloo ranks shard a seeded global batch with no data-path collective, and
the shards reassemble to exactly the global batch (CPU only; uses the reference operators as the
per-rank "model" when they are built, a checksum otherwise)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from onenew_b200.sharding import shard_range  # noqa: E402


def test_shard_range_partitions():
    for world in (1, 2, 4, 8):
        cuts = [shard_range(256, world, r) for r in range(world)]
        assert cuts[0][0] == 0 and cuts[-1][1] == 256
        assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        shard_range(10, 4, 0)
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import bench
    a, b = shard_range(8, world, rank)
    x = bench.make_inputs("resnet50", b - a, 100 + a)                    # same seeding rule as bench.py
    y = x.reshape(b - a, -1).astype(np.float64).sum(axis=1)        # stands in for the per-image result
    np.save(os.path.join(out_dir, f"r{rank}.npy"), y)
    # the only communication: the barrier and the max-over-ranks of the step time
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_without_exchange(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.concatenate([np.load(tmp_path / f"r{r}.npy") for r in range(world)])
    sys.path.insert(0, ROOT)
    import bench
    whole = bench.make_inputs("resnet50", 8, 100)     # the global batch, seeded per image index
    assert np.array_equal(got, whole.reshape(8, -1).astype(np.float64).sum(axis=1))
