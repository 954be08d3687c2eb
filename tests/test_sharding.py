"""The multi-GPU split of the batch axis, on CPU: ranges tile the batch, and a
world of two gloo ranks, each taking its own range with no data exchanged between
them, reproduces the single-rank result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import harness
from metal_linalg_torch import shard_batch


@pytest.mark.parametrize("batch", [0, 1, 7, 8, 1024, 262144])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_ranges_tile_the_batch(batch, world):
    ranges = [shard_batch(batch, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == batch
    for (b0, e0), (b1, e1) in zip(ranges, ranges[1:]):
        assert e0 == b1
    sizes = [e - b for b, e in ranges]
    assert max(sizes) - min(sizes) <= 1


def test_bad_rank_is_rejected():
    with pytest.raises(ValueError):
        shard_batch(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, batch, path):
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [os.path.join(here, "oracle"), os.path.join(here, "metal-linalg_b200")]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import harness as h
    from metal_linalg_torch import shard_batch as shard, workloads
    a = workloads.generate("c1_32x32", batch=batch).numpy()
    b0, b1 = shard(batch, rank, world)
    # each rank factors its own range (the CPU oracle stands in for the GPU here:
    # the split, not the kernel, is under test) and nothing crosses ranks
    q, r = h.oracle_qr(a[b0:b1])
    np.savez(f"{path}.{rank}.npz", q=q, r=r, b0=b0, b1=b1)
    # the bench's timing pattern: barrier, then the max over ranks
    dist.barrier()
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.destroy_process_group()


def test_two_ranks_reproduce_one(tmp_path):
    from metal_linalg_torch import workloads
    batch, world = 37, 2
    path = str(tmp_path / "shard")
    mp.spawn(_rank_main, args=(world, _free_port(), batch, path), nprocs=world, join=True)
    a = workloads.generate("c1_32x32", batch=batch).numpy()
    q_all, r_all = harness.oracle_qr(a)
    covered = 0
    for rank in range(world):
        z = np.load(f"{path}.{rank}.npz")
        b0, b1 = int(z["b0"]), int(z["b1"])
        assert np.array_equal(z["q"], q_all[b0:b1]) and np.array_equal(z["r"], r_all[b0:b1])
        covered += b1 - b0
    assert covered == batch
