"""The batch axis over the GPUs of one machine.

Matrices of a batch are independent, so a batch is split into contiguous ranges,
one per GPU, with no exchange between them: no collective and no NCCL. The
reference has one GPU and nothing like this; the split follows its batch
chunking (src/qr_householder.mm:323-344), a chunk per device instead of a chunk
per command buffer.

Two ways to run on several GPUs:
  * one process per GPU (torchrun): each rank calls `shard_batch(batch, rank,
    world)` for its range and `metal_linalg_torch.qr` on its own shard;
  * one process driving several GPUs: `qr_sharded([a0, a1, ...])` on tensors
    that already live on their GPUs enqueues every shard's kernels on its
    device's current stream without waiting for any of them.
"""
import torch


def shard_batch(batch, rank, world):
    """The contiguous range [begin, end) of a batch of `batch` matrices that rank
    `rank` of `world` owns; ranges differ in size by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"shard_batch: rank {rank} of {world}")
    return batch * rank // world, batch * (rank + 1) // world


def qr_sharded(shards, mode="reduced"):
    """QR of each tensor of `shards` on the GPU it lives on. Returns a list of
    (Q, R), in order. Nothing is copied between devices and nothing is waited
    for: each result is ready on its device's current stream."""
    from . import qr
    out = []
    for a in shards:
        if not isinstance(a, torch.Tensor) or a.device.type != "cuda":
            raise ValueError("qr_sharded: every shard must be a CUDA tensor on the GPU that is to factor it")
        out.append(qr(a, mode))
    return out
