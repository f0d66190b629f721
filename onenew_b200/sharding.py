"""Batch sharding for multi-GPU inference: images are independent, so a global batch is cut into
contiguous per-rank slices and nothing is exchanged between ranks (the reference itself is strictly
per-image, host/ops/conv.h:43).  Rank r of `world` takes images [start, stop)."""


def shard_range(global_batch, world, rank):
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per
