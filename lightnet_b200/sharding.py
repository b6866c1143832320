"""Batch sharding of the detector over several GPUs: one process per GPU, no collective on the data path.

Images are independent, so rank r runs the whole network on its own contiguous slice of the batch and only the
detections (a few KB per image) travel, over the host, after the device work is done.  The reference has no multi-GPU
path of its own: its executor owns one device (lightnet-runtime/src/runtime/gpu_types.rs:227-244) and a caller who
wants several runs one executor per device; this module is that caller.

`torch.distributed` is the only plumbing (backend "nccl" with GPUs, "gloo" in CPU tests); nothing here touches device
memory, so the logic is testable without a GPU by passing any callable as the per-rank detector.
"""
from __future__ import annotations

import numpy as np


def shard_bounds(total: int, world: int):
    """[(start, stop)] per rank: contiguous, in rank order, sizes differing by at most one (earlier ranks take the extra)."""
    if world <= 0:
        raise ValueError("world must be positive")
    if total < 0:
        raise ValueError("total must not be negative")
    base, extra = divmod(total, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def pad_to_capacity(images: np.ndarray, capacity: int) -> np.ndarray:
    """A network is built for a fixed batch; a short (or empty) shard is padded with zero images whose detections are dropped."""
    n = images.shape[0]
    if n > capacity:
        raise ValueError("shard of %d images exceeds the per-rank batch %d" % (n, capacity))
    if n == capacity:
        return images
    pad = np.zeros((capacity - n,) + images.shape[1:], images.dtype)
    return np.concatenate([images, pad], 0)


class ShardedDetector:
    """detect(images) over all ranks of a process group.

    detect_fn(images[capacity, C, H, W]) -> list of `capacity` per-image detection arrays; every rank passes its own (on a
    GPU box: `GpuExecutableNetwork.detect` of a network created with batch = capacity on that rank's device).
    Every rank calls `detect` with the same global batch (or rank 0's is broadcast with broadcast_input=True) and every
    rank gets the detections of all images, in input order."""

    def __init__(self, detect_fn, capacity: int, group=None):
        import torch.distributed as dist

        self.detect_fn = detect_fn
        self.capacity = int(capacity)
        self.group = group
        self.dist = dist
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def detect(self, images: np.ndarray, broadcast_input: bool = False):
        if broadcast_input and self.world > 1:
            box = [images if self.rank == 0 else None]
            self.dist.broadcast_object_list(box, src=0, group=self.group)
            images = box[0]
        total = images.shape[0]
        if total > self.capacity * self.world:
            raise ValueError("%d images exceed %d ranks x batch %d" % (total, self.world, self.capacity))
        start, stop = shard_bounds(total, self.world)[self.rank]
        local = []
        if stop > start:
            local = list(self.detect_fn(pad_to_capacity(np.ascontiguousarray(images[start:stop]), self.capacity)))[: stop - start]
        if self.world == 1:
            return local
        parts = [None] * self.world
        self.dist.all_gather_object(parts, local, group=self.group)
        out = []
        for p in parts:
            out.extend(p)
        if len(out) != total:
            raise RuntimeError("gathered %d detection lists for %d images" % (len(out), total))
        return out


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Timing convention of the benchmark: a multi-GPU step takes as long as its slowest rank."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
