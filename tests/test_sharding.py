"""Multi-GPU host logic on CPU: two gloo ranks shard a batch, run a stand-in detector, gather detections."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from lightnet_b200 import sharding


def fake_detect(images):
    """Stand-in for a per-rank network: one record per image that encodes its content, variable count per image."""
    out = []
    for img in images:
        n = int(img.sum()) % 4
        out.append(np.full((n, 7), float(img.sum()), np.float32))
    return out


def worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        det = sharding.ShardedDetector(fake_detect, capacity=3)
        rng = np.random.default_rng(0)
        ok = True
        for total in (6, 5, 1, 0):   # full, ragged, one rank idle, empty
            images = rng.integers(0, 9, (total, 1, 2, 2)).astype(np.float32)
            got = det.detect(images)
            ref = fake_detect(images)
            ok &= len(got) == total and all(np.array_equal(a, b) for a, b in zip(got, ref))
        # broadcast from rank 0: the other rank passes garbage
        images = rng.integers(0, 9, (4, 1, 2, 2)).astype(np.float32)
        got = det.detect(images if rank == 0 else np.zeros((1, 1, 2, 2), np.float32), broadcast_input=True)
        box = [images if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ok &= all(np.array_equal(a, b) for a, b in zip(got, fake_detect(box[0])))
        try:
            det.detect(np.zeros((7, 1, 2, 2), np.float32))
            ok = False
        except ValueError:
            pass
        ok &= sharding.max_over_ranks(10.0 + rank) == 10.0 + world - 1
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_shard_bounds():
    assert sharding.shard_bounds(64, 8) == [(8 * r, 8 * r + 8) for r in range(8)]
    assert sharding.shard_bounds(5, 2) == [(0, 3), (3, 5)]
    assert sharding.shard_bounds(1, 4) == [(0, 1), (1, 1), (1, 1), (1, 1)]
    assert sharding.shard_bounds(0, 2) == [(0, 0), (0, 0)]
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 0)
    x = np.ones((2, 3, 4, 4), np.float32)
    assert sharding.pad_to_capacity(x, 4).shape == (4, 3, 4, 4) and sharding.pad_to_capacity(x, 4)[2:].sum() == 0
    with pytest.raises(ValueError):
        sharding.pad_to_capacity(x, 1)


def test_sharded_detect_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert results.get(0) and results.get(1)
