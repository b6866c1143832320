"""Seeded synthetic weights and inputs of the benchmark configurations (no dataset or .weights file is
needed: every benchmark uses random-init networks and uniform images)."""
from __future__ import annotations

import numpy as np


def he_weights(layers, seed: int = 0, bn_identity: bool = True) -> np.ndarray:
    """Darknet .weights payload (per conv: biases, [scales, mean, variance], weights) for a list of layer-info
    dicts: conv weights He-normal N(0, sqrt(2/fan_in)), biases 0, BN gamma=1 beta=0 mean=0 var=1.
    bn_identity=False draws plausible BN statistics instead, to exercise the fold."""
    rng = np.random.default_rng(seed)
    parts = []
    for l in layers:
        if l["kind"] != "conv":
            continue
        f, c, k = l["filters"], l["in_c"] // l.get("groups", 1), l["size"]   # channels each filter reads
        fan_in = c * k * k
        if bn_identity or not l["bn"]:
            parts.append(np.zeros(f, np.float32) if bn_identity else rng.normal(0, 0.1, f).astype(np.float32))
        else:
            parts.append(rng.normal(0, 0.1, f).astype(np.float32))
        if l["bn"]:
            if bn_identity:
                parts += [np.ones(f, np.float32), np.zeros(f, np.float32), np.ones(f, np.float32)]
            else:
                parts += [rng.uniform(0.5, 1.5, f).astype(np.float32), rng.normal(0, 0.2, f).astype(np.float32),
                          rng.uniform(0.5, 2.0, f).astype(np.float32)]
        parts.append(rng.normal(0, np.sqrt(2.0 / fan_in), f * fan_in).astype(np.float32))
    return np.concatenate(parts)


def uniform_images(batch, channels, height, width, seed: int = 1) -> np.ndarray:
    return np.random.default_rng(seed).random((batch, channels, height, width), dtype=np.float32)


COCO_ANCHORS = [(10, 13), (16, 30), (33, 23), (30, 61), (62, 45), (59, 119), (116, 90), (156, 198), (373, 326)]


def stress_heads(batch, grids=(80, 40, 20), classes=80, seed: int = 2, obj_mu: float = -4.0, chunk: int = 16):
    """Raw [yolo] head tensors of the decode + NMS stress workload: 3 anchors per cell, xy logits N(0,1), wh logits
    N(0,0.5) (the decode multiplies exp(wh) by the anchors), objectness and class logits N(obj_mu, 2).
    Returns one f32 array [batch, 3*(5+classes), g, g] per grid, generated `chunk` images at a time."""
    rng = np.random.default_rng(seed)
    heads = []
    for g in grids:
        t = np.empty((batch, 3, 5 + classes, g, g), np.float32)
        for b0 in range(0, batch, chunk):
            b1 = min(batch, b0 + chunk)
            n = b1 - b0
            t[b0:b1, :, 0:2] = rng.standard_normal((n, 3, 2, g, g), dtype=np.float32)
            t[b0:b1, :, 2:4] = rng.standard_normal((n, 3, 2, g, g), dtype=np.float32) * np.float32(0.5)
            t[b0:b1, :, 4:] = rng.standard_normal((n, 3, 1 + classes, g, g), dtype=np.float32) * np.float32(2.0) + np.float32(obj_mu)
        heads.append(t.reshape(batch, 3 * (5 + classes), g, g))
    return heads


def stress_head_specs(grids=(80, 40, 20), classes=80):
    return [dict(gw=g, gh=g, classes=classes, anchors=COCO_ANCHORS[3 * i:3 * i + 3], scale_x_y=1.0, new_coords=0) for i, g in enumerate(grids)]
