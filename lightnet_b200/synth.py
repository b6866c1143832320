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
        f, c, k = l["filters"], l["in_c"], l["size"]
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
