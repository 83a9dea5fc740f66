"""Seeded synthetic tensors that are bit-identical on every machine and library version.

A counter-based integer hash (splitmix64 finaliser) drives everything, so fixtures need to store
only outputs: the inputs are regenerated from (seed, shape).  Values are the centred sum of four
uniforms scaled to the requested standard deviation -- bell-shaped like the N(0, sigma) inputs the
benchmark configurations describe, with exact zeros and both signs present.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def bell(seed: int, shape, sigma: float = 1.0) -> np.ndarray:
    """fp32 tensor, mean 0, standard deviation ~sigma, values on a grid of 1/2048 * sigma * sqrt(3)."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x100000001B3)
        h = _mix(idx)
    parts = [((h >> np.uint64(16 * i)) & np.uint64(0xFFFF)).astype(np.int64) for i in range(4)]
    s = parts[0] + parts[1] + parts[2] + parts[3] - 2 * 65535          # in [-131070, 131070], variance 4*(65536^2)/12
    scale = np.float32(sigma / (65536.0 * np.sqrt(4.0 / 12.0)))
    return (s.astype(np.float32) * scale).reshape(shape)


def uniform01(seed: int, shape) -> np.ndarray:
    """fp32 tensor in [0, 1) on a 2^-24 grid."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x100000001B3)
        h = _mix(idx)
    return ((h >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)).reshape(shape)


def conv_case(seed: int, batch: int, c: int, h: int, w: int, n: int, ks: int):
    """(x [batch,c,h,w] ~ sigma 1, weights [n,c,ks,ks] ~ sigma 0.05, biases [n] ~ sigma 0.01)."""
    x = bell(seed * 3 + 1, (batch, c, h, w), 1.0)
    wt = bell(seed * 3 + 2, (n, c, ks, ks), 0.05)
    b = bell(seed * 3 + 3, (n,), 0.01)
    return x, wt, b
