"""Seeded synthetic tensors for the benchmark configurations.

The reference draws every weight and input from an unseeded ``Random()`` (for
example lib/layertypes/denseLayer.dart:33), so reproducible inputs need a
generator of our own.  This one is counter based: element ``i`` of tensor
``tensor_id`` under ``seed`` depends only on that triple, so any shard of a tensor
can be produced on any rank without generating the rest.

    u64   = splitmix64(seed * 0x9E3779B97F4A7C15 + tensor_id * 0xD1B54A32D192ED03 + counter)
    U[0,1) = (u64 >> 11) * 2**-53
    N(0,1) = Box-Muller over the pair (2i, 2i+1) of uniforms, cosine branch

Values are produced in float64 and rounded once to float32; checkers widen those
float32 values back to float64 so that input quantisation is never charged to a
kernel.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _key(seed: int, tensor_id: int) -> np.uint64:
    return np.uint64((seed * 0x9E3779B97F4A7C15 + tensor_id * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF)


def uniform01(seed: int, tensor_id: int, n: int, offset: int = 0) -> np.ndarray:
    """n float64 uniforms in [0,1), elements offset..offset+n-1 of the stream."""
    with np.errstate(over="ignore"):
        ctr = (np.arange(offset, offset + n, dtype=np.uint64) + _key(seed, tensor_id)) & _M64
    return (_splitmix64(ctr) >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)


def uniform(seed, tensor_id, shape, lo=0.0, hi=1.0, offset=0, dtype=np.float32):
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(seed, tensor_id, n, offset)).reshape(shape).astype(dtype)


def normal(seed, tensor_id, shape, std=1.0, offset=0, dtype=np.float32):
    n = int(np.prod(shape))
    u = uniform01(seed, tensor_id, 2 * n, 2 * offset)
    u1 = 1.0 - u[0::2]          # (0,1]
    u2 = u[1::2]
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (std * z).reshape(shape).astype(dtype)


def integers(seed, tensor_id, shape, high, offset=0):
    n = int(np.prod(shape))
    return np.minimum((uniform01(seed, tensor_id, n, offset) * high).astype(np.int64), high - 1).reshape(shape).astype(np.int32)


def xavier_uniform(seed, tensor_id, fan_in, fan_out, dtype=np.float32):
    a = float(np.sqrt(6.0 / (fan_in + fan_out)))
    return uniform(seed, tensor_id, (fan_in, fan_out), -a, a, dtype=dtype)
