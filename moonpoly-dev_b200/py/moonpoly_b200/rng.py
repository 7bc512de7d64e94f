"""Stateless, platform-independent input generator for tests and benchmarks.

    r(seed, stream, i) = splitmix64( splitmix64(seed XOR (stream << 56)) + i )

uniform u = (r >> 11) * 2**-53; normals by Box-Muller on (r(2i), r(2i+1)).
One stream id per tensor: A = 0, B / W = 1, a_scales = 2, b_scales = 3,
shape draws = 4, bias = 5.  The generator does not depend on torch's (device-
and version-dependent) generators, so every box sees identical inputs.
"""
from __future__ import annotations

import numpy as np

STREAM_A, STREAM_B, STREAM_A_SCALE, STREAM_B_SCALE, STREAM_SHAPES, STREAM_BIAS = range(6)

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def raw(seed: int, stream: int, count: int, offset: int = 0) -> np.ndarray:
    base = _splitmix64(np.array([(seed ^ (stream << 56)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0]
    idx = np.arange(offset, offset + count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _splitmix64((base + idx) & _M64)


def uniform01(seed: int, stream: int, count: int, offset: int = 0) -> np.ndarray:
    return (raw(seed, stream, count, offset) >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)


def uniform(seed: int, stream: int, shape, lo: float, hi: float, dtype=np.float32) -> np.ndarray:
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(seed, stream, n)).astype(dtype).reshape(shape)


def normal(seed: int, stream: int, shape, scale: float = 1.0, dtype=np.float16) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, dtype=dtype)
    chunk = 1 << 22                      # bound temporaries for GB-sized tensors
    for s in range(0, n, chunk):
        c = min(chunk, n - s)
        u = uniform01(seed, stream, 2 * c, 2 * s)
        u1 = np.maximum(u[0::2], 2.0 ** -53)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u[1::2])
        out[s:s + c] = (scale * z).astype(dtype)
    return out.reshape(shape)


def int8_uniform(seed: int, stream: int, shape, lo: int = -127, hi: int = 127) -> np.ndarray:
    n = int(np.prod(shape))
    span = np.uint64(hi - lo + 1)
    return ((raw(seed, stream, n) >> np.uint64(16)) % span).astype(np.int64).__add__(lo).astype(np.int8).reshape(shape)


def small_ints(seed: int, stream: int, shape, lo: int = -2, hi: int = 2, dtype=np.float16) -> np.ndarray:
    """Integer-valued entries, the value range the reference's CTest programmes use
    (TensorFillRandomUniform(view, 1, 2, -2, bits=0)): every product and partial sum
    is exact, so any correct GEMM reproduces the result bit for bit."""
    n = int(np.prod(shape))
    span = np.uint64(hi - lo + 1)
    return (((raw(seed, stream, n) >> np.uint64(16)) % span).astype(np.int64) + lo).astype(dtype).reshape(shape)


def log_uniform_ints(seed: int, stream: int, count: int, lo: int, hi: int) -> list[int]:
    """M_i = clamp(round(hi ** u_i), lo, hi), u ~ U[0,1): the INT8 scaled_mm M draws."""
    u = uniform01(seed, stream, count)
    vals = np.rint(np.power(float(hi), u)).astype(np.int64)
    return [int(v) for v in np.clip(vals, lo, hi)]


def mixed_batch_sizes(seed: int, stream: int, count: int) -> list[int]:
    """70 % decode (M in [1,256]) / 30 % prefill (M in [512,8192]) token batches."""
    u = uniform01(seed, stream, 2 * count)
    out = []
    for i in range(count):
        pick, v = u[2 * i], u[2 * i + 1]
        out.append(1 + int(v * 256) if pick < 0.7 else 512 + int(v * (8192 - 512 + 1)))
    return out
