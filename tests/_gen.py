"""Deterministic synthetic inputs for the parity tests.

Values come from integer hashing only (no libm, no numpy RNG stream), so the
same (seed, shape) gives the same bits on every machine and numpy version:
the golden fixtures store outputs only and regenerate their inputs from here.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(x):
    """splitmix64 finaliser on a uint64 array."""
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def uniform_u32(seed, shape):
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        ctr = np.arange(n, dtype=np.uint64) + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        return (_mix(ctr) >> np.uint64(32)).astype(np.uint32).reshape(shape)


def normal(seed, shape, std=1.0):
    """Approximately N(0, std^2) float32: sum of twelve 16-bit uniforms - 6
    (Irwin-Hall), every step exact in float32."""
    n = int(np.prod(shape))
    acc = np.zeros(n, dtype=np.int64)
    with np.errstate(over="ignore"):
        base = np.arange(n, dtype=np.uint64) * np.uint64(3) + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        for r in range(3):
            h = _mix(base + np.uint64(r))
            for s in (0, 16, 32, 48):
                acc += ((h >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.int64)
    x = (acc.astype(np.float32) / np.float32(65536.0)) - np.float32(6.0)
    if std != 1.0:
        x = x * np.float32(std)
    return x.reshape(shape).astype(np.float32)


def randint(seed, lo, hi, shape=()):
    """Integers uniform in [lo, hi] (inclusive)."""
    u = uniform_u32(seed, shape if shape else (1,)).astype(np.int64)
    out = lo + (u % (hi - lo + 1))
    return out if shape else int(out[0])
