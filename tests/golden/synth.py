"""Portable synthetic-data helpers shared by the golden-vector generator and the tests.

Large inputs are not stored in the fixtures; they are regenerated from a seed with the integer
hash below, which uses only wrapping uint64 arithmetic and therefore yields identical bits on any
machine and numpy version.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(z):
    """splitmix64 finaliser on a uint64 array."""
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def hash_u64(seed, n):
    with np.errstate(over="ignore"):
        base = _mix(np.full(1, seed, dtype=np.uint64))[0]
        return _mix(np.arange(n, dtype=np.uint64) * np.uint64(0xD1342543DE82EF95) + base)


def uniform(seed, shape, lo=0.0, hi=1.0):
    """float32 uniform in [lo, hi) with 24 random mantissa bits."""
    n = int(np.prod(shape))
    u = (hash_u64(seed, n) >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return (lo + (hi - lo) * u).astype(np.float32).reshape(shape)


def normal(seed, shape, mean=0.0, std=1.0):
    """float32 normal via Box-Muller on two hashed uniforms."""
    n = int(np.prod(shape))
    u1 = ((hash_u64(seed, n) >> np.uint64(11)).astype(np.float64) + 1.0) / float(1 << 53)
    u2 = (hash_u64(seed ^ 0x5DEECE66D, n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).astype(np.float32).reshape(shape)


def integers(seed, shape, lo, hi):
    """int64 uniform in [lo, hi)."""
    n = int(np.prod(shape))
    return (lo + (hash_u64(seed, n) % np.uint64(hi - lo)).astype(np.int64)).reshape(shape)


def anchor_pairs(seed, n_detectors, n_anchors, n_inputs):
    """int32 [Nt, Nc, 2] anchor pairs with distinct ends inside a pair, uniform over the inputs."""
    a1 = integers(seed, (n_detectors, n_anchors), 0, n_inputs)
    off = integers(seed + 1, (n_detectors, n_anchors), 1, n_inputs)
    a2 = (a1 + off) % n_inputs
    return np.stack([a1, a2], axis=-1).astype(np.int32)


def sparse_images(seed, shape, density=0.19, lo=0.5, hi=1.0):
    """float32 tensor, `density` of the entries uniform in [lo, hi), the rest exactly zero."""
    mask = uniform(seed, shape) < density
    vals = uniform(seed + 7, shape, lo, hi)
    return np.where(mask, vals, np.float32(0.0)).astype(np.float32)
