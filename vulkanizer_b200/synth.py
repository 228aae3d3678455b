"""Seeded synthetic operands for the tests and the benchmark.

One counter-based generator (splitmix64 of seed and element index) defines every input, so "the same seeded
inputs" means the same bits on every machine and numpy version. Shapes and distributions restate the five
benchmark configurations: uniform[-1, 1] fp32, normal(0, sigma) rounded to f16 / bf16, uniform integers in
[-127, 127]. Values are produced in blocks so that a 8192 x 8192 operand needs no more than a few hundred MB
of host memory at a time.
"""
from __future__ import annotations

import numpy as np

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (x + np.uint64(0x9E3779B97F4A7C15)) & _MASK
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _MASK
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _MASK
        return z ^ (z >> np.uint64(31))


def _bits(seed: int, stream: int, first: int, count: int) -> np.ndarray:
    idx = np.arange(first, first + count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        key = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream))
        return _splitmix64(idx ^ key)


def _unit(seed: int, stream: int, first: int, count: int) -> np.ndarray:
    """Uniform in [0, 1) with 53 random bits."""
    return (_bits(seed, stream, first, count) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def uniform(seed: int, count: int, lo: float = -1.0, hi: float = 1.0, first: int = 0) -> np.ndarray:
    return (lo + (hi - lo) * _unit(seed, 0, first, count)).astype(np.float32)


def normal(seed: int, count: int, sigma: float = 1.0, first: int = 0) -> np.ndarray:
    """Box-Muller on two independent streams; element i depends on (seed, i) only."""
    u1 = 1.0 - _unit(seed, 1, first, count)  # (0, 1]
    u2 = _unit(seed, 2, first, count)
    return (sigma * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def int8_uniform(seed: int, count: int, first: int = 0) -> np.ndarray:
    """Integers uniform in [-127, 127]."""
    return ((_bits(seed, 3, first, count) >> np.uint64(16)) % np.uint64(255)).astype(np.int64).astype(np.int16).__sub__(127).astype(np.int8)


def blocks(total: int, block: int = 1 << 24):
    first = 0
    while first < total:
        n = min(block, total - first)
        yield first, n
        first += n
