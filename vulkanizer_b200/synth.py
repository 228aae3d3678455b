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


# ---- the same generator on a torch device, for operands too large to make on the host in reasonable time ----
#
# Integers are 64-bit two's complement, whose products and sums agree with the unsigned ones above in every bit; logical right
# shifts are arithmetic shifts with the sign extension masked off. The uniform values are therefore identical; the normal ones
# go through log, sqrt and cos in float64 like the numpy form, whose last-place differences between math libraries vanish in
# the rounding to float32 except in about one value in 10^8 (tests/test_oracle_cpu.py compares the two forms).

def _i64(value: int) -> int:
    value &= 0xFFFFFFFFFFFFFFFF
    return value - (1 << 64) if value >= (1 << 63) else value


def _lsr(x, n: int):
    return (x >> n) & ((1 << (64 - n)) - 1)


def _splitmix64_torch(x):
    z = x + _i64(0x9E3779B97F4A7C15)
    z = (z ^ _lsr(z, 30)) * _i64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _i64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def _unit_torch(torch, seed: int, stream: int, first: int, count: int, device):
    key = int(_splitmix64(np.array([(seed * 0x100000001B3 + stream) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0])
    idx = torch.arange(first, first + count, dtype=torch.int64, device=device)
    bits = _splitmix64_torch(idx ^ _i64(key))
    return _lsr(bits, 11).to(torch.float64) * (1.0 / 9007199254740992.0)


def normal_torch(torch, seed: int, count: int, sigma: float = 1.0, first: int = 0, device="cuda"):
    """normal() above as a float32 tensor on `device`."""
    u1 = 1.0 - _unit_torch(torch, seed, 1, first, count, device)
    u2 = _unit_torch(torch, seed, 2, first, count, device)
    return (sigma * torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * np.pi * u2)).to(torch.float32)


def fill_normal_torch(torch, out, seed: int, sigma: float = 1.0, first: int = 0, block: int = 1 << 24):
    """Fills the 1-d tensor `out` (any floating type) with elements first .. first + len(out) of the normal stream of `seed`,
    rounded from float32 to out's type (round to nearest even, as the host-side conversions do)."""
    for start in range(0, out.numel(), block):
        n = min(block, out.numel() - start)
        out[start:start + n] = normal_torch(torch, seed, n, sigma, first + start, out.device).to(out.dtype)
    return out
