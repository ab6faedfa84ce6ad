"""The random numbers of random-weights models restated in numpy (test infrastructure): the library's
host generator (model folders) and its device fill kernel (`csrc/utility.cu`) must both give
these values bit for bit; the definition is that of `csrc/random_init.h`.

    key(seed, name) = fnv1a64(name) ^ (seed * G)            G = 0x9E3779B97F4A7C15, 64-bit wrap-around
    base            = fin(key + G)                           fin = the splitmix64 finaliser
    r_j(i)          = fin(base + (3 i + j + 1) G), j = 0..2
    z(i)            = sum of the twelve 16-bit fields of r_0..r_2, minus 393210
    value(i)        = float32(z(i)) * (std / 65536) + mean   each operation rounded once in float32

The reference has no random models (its tests randomise tensors per operator, test/checker.cpp:162-204).
"""
from __future__ import annotations

import numpy as np

_G = np.uint64(0x9E3779B97F4A7C15)
_M64 = (1 << 64) - 1


def _fin(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def random_key(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h ^ ((int(seed) * 0x9E3779B97F4A7C15) & _M64)


def random_values(seed: int, name: str, n: int, std: float = 0.02, mean: float = 0.0) -> np.ndarray:
    """float32 [n]: values 0..n-1 of the stream of (seed, name)."""
    with np.errstate(over="ignore"):
        base = _fin(np.array([random_key(seed, name)], dtype=np.uint64) + _G)[0]
        total = np.zeros(n, dtype=np.int64)
        i3 = np.arange(n, dtype=np.uint64) * np.uint64(3)
        for j in (1, 2, 3):
            r = _fin(base + (i3 + np.uint64(j)) * _G)
            for shift in (0, 16, 32, 48):
                total += ((r >> np.uint64(shift)) & np.uint64(0xFFFF)).astype(np.int64)
    z = (total - 393210).astype(np.float32)
    scale = np.float32(std) / np.float32(65536.0)
    return (z * scale + np.float32(mean)).astype(np.float32)


def to_bfloat16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> the 16 bits of the nearest bfloat16 (ties to even), as uint16."""
    u = x.astype(np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)
