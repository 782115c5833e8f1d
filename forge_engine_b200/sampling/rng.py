"""The counter-based uniform the sampling kernel draws with, restated in Python.

``uniform(seed, counter)`` returns exactly the float the kernel computes for the same
pair, so a sampled sequence can be reproduced on the host: seed = the request's seed,
counter = how many tokens the request has sampled before this one.
"""

from __future__ import annotations

_MASK = (1 << 64) - 1


def splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, counter: int) -> float:
    """24 random bits scaled into [0, 1)."""
    mixed = splitmix64(splitmix64(seed & _MASK) ^ ((counter * 0xD1342543DE82EF95) & _MASK))
    return (mixed >> 40) / 16777216.0
