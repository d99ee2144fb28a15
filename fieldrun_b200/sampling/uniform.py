"""Uniform numbers for sampling, as a function of (seed, request, step).

A counter-based generator (the SplitMix64 finaliser over a mixed counter) instead
of a stateful one: the number a request's n-th token is drawn with does not
depend on which other requests run beside it or in which order batches finish.
The value has 24 random bits, so it is exact in float32 and always below 1.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) for the ``step``-th generated token of request ``request``."""
    h = _mix(seed & _MASK)
    h = _mix(h ^ (request & _MASK))
    h = _mix(h ^ (step & _MASK))
    return (h >> 40) / float(1 << 24)
