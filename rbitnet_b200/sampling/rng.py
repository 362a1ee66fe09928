"""Counter-based uniform numbers for sampling: u = f(seed, request index, step).

The reference draws from an unseeded thread RNG
(crates/bitnet-core/src/llama/runtime.rs:62, :98), so its samples cannot be
repeated.  Here a draw depends only on the seed, on which request it is for and
on how many tokens that request has produced, never on the batch it ran in or
on the slot it held.
"""
from __future__ import annotations

_M = (1 << 64) - 1


def _mix(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M
    return x ^ (x >> 31)


def uniform(seed: int, request: int, step: int) -> float:
    """A float32-exact number in [0, 1)."""
    h = _mix(_mix(_mix(seed & _M) ^ (request & _M)) ^ (step & _M))
    return (h >> 40) / float(1 << 24)


def uniforms(seed: int, requests, steps):
    """``uniform(seed, r, s)`` for every pair of the two equally long sequences, as float32 values
    in a numpy array (the same numbers, made with wrapping 64-bit integer arithmetic)."""
    import numpy as np
    r = np.asarray(requests, dtype=np.uint64)
    t = np.asarray(steps, dtype=np.uint64)

    def mix(x):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))

    with np.errstate(over="ignore"):
        h = mix(mix(np.uint64(_mix(seed & _M)) ^ r) ^ t)
    return ((h >> np.uint64(40)).astype(np.float64) / float(1 << 24)).astype(np.float32)
