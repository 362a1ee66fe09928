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
