"""Position encodings.

Rotary: each head's pairs are rotated by angle = pos * theta^(-2i/D), the
inverse frequencies and the angle in float32
(crates/bitnet-core/src/llama/model.rs:122-136).  ``pairing`` "interleaved"
rotates (2i, 2i+1) as the reference does; "half" rotates (i, i+D/2), the row
order of checkpoints with Hugging Face tensor names.  Keys are cached after the
rotation, values are not rotated (:242-257).
"""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, pairing: str = "half", max_positions: int = 0):
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, found {head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.head_dim, self.theta, self.pairing = int(head_dim), float(theta), pairing
        self.max_positions = int(max_positions)
        self.inv_freq = None

    def bind(self, weights, ops):
        i = torch.arange(self.head_dim // 2, dtype=torch.float32)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), 2.0 * i / self.head_dim)
        self.inv_freq = inv.to(ops.device)

    def rotary(self):
        return self.inv_freq, self.pairing == "interleaved", self.head_dim


class NoPositionEncoding(PositionEncoding):
    """Positions enter only through the causal mask."""
    def __init__(self, **_):
        pass


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
