"""Interfaces of the parts a layer is put together from.

A part gets its sizes and constants as constructor parameters, says which
weights it needs (``weight_shapes``), receives them (``bind``) and then runs on
the tokens of a step (``forward``).  Kernels are reached only through
``ctx.ops``; a part never asks which model it is in.

Roles:
  norm              forward(ctx, x[T,E] float32) -> h[T,E] in the compute dtype
  position          describes how positions enter a mixer (``rotary()``)
  mixer             forward(ctx, h, entry, accumulate_into) ; adds its result to the
                    float32 residual stream; may need cache (``cache_need``) and
                    fixed-size per-sequence state (``state_need``)
  feed_forward      forward(ctx, h, accumulate_into)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer stores per position.  Layers with equal needs share a cache group
    (one pool of pages per stored tensor); ``window`` None means every earlier position is kept.

    By default two tensors are stored per position, keys and values, each of ``n_kv_heads``
    heads of ``head_dim`` values.  ``streams`` names other contents: a tuple of (heads, width)
    pairs, one per stored tensor, for instance ``((1, 96),)`` for a mixer that keeps one vector
    per position, or keys and values of different widths."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    streams: Optional[Tuple[Tuple[int, int], ...]] = None

    def stream_shapes(self) -> Tuple[Tuple[int, int], ...]:
        if self.streams is not None:
            return tuple((int(h), int(w)) for h, w in self.streams)
        return ((self.n_kv_heads, self.head_dim), (self.n_kv_heads, self.head_dim))


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence: a tensor of ``shape`` and ``dtype`` per slot,
    zeroed when the slot is handed out."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    role = ""

    def weight_shapes(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """key -> (shape, "matrix" | "norm")"""
        return {}

    def bind(self, weights: Dict[str, torch.Tensor], ops) -> None:
        """Take the weights (already on the device, as stored in the files)."""


class Norm(Part):
    role = "norm"

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    role = "position"

    def rotary(self):
        """None, or (inv_freq float32 [D/2] device tensor, interleaved: bool, rot_dim)."""
        return None


class Mixer(Part):
    role = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx, h: torch.Tensor, entry: int, accumulate_into: torch.Tensor) -> None:
        """h[T, E]: the normed input rows of this step's tokens.  ``entry`` is the
        index of this run in the schedule (``ctx.cache_view(entry)``,
        ``ctx.state_view(entry)``).  The result is added to ``accumulate_into``."""
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"

    def forward(self, ctx, h: torch.Tensor, accumulate_into: torch.Tensor) -> None:
        raise NotImplementedError
