"""RMSNorm: y = x * w / sqrt(mean(x^2) + eps), all in float32
(crates/bitnet-core/src/llama/model.rs:93-100).  The weight multiplies directly (no 1+w)."""
from __future__ import annotations

import torch

from .base import Norm
from .registry import register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def weight_shapes(self):
        return {"weight": ((self.width,), "norm")}

    def bind(self, weights, ops):
        # exact in float32 whatever the stored dtype
        self.weight = weights["weight"].to(torch.float32).contiguous()

    def forward(self, ctx, x):
        return ctx.ops.rmsnorm(x, self.weight, self.eps)


register_part("norm", "rmsnorm", RMSNorm)
