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

    def deferred(self, ops):
        """What a product before this norm needs to prepare it, if the operations can fold a norm
        into the products around it (see ``PreNormBlock``); else None."""
        make = getattr(ops, "norm_request", None)
        return make(self.weight, self.eps) if make is not None else None


register_part("norm", "rmsnorm", RMSNorm)
