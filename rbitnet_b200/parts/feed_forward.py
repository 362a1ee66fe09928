"""Dense gated feed-forward: down( act(gate h) * (up h) ), act = SiLU, no bias
(crates/bitnet-core/src/llama/model.rs:116-120, 296-306).  The activation and
the product are float32 before any rounding to the compute dtype."""
from __future__ import annotations

from .base import FeedForward
from .registry import register_part


class GatedDense(FeedForward):
    def __init__(self, width: int, inner: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated feed-forward: activation {activation!r} is not built (only 'silu')")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.w_gate_up = self.w_down = None

    def weight_shapes(self):
        return {"gate": ((self.inner, self.width), "matrix"), "up": ((self.inner, self.width), "matrix"),
                "down": ((self.width, self.inner), "matrix")}

    def bind(self, weights, ops):
        self.w_gate_up = ops.prepare_gate_up(weights["gate"], weights["up"])
        self.w_down = ops.prepare_linear([weights["down"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    def forward(self, ctx, h, accumulate_into, then_norm=None):
        t = ctx.ops.gated_linear(h, self.w_gate_up)        # silu(gate h) * (up h)
        if then_norm is None:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into)
        else:
            ctx.ops.linear(t, self.w_down, accumulate_into=accumulate_into, then_norm=then_norm)


register_part("feed_forward", "gated_dense", GatedDense)
