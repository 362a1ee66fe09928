"""Arrangement of a layer's parts.  "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x))
(crates/bitnet-core/src/llama/model.rs:237-306).  The residual stream x is float32."""
from __future__ import annotations

from .registry import register_part, build_part


class PreNormBlock:
    def __init__(self, spec):
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.feed_forward = build_part("feed_forward", spec.feed_forward)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.ffn_norm = build_part("norm", spec.ffn_norm)

    def parts(self):
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}

    def run(self, ctx, x, entry: int) -> None:
        h = self.mixer_norm.forward(ctx, x)
        self.mixer.forward(ctx, h, entry, accumulate_into=x)
        h = self.ffn_norm.forward(ctx, x)
        self.feed_forward.forward(ctx, h, accumulate_into=x)


register_part("block", "pre_norm", PreNormBlock)
