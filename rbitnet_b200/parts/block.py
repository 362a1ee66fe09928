"""Arrangement of a layer's parts.  "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x))
(crates/bitnet-core/src/llama/model.rs:237-306).  The residual stream x is float32.

An arrangement is a class built from a ``BlockSpec`` with ``parts()`` (name -> part, every part
whose weights are to be bound; the names are those of ``BlockSpec.parts``) and
``run(ctx, x, entry)``.  ``build_parts`` makes every part a spec names, whatever it is called."""
from __future__ import annotations

from .registry import register_part, build_part


def build_parts(spec) -> dict:
    """name -> part for every entry of ``spec.parts``."""
    return {name: build_part(spec.role_of(name), ps) for name, ps in spec.parts.items()}


class PreNormBlock:
    def __init__(self, spec):
        self.spec = spec
        self._parts = build_parts(spec)
        missing = [n for n in ("mixer", "feed_forward", "mixer_norm", "ffn_norm") if n not in self._parts]
        if missing:
            raise ValueError(f"a pre_norm block needs the parts {missing}")
        self.mixer, self.feed_forward = self._parts["mixer"], self._parts["feed_forward"]
        self.mixer_norm, self.ffn_norm = self._parts["mixer_norm"], self._parts["ffn_norm"]

    def parts(self):
        return self._parts

    def run(self, ctx, x, entry: int) -> None:
        h = self.mixer_norm.forward(ctx, x)
        self.mixer.forward(ctx, h, entry, accumulate_into=x)
        h = self.ffn_norm.forward(ctx, x)
        self.feed_forward.forward(ctx, h, accumulate_into=x)


register_part("block", "pre_norm", PreNormBlock)
