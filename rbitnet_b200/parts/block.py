"""Arrangement of a layer's parts.  "pre_norm": x += mixer(norm(x)); x += feed_forward(norm(x))
(crates/bitnet-core/src/llama/model.rs:237-306).  The residual stream x is float32.

A norm between two products.  For a few tokens a norm is a kernel that does a microsecond of work
and costs three in a chain of dependent launches.  Where the operations offer it
(``ops.norm_request``), the norm's own part says what it needs (``deferred``) and the parts on both
sides say that they pass it on (``folds_norms``), the block asks the part before a norm to have its
last product leave the rows times the norm's weights, with their sums of squares, and gives those
to the part after the norm, whose first product multiplies its sums by each row's factor.  Parts
that know nothing of this get the normed rows as before.

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

    #: ``run`` takes the rows of its first norm from the block before and leaves them for the block after
    chains_norms = True

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _request(ctx, norm, before):
        """A request to the part before ``norm``, if both know how."""
        if norm is None or not getattr(before, "folds_norms", False):
            return None
        deferred = getattr(norm, "deferred", None)
        return deferred(ctx.ops) if deferred is not None else None

    @staticmethod
    def _rows_for(ctx, part, norm, x, pending):
        """The input of ``part``: what the part before left if ``part`` takes it, else the normed rows."""
        if pending is None:
            return norm.forward(ctx, x)
        return pending if getattr(part, "folds_norms", False) else ctx.ops.normed(pending)

    def run(self, ctx, x, entry: int, pending=None, next_norm=None):
        """``pending``: what the block before left for this block's first norm (or None).  Returns what
        it leaves for ``next_norm``, the first norm of the block after (or None)."""
        h = self._rows_for(ctx, self.mixer, self.mixer_norm, x, pending)
        request = self._request(ctx, self.ffn_norm, self.mixer)
        if request is None:
            self.mixer.forward(ctx, h, entry, accumulate_into=x)
        else:
            self.mixer.forward(ctx, h, entry, accumulate_into=x, then_norm=request)
        h = self._rows_for(ctx, self.feed_forward, self.ffn_norm, x, request.result if request is not None else None)
        request = self._request(ctx, next_norm, self.feed_forward)
        if request is None:
            self.feed_forward.forward(ctx, h, accumulate_into=x)
            return None
        self.feed_forward.forward(ctx, h, accumulate_into=x, then_norm=request)
        return request.result


register_part("block", "pre_norm", PreNormBlock)
