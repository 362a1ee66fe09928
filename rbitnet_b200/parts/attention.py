"""Grouped-query attention over the cache, as a mixer.

q = Wq h, k = Wk h, v = Wv h without bias; q and k take the position encoding;
k and v are appended to the sequence's cache; query head h reads kv head
h // (H/K); score = (q.k) * scale over the keys the mask allows (causal, and a
window if given); softmax in float32; o = P v; result Wo o is added to the
residual stream.  crates/bitnet-core/src/llama/model.rs:238-294
"""
from __future__ import annotations

import math
from typing import Optional

from .base import Mixer, CacheNeed
from .registry import register_part, build_part
from .spec import PartSpec


class Attention(Mixer):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: Optional[dict] = None, window: Optional[int] = None,
                 scale: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        self.width, self.n_heads, self.n_kv_heads, self.head_dim = width, n_heads, n_kv_heads, head_dim
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        position = position or {"kind": "none", "params": {}}
        self.position = build_part("position", PartSpec(position["kind"], dict(position.get("params", {}))))
        self.w_qkv = self.w_q = self.w_o = None

    def weight_shapes(self):
        H, K, D, E = self.n_heads, self.n_kv_heads, self.head_dim, self.width
        return {"q": ((H * D, E), "matrix"), "k": ((K * D, E), "matrix"),
                "v": ((K * D, E), "matrix"), "o": ((E, H * D), "matrix")}

    def cache_need(self):
        return CacheNeed(self.n_kv_heads, self.head_dim, self.window)

    def bind(self, weights, ops):
        self.position.bind({}, ops)
        # one product for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = ops.prepare_linear([weights["q"], weights["k"], weights["v"]])
        self.w_q = None  # for a run that reads another layer's cache: the q rows of w_qkv, as a view
        self.w_o = ops.prepare_linear([weights["o"]])

    #: ``h`` may be rows with their norm pending, and ``then_norm`` is handed to the last product
    folds_norms = True

    def forward(self, ctx, h, entry, accumulate_into, then_norm=None):
        ops = ctx.ops
        view = ctx.cache_view(entry)
        if view.writes:
            w = self.w_qkv
        else:
            if self.w_q is None:
                self.w_q = ops.rows_of(self.w_qkv, 0, self.n_heads * self.head_dim)
            w = self.w_q
        q = ops.project_rotate_append(h, w, self.position.rotary(), ctx.meta, view, self.n_heads)
        a = ops.attention(q, ctx.meta, view, self.n_heads, self.scale, self.window)
        if then_norm is None:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into)
        else:
            ops.linear(a, self.w_o, accumulate_into=accumulate_into, then_norm=then_norm)


register_part("mixer", "attention", Attention)
