"""A model at run time: the parts of a ``ModelSpec`` with their weights on the device,
run over the tokens of one step in the order the schedule gives.

Embedding -> scheduled layers -> rows whose logits are wanted -> final norm ->
head (crates/bitnet-core/src/llama/model.rs:230-232, :236-307, :309-315).  Only
the wanted rows go through the final norm and the head.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..parts import ModelSpec, build_block, build_part
from ..weights import check_tensors


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], ops):
        for n in check_tensors(spec.expected_shapes(), tensors, ignorable=spec.ignorable):
            tensors = {k: v for k, v in tensors.items() if k != n}
        self.spec, self.ops = spec, ops
        self.width, self.vocab_size = spec.width, spec.vocab_size
        dev = ops.device
        self.blocks = []
        for blk in spec.layers:
            block = build_block(blk)
            for name, part in block.parts().items():
                weights = {key: tensors[blk.names[f"{name}.{key}"]].to(dev)
                           for key in part.weight_shapes()}
                part.bind(weights, ops)
            self.blocks.append(block)
        self.embedding_scale, self.logit_scale = float(spec.embedding_scale), float(spec.logit_scale)
        self.final_norm = build_part("norm", spec.final_norm)
        self.final_norm.bind({k: tensors[n].to(dev) for k, n in spec.final_norm_names.items()}, ops)
        self.embedding = ops.prepare_embedding(tensors[spec.embedding_name])
        if spec.head_name is None:
            self.head = ops.prepare_linear([self.embedding])     # tied: the table itself
        else:
            self.head = ops.prepare_linear([tensors[spec.head_name].to(dev)])
        for e, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {e} names layer {entry.layer}, which does not exist")
            if entry.reads_cache_of is not None and not 0 <= entry.reads_cache_of < e:
                raise ValueError(f"schedule entry {e} may only read the cache of an earlier entry")

    @staticmethod
    def _mixer_of(block, layer: int):
        """The part of a block that may need cache or state: its one mixer (None if it has none)."""
        from ..parts.base import Mixer
        mixers = [p for p in block.parts().values() if isinstance(p, Mixer)]
        if len(mixers) > 1:
            raise ValueError(f"layer {layer} has {len(mixers)} mixers; a cache entry belongs to one run of one "
                             "mixer, so give each mixer a layer of its own")
        return mixers[0] if mixers else None

    # what the cache has to provide
    def cache_plan(self):
        cache_needs, reads, state_needs = {}, {}, {}
        for e, entry in enumerate(self.spec.schedule):
            mixer = self._mixer_of(self.blocks[entry.layer], entry.layer)
            if mixer is None:
                continue
            need = mixer.cache_need()
            if need is not None:
                if entry.reads_cache_of is None:
                    cache_needs[e] = need
                else:
                    reads[e] = entry.reads_cache_of
                    src = self._mixer_of(self.blocks[self.spec.schedule[entry.reads_cache_of].layer], -1)
                    theirs = src.cache_need() if src is not None else None
                    if theirs is not None and theirs.window and (not need.window or need.window > theirs.window):
                        raise ValueError(f"schedule entry {e} sees {need.window or 'all'} keys but reads the cache of "
                                         f"entry {entry.reads_cache_of}, which keeps only the last {theirs.window}")
            st = mixer.state_need()
            if st is not None:
                state_needs[e] = st
        return cache_needs, reads, state_needs

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.head.w)
        for b in self.blocks:
            for part in b.parts().values():
                for v in vars(part).values():
                    w = getattr(v, "w", None)
                    if isinstance(w, torch.Tensor):
                        add(w)
        return total

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns float32 logits [wanted rows, vocab] or None."""
        ops, meta = ctx.ops, ctx.meta
        x = ops.embed(meta.token_ids, self.embedding, self.embedding_scale)   # float32 residual stream [T, E]
        schedule, pending = self.spec.schedule, None
        for e, entry in enumerate(schedule):
            block = self.blocks[entry.layer]
            if not getattr(block, "chains_norms", False):
                block.run(ctx, x, e)
                continue
            # a block that can hand the rows of the next block's first norm on (see parts/block.py)
            after = self.blocks[schedule[e + 1].layer] if e + 1 < len(schedule) else None
            next_norm = after.first_norm() if getattr(after, "chains_norms", False) else None
            pending = block.run(ctx, x, e, pending=pending, next_norm=next_norm)
        if meta.n_want == 0:
            return None
        rows = x if meta.want_every_row else ops.gather_rows(x, meta.want_rows)
        h = self.final_norm.forward(ctx, rows)
        return ops.linear(h, self.head, out_dtype=torch.float32, scale=self.logit_scale)
