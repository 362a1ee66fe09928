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
        check_tensors(spec.expected_shapes(), tensors)
        self.spec, self.ops = spec, ops
        self.width, self.vocab_size = spec.width, spec.vocab_size
        dev = ops.device
        self.blocks = []
        for blk in spec.layers:
            block = build_block(blk)
            for role, part in block.parts().items():
                weights = {key: tensors[blk.names[f"{role}.{key}"]].to(dev)
                           for key in part.weight_shapes()}
                part.bind(weights, ops)
            self.blocks.append(block)
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

    # what the cache has to provide
    def cache_plan(self):
        cache_needs, reads, state_needs = {}, {}, {}
        for e, entry in enumerate(self.spec.schedule):
            mixer = self.blocks[entry.layer].mixer
            need = mixer.cache_need()
            if need is not None:
                if entry.reads_cache_of is None:
                    cache_needs[e] = need
                else:
                    reads[e] = entry.reads_cache_of
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
        x = ops.embed(meta.token_ids, self.embedding)            # float32 residual stream [T, E]
        for e, entry in enumerate(self.spec.schedule):
            self.blocks[entry.layer].run(ctx, x, e)
        if meta.n_want == 0:
            return None
        rows = x if meta.want_every_row else ops.gather_rows(x, meta.want_rows)
        h = self.final_norm.forward(ctx, rows)
        return ops.linear(h, self.head, out_dtype=torch.float32)
