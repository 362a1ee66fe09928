"""Pure data that describes a model: which parts each layer is made of, with what
sizes, under which tensor names, and in which order the layers run.

An architecture's builder turns its configuration into a ``ModelSpec``.  The
engine builds the parts from it; nothing below the builder knows which model
it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part: ``kind`` is its name in the part registry, ``params`` its sizes and constants."""
    kind: str
    params: dict = field(default_factory=dict)


@dataclass
class BlockSpec:
    """One layer: a mixer and a feed-forward, each behind a norm, arranged by ``arrangement``.

    ``names`` maps a part-local weight key ("mixer.q", "feed_forward.down",
    "mixer_norm.weight", ...) to the tensor's full name in the weight files.
    """
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    names: Dict[str, str]
    arrangement: str = "pre_norm"


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``reads_cache_of`` names an EARLIER entry of the schedule
    whose keys and values this run reads instead of writing its own."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    width: int
    vocab_size: int
    embedding_name: str
    layers: List[BlockSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    final_norm_names: Dict[str, str]
    #: tensor name of the output matrix [vocab, width]; None: the embedding table is used
    head_name: Optional[str]
    #: longest sequence the model's position encoding is defined for
    max_positions: int
    stop_ids: List[int] = field(default_factory=list)

    def tensor_table(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """name -> (shape, init kind) of every tensor the model needs."""
        from .registry import build_part
        table: Dict[str, Tuple[Tuple[int, ...], str]] = {
            self.embedding_name: ((self.vocab_size, self.width), "matrix")}
        for blk in self.layers:
            for role in ("mixer", "feed_forward", "mixer_norm", "ffn_norm"):
                part = build_part(role, getattr(blk, role))
                for key, (shape, kind) in part.weight_shapes().items():
                    table[blk.names[f"{role}.{key}"]] = (tuple(shape), kind)
        norm = build_part("norm", self.final_norm)
        for key, (shape, kind) in norm.weight_shapes().items():
            table[self.final_norm_names[key]] = (tuple(shape), kind)
        if self.head_name is not None:
            table[self.head_name] = ((self.vocab_size, self.width), "matrix")
        return table

    def expected_shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: s for n, (s, _) in self.tensor_table().items()}
