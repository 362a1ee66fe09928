"""Pure data that describes a model: which parts each layer is made of, with what
sizes, under which tensor names, and in which order the layers run.

An architecture's builder turns its configuration into a ``ModelSpec``.  The
engine builds the parts from it; nothing below the builder knows which model
it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


#: the registry role of a block's well-known part names; other names carry their role in the PartSpec
_ROLE_OF_NAME = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "ffn_norm": "norm"}


@dataclass
class PartSpec:
    """One part: ``kind`` is its name in the part registry, ``params`` its sizes and constants,
    ``role`` the registry it is looked up in (may stay empty for a block's well-known names)."""
    kind: str
    params: dict = field(default_factory=dict)
    role: str = ""


class BlockSpec:
    """One layer: named parts, put together by ``arrangement`` (a kind of the "block" registry).

    ``parts`` maps a name the arrangement knows ("mixer", "feed_forward", "mixer_norm",
    "ffn_norm" for the pre-norm block; any other names for another arrangement) to the part's
    spec.  ``names`` maps "<part name>.<weight key>" ("mixer.q", "ffn_norm.weight", ...) to
    the tensor's full name in the weight files.  A block may have any number of parts: its
    weights are declared by walking ``parts``, whatever they are called.

    The four well-known names can also be given as keyword arguments and read or set as
    attributes (``spec.mixer = PartSpec(...)``).
    """

    def __init__(self, parts: Optional[Dict[str, PartSpec]] = None, names: Optional[Dict[str, str]] = None,
                 arrangement: str = "pre_norm", **named: PartSpec):
        self.parts: Dict[str, PartSpec] = dict(parts or {})
        self.parts.update(named)
        self.names: Dict[str, str] = dict(names or {})
        self.arrangement = arrangement

    def role_of(self, name: str) -> str:
        role = self.parts[name].role or _ROLE_OF_NAME.get(name, "")
        if not role:
            raise ValueError(f"block part {name!r} has no role: give PartSpec(..., role=...)")
        return role

    def __getattr__(self, name):
        parts = self.__dict__.get("parts")
        if parts is not None and name in parts:
            return parts[name]
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if isinstance(value, PartSpec):
            self.parts[name] = value
        else:
            object.__setattr__(self, name, value)

    def __repr__(self):
        return f"BlockSpec({self.arrangement!r}, parts={self.parts!r})"


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
    #: the embedded rows are multiplied by this (1.0: as stored), in the embedding kernel
    embedding_scale: float = 1.0
    #: the logits are multiplied by this (1.0: the plain product), in the head product's epilogue
    logit_scale: float = 1.0
    #: name patterns (fnmatch) of tensors a model folder may hold that the model does not use
    ignorable: List[str] = field(default_factory=list)

    def tensor_table(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """name -> (shape, init kind) of every tensor the model needs."""
        from .registry import build_part
        table: Dict[str, Tuple[Tuple[int, ...], str]] = {
            self.embedding_name: ((self.vocab_size, self.width), "matrix")}
        for i, blk in enumerate(self.layers):
            for name, part_spec in blk.parts.items():
                part = build_part(blk.role_of(name), part_spec)
                for key, (shape, kind) in part.weight_shapes().items():
                    if f"{name}.{key}" not in blk.names:
                        raise ValueError(f"layer {i}: no tensor name for weight {name}.{key}")
                    table[blk.names[f"{name}.{key}"]] = (tuple(shape), kind)
        norm = build_part("norm", self.final_norm)
        for key, (shape, kind) in norm.weight_shapes().items():
            table[self.final_norm_names[key]] = (tuple(shape), kind)
        if self.head_name is not None:
            table[self.head_name] = ((self.vocab_size, self.width), "matrix")
        return table

    def expected_shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: s for n, (s, _) in self.tensor_table().items()}
