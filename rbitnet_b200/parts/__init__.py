from .spec import PartSpec, BlockSpec, ScheduleEntry, ModelSpec
from .base import Part, Norm, PositionEncoding, Mixer, FeedForward, CacheNeed, StateNeed
from .registry import register_part, unregister_part, known_parts, build_part, build_block
from .norm import RMSNorm
from .position import RotaryEncoding, NoPositionEncoding
from .attention import Attention
from .feed_forward import GatedDense
from .block import PreNormBlock

__all__ = ["PartSpec", "BlockSpec", "ScheduleEntry", "ModelSpec", "Part", "Norm", "PositionEncoding",
           "Mixer", "FeedForward", "CacheNeed", "StateNeed", "register_part", "unregister_part",
           "known_parts", "build_part", "build_block", "RMSNorm", "RotaryEncoding", "NoPositionEncoding", "Attention",
           "GatedDense", "PreNormBlock"]
