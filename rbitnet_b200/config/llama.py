"""LlamaConfig: the dense Llama decoder's hyper-parameters, by config.json key.

Defaults and checks follow the reference's reader of the same quantities
(crates/bitnet-core/src/llama/config.rs:40-122): key/value heads default to the
number of heads (:56), heads must be a multiple of key/value heads (:57-61),
the head size must be even (:68-72), theta defaults to 10000 (:94-97), the
norm's eps to 1e-5 (:99-102) and the context to 2048 (:104-108).  The
reference derives head_dim = hidden/heads and its weight checks pin
heads*head_dim = hidden (crates/bitnet-core/src/llama/model.rs:182-185); here
``head_dim`` is an optional key with that default, and the same product rule.
The reference silently clamps the context to 8192; here the limit of a run is
the engine's ``max_seq`` option instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, List, Optional, Union

from .base import ModelConfig, ConfigError


@dataclass
class LlamaConfig(ModelConfig):
    architecture: ClassVar[str] = "LlamaForCausalLM"
    required: ClassVar[tuple] = ("hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "vocab_size")
    pinned: ClassVar[dict] = {"hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
                              "rope_scaling": None}

    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    intermediate_size: int = 0
    vocab_size: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 2048
    tie_word_embeddings: bool = False
    eos_token_id: Union[int, List[int], None] = None
    bos_token_id: Optional[int] = None
    #: "half": rotate pairs (i, i+D/2), the row order of checkpoints with
    #: Hugging Face tensor names; "interleaved": pairs (2i, 2i+1), literally
    #: crates/bitnet-core/src/llama/model.rs:122-136.
    rope_pairing: str = "half"
    #: None: every earlier key is seen (the reference's only mask, the loop
    #: bound of crates/bitnet-core/src/llama/model.rs:266).
    sliding_window: Optional[int] = None
    hidden_act: str = "silu"

    def validate(self) -> None:
        H = self.num_attention_heads
        if self.num_key_value_heads is None:
            self.num_key_value_heads = H
        K = self.num_key_value_heads
        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                     "intermediate_size", "vocab_size", "max_position_embeddings"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config.json: {name} must be a positive integer, found {v!r}")
        if K <= 0 or H % K != 0:
            raise ConfigError(
                f"config.json: invalid num_attention_heads / num_key_value_heads ({H} / {K})")
        if self.head_dim is None:
            if self.hidden_size % H != 0:
                raise ConfigError(
                    f"config.json: hidden_size {self.hidden_size} not divisible by "
                    f"num_attention_heads {H}")
            self.head_dim = self.hidden_size // H
        if H * self.head_dim != self.hidden_size:
            raise ConfigError(
                f"config.json: num_attention_heads*head_dim = {H * self.head_dim} must equal "
                f"hidden_size {self.hidden_size}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: invalid head_dim {self.head_dim}: must be even")
        if self.rope_pairing not in ("half", "interleaved"):
            raise ConfigError(f"config.json: rope_pairing {self.rope_pairing!r} "
                              "must be 'half' or 'interleaved'")
        if not (self.rope_theta > 0):
            raise ConfigError(f"config.json: rope_theta must be positive, found {self.rope_theta}")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, found {self.rms_norm_eps}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            raise ConfigError("config.json: sliding_window must be positive or null")

    @property
    def stop_ids(self) -> List[int]:
        e = self.eos_token_id
        if e is None:
            return []
        return list(e) if isinstance(e, (list, tuple)) else [int(e)]
