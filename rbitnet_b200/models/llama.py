"""The dense Llama decoder as data: which parts its layers are made of, and its tensor names.

Structure (crates/bitnet-core/src/llama/model.rs:219-316): embedding, L identical
pre-norm blocks (RMSNorm, rotary grouped-query attention, RMSNorm, SiLU-gated
feed-forward), a final RMSNorm with the same eps, a linear head (the embedding
table when ``tie_word_embeddings``).  Tensor names are the Hugging Face ones;
the reference reads the same tensors under GGUF names
(crates/bitnet-core/src/llama/model.rs:146-179).
"""
from __future__ import annotations

from ..config import LlamaConfig, register_architecture
from ..parts import PartSpec, BlockSpec, ScheduleEntry, ModelSpec

_LAYER_NAMES = {
    "mixer_norm.weight": "input_layernorm.weight",
    "mixer.q": "self_attn.q_proj.weight",
    "mixer.k": "self_attn.k_proj.weight",
    "mixer.v": "self_attn.v_proj.weight",
    "mixer.o": "self_attn.o_proj.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "feed_forward.gate": "mlp.gate_proj.weight",
    "feed_forward.up": "mlp.up_proj.weight",
    "feed_forward.down": "mlp.down_proj.weight",
}


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = {"kind": "rotary", "params": {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                             "pairing": cfg.rope_pairing,
                                             "max_positions": cfg.max_position_embeddings}}
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(BlockSpec(parts=dict(
            mixer=PartSpec("attention", {"width": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                                         "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                                         "position": position, "window": cfg.sliding_window}),
            feed_forward=PartSpec("gated_dense", {"width": cfg.hidden_size, "inner": cfg.intermediate_size,
                                                  "activation": cfg.hidden_act}),
            mixer_norm=norm, ffn_norm=norm),
            names={k: f"model.layers.{i}.{v}" for k, v in _LAYER_NAMES.items()},
            arrangement="pre_norm"))
    return ModelSpec(
        width=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding_name="model.embed_tokens.weight",
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=norm, final_norm_names={"weight": "model.norm.weight"},
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings,
        stop_ids=cfg.stop_ids,
        # buffers some exporters store; an output matrix stored beside a tied embedding
        ignorable=["*.rotary_emb.inv_freq"] + (["lm_head.weight"] if cfg.tie_word_embeddings else []))


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec)
