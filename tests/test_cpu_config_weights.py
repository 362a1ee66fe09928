"""Configuration, registry and weight errors (no GPU)."""
import json

import pytest
import torch

from tiny import TINY_A, TINY_B
from rbitnet_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config,
                                 known_architectures, get_architecture)
from rbitnet_b200.weights import (WeightError, check_tensors, read_model_tensors, read_safetensors,
                                  write_safetensors, write_random_model, random_tensors)
import plain_llama as plain


def test_defaults_follow_the_reference():
    c = config_from_dict(dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=1,
                              num_attention_heads=4, intermediate_size=100, vocab_size=50))
    assert c.num_key_value_heads == 4          # config.rs:56
    assert c.head_dim == 16                    # config.rs:62
    assert c.rope_theta == 10000.0             # config.rs:94-97
    assert c.rms_norm_eps == 1e-5              # config.rs:99-102
    assert c.max_position_embeddings == 2048   # config.rs:104-108
    assert c.tie_word_embeddings is False and c.stop_ids == []


def test_both_tiny_configurations_parse_and_differ():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    for f in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
              "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps", "max_position_embeddings",
              "tie_word_embeddings", "rope_pairing"):
        assert getattr(a, f) != getattr(b, f), f


@pytest.mark.parametrize("change,fragment", [
    ({"hidden_size": None}, "missing hidden_size"),
    ({"num_hidden_layers": None}, "missing num_hidden_layers"),
    ({"num_attention_heads": None}, "missing num_attention_heads"),
    ({"intermediate_size": None}, "missing intermediate_size"),
    ({"vocab_size": None}, "missing vocab_size"),
    ({"num_key_value_heads": 3}, "num_attention_heads / num_key_value_heads"),
    ({"head_dim": 20}, "must equal hidden_size"),
    ({"hidden_size": 60, "head_dim": 15}, "must be even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "linear"}}, "rope_scaling"),
    ({"rope_pairing": "odd"}, "rope_pairing"),
    ({"vocab_size": -3}, "positive integer"),
    ({"architectures": ["NopeForCausalLM"]}, "unknown architecture"),
    ({"architectures": None}, "missing architectures"),
])
def test_config_errors(change, fragment):
    d = dict(TINY_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert fragment in str(e.value)


def test_eos_ids_and_registry():
    d = dict(TINY_A, eos_token_id=[3, 9])
    assert config_from_dict(d).stop_ids == [3, 9]
    assert config_from_dict(dict(TINY_A, eos_token_id=2)).stop_ids == [2]
    assert "LlamaForCausalLM" in known_architectures()
    assert get_architecture("LlamaForCausalLM").config_cls is LlamaConfig


def test_config_json_problems(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)


def _spec(cfgd):
    cfg = config_from_dict(cfgd)
    return cfg, get_architecture(cfg.architecture).build_spec(cfg)


def test_tensor_table_matches_the_architecture():
    for cfgd, n_params in ((TINY_A, 108864), (TINY_B, 369312)):
        cfg, spec = _spec(cfgd)
        table = spec.expected_shapes()
        assert sum(int(torch.tensor(s).prod()) for s in table.values()) == n_params
        assert ("lm_head.weight" in table) == (not cfg.tie_word_embeddings)
        assert table["model.layers.0.self_attn.k_proj.weight"] == (cfg.num_key_value_heads * cfg.head_dim, cfg.hidden_size)
        assert table["model.layers.0.mlp.down_proj.weight"] == (cfg.hidden_size, cfg.intermediate_size)


def test_random_model_folder_round_trip(tmp_path):
    cfg, spec = _spec(TINY_B)
    write_random_model(tmp_path, cfg, seed=5)
    assert load_config(tmp_path).to_dict() == cfg.to_dict()
    t = read_model_tensors(tmp_path)
    check_tensors(spec.expected_shapes(), t)
    again = random_tensors(spec, 5)
    other = random_tensors(spec, 6)
    for name in t:
        assert torch.equal(t[name], again[name])
        assert not torch.equal(t[name], other[name])
    # the independent reader of the plain implementation sees the same bytes
    _, pt = plain.load_folder(tmp_path)
    assert all(torch.equal(pt[n], t[n]) for n in t)
    norm = t["model.layers.1.input_layernorm.weight"]
    assert abs(float(norm.mean()) - 1.0) < 0.02 and 0.005 < float(t["lm_head.weight"].std()) < 0.04


def test_dtypes_on_the_way_in(tmp_path):
    tensors = {"a": torch.randn(3, 4), "b": torch.randn(3, 4).to(torch.bfloat16),
               "c": torch.randn(2, 2).to(torch.float16), "d": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    write_safetensors(tmp_path / "x.safetensors", tensors)
    got = read_safetensors(tmp_path / "x.safetensors")
    assert got["a"].dtype == torch.float32 and torch.equal(got["a"], tensors["a"])       # 32-bit stays
    assert got["b"].dtype == torch.bfloat16 and torch.equal(got["b"], tensors["b"])
    assert got["c"].dtype == torch.float16 and torch.equal(got["c"], tensors["c"])       # half stays exact
    assert got["d"].dtype == torch.int32 and got["d"].tolist() == tensors["d"].tolist()  # integer tables


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    _, spec = _spec(TINY_A)
    t = random_tensors(spec, 0)
    del t["model.norm.weight"], t["model.layers.1.mlp.up_proj.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    t["extra.bias"] = torch.zeros(3)
    with pytest.raises(WeightError) as e:
        check_tensors(spec.expected_shapes(), t)
    msg = str(e.value)
    assert "missing (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected (1): extra.bias" in msg
    assert "model.layers.0.self_attn.q_proj.weight expected [64, 64] found [64, 32]" in msg


def test_broken_files(tmp_path):
    with pytest.raises(WeightError, match="no model.safetensors"):
        read_model_tensors(tmp_path)
    cfg, _ = _spec(TINY_A)
    write_random_model(tmp_path, cfg, 0)
    f = tmp_path / "model.safetensors"
    raw = f.read_bytes()
    f.write_bytes(raw[:len(raw) // 2])
    with pytest.raises(WeightError, match="outside the file"):
        read_model_tensors(tmp_path)
    f.write_bytes(raw[:4])
    with pytest.raises(WeightError, match="truncated"):
        read_model_tensors(tmp_path)
    f.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError, match="header length"):
        read_model_tensors(tmp_path)
    hdr = json.dumps({"t": {"dtype": "Q9", "shape": [1], "data_offsets": [0, 4]}}).encode()
    f.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0\0\0\0")
    with pytest.raises(WeightError, match="unknown dtype"):
        read_model_tensors(tmp_path)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 4]}}).encode()
    f.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0\0\0\0")
    with pytest.raises(WeightError, match="needs 12"):
        read_model_tensors(tmp_path)


def test_sharded_folder(tmp_path):
    _, spec = _spec(TINY_A)
    t = random_tensors(spec, 1)
    names = sorted(t)
    half = len(names) // 2
    write_safetensors(tmp_path / "s1.safetensors", {n: t[n] for n in names[:half]})
    write_safetensors(tmp_path / "s2.safetensors", {n: t[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    got = read_model_tensors(tmp_path)
    check_tensors(spec.expected_shapes(), got)
    (tmp_path / "s2.safetensors").unlink()
    with pytest.raises(WeightError, match="not in the folder"):
        read_model_tensors(tmp_path)


def test_harmless_extras_are_left_out_with_a_warning_and_others_are_an_error():
    """crates/bitnet-core/src/llama/model.rs:54-60 looks tensors up by name and never sees extras."""
    cfg, spec = _spec(TINY_A)                     # tied head
    t = random_tensors(spec, 0)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["lm_head.weight"] = torch.zeros(cfg.vocab_size, cfg.hidden_size)
    with pytest.warns(UserWarning, match="rotary_emb.inv_freq"):
        ignored = check_tensors(spec.expected_shapes(), t, ignorable=spec.ignorable)
    assert ignored == ["lm_head.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    with pytest.warns(UserWarning), pytest.raises(WeightError, match=r"unexpected \(1\): model.layers.0.self_attn.q_proj.bias"):
        check_tensors(spec.expected_shapes(), t, ignorable=spec.ignorable)
    _, spec_b = _spec(TINY_B)                     # untied: lm_head.weight is needed, not ignorable
    assert "lm_head.weight" not in spec_b.ignorable and "lm_head.weight" in spec_b.expected_shapes()


def test_random_values_are_a_function_of_seed_name_and_index():
    """crates/bitnet-core/src/model/toy.rs:16-30: one deterministic generator wherever it runs."""
    from rbitnet_b200.weights.random_init import random_tensor, reference_value, random_values, _tensor_key
    t = random_tensor("model.layers.1.mlp.up_proj.weight", (5, 7), "matrix", 9)
    for i in (0, 1, 17, 34):
        assert float(t.view(-1)[i]) == reference_value(9, "model.layers.1.mlp.up_proj.weight", i)
    # any part of a tensor can be made alone
    key = _tensor_key(9, "model.layers.1.mlp.up_proj.weight")
    scale = torch.tensor(0.02 / (8.0 * (65536.0 ** 2 - 1.0) / 12.0) ** 0.5, dtype=torch.float32)
    assert torch.equal(random_values(key, 10, 6) * scale, t.view(-1)[10:16])
    # other seed, other name: other values
    assert not torch.equal(t, random_tensor("model.layers.1.mlp.up_proj.weight", (5, 7), "matrix", 10))
    assert not torch.equal(t, random_tensor("model.layers.0.mlp.up_proj.weight", (5, 7), "matrix", 9))
    big = random_tensor("w", (512, 512), "matrix", 1)
    assert abs(float(big.std()) - 0.02) < 2e-4 and abs(float(big.mean())) < 2e-4
    n = random_tensor("n", (4096,), "norm", 1)
    assert abs(float(n.mean()) - 1.0) < 2e-3 and abs(float(n.std()) - 0.02) < 2e-3
    b = random_tensor("w", (512, 512), "matrix", 1, dtype=torch.bfloat16)       # made in float32, then rounded
    assert torch.equal(b, big.to(torch.bfloat16))
