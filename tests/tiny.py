"""The two tiny configurations the tests use.  They differ in every size and option:
head counts and grouping, sizes that are no power of two, layers, vocabulary, eps, theta,
rotary pairing, tied or untied head."""
import torch

TINY_A = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=128,
              tie_word_embeddings=True, rope_pairing="interleaved", hidden_act="silu")
TINY_B = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=96,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256,
              vocab_size=384, rope_theta=500000.0, rms_norm_eps=1e-6, max_position_embeddings=256,
              tie_word_embeddings=False, rope_pairing="half", hidden_act="silu")
# (config, weight seed, prompt lengths, prompt seed, decode steps)
WORKLOADS = {"A": (TINY_A, 0, [5, 9, 3], 1, 8), "B": (TINY_B, 2, [1, 17, 6, 11], 3, 12)}


def prompts(lengths, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
