"""The plain implementation checked against itself: its whole-sequence form against a
literal, one-token-at-a-time restatement of the reference's forward loop
(crates/bitnet-core/src/llama/model.rs:219-316), and its parts against hand values."""
import math

import torch

import plain_llama as plain
from tiny import TINY_A, TINY_B, prompts
from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors


def _tensors(cfgd, seed):
    cfg = config_from_dict(cfgd)
    return random_tensors(get_architecture(cfg.architecture).build_spec(cfg), seed)


def literal_forward(cfg, tensors, tokens):
    """Scalar-loop restatement, token by token with an explicit cache, float64."""
    c = plain.normalise_config(cfg)
    E, H, K, D = c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    L, eps, theta = c["num_hidden_layers"], c["rms_norm_eps"], c["rope_theta"]
    t64 = {k: v.double() for k, v in tensors.items()}
    kc = [[] for _ in range(L)]
    vc = [[] for _ in range(L)]
    out = []

    def norm(x, w):
        s = sum(float(v) ** 2 for v in x) / len(x)
        return x * w / math.sqrt(s + eps)

    def rot(s, pos):
        s = s.clone()
        half = D // 2
        for i in range(half):
            inv = float(1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32),
                                        torch.tensor(2.0 * i / D, dtype=torch.float32)))
            ang = float(torch.tensor(pos, dtype=torch.float32) * torch.tensor(inv, dtype=torch.float32))
            a, b = (2 * i, 2 * i + 1) if c["rope_pairing"] == "interleaved" else (i, i + half)
            x0, x1 = float(s[a]), float(s[b])
            s[a] = x0 * math.cos(ang) - x1 * math.sin(ang)
            s[b] = x0 * math.sin(ang) + x1 * math.cos(ang)
        return s

    for pos, tok in enumerate(tokens):
        x = t64["model.embed_tokens.weight"][tok].clone()
        for il in range(L):
            lw = plain.layer_weights(t64, il, torch.float64)
            h = norm(x, lw["attn_norm"])
            q, k, v = lw["q"] @ h, lw["k"] @ h, lw["v"] @ h
            q = torch.cat([rot(q[i * D:(i + 1) * D], pos) for i in range(H)])
            k = torch.cat([rot(k[i * D:(i + 1) * D], pos) for i in range(K)])
            kc[il].append(k)
            vc[il].append(v)
            attn = torch.zeros(E, dtype=torch.float64)
            for qh in range(H):
                kvh = qh // (H // K)
                sc = torch.tensor([float(q[qh * D:(qh + 1) * D] @ kc[il][p][kvh * D:(kvh + 1) * D]) / math.sqrt(D)
                                   for p in range(pos + 1)], dtype=torch.float64)
                pr = torch.exp(sc - sc.max())
                pr = pr / pr.sum()
                for p in range(pos + 1):
                    attn[qh * D:(qh + 1) * D] += pr[p] * vc[il][p][kvh * D:(kvh + 1) * D]
            x = x + lw["o"] @ attn
            h2 = norm(x, lw["ffn_norm"])
            g = lw["gate"] @ h2
            x = x + lw["down"] @ ((g / (1 + torch.exp(-g))) * (lw["up"] @ h2))
        xn = norm(x, t64["model.norm.weight"])
        head = t64["model.embed_tokens.weight"] if c["tie_word_embeddings"] else t64["lm_head.weight"]
        out.append(head @ xn)
    return torch.stack(out)


def test_whole_sequence_form_equals_the_literal_loop():
    for cfgd, seed in ((TINY_A, 0), (TINY_B, 2)):
        t = _tensors(cfgd, seed)
        for name in t:
            if "q_proj" in name or "k_proj" in name:
                t[name] = t[name] * 6
        p = prompts([11], cfgd["vocab_size"], 4)[0]
        a = plain.forward(cfgd, t, p, torch.float64)
        b = literal_forward(cfgd, t, p)
        assert float((a - b).abs().max()) < 1e-9


def test_rmsnorm_silu_softmax_hand_values():
    x = torch.tensor([3.0, 4.0], dtype=torch.float64)
    y = plain.rmsnorm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    r = 1 / math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([6.0 * r, 2.0 * r], dtype=torch.float64))
    assert abs(float(plain.silu(torch.tensor(1.0))) - 1 / (1 + math.exp(-1))) < 1e-7
    s = plain.softmax_rows(torch.tensor([[0.0, math.log(3.0)]], dtype=torch.float64))
    assert torch.allclose(s, torch.tensor([[0.25, 0.75]], dtype=torch.float64))


def test_rope_pairings_are_one_function_up_to_a_row_permutation():
    D, T = 16, 7
    x = torch.randn(T, 2, D, dtype=torch.float64)
    pos = torch.arange(T) + 3
    perm = torch.empty(D, dtype=torch.long)            # half index j -> interleaved index
    perm[:D // 2] = torch.arange(0, D, 2)
    perm[D // 2:] = torch.arange(1, D, 2)
    half = plain.rope(x, pos, 10000.0, "half")
    inter = plain.rope(x[..., torch.argsort(perm)], pos, 10000.0, "interleaved")
    assert torch.allclose(inter[..., perm], half, atol=1e-12)
    # rotation by position 0 is the identity; norms are kept
    assert torch.allclose(plain.rope(x, torch.zeros(T, dtype=torch.long), 5e5, "half"), x)
    assert torch.allclose(half.norm(dim=-1), x.norm(dim=-1))


def test_attention_is_causal_grouped_and_windowed():
    T, H, K, D = 6, 4, 2, 8
    q, k, v = (torch.randn(T, n, D, dtype=torch.float64) for n in (H, K, K))
    out = plain.attention(q, k, v).reshape(T, H, D)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # first token, groups
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0                                                         # the future is unseen
    assert torch.allclose(plain.attention(q, k2, v2).reshape(T, H, D)[:4], out[:4])
    w = plain.attention(q, k, v, window=2).reshape(T, H, D)
    k3, v3 = k.clone(), v.clone()
    k3[:3], v3[:3] = 5.0, 5.0                                                          # beyond the window
    assert torch.allclose(plain.attention(q, k3, v3, window=2).reshape(T, H, D)[4:], w[4:])
    assert not torch.allclose(w[5], out[5])


def test_sampling_rules():
    z = torch.tensor([0.1, float("nan"), 2.0, 2.0, -1.0])
    assert plain.greedy_token(z) == 2                       # NaN as -inf, lowest index on a tie
    assert plain.temperature_token(torch.tensor([0.0, 0.0, 0.0, 0.0]), 1.0, 0.49) == 1
    assert plain.temperature_token(torch.tensor([0.0, 0.0, 0.0, 0.0]), 1.0, 0.51) == 2
    assert plain.temperature_token(torch.tensor([0.0, 50.0]), 0.5, 0.999) == 1
    assert plain.temperature_token(torch.tensor([1.0, 2.0]), 1.0, 0.0) == 0


def test_schedule_with_a_repeated_layer_and_a_shared_cache_changes_the_result():
    t = _tensors(TINY_A, 0)
    p = prompts([9], 256, 1)[0]
    a = plain.forward(TINY_A, t, p)
    b = plain.forward(TINY_A, t, p, schedule=[(0, None), (1, None), (0, None)])
    c = plain.forward(TINY_A, t, p, schedule=[(0, None), (1, 0)])
    assert not torch.allclose(a, b) and not torch.allclose(a, c)


def test_plain_implementation_and_weight_generator_against_committed_numbers():
    """tests/golden/plain_tiny.json was written by tests/golden/make_golden.py: the oracle's logits for a
    fixed prompt on the seeded random weights of both tiny configurations.  (No output of the
    reference's own code exists to compare with: it cannot be compiled here.)"""
    import importlib.util
    import json
    from pathlib import Path
    here = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_golden", here / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    want = json.loads((here / "plain_tiny.json").read_text())
    got = mod.golden()
    for name in ("A", "B"):
        assert got[name]["prompt"] == want[name]["prompt"]
        assert got[name]["first_weights"] == want[name]["first_weights"]              # bit for bit
        assert got[name]["argmax_per_row"] == want[name]["argmax_per_row"]
        for a, b in zip(got[name]["last_row_first_8"], want[name]["last_row_first_8"]):
            assert abs(a - b) <= 1e-9 * max(1.0, abs(b))          # float64 sums may be ordered otherwise on another CPU
        assert abs(got[name]["sum_abs"] - want[name]["sum_abs"]) <= 1e-9 * want[name]["sum_abs"]
