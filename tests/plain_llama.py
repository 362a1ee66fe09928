"""Plain, slow Llama decoder: whole sequences, no cache, one function per part.

This is the oracle that the engine is compared with.  It is written from the
formulas of azerothl/Rbitnet's dense Llama forward and shares no code with the
product package (it imports nothing from ``rbitnet_b200``).  The reference's
own model code is Rust and cannot be compiled here (no Rust toolchain, and its
model only loads GGUF files), so this file rests on the formulas alone; every
function cites the reference lines it restates.

All math runs in the dtype asked for (float64 in most tests, so that it is a
neutral judge of the 32-bit engine path) and where the tensors are: on the CPU,
or on the GPU with torch's float64 operations for configurations of real layer
sizes, whose oracle would take minutes on the CPU.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# --------------------------------------------------------------------------- parts

def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * w / sqrt(mean(x^2) + eps) over the last axis.

    crates/bitnet-core/src/llama/model.rs:93-100
    """
    s = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * w * (1.0 / torch.sqrt(s + eps))


def silu(x: torch.Tensor) -> torch.Tensor:
    """v / (1 + exp(-v)).  crates/bitnet-core/src/llama/model.rs:116-120"""
    return x / (1.0 + torch.exp(-x))


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """Max-subtracted softmax over the last axis.

    crates/bitnet-core/src/llama/model.rs:102-114
    """
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True)


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """angle[p, i] = pos_p * theta^(-2i/D), i < D/2, built in float32 as the
    reference does (powf and the product are f32).

    crates/bitnet-core/src/llama/model.rs:126-128
    """
    i = torch.arange(head_dim // 2, dtype=torch.float32)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * i / head_dim)
    return positions.to(torch.float32)[:, None] * inv.to(positions.device)[None, :]


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float, pairing: str) -> torch.Tensor:
    """Rotate x[T, heads, D] by position.

    pairing "interleaved": pairs (2i, 2i+1), the reference's own
    (crates/bitnet-core/src/llama/model.rs:122-136).
    pairing "half": pairs (i, i+D/2), the order Hugging Face named checkpoints
    keep; it is the same function up to a fixed permutation of the rows of the
    q and k projections.
    """
    D = x.shape[-1]
    ang = rope_angles(positions, D, theta).to(x.dtype)
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    out = torch.empty_like(x)
    if pairing == "interleaved":
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
    elif pairing == "half":
        h = D // 2
        x0, x1 = x[..., :h], x[..., h:]
        out[..., :h] = x0 * c - x1 * s
        out[..., h:] = x0 * s + x1 * c
    else:
        raise ValueError(pairing)
    return out


def attention(q, k, v, window=None):
    """Causal grouped-query attention of one whole sequence.

    q [T, H, D] and k [T, K, D] are already rotated; v [T, K, D].  Query head h
    reads kv head h // (H/K); scores are (q.k) * 1/sqrt(D), the scale applied
    to the finished dot product; token t sees keys 0..t (and, with a window w,
    only the last w of them).

    crates/bitnet-core/src/llama/model.rs:260-289
    """
    T, H, D = q.shape
    K = k.shape[1]
    G = H // K
    scale = 1.0 / math.sqrt(D)
    out = torch.zeros(T, H, D, dtype=q.dtype, device=q.device)
    t_idx = torch.arange(T, device=q.device)
    allowed = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        allowed &= t_idx[None, :] > (t_idx[:, None] - window)
    for h in range(H):
        kh = h // G
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = softmax_rows(s)
        out[:, h, :] = p @ v[:, kh, :]
    return out.reshape(T, H * D)


def attention_mixer(x, lw, cfg, positions, shared_kv=None):
    """q, k, v projections, rotation of q and k, attention, output projection.

    Returns (y, (k_rot, v)) so that another layer may read this layer's keys
    and values.  crates/bitnet-core/src/llama/model.rs:238-291
    """
    T = x.shape[0]
    H, K, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ lw["q"].T).reshape(T, H, D)
    q = rope(q, positions, cfg["rope_theta"], cfg["rope_pairing"])
    if shared_kv is None:
        k = (x @ lw["k"].T).reshape(T, K, D)
        v = (x @ lw["v"].T).reshape(T, K, D)
        k = rope(k, positions, cfg["rope_theta"], cfg["rope_pairing"])
    else:
        k, v = shared_kv
    a = attention(q, k, v, cfg.get("sliding_window"))
    return a @ lw["o"].T, (k, v)


def gated_mlp(x, lw):
    """down( silu(gate x) * (up x) ).  crates/bitnet-core/src/llama/model.rs:297-303"""
    return (silu(x @ lw["gate"].T) * (x @ lw["up"].T)) @ lw["down"].T


def block(x, lw, cfg, positions, shared_kv=None):
    """Pre-norm block: x += attn(norm(x)); x += mlp(norm(x)).

    crates/bitnet-core/src/llama/model.rs:237-306
    """
    y, kv = attention_mixer(rmsnorm(x, lw["attn_norm"], cfg["rms_norm_eps"]), lw, cfg, positions, shared_kv)
    x = x + y
    x = x + gated_mlp(rmsnorm(x, lw["ffn_norm"], cfg["rms_norm_eps"]), lw)
    return x, kv


# --------------------------------------------------------------------------- model

def normalise_config(cfg: dict) -> dict:
    """Fill the defaults the reference uses (crates/bitnet-core/src/llama/config.rs:56,
    62, 94-108): kv heads = heads, head_dim = hidden/heads, theta 10000, eps 1e-5."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("tie_word_embeddings", False)
    c.setdefault("rope_pairing", "half")
    c.setdefault("sliding_window", None)
    return c


def layer_weights(tensors: dict, i: int, dtype) -> dict:
    p = f"model.layers.{i}."
    names = {
        "attn_norm": "input_layernorm.weight",
        "q": "self_attn.q_proj.weight",
        "k": "self_attn.k_proj.weight",
        "v": "self_attn.v_proj.weight",
        "o": "self_attn.o_proj.weight",
        "ffn_norm": "post_attention_layernorm.weight",
        "gate": "mlp.gate_proj.weight",
        "up": "mlp.up_proj.weight",
        "down": "mlp.down_proj.weight",
    }
    return {k: tensors[p + n].to(dtype) for k, n in names.items()}


def forward(cfg: dict, tensors: dict, tokens, dtype=torch.float64, schedule=None, rows=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence of token ids (with ``rows``: of those positions only).

    ``schedule`` is a list of (layer index, index of the earlier schedule entry
    whose keys and values this entry reads, or None); the default runs every
    layer once in order.  crates/bitnet-core/src/llama/model.rs:219-316
    """
    cfg = normalise_config(cfg)
    ids = torch.as_tensor(tokens, dtype=torch.long)
    if int(ids.max()) >= cfg["vocab_size"] or int(ids.min()) < 0:
        raise ValueError("token id out of range")
    table = tensors["model.embed_tokens.weight"]
    ids = ids.to(table.device)
    positions = torch.arange(ids.shape[0], device=table.device)
    x = table[ids].to(dtype)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, reads in schedule:
        lw = layer_weights(tensors, layer, dtype)
        x, kv = block(x, lw, cfg, positions, None if reads is None else kvs[reads])
        kvs.append(kv)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long, device=x.device)]
    xn = rmsnorm(x, tensors["model.norm.weight"].to(dtype), cfg["rms_norm_eps"])
    head = (table if cfg["tie_word_embeddings"] else tensors["lm_head.weight"]).to(dtype)
    return xn @ head.T


# --------------------------------------------------------------------------- sampling and generation

def greedy_token(logits: torch.Tensor) -> int:
    """Index of the largest logit, NaN counted as -inf; the lowest index wins a
    tie (the reference's max_by keeps the last of equal maxima; the engine
    documents the lowest).  crates/bitnet-core/src/llama/runtime.rs:82-93"""
    z = torch.where(torch.isnan(logits), torch.full_like(logits, float("-inf")), logits)
    return int(torch.argmax(z))


def temperature_cdf(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Cumulative sums of exp(z/T - max) in index order, in float64.

    crates/bitnet-core/src/llama/runtime.rs:94-101
    """
    z = logits.to(torch.float64) / temperature
    e = torch.exp(z - z.max())
    return torch.cumsum(e, dim=0)


def temperature_token(logits: torch.Tensor, temperature: float, u: float) -> int:
    """First index whose cumulative sum reaches u * total; the last index if
    none does.  crates/bitnet-core/src/llama/runtime.rs:98-106"""
    c = temperature_cdf(logits, temperature)
    r = u * float(c[-1])
    hit = torch.nonzero(c >= r)
    return int(hit[0]) if hit.numel() else logits.numel() - 1


def generate_greedy(cfg, tensors, prompt, max_new_tokens, stop_ids=(), dtype=torch.float64):
    """Greedy generation by running the whole sequence again for every token.
    A sampled stop token ends the sequence and is not emitted.

    crates/bitnet-core/src/llama/runtime.rs:50-73
    """
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        nxt = greedy_token(forward(cfg, tensors, seq, dtype)[-1])
        if nxt in stop_ids:
            break
        out.append(nxt)
        seq.append(nxt)
    return out


# --------------------------------------------------------------------------- files (independent of the package)

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = bytearray(raw[base + a: base + b])
        t = torch.frombuffer(buf, dtype=dt) if b > a else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, read_safetensors(folder / "model.safetensors")
