"""Writes tests/golden/plain_tiny.json: logits of the plain implementation (tests/plain_llama.py, float64)
for the two tiny configurations with the seeded random weights of rbitnet_b200.weights.random_init.

The plain implementation rests on the formulas of azerothl/Rbitnet's Llama forward
(crates/bitnet-core/src/llama/model.rs:93-136, 219-316) alone: the reference is a Rust workspace that
cannot be compiled here (no Rust toolchain) and loads GGUF files only, so there is no output of the
reference's own code to commit.  This file pins the oracle and the weight generator instead: a change to
either shows as a difference against these numbers.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import plain_llama as plain  # noqa: E402
from tiny import TINY_A, TINY_B, prompts  # noqa: E402


def golden():
    from rbitnet_b200.config import config_from_dict
    from rbitnet_b200.config.registry import get_architecture
    from rbitnet_b200.weights import random_tensors
    out = {}
    for name, cfg, seed in (("A", TINY_A, 0), ("B", TINY_B, 2)):
        c = config_from_dict(cfg)
        tensors = random_tensors(get_architecture(c.architecture).build_spec(c), seed)
        p = prompts([12], cfg["vocab_size"], seed=5)[0]
        logits = plain.forward(cfg, tensors, p, torch.float64)
        out[name] = {"weight_seed": seed, "prompt": p,
                     "first_weights": tensors["model.embed_tokens.weight"].view(-1)[:4].tolist(),
                     "last_row_first_8": logits[-1, :8].tolist(),
                     "argmax_per_row": logits.argmax(dim=1).tolist(),
                     "sum_abs": float(logits.abs().sum())}
    return out


if __name__ == "__main__":
    path = Path(__file__).resolve().parent / "plain_tiny.json"
    path.write_text(json.dumps(golden(), indent=1) + "\n")
    print(f"wrote {path}")
