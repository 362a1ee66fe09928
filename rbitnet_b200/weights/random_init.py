"""Random weights from a configuration and a seed.

The reference has a no-file mode that builds a small model from a seed
(RBITNET_TOY / RBITNET_TOY_SEED, crates/bitnet-core/src/inference.rs:24-36,
crates/bitnet-core/src/model/toy.rs:16-30).  Here the same idea serves the real
architecture: every matrix ~ N(0, 0.02), every norm weight 1 + N(0, 0.02), each
tensor from a generator keyed by (seed, tensor name) so that any tensor can be
made again alone.  ``write_random_model`` writes a model folder (config.json,
model.safetensors) that loads like any other.
"""
from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Dict

import torch

from .safetensors_io import write_safetensors

STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 62) - 1)


def random_tensor(name: str, shape, kind: str, seed: int, dtype=torch.float32,
                  device="cpu") -> torch.Tensor:
    """kind "matrix": N(0, 0.02); kind "norm": 1 + N(0, 0.02).  Values are drawn
    in float32 and then rounded to ``dtype``."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    t = torch.randn(tuple(shape), generator=g, dtype=torch.float32, device=device) * STD
    if kind == "norm":
        t += 1.0
    elif kind != "matrix":
        raise ValueError(f"unknown init kind {kind!r}")
    return t.to(dtype)


def random_tensors(spec, seed: int, dtype=torch.float32, device="cpu") -> Dict[str, torch.Tensor]:
    """All tensors of a ModelSpec (``spec.tensor_table()``: name -> (shape, kind))."""
    return {name: random_tensor(name, shape, kind, seed, dtype, device)
            for name, (shape, kind) in spec.tensor_table().items()}


def write_random_model(folder, config, seed: int, dtype=torch.float32) -> Path:
    """Write config.json and model.safetensors for ``config`` (a ModelConfig)."""
    from ..config.registry import get_architecture
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    spec = get_architecture(config.architecture).build_spec(config)
    config.save(folder)
    write_safetensors(folder / "model.safetensors", random_tensors(spec, seed, dtype),
                      metadata={"format": "pt", "seed": seed})
    return folder
