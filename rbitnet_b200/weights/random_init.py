"""Random weights from a configuration and a seed.

The reference has a no-file mode that builds a small model from a seed with one
deterministic generator, the same wherever it runs (RBITNET_TOY /
RBITNET_TOY_SEED, crates/bitnet-core/src/inference.rs:24-36; the generator
crates/bitnet-core/src/model/toy.rs:16-30).  Here the same idea serves the real
architecture: every matrix ~ N(0, 0.02), every norm weight 1 + N(0, 0.02).

Every value is a function of (seed, tensor name, element index) alone, made
with wrapping 64-bit integer arithmetic and one float32 multiplication, so the
CPU and the GPU fill bit-identical values, any tensor (or any part of one) can
be made again alone, and a 16 GB model never has to cross the bus:

    key   = first 8 bytes of sha256("<seed>:<name>")
    x     = key ^ (index * 0x9E3779B97F4A7C15)
    h1,h2 = mix64(x), mix64(x ^ 0xD1B54A32D192ED03)       (the splitmix64 finaliser)
    s     = the sum of the eight 16-bit fields of h1 and h2      (0 .. 8 * 65535)
    value = float32(s - 4 * 65535) * float32(0.02 / sqrt(8 * (65536^2 - 1) / 12))

a sum of eight uniform integers: mean 0, deviation 0.02, bell-shaped, within 4.9 deviations.
``write_random_model`` writes a model folder (config.json, model.safetensors) that
loads like any other; ``Engine.from_random`` makes the same tensors on the device.
"""
from __future__ import annotations

import hashlib
import math
from pathlib import Path
from typing import Dict

import torch

from .safetensors_io import write_safetensors

STD = 0.02
_M64 = (1 << 64) - 1
_GOLD = 0x9E3779B97F4A7C15
_SECOND = 0xD1B54A32D192ED03
_MUL1, _MUL2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
#: deviation of a sum of eight uniform integers of 0..65535
_SUM_STD = math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)
#: elements made at a time (a handful of int64 temporaries of this size are live)
_CHUNK = 1 << 24


def _signed(c: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    return c - (1 << 64) if c >= (1 << 63) else c


def _tensor_key(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64's finaliser on int64 tensors; right shifts are made logical by masking."""
    x = x + _signed(_GOLD)
    x = (x ^ ((x >> 30) & ((1 << 34) - 1))) * _signed(_MUL1)
    x = (x ^ ((x >> 27) & ((1 << 37) - 1))) * _signed(_MUL2)
    return x ^ ((x >> 31) & ((1 << 33) - 1))


def _field_sum(h: torch.Tensor) -> torch.Tensor:
    return (h & 0xFFFF) + ((h >> 16) & 0xFFFF) + ((h >> 32) & 0xFFFF) + ((h >> 48) & 0xFFFF)


def random_values(key: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """float32 values of elements ``start .. start+count-1`` of the tensor with this key,
    deviation 1 (before the scale to 0.02)."""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    x = (idx * _signed(_GOLD)) ^ _signed(key)
    s = _field_sum(_mix64(x)) + _field_sum(_mix64(x ^ _signed(_SECOND)))
    return (s - 4 * 65535).to(torch.float32)


def reference_value(seed: int, name: str, index: int) -> float:
    """The same value from Python integers (slow; for tests and for documentation)."""
    def mix(x):
        x = (x + _GOLD) & _M64
        x = ((x ^ (x >> 30)) * _MUL1) & _M64
        x = ((x ^ (x >> 27)) * _MUL2) & _M64
        return x ^ (x >> 31)
    x = _tensor_key(seed, name) ^ ((index * _GOLD) & _M64)
    s = 0
    for h in (mix(x), mix(x ^ _SECOND)):
        s += sum((h >> sh) & 0xFFFF for sh in (0, 16, 32, 48))
    return float(torch.tensor(float(s - 4 * 65535), dtype=torch.float32)
                 * torch.tensor(STD / _SUM_STD, dtype=torch.float32))


def random_tensor(name: str, shape, kind: str, seed: int, dtype=torch.float32,
                  device="cpu") -> torch.Tensor:
    """kind "matrix": N(0, 0.02); kind "norm": 1 + N(0, 0.02).  Values are made
    in float32 and then rounded to ``dtype``."""
    if kind not in ("matrix", "norm"):
        raise ValueError(f"unknown init kind {kind!r}")
    shape = tuple(int(s) for s in shape)
    n = math.prod(shape)
    key = _tensor_key(seed, name)
    out = torch.empty(n, dtype=dtype, device=device)
    scale = torch.tensor(STD / _SUM_STD, dtype=torch.float32, device=device)
    for a in range(0, n, _CHUNK):
        c = min(_CHUNK, n - a)
        v = random_values(key, a, c, device) * scale
        if kind == "norm":
            v = v + 1.0
        out[a:a + c] = v.to(dtype)
    return out.view(shape)


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
