"""Shared pieces of the tests: model folders with random weights, and the one place
where tolerances are stated."""
from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_llama as plain
from rbitnet_b200.config import config_from_dict
from rbitnet_b200.config.registry import get_architecture
from rbitnet_b200.weights import random_tensors, write_safetensors

# Tolerances (absolute, relative to the largest reference value) against the plain
# implementation run in float64 on the same stored weights.
# float32: rounding of float32 sums only.  The products add up to 14,336 terms one after the other
# in float32 (the reference's order, crates/bitnet-core/src/llama/model.rs:72-74), whose rounding
# errors walk to about sqrt(terms) * 2^-24 of the result: the largest error seen over all tests is
# 6.4e-6 of the largest logit (the Llama-3-8B layer sizes; the tiny configurations stay below 1e-6),
# so the band is the reference's own guideline of 1e-5 (docs/GOLDEN_TESTS.md:24) plus twice that.
# bfloat16: activations between kernels and the cache are rounded to bfloat16 (8 bits of mantissa)
# nine times per layer; the residual stream, norms, softmax and sums are float32.  See bf16_rtol;
# the default is its value for the three layers of the deeper tiny configuration.
TOL = {"float32": (1e-5, 2e-5), "bfloat16": (0.0, 2e-2)}


#: largest error seen per dtype, as a fraction of the largest reference value (printed at the end of a run)
WORST = {}


def bf16_rtol(layers: int) -> float:
    """The bfloat16 band for a model of ``layers`` layers, as a fraction of the largest reference
    value.  A layer rounds to bfloat16 at nine places (the normed inputs, q/k/v, the cache, P, the
    attention output, the gated activation), which moves the logits by up to about 1 % of the
    largest one at any width when attention scores have a deviation of about one (measured: 0.9 to
    1.1 % for one and two layers of the Llama-3-8B, Llama-2-7B and TinyLlama layer sizes, 1.8 % for
    eight layers; scores twice as spread give twice the error, which is why the tests scale q and k
    by 1 / (0.02 sqrt(width))); the layers' errors are independent and add in quadrature."""
    return 1.2e-2 * max(1.0, float(layers)) ** 0.5


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "", rtol=None):
    got, ref = got.detach().double().cpu(), ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    atol, default_rtol = TOL[dtype]
    rtol = default_rtol if rtol is None else rtol
    scale = float(ref.abs().max())
    err = float((got - ref).abs().max())
    import os
    key = (dtype, os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0].split("::", 1)[-1])
    WORST[key] = max(WORST.get(key, 0.0), err / max(scale, 1e-30))
    assert err <= atol + rtol * scale, f"{what}: max error {err:.3e} > {atol} + {rtol} * {scale:.3e} ({dtype})"
    return err


def sharpen(tensors: dict, factor: float) -> dict:
    """Scale every query and key projection so that attention scores spread out (random
    small weights give nearly uniform attention, which would hide a wrong mask or position)."""
    out = dict(tensors)
    for name in tensors:
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            out[name] = tensors[name] * factor
    return out


def make_model_dir(folder, cfg_dict: dict, seed: int, store: str = "float32", factor: float = 4.0) -> Path:
    """Writes config.json and model.safetensors; ``store`` is the dtype on file."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(cfg_dict)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    tensors = sharpen(random_tensors(spec, seed), factor)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store]
    tensors = {k: v.to(dt) for k, v in tensors.items()}
    (folder / "config.json").write_text(json.dumps(cfg_dict))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


class PlainModel:
    """The plain implementation on a model folder, with whole-sequence logits cached."""

    def __init__(self, folder):
        self.cfg, self.tensors = plain.load_folder(folder)
        self._memo = {}

    def logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.tensors, list(tokens), torch.float64)
        return self._memo[key]
