"""Weights by tensor name: checked against what the model's parts expect.

The model (built from its configuration) says which tensors it needs and their
shapes; ``check_tensors`` compares that with what a folder holds and raises ONE
error that lists every missing tensor, every unexpected tensor and every wrong
shape.  The reference checks element counts tensor by tensor and stops at the
first mismatch (crates/bitnet-core/src/llama/model.rs:147-194, messages such as
"layer {i} weight shape mismatch" and "missing tensor (tried [...])", :55-57);
full shapes and a complete list are this library's choice.
"""
from __future__ import annotations

from typing import Dict, Mapping, Tuple

import torch

from .safetensors_io import WeightError, read_model_tensors


def check_tensors(expected: Mapping[str, Tuple[int, ...]], found: Mapping[str, torch.Tensor],
                  where: str = "weights") -> None:
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected]
    wrong = [(n, tuple(expected[n]), tuple(found[n].shape)) for n in expected
             if n in found and tuple(found[n].shape) != tuple(expected[n])]
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not fit the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(
            f"{n} expected {list(e)} found {list(f)}" for n, e, f in sorted(wrong)))
    raise WeightError("\n".join(lines))


def load_checked(folder, expected: Mapping[str, Tuple[int, ...]]) -> Dict[str, torch.Tensor]:
    tensors = read_model_tensors(folder)
    check_tensors(expected, tensors, where=str(folder))
    return tensors
