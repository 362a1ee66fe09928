"""Weights by tensor name: checked against what the model's parts expect.

The model (built from its configuration) says which tensors it needs and their
shapes; ``check_tensors`` compares that with what a folder holds and raises ONE
error that lists every missing tensor, every unexpected tensor and every wrong
shape.  The reference checks element counts tensor by tensor and stops at the
first mismatch (crates/bitnet-core/src/llama/model.rs:147-194, messages such as
"layer {i} weight shape mismatch" and "missing tensor (tried [...])", :55-57);
full shapes and a complete list are this library's choice.  The reference looks
tensors up by name and never sees extras (:54-60); here an extra tensor is an
error unless the architecture names it as harmless (buffers that some exporters
store, an output matrix beside a tied embedding): those are listed in a warning
and left out.
"""
from __future__ import annotations

import fnmatch
import warnings
from typing import Dict, List, Mapping, Sequence, Tuple

import torch

from .safetensors_io import WeightError, read_model_tensors


def check_tensors(expected: Mapping[str, Tuple[int, ...]], found: Mapping[str, torch.Tensor],
                  where: str = "weights", ignorable: Sequence[str] = ()) -> List[str]:
    """Raises one ``WeightError`` for everything that does not fit.  ``ignorable``: name
    patterns (``fnmatch``) of tensors the model does not use and may find; those present are
    named in a warning and returned."""
    missing = [n for n in expected if n not in found]
    extra = [n for n in found if n not in expected]
    ignored = sorted(n for n in extra if any(fnmatch.fnmatchcase(n, p) for p in ignorable))
    unexpected = [n for n in extra if n not in ignored]
    if ignored:
        warnings.warn(f"{where}: {len(ignored)} tensors the model does not use were left out: "
                      + ", ".join(ignored[:8]) + (", ..." if len(ignored) > 8 else ""))
    wrong = [(n, tuple(expected[n]), tuple(found[n].shape)) for n in expected
             if n in found and tuple(found[n].shape) != tuple(expected[n])]
    if not (missing or unexpected or wrong):
        return ignored
    lines = [f"{where}: the tensors do not fit the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(
            f"{n} expected {list(e)} found {list(f)}" for n, e, f in sorted(wrong)))
    raise WeightError("\n".join(lines))


def load_checked(folder, expected: Mapping[str, Tuple[int, ...]],
                 ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    tensors = read_model_tensors(folder)
    for n in check_tensors(expected, tensors, where=str(folder), ignorable=ignorable):
        del tensors[n]
    return tensors
