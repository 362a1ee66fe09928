"""Reader and writer of the safetensors container, by tensor name.

Format: 8 bytes little-endian header length n, n bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__``), then the raw little-endian data.  The file is memory-mapped
and tensors are views into the map, so a 16 GB model is not copied on the host
before it goes to the device.

Dtypes on the way in: BF16 stays bfloat16, F32 stays float32, F16 stays float16
(the engine converts it to its compute dtype, exactly so for float32), F64
becomes float32, integer tables become int32.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict

import numpy as np
import torch


class WeightError(ValueError):
    """A weight file that cannot be read, or that does not fit the model."""


_NP = {"F32": (np.dtype("<f4"), torch.float32), "F16": (np.dtype("<f2"), torch.float16),
       "BF16": (np.dtype("<u2"), torch.bfloat16), "F64": (np.dtype("<f8"), torch.float64),
       "I64": (np.dtype("<i8"), torch.int64), "I32": (np.dtype("<i4"), torch.int32),
       "I16": (np.dtype("<i2"), torch.int16), "I8": (np.dtype("i1"), torch.int8),
       "U8": (np.dtype("u1"), torch.uint8), "BOOL": (np.dtype("u1"), torch.bool)}
_NAME_OF = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
            torch.float64: "F64", torch.int64: "I64", torch.int32: "I32"}


def _storage_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.float16):
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.int32):
        return t.to(torch.int32)
    return t


def read_header(path) -> tuple:
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise WeightError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise WeightError(f"{path}: header length {n} exceeds the file's {size} bytes")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightError(f"{path}: header is not valid JSON ({e})") from None
    if not isinstance(header, dict):
        raise WeightError(f"{path}: header must be a JSON object")
    return header, 8 + n, size


def read_safetensors(path) -> Dict[str, torch.Tensor]:
    """All tensors of one file, as views of a private memory map (CPU tensors)."""
    path = Path(path)
    header, base, size = read_header(path)
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dt, shape, (a, b) = info["dtype"], list(info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise WeightError(f"{path}: malformed header entry for {name!r}") from None
        if dt not in _NP:
            raise WeightError(f"{path}: tensor {name!r} has unknown dtype {dt!r}")
        npdt, tdt = _NP[dt]
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if a < 0 or b < a or base + b > size:
            raise WeightError(f"{path}: tensor {name!r} data [{a},{b}) lies outside the file "
                              f"(truncated? {size - base} data bytes present)")
        if b - a != count * npdt.itemsize:
            raise WeightError(f"{path}: tensor {name!r} has {b - a} bytes but shape {shape} "
                              f"of {dt} needs {count * npdt.itemsize}")
        arr = np.frombuffer(mm, dtype=npdt, count=count, offset=base + a)
        t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t.to(torch.bool)
        out[name] = _storage_dtype(t.reshape(shape))
    return out


def read_model_tensors(folder) -> Dict[str, torch.Tensor]:
    """Tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` names."""
    folder = Path(folder)
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    if single.is_file():
        return read_safetensors(single)
    if index.is_file():
        try:
            wm = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError) as e:
            raise WeightError(f"{index}: no weight_map ({e})") from None
        out: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(wm.values())):
            if not (folder / shard).is_file():
                raise WeightError(f"{index}: names shard {shard!r}, which is not in the folder")
            out.update(read_safetensors(folder / shard))
        return out
    raise WeightError(f"{folder}: no model.safetensors (or model.safetensors.index.json)")


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAME_OF:
            raise WeightError(f"cannot write tensor {name!r} of dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME_OF[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
