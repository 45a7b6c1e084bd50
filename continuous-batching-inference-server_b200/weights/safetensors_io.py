"""Reading and writing ``model.safetensors`` by tensor name.

File format: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the raw
little-endian tensor bytes.  The reference's weight file is a flat run of fp32
without names or shapes (python/export_weights.py:4-19, src/model_weights.cpp:46-72);
truncation is its only check (src/model_weights.cpp:23-25).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
           "U8": torch.uint8, "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightsError(ValueError):
    """A weight file that cannot be read or does not fit the model."""


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Returns ``{name: tensor}`` on the CPU in the stored dtype (copied out of the file)."""
    if not os.path.isfile(path):
        raise WeightsError(f"{path} does not exist")
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        if size < 8:
            raise WeightsError(f"{path}: too short for a safetensors header ({size} bytes)")
        (hlen,) = struct.unpack("<Q", f.read(8))
        if 8 + hlen > size:
            raise WeightsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: header is not JSON: {e}") from None
        base = 8 + hlen
        out: Dict[str, torch.Tensor] = {}
        problems = []
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        try:
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                dt = _DTYPES.get(meta.get("dtype"))
                if dt is None:
                    problems.append(f"{name}: unknown dtype {meta.get('dtype')!r}")
                    continue
                shape = list(meta["shape"])
                b, e = meta["data_offsets"]
                numel = 1
                for s in shape:
                    numel *= s
                want = numel * torch.empty((), dtype=dt).element_size()
                if e - b != want:
                    problems.append(f"{name}: {e - b} bytes stored, shape {shape} needs {want}")
                    continue
                if b < 0 or base + e > size:
                    problems.append(f"{name}: data_offsets [{b}, {e}) lie outside the file")
                    continue
                if numel == 0:
                    out[name] = torch.empty(shape, dtype=dt)
                    continue
                buf = bytearray(mm[base + b: base + e])
                out[name] = torch.frombuffer(buf, dtype=dt).reshape(shape)
        finally:
            if mm is not None:
                mm.close()
    if problems:
        raise WeightsError(f"{path}: " + "; ".join(problems))
    return out


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"{name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
