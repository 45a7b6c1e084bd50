"""Weights of a model folder, matched by name against what the model's parts declare.

Floating tensors stored in 16 bits are kept as bfloat16, tensors stored in 32 bits
stay 32-bit, integer tables become int32.  A folder that does not fit the model
gives ONE error that lists every missing tensor, every unexpected tensor and every
wrong shape.  (The reference reads positionally and notices only a short file:
src/model_weights.cpp:22-32.)
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Dict, Iterable, Sequence, Tuple

import torch

from .safetensors_io import WeightsError, read_safetensors


ROLES = ("matrix", "table", "vector", "norm_weight", "norm_bias")


@dataclass(frozen=True)
class TensorDecl:
    """A tensor that a part expects: full name, shape, and role.

    role "matrix" / "table": used by matrix products or row lookups, held in the
    compute dtype; "vector": a bias, "norm_weight" / "norm_bias": the scale and shift of
    a norm; these three are always applied in 32-bit.  The role, never the name, tells
    the random-weights mode how to draw a tensor (a norm's scale is drawn around 1).
    """
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"

    def __post_init__(self):
        if self.role not in ROLES:
            raise ValueError(f"tensor {self.name!r}: role {self.role!r} is not one of {sorted(ROLES)}")


def _stored_form(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float16,):
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if not t.is_floating_point() and t.dtype != torch.int32:
        return t.to(torch.int32)
    return t


def read_model_tensors(folder: str) -> Dict[str, torch.Tensor]:
    """All tensors of ``folder/model.safetensors`` with a leading ``transformer.`` stripped."""
    raw = read_safetensors(os.path.join(folder, "model.safetensors"))
    out = {}
    for name, t in raw.items():
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        out[name] = _stored_form(t)
    return out


def check_tensors(declared: Sequence[TensorDecl], tensors: Dict[str, torch.Tensor],
                  ignored: Iterable[str] = (), where: str = "weights") -> None:
    """Raises one WeightsError naming all missing, unexpected and misshapen tensors."""
    want = {d.name: tuple(d.shape) for d in declared}
    ignore = [re.compile(p) for p in ignored]
    missing = sorted(n for n in want if n not in tensors)
    unexpected = sorted(n for n in tensors if n not in want and not any(p.search(n) for p in ignore))
    wrong = sorted(f"{n}: stored {tuple(tensors[n].shape)}, model needs {want[n]}"
                   for n in want if n in tensors and tuple(tensors[n].shape) != want[n])
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightsError(f"{where} do not fit the model: " + " | ".join(parts))
