"""Random weights from a configuration and a seed, and a model folder made of them.

Each tensor is drawn from its own generator keyed by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist.  The reference seeds
torch once and takes torch's default initialisers (python/model.py:73-77).
"""
from __future__ import annotations

import json
import os
import zlib
from dataclasses import dataclass
from typing import Dict, Sequence

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


@dataclass(frozen=True)
class InitScheme:
    """Standard deviations of the draws; means are 0 except norm weights (1)."""
    matrix_std: float = 0.02
    bias_std: float = 0.0
    norm_weight_std: float = 0.0
    norm_bias_std: float = 0.0


def random_tensors(declared: Sequence[TensorDecl], seed: int, scheme: InitScheme = InitScheme(),
                   dtype: torch.dtype = torch.bfloat16, device: str = "cpu",
                   draw_on: str = None) -> Dict[str, torch.Tensor]:
    """One tensor per declaration, on ``device``.  How a tensor is drawn follows from its declared
    role alone.  ``draw_on`` names the device whose generator draws the values (default: ``device``):
    torch's CPU and CUDA generators give different values for one seed, so values that another
    program has to draw again (a plain implementation on the CPU) are drawn with ``draw_on="cpu"``."""
    draw_on = draw_on or device
    by_role = {"norm_weight": (1.0, scheme.norm_weight_std), "norm_bias": (0.0, scheme.norm_bias_std),
               "vector": (0.0, scheme.bias_std), "matrix": (0.0, scheme.matrix_std),
               "table": (0.0, scheme.matrix_std)}
    out = {}
    for d in declared:
        g = torch.Generator(device=draw_on)
        g.manual_seed((int(seed) * 1000003 + zlib.crc32(d.name.encode())) & 0x7FFFFFFFFFFFFFFF)
        mean, std = by_role[d.role]
        if std == 0.0:
            t = torch.full(d.shape, mean, dtype=torch.float32, device=device)
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device=draw_on).normal_(mean, std, generator=g)
        out[d.name] = t.to(dtype).to(device)
    return out


def write_model_folder(folder: str, config, seed: int, scheme: InitScheme = InitScheme(),
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes ``config.json`` and ``model.safetensors`` of a random model of ``config``."""
    from ..models.model import declared_tensors  # parts declare their tensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    tensors = random_tensors(declared_tensors(config.model_spec()), seed, scheme, dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
