"""LayerNorm with the residual add folded in."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, Norm, register_norm


class LayerNorm(Norm):
    """y = (x - mean) * rsqrt(var + eps) * weight + bias over the last dim, biased variance,
    statistics in 32-bit (reference: kernels/elementwise.cu:21-57; eps is a literal there, :51)."""

    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        if not 0 < self.width <= ops.NORM_MAX_WIDTH:
            raise ValueError(f"LayerNorm: width {self.width} is outside 1..{ops.NORM_MAX_WIDTH}, the widest row the kernel takes")
        self.weight = self.bias = None

    def tensors(self, prefix):
        return [TensorDecl(prefix + "weight", (self.width,), "norm_weight"),
                TensorDecl(prefix + "bias", (self.width,), "norm_bias")]

    def load(self, prefix, tensors, dtype, device):
        self.weight = self._vector(tensors[prefix + "weight"], device)
        self.bias = self._vector(tensors[prefix + "bias"], device)

    def as_layernorm(self):
        return (self.weight, self.bias, self.eps) if self.weight is not None and self.bias is not None else None

    def forward(self, ctx, x, delta: Optional[Delta], rows=None, out_dtype=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype or ctx.dtype, device=x.device)
        ops.add_layernorm(x, delta.value if delta else None, delta.bias if delta else None,
                          self.weight, self.bias, self.eps, out, rows)
        return out


class NoNorm(Norm):
    """No normalisation: adds what is pending to the residual stream and hands the rows on in the
    compute dtype (for a model without a final norm)."""

    def __init__(self, width: int):
        self.width = int(width)
        if not 0 < self.width <= ops.NORM_MAX_WIDTH:
            raise ValueError(f"width {self.width} is outside 1..{ops.NORM_MAX_WIDTH}, the widest row the kernel takes")

    def forward(self, ctx, x, delta: Optional[Delta], rows=None, out_dtype=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype or ctx.dtype, device=x.device)
        ops.add_layernorm(x, delta.value if delta else None, delta.bias if delta else None, None, None, 0.0, out, rows)
        return out


register_norm("layernorm", LayerNorm)
register_norm("none", NoNorm)
