"""Position encodings."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import PositionEncoding, register_position


class LearnedPositions(PositionEncoding):
    """A learned row per absolute position, added to the token's row at the input:
    x[r] = wte[tok[r]] + wpe[pos[r]] (reference: python/model.py:65-66, kernels/elementwise.cu:7-17).
    Keys are cached as projected; nothing is applied to them later."""

    def __init__(self, width: int, n_positions: int, tensor: str = "wpe.weight"):
        self.width, self.n_positions, self.tensor = int(width), int(n_positions), tensor
        self.table = None

    def tensors(self, prefix):
        return [TensorDecl(prefix + self.tensor, (self.n_positions, self.width), "table")]

    def load(self, prefix, tensors, dtype, device):
        self.table = self._matrix(tensors[prefix + self.tensor], dtype, device)

    def embed(self, ctx, token_table, multiplier: float = 1.0):
        x = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=token_table.device)
        ops.embed_pos_add(ctx.tokens, ctx.positions, token_table, self.table, x, ctx.error_flag, multiplier)
        return x


class NoPositions(PositionEncoding):
    """Token rows only (for mixers that carry order themselves)."""

    def __init__(self, width: int):
        self.width = int(width)

    def embed(self, ctx, token_table, multiplier: float = 1.0):
        x = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=token_table.device)
        ops.embed_pos_add(ctx.tokens, ctx.positions, token_table, None, x, ctx.error_flag, multiplier)
        return x


register_position("learned", LearnedPositions)
register_position("none", NoPositions)
