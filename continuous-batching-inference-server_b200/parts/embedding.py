"""The model's input: token rows from a table."""
from __future__ import annotations

from ..weights.loader import TensorDecl
from .base import Embedding, register_embedding


class TokenTable(Embedding):
    """x[r] = table[tok[r]] * multiplier + what the position encoding adds at the input
    (reference: python/model.py:65-66 has no multiplier; kernels/elementwise.cu:7-17).  The lookup and
    the position encoding's addition are one kernel, so the encoding's ``embed`` is handed the table."""

    def __init__(self, vocab_size: int, width: int, tensor: str = "wte.weight", multiplier: float = 1.0):
        self.vocab_size, self.width, self.tensor, self.multiplier = int(vocab_size), int(width), tensor, float(multiplier)
        self.table = None

    def tensors(self, prefix):
        return [TensorDecl(prefix + self.tensor, (self.vocab_size, self.width), "table")]

    def load(self, prefix, tensors, dtype, device):
        self.table = self._matrix(tensors[prefix + self.tensor], dtype, device)

    def forward(self, ctx, position):
        if self.multiplier == 1.0:
            return position.embed(ctx, self.table)
        return position.embed(ctx, self.table, multiplier=self.multiplier)


register_embedding("token_table", TokenTable)
