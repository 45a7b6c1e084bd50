"""The model's output: logits over the vocabulary at the wanted rows."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Head, register_head


class LinearHead(Head):
    """logits = soft_cap(logit_scale * (norm(x)[rows] @ W^T + bias)) in 32-bit, W ``[vocab, width]``.
    ``tensor`` None ties W to the embedding's table; ``bias`` names a bias tensor or is None;
    ``soft_cap`` c > 0 maps a logit v to c * tanh(v / c).  The reference's head has neither bias,
    scale nor cap and runs on every row (python/model.py:69-70, src/transformer.cpp:92-93); here only
    the rows whose logits are wanted reach it."""

    def __init__(self, vocab_size: int, width: int, tensor: Optional[str] = None, bias: Optional[str] = None,
                 logit_scale: float = 1.0, soft_cap: float = 0.0):
        self.vocab_size, self.width, self.tensor, self.bias_name = int(vocab_size), int(width), tensor, bias
        self.logit_scale, self.soft_cap = float(logit_scale), float(soft_cap)
        self.weight = self.bias = None

    def tensors(self, prefix):
        out = []
        if self.tensor is not None:
            out.append(TensorDecl(prefix + self.tensor, (self.vocab_size, self.width), "matrix"))
        if self.bias_name is not None:
            out.append(TensorDecl(prefix + self.bias_name, (self.vocab_size,), "vector"))
        return out

    def tie(self, embedding):
        if self.tensor is None:
            if embedding.table is None or tuple(embedding.table.shape) != (self.vocab_size, self.width):
                raise ValueError("a tied head needs an embedding with a table of [vocab, width]")
            self.weight = embedding.table

    def load(self, prefix, tensors, dtype, device):
        if self.tensor is not None:
            self.weight = self._matrix(tensors[prefix + self.tensor], dtype, device)
        if self.bias_name is not None:
            self.bias = self._vector(tensors[prefix + self.bias_name], device)

    def streamed_weights(self):
        return [self.weight]

    def forward(self, ctx, x, pending, final_norm):
        if ctx.n_logit_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=x.device)
        h = final_norm.forward(ctx, x, pending, rows=ctx.logit_rows)
        logits = ops.linear(h, self.weight, None, None, out_dtype=torch.float32)
        if self.bias is not None:
            ops.bias_act(logits, self.bias, None)
        if self.logit_scale != 1.0 or self.soft_cap > 0.0:
            ops.scale_soft_cap(logits, self.logit_scale, self.soft_cap)
        return logits


register_head("linear", LinearHead)
