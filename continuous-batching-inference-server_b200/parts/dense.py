"""Dense feed-forward."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Delta, FeedForward, register_feed_forward


class DenseFeedForward(FeedForward):
    """act(h @ W1 + b1) @ W2 + b2 with the activation taken on the 32-bit sum
    (reference: python/model.py:50, src/transformer.cpp:86-88).  Weights come in GPT-2's
    Conv1D layout [in, out] and are kept transposed, [out, in]."""

    def __init__(self, width: int, inner: int, activation: str,
                 names=("mlp.c_fc", "mlp.c_proj")):
        if activation not in ops.ACT:
            raise ValueError(f"activation {activation!r} is not one of {sorted(k for k in ops.ACT if k)}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.fc, self.proj = names
        self.w1 = self.b1 = self.w2 = self.b2 = None

    def tensors(self, prefix):
        return [TensorDecl(f"{prefix}{self.fc}.weight", (self.width, self.inner)),
                TensorDecl(f"{prefix}{self.fc}.bias", (self.inner,), "vector"),
                TensorDecl(f"{prefix}{self.proj}.weight", (self.inner, self.width)),
                TensorDecl(f"{prefix}{self.proj}.bias", (self.width,), "vector")]

    def load(self, prefix, tensors, dtype, device):
        self.w1 = self._matrix_nk(tensors[f"{prefix}{self.fc}.weight"], dtype, device)
        self.b1 = self._vector(tensors[f"{prefix}{self.fc}.bias"], device)
        self.w2 = self._matrix_nk(tensors[f"{prefix}{self.proj}.weight"], dtype, device)
        self.b2 = self._vector(tensors[f"{prefix}{self.proj}.bias"], device)

    def streamed_weights(self):
        return [self.w1, self.w2]

    def fuses_norm(self, ctx, norm):
        return ops.ln_linear_takes(ctx, norm, self.w1) and self.inner % 8 == 0

    def forward_residual(self, ctx, x, norm):
        a = torch.empty((ctx.n_rows, self.inner), dtype=ctx.dtype, device=x.device)
        ops.ln_linear(x, *norm.as_layernorm(), self.w1, self.b1, self.activation, a)
        ops.gemm_small_m(a, self.w2, self.b2, None, x, accumulate=True)

    def forward(self, ctx, h):
        a = ops.linear(h, self.w1, self.b1, self.activation)
        if ops.linear_add_takes(a, self.w2, ctx.residual):         # the product adds into the residual stream itself
            ops.linear_add(a, self.w2, self.b2, ctx.residual)
            return None
        return Delta(ops.linear(a, self.w2, None, None, out_dtype=torch.float32), self.b2)


register_feed_forward("dense", DenseFeedForward)
