"""Causal attention over the paged cache."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import CacheNeed, Delta, Mixer, register_mixer


class PagedAttention(Mixer):
    """q|k|v = h @ c_attn + b; this step's k and v go into the layer's pages; every row attends
    to the keys of its request up to its own position (inside ``window`` if one is set), scores
    scaled by ``scale``, softmax in 32-bit; the heads' outputs side by side go through c_proj
    (reference: python/model.py:36-46, kernels/attention.cu:7-19 and 57-98,
    src/transformer.cpp:71-83).  ``n_kv_head`` < ``n_head`` shares each key/value head among
    n_head/n_kv_head query heads.  With ``own_kv=False`` the layer projects only queries and
    reads the cache of another layer."""

    def __init__(self, width: int, n_head: int, n_kv_head: int, head_dim: int, scale: float, window: int = 0,
                 own_kv: bool = True, names=("attn.c_attn", "attn.c_proj")):
        if n_head % n_kv_head:
            raise ValueError(f"n_head={n_head} is not a multiple of n_kv_head={n_kv_head}")
        if not 0 < int(head_dim) <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"head_dim={head_dim} is outside 1..{ops.ATTENTION_MAX_HEAD_DIM}, the largest head "
                             f"any attention kernel takes")
        self.width, self.n_head, self.n_kv_head, self.head_dim = int(width), int(n_head), int(n_kv_head), int(head_dim)
        self.scale, self.window, self.own_kv = float(scale), int(window), bool(own_kv)
        self.qkv_name, self.proj_name = names
        self.d_q = self.n_head * self.head_dim
        self.d_kv = self.n_kv_head * self.head_dim
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    @property
    def qkv_width(self):
        return self.d_q + (2 * self.d_kv if self.own_kv else 0)

    def cache_need(self):
        return CacheNeed.keys_values(self.n_kv_head, self.head_dim, self.window) if self.own_kv else None

    def tensors(self, prefix):
        return [TensorDecl(f"{prefix}{self.qkv_name}.weight", (self.width, self.qkv_width)),
                TensorDecl(f"{prefix}{self.qkv_name}.bias", (self.qkv_width,), "vector"),
                TensorDecl(f"{prefix}{self.proj_name}.weight", (self.d_q, self.width)),
                TensorDecl(f"{prefix}{self.proj_name}.bias", (self.width,), "vector")]

    def load(self, prefix, tensors, dtype, device):
        self.w_qkv = self._matrix_nk(tensors[f"{prefix}{self.qkv_name}.weight"], dtype, device)
        self.b_qkv = self._vector(tensors[f"{prefix}{self.qkv_name}.bias"], device)
        self.w_o = self._matrix_nk(tensors[f"{prefix}{self.proj_name}.weight"], dtype, device)
        self.b_o = self._vector(tensors[f"{prefix}{self.proj_name}.bias"], device)

    def streamed_weights(self):
        return [self.w_qkv, self.w_o]

    def fuses_norm(self, ctx, norm):
        return ops.ln_linear_takes(ctx, norm, self.w_qkv)

    def forward_residual(self, ctx, x, norm, cache, state):
        qkv = torch.empty((ctx.n_rows, self.qkv_width), dtype=ctx.dtype, device=x.device)
        ops.ln_linear(x, *norm.as_layernorm(), self.w_qkv, self.b_qkv, None, qkv)
        out = self._attend(ctx, qkv, cache)
        ops.gemm_small_m(out, self.w_o, self.b_o, None, x, accumulate=True)

    def forward(self, ctx, h, cache, state):
        out = self._attend(ctx, ops.linear(h, self.w_qkv, self.b_qkv), cache)
        if ops.linear_add_takes(out, self.w_o, ctx.residual):      # the product adds into the residual stream itself
            ops.linear_add(out, self.w_o, self.b_o, ctx.residual)
            return None
        return Delta(ops.linear(out, self.w_o, None, None, out_dtype=torch.float32), self.b_o)

    def _attend(self, ctx, qkv, cache):
        if cache is None:
            raise RuntimeError("attention needs a cache: its own or the layer's it reads")
        pe = ctx.position_encoding
        if pe is not None and pe.acts_in_mixer:      # e.g. a rotation of queries and keys, before the keys are cached
            pe.apply_in_mixer(ctx, qkv[:, :self.d_q], qkv[:, self.d_q:self.d_q + self.d_kv] if self.own_kv else None,
                              self.head_dim)
        view = ctx.groups[cache.group]
        out = torch.empty((ctx.n_rows, self.d_q), dtype=qkv.dtype, device=qkv.device)
        ctx.attention(self, qkv, cache, view, out)      # stores this step's k, v (if own_kv), then attends
        return out


register_mixer("attention", PagedAttention)
