"""Block arrangements."""
from __future__ import annotations

import struct

import torch

from ..kernels import ops
from .attention import PagedAttention
from .base import Block, register_block
from .dense import DenseFeedForward
from .layernorm import LayerNorm


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))   (reference: python/model.py:48-51).
    Each add is folded into the norm that follows it, so a layer's feed-forward output
    is handed on as pending and added by the next layer's first norm (or the final norm).

    With ``CBIS_FUSED_DECODE=1`` a decode step (single tokens only, up to 16 rows, bfloat16) of consecutive blocks
    made of LayerNorm, paged attention with keys of its own (head size 64 or 128) and a dense feed-forward runs as ONE
    persistent kernel for the whole run of layers (``ops.decode_layers``); everything else, and by default this too
    (the chain of kernels is the faster of the two as measured), runs part by part."""

    def forward(self, ctx, x, pending, cache, state):
        # A part that normalises inside its own first kernel and adds into the residual stream (a decode step of a
        # few rows: two kernels fewer per layer) is handed the stream; any other gets normalised rows and hands
        # back what is to be added.
        if self.mixer.fuses_norm(ctx, self.norm_mixer):
            if pending is not None:
                ops.add_delta(x, pending.value, pending.bias)
            self.mixer.forward_residual(ctx, x, self.norm_mixer, cache, state)
            d = None
        else:
            h = self.norm_mixer.forward(ctx, x, pending)
            ctx.residual = x          # a part may add its result into the stream itself and hand back None
            d = self.mixer.forward(ctx, h, cache, state)
            ctx.residual = None
        if self.feed_forward.fuses_norm(ctx, self.norm_feed_forward):
            if d is not None:
                ops.add_delta(x, d.value, d.bias)
            self.feed_forward.forward_residual(ctx, x, self.norm_feed_forward)
            return None
        h = self.norm_feed_forward.forward(ctx, x, d)
        ctx.residual = x
        d = self.feed_forward.forward(ctx, h)
        ctx.residual = None
        return d

    # ---- a run of layers in one kernel ----------------------------------------------------------------
    def _static_run_key(self, cache):
        """The part of ``run_key`` that does not depend on the step; None if this block cannot take part."""
        key = getattr(self, "_run_key", False)
        if key is not False:
            return key
        a, f, n1, n2 = self.mixer, self.feed_forward, self.norm_mixer, self.norm_feed_forward
        key = None
        if (type(a) is PagedAttention and type(f) is DenseFeedForward and type(n1) is LayerNorm and type(n2) is LayerNorm
                and a.own_kv and a.head_dim in (64, 128) and cache is not None and cache.page_size % 16 == 0
                and a.width == f.width == n1.width == n2.width and a.width % 8 == 0 and f.inner % 8 == 0
                and a.w_qkv is not None and a.w_qkv.is_cuda and a.w_qkv.dtype == torch.bfloat16):
            key = ("decode_layers", a.width, a.n_head, a.n_kv_head, a.head_dim, f.inner, f.activation, a.window, a.scale,
                   cache.group, cache.page_size)
        self._run_key = key
        return key

    def run_key(self, ctx, cache, state):
        if (not ops.USE_FUSED_DECODE or ctx.dtype != torch.bfloat16 or ctx.n_rows != ctx.n_decode
                or not 1 <= ctx.n_rows <= ops.FUSED_DECODE_MAX_ROWS or ctx.runner is None):
            return None
        pe = ctx.position_encoding
        if pe is not None and pe.acts_in_mixer:
            return None
        return self._static_run_key(cache)

    @classmethod
    def forward_run(cls, ctx, blocks, x, pending, caches, states):
        plans = ctx.runner.__dict__.setdefault("_decode_layer_plans", {})
        pkey = tuple(id(b) for b in blocks)
        plan = plans.get(pkey)
        if plan is None:
            try:
                plan = _DecodeLayersPlan(blocks, caches, x.device)
            except ops.KernelError:        # sizes the kernel does not take: this run goes part by part, for good
                plan = False
            plans[pkey] = plan
        if plan is False:
            return super().forward_run(ctx, blocks, x, pending, caches, states)
        if pending is not None:            # what the layer before left to be added
            ops.add_delta(x, pending.value, pending.bias)
        try:
            plan.run(ctx, x)
        except ops.KernelError as err:
            if "CUDA error" in str(err):
                raise
            plans[pkey] = False            # refused before anything was launched
            return super().forward_run(ctx, blocks, x, None, caches, states)
        return None                        # x is up to date


class _DecodeLayersPlan:
    """What ``ops.decode_layers`` needs for a run of layers, made once: the TMA descriptors of the weights, the
    per-layer record of pointers, and scratch for q|k|v, the attention's output and the feed-forward's hidden rows."""

    def __init__(self, blocks, caches, device):
        a, f = blocks[0].mixer, blocks[0].feed_forward
        self.n_layers = len(blocks)
        self.d, self.n_head, self.n_kv_head, self.hd, self.F = a.width, a.n_head, a.n_kv_head, a.head_dim, f.inner
        self.act, self.window, self.scale = f.activation, a.window, a.scale
        self.group, self.page_size = caches[0].group, caches[0].page_size
        n_qkv = a.d_q + 2 * a.d_kv
        self.blocks = ops.decode_layers_blocks(min(n_qkv, self.d, self.F))
        maps, recs = [], []
        for b, cache in zip(blocks, caches):
            m, ff, n1, n2 = b.mixer, b.feed_forward, b.norm_mixer, b.norm_feed_forward
            for w in (m.w_qkv, m.w_o, ff.w1, ff.w2):
                maps.append(ops.decode_layers_map(w, self.blocks))
            ptrs = [t.data_ptr() for t in (n1.weight, n1.bias, m.b_qkv, m.b_o, n2.weight, n2.bias, ff.b1, ff.b2,
                                           cache.k, cache.v)]
            recs.append(struct.pack("<10Q2f", *ptrs, n1.eps, n2.eps))
        if len(recs[0]) != ops.decode_layers_desc_bytes():
            raise ops.KernelError("decode_layers: the per-layer record does not have the kernel's size")
        self.maps = torch.cat(maps).to(device)
        self.layers = torch.frombuffer(bytearray(b"".join(recs)), dtype=torch.uint8).to(device)
        rows = ops.FUSED_DECODE_MAX_ROWS
        self.qkv = torch.zeros((rows, n_qkv), dtype=torch.bfloat16, device=device)
        self.attn = torch.zeros((rows, a.d_q), dtype=torch.bfloat16, device=device)
        self.hidden = torch.zeros((rows, self.F), dtype=torch.bfloat16, device=device)
        self.grid_counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.keep = [(b, c) for b, c in zip(blocks, caches)]      # the records hold their addresses

    def run(self, ctx, x):
        M = ctx.n_rows
        nsplit = ops.decode_layers_splits(M, self.n_head, ctx.ctx_limit, self.blocks)
        part, counters = ctx.decode_scratch(ops.decode_scratch_floats(M, self.n_head, self.hd, nsplit), M * self.n_head)
        view = ctx.groups[self.group]
        self.grid_counter.zero_()
        ops.decode_layers(self.maps, self.layers, self.n_layers, self.blocks, M, self.d, self.n_head, self.n_kv_head,
                          self.hd, self.F, self.page_size, self.act, self.window, self.scale, nsplit, x, self.qkv,
                          self.attn, self.hidden, view.block_table, ctx.row_seq, ctx.positions, view.slot_mapping, part,
                          counters, self.grid_counter, getattr(self, "trace", None))


register_block("pre_norm", PreNormBlock)
