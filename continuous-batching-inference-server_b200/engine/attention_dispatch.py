"""Chooses the attention kernel for the rows of a step.

Rows of one-token segments (decoding) come first, the rows of longer segments (portions of
prompts) after them, so each kind is one run of rows.  All kernels read the same pages and
keep the same contract: the query at position p sees the keys of its own request up to p.
"""
from __future__ import annotations

from ..kernels import ops


def run_attention(ctx, mixer, qkv, cache, view, out) -> None:
    q = qkv[:, :mixer.d_q]
    ops.paged_attention_generic(q, cache.k, cache.v, view.block_table, ctx.row_seq, ctx.positions, out,
                                mixer.n_head, mixer.n_kv_head, mixer.head_dim, cache.page_size, mixer.scale,
                                mixer.window)
