"""Chooses the attention kernels for the rows of a step, and stores the step's keys and values.

Rows of one-token segments (decoding) come first, the rows of longer segments (portions of
prompts) after them, so each kind is one run of rows.  All kernels read the same pages and
keep the same contract: the query at position p sees the keys of its own request up to p
(inside the window, if the mixer has one).

* bfloat16, head size a multiple of 8, decoding rows: the split-KV decode kernel, which also
  stores the current token's key and value;
* bfloat16, head size 64 or 128, page size a power of two, longer segments: the TMA + tcgen05 kernel,
  after the cache-write kernel; other head sizes in steps of 16 up to 128 (and these two with
  CBIS_TCGEN05=0): the tiled mma.sync kernel;
* 32-bit, head size in steps of 16 up to 128, longer segments: the tiled 32-bit kernel (decoding rows: the general
  kernel);
* everything else: the general kernel, after the cache-write kernel.
"""
from __future__ import annotations

import torch

from ..kernels import ops


def _key_chunks(ctx, mixer, nd, T, hd, row_tile=64, blocks_per_tile=1, blocks_per_sm=8, min_chunk=256):
    """Few rows behind a long context give the tiled kernels too few blocks: the keys are then cut into chunks over
    more blocks, whose partial results (in the step's scratch memory) a second kernel merges."""
    limit = ctx.ctx_limit
    chunks = ops.prefill_key_chunks(-(-ctx.max_seg_rows // row_tile), mixer.n_head, ctx.n_segments - nd, limit,
                                    blocks_per_tile, blocks_per_sm, min_chunk)
    partial = None
    if chunks[0] > 1:
        partial, _ = ctx.decode_scratch((T - nd) * mixer.n_head * chunks[0] * (hd + 4), 1)
    return chunks, partial


def _general_chunks(ctx, mixer, rows, hd):
    """The general kernel gives a warp to every (row, head): a few rows behind a long context are cut the same way."""
    limit = ctx.ctx_limit
    chunks = ops.generic_key_chunks(rows, mixer.n_head, limit, hd)
    partial = None
    if chunks[0] > 1:
        partial, _ = ctx.decode_scratch(rows * mixer.n_head * chunks[0] * (hd + 4), 1)
    return chunks, partial


def run_attention(ctx, mixer, qkv, cache, view, out) -> None:
    nd = ctx.n_decode
    T = ctx.n_rows
    hd, ps = mixer.head_dim, cache.page_size
    k_off, v_off = mixer.d_q, mixer.d_q + mixer.d_kv
    fast_decode = qkv.dtype == torch.bfloat16 and hd % 8 == 0 and hd <= 256 and nd > 0
    first_general = nd if fast_decode else 0
    if fast_decode:
        limit = ctx.ctx_limit
        nsplit = ops.decode_splits(nd, mixer.n_head, limit)
        scratch = counters = None
        if nsplit > 1:
            scratch, counters = ctx.decode_scratch(ops.decode_scratch_floats(nd, mixer.n_head, hd, nsplit),
                                                   nd * mixer.n_head)
        ops.paged_decode_bf16(qkv[:nd], k_off if mixer.own_kv else -1, v_off if mixer.own_kv else -1, cache.k, cache.v,
                              view.block_table, ctx.row_seq, ctx.positions, view.slot_mapping, out[:nd], scratch, counters,
                              mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale, mixer.window, nsplit)
    if first_general < T:
        r = slice(first_general, T)
        if mixer.own_kv:
            ops.kv_write(qkv[r], k_off, v_off, cache.k, cache.v, view.slot_mapping[r], mixer.n_kv_head, hd, ps)
        tiled = qkv.dtype == torch.bfloat16 and ps & (ps - 1) == 0 and first_general == nd
        if tiled and hd in (64, 128) and 8 <= ps <= 128 and ops.USE_TCGEN05:
            # TMA + tcgen05: q and out keep their full row numbering, the kernel finds its rows through cu_rows
            chunks, partial = _key_chunks(ctx, mixer, nd, T, hd, row_tile=128, blocks_per_tile=2, blocks_per_sm=2, min_chunk=8192)
            ops.paged_prefill_tc5(qkv, cache.k, cache.v, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                  ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                  mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        if tiled and hd % 16 == 0 and 16 <= hd <= 128:
            chunks, partial = _key_chunks(ctx, mixer, nd, T, hd)
            ops.paged_prefill_bf16(qkv, cache.k, cache.v, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                   ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                   mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        if qkv.dtype == torch.float32 and hd % 16 == 0 and 16 <= hd <= 128 and ops.USE_TILED_F32:
            # 32-bit: decoding rows through the general kernel, the longer segments 64 rows to a block
            if nd > 0:
                d = slice(0, nd)
                chunks, partial = _general_chunks(ctx, mixer, nd, hd)
                ops.paged_attention_generic(qkv[d, :mixer.d_q], cache.k, cache.v, view.block_table, ctx.row_seq[d],
                                            ctx.positions[d], out[d], mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale,
                                            mixer.window, chunks, partial)
            if ctx.n_segments > nd:
                chunks, partial = _key_chunks(ctx, mixer, nd, T, hd)
                ops.paged_prefill_f32(qkv, cache.k, cache.v, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                      ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                      mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        chunks, partial = _general_chunks(ctx, mixer, T - first_general, hd)
        ops.paged_attention_generic(qkv[r, :mixer.d_q], cache.k, cache.v, view.block_table, ctx.row_seq[r],
                                    ctx.positions[r], out[r], mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale,
                                    mixer.window, chunks, partial)
