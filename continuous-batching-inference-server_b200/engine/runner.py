"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step holds portions of prompts beside single decoded tokens, cut anywhere.  It runs only
the tokens it is given, as one batch, and returns the logits at the wanted places.  The
reference's ``TransformerRunner::forward_step`` (src/transformer.cpp:44-99) takes rows
``(token, position, seq_id)``, copies a whole 2048-entry page table per ROW to the device
(:52-63) and returns every row's logits to the host (:95-98).  Here a step is a list of
segments; one packed int32 buffer per step carries tokens, positions, each group's block
table per REQUEST and token slots; only wanted rows reach the head; logits stay on the device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CachePool
from ..kernels import ops
from .attention_dispatch import run_attention


class StepError(ValueError):
    """A step that does not fit the cache's state or the engine's limits."""


@dataclass
class StepEntry:
    """Tokens ``tokens`` of the request in ``slot`` at positions ``start``..; logits are wanted
    at the places ``want`` (indices into ``tokens``)."""
    slot: int
    start: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


@dataclass
class GroupView:
    """What the layers of one cache group see of a step."""
    block_table: torch.Tensor     # int32 [S, max_blocks]: logical page -> physical page (-1: given back)
    slot_mapping: torch.Tensor    # int32 [T]: token slot (page * page_size + offset) of each row
    max_blocks: int


class StepContext:
    """Everything a part may read about the running step.  Rows are ordered: all segments of one
    token first (``n_decode`` of them), then the longer segments, each segment's rows in a run."""

    def __init__(self):
        self.dtype: torch.dtype = torch.float32
        self.n_rows = 0
        self.n_segments = 0
        self.n_decode = 0                       # leading segments that hold exactly one token
        self.tokens = self.positions = self.row_seq = None          # int32 [T]
        self.seg_slot = self.seg_start = self.seg_ctx = None        # int32 [S]: state slot, first position, length after the step
        self.cu_rows = None                                          # int32 [S+1]
        self.logit_rows = None                                       # int32 [R]
        self.n_logit_rows = 0
        self.groups: List[GroupView] = []
        self.error_flag = None
        self.host_seg_rows: List[int] = []     # rows of each segment (host copy)
        self.host_seg_ctx: List[int] = []
        self.max_seg_rows = 0
        self.max_ctx = 0
        self.pool: Optional[CachePool] = None
        self.scratch: Dict[str, torch.Tensor] = {}

    def layer_cache(self, li: int):
        return self.pool.layer_cache.get(li)

    def layer_state(self, li: int):
        return self.pool.state.get(li)

    def attention(self, mixer, qkv, cache, view, out):
        run_attention(self, mixer, qkv, cache, view, out)


class ModelRunner:
    def __init__(self, model, pool: CachePool, *, max_batched_tokens: int = 512, max_num_seqs: int = 16):
        self.model, self.pool = model, pool
        self.max_tokens, self.max_seqs = int(max_batched_tokens), int(max_num_seqs)
        self.device = model.device
        T, S = self.max_tokens, self.max_seqs
        self._layout: Dict[str, tuple] = {}
        off = 0

        def field_(name, n):
            nonlocal off
            self._layout[name] = (off, n)
            off += (n + 3) // 4 * 4      # 16-byte aligned fields

        for name in ("tokens", "positions", "row_seq", "logit_rows"):
            field_(name, T)
        for name in ("seg_slot", "seg_start", "seg_ctx"):
            field_(name, S)
        field_("cu_rows", S + 1)
        self._n_groups = len(pool.groups)
        for g in range(self._n_groups):
            field_(f"slot_mapping{g}", T)
            field_(f"block_table{g}", S * pool.max_blocks(g))
        self._host = torch.zeros(off, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
            else torch.zeros(off, dtype=torch.int32)
        self._host_np = self._host.numpy()
        self._dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copied = None    # event after the last host->device copy of the packed buffer

    # ------------------------------------------------------------------
    def _dev_view(self, name, n=None):
        o, full = self._layout[name]
        return self._dev[o:o + (full if n is None else n)]

    def _host_view(self, name, n=None):
        o, full = self._layout[name]
        return self._host_np[o:o + (full if n is None else n)]

    def validate(self, entries: Sequence[StepEntry]) -> None:
        spec, mgr = self.model.spec, self.pool.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_seqs:
            raise StepError(f"{len(entries)} requests in one step; the engine was made for {self.max_seqs}")
        total = sum(len(e.tokens) for e in entries)
        if total > self.max_tokens:
            raise StepError(f"{total} tokens in one step; the engine was made for {self.max_tokens}")
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot}: an entry without tokens")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not mgr.live(e.slot):
                raise StepError(f"slot {e.slot} holds no request")
            if e.start < 0 or e.start + n > spec.max_positions:
                raise StepError(f"slot {e.slot}: positions {e.start}..{e.start + n - 1} exceed the model's "
                                f"{spec.max_positions} positions")
            if mgr.length(e.slot) != e.start + n:
                raise StepError(f"slot {e.slot}: the cache holds room for {mgr.length(e.slot)} tokens, the step "
                                f"brings tokens {e.start}..{e.start + n - 1}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= spec.vocab_size:
                raise StepError(f"slot {e.slot}: token id {lo if lo < 0 else hi} outside the vocabulary of "
                                f"{spec.vocab_size}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} outside its {n} tokens")

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Packs the step into the host buffer, copies it over, returns the views."""
        self.validate(entries)
        if self._copied is not None:
            self._copied.synchronize()   # the last step's copy must have left the pinned buffer
        mgr, pool = self.pool.manager, self.pool
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        tokens, positions, row_seq = (self._host_view(n, T) for n in ("tokens", "positions", "row_seq"))
        seg_slot, seg_start, seg_ctx = (self._host_view(n, S) for n in ("seg_slot", "seg_start", "seg_ctx"))
        cu = self._host_view("cu_rows", S + 1)
        row0_of_entry = [0] * S
        r = 0
        cu[0] = 0
        for s, ei in enumerate(order):
            e = entries[ei]
            n = len(e.tokens)
            row0_of_entry[ei] = r
            tokens[r:r + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[r:r + n] = np.arange(e.start, e.start + n, dtype=np.int32)
            row_seq[r:r + n] = s
            seg_slot[s], seg_start[s], seg_ctx[s] = e.slot, e.start, e.start + n
            r += n
            cu[s + 1] = r
        want_rows = [row0_of_entry[ei] + w for ei, e in enumerate(entries) for w in e.want]
        R = len(want_rows)
        if R:
            self._host_view("logit_rows", R)[:] = np.asarray(want_rows, dtype=np.int32)
        for g in range(self._n_groups):
            ps, mb = pool.page_size, pool.max_blocks(g)
            sm = self._host_view(f"slot_mapping{g}", T)
            bt = self._host_view(f"block_table{g}", S * mb).reshape(S, mb)
            for s, ei in enumerate(order):
                e = entries[ei]
                table = np.asarray(mgr.block_table(e.slot, g), dtype=np.int32)
                bt[s, :len(table)] = table
                bt[s, len(table):] = -1
                pos = positions[cu[s]:cu[s + 1]]
                sm[cu[s]:cu[s + 1]] = table[pos // ps] * ps + pos % ps
        self._dev.copy_(self._host, non_blocking=True)
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record()

        ctx = StepContext()
        ctx.dtype, ctx.pool, ctx.error_flag = self.model.dtype, pool, self.error_flag
        ctx.n_rows, ctx.n_segments, ctx.n_logit_rows = T, S, R
        ctx.n_decode = sum(1 for e in entries if len(e.tokens) == 1)
        ctx.tokens, ctx.positions, ctx.row_seq = (self._dev_view(n, T) for n in ("tokens", "positions", "row_seq"))
        ctx.seg_slot, ctx.seg_start, ctx.seg_ctx = (self._dev_view(n, S) for n in ("seg_slot", "seg_start", "seg_ctx"))
        ctx.cu_rows = self._dev_view("cu_rows", S + 1)
        ctx.logit_rows = self._dev_view("logit_rows", R)
        ctx.host_seg_rows = [len(entries[ei].tokens) for ei in order]
        ctx.host_seg_ctx = [entries[ei].start + len(entries[ei].tokens) for ei in order]
        ctx.max_seg_rows, ctx.max_ctx = max(ctx.host_seg_rows), max(ctx.host_seg_ctx)
        for g in range(self._n_groups):
            mb = pool.max_blocks(g)
            ctx.groups.append(GroupView(self._dev_view(f"block_table{g}", S * mb).view(S, mb),
                                        self._dev_view(f"slot_mapping{g}", T), mb))
        return ctx

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one step; returns float32 logits ``[wanted, vocab]`` on the device, in the order
        of the entries and of each entry's ``want``.  The cache manager must already hold room
        for the step's tokens (``manager.append``)."""
        ctx = self.build_context(entries)
        return self.model.forward(ctx)
