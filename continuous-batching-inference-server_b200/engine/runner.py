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
        self.runner = None
        self.fixed_shapes = False              # the step is being captured for replay: no size may depend on this batch
        self.max_positions = 0

    def layer_cache(self, li: int):
        return self.pool.layer_cache.get(li)

    def layer_state(self, li: int):
        return self.pool.state.get(li)

    def attention(self, mixer, qkv, cache, view, out):
        """Stores this step's keys/values of ``mixer`` (if it keeps its own) and attends over the pages."""
        run_attention(self, mixer, qkv, cache, view, out)

    def decode_scratch(self, n_floats: int, n_counters: int):
        """(float scratch, zeroed int32 counters) for kernels that split work and merge it in the last block."""
        return self.runner.scratch(n_floats, n_counters)


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
        # decode-only steps replay a captured CUDA graph unless a part reads device values on the host
        self.use_graphs = all(getattr(part, "capturable", True)
                              for layer in model.layers for _, part in layer.parts())
        self._graphs: Dict[int, tuple] = {}      # rows of a decode-only step -> (graph, context, logits)
        worst = heads = 0
        for layer in model.layers:
            m = layer.mixer
            if hasattr(m, "n_head") and hasattr(m, "head_dim"):
                worst = max(worst, ops.decode_scratch_floats(S, m.n_head, m.head_dim, 32))
                heads = max(heads, m.n_head)
        self._scratch = torch.empty(max(worst, 1), dtype=torch.float32, device=self.device)
        self._counters = torch.zeros(max(S * heads, 1), dtype=torch.int32, device=self.device)
        self.graph_replays = 0
        self._table_cache: Dict[tuple, tuple] = {}   # (slot, group) -> (request id, pages, numpy row)

    # ------------------------------------------------------------------
    def _dev_view(self, name, n=None):
        o, full = self._layout[name]
        return self._dev[o:o + (full if n is None else n)]

    def _host_view(self, name, n=None):
        o, full = self._layout[name]
        return self._host_np[o:o + (full if n is None else n)]

    def bytes_per_step_h2d(self) -> int:
        """Bytes of the packed step description copied from pinned host memory every step."""
        return self._host.numel() * 4

    def scratch(self, n_floats: int, n_counters: int):
        """Float scratch for partial results and int32 counters (zero between launches) shared by the
        kernels of a step; both grow if a part asks for more than the built-in attention needs."""
        if n_floats > self._scratch.numel() or n_counters > self._counters.numel():
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("kernel scratch would have to grow during graph capture")
            if n_floats > self._scratch.numel():
                self._scratch = torch.empty(n_floats, dtype=torch.float32, device=self.device)
            if n_counters > self._counters.numel():
                self._counters = torch.zeros(n_counters, dtype=torch.int32, device=self.device)
        return self._scratch, self._counters

    def validate(self, entries: Sequence[StepEntry], reserved_ahead: bool = False) -> None:
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
            if reserved_ahead and mgr.length(e.slot) >= e.start + n:
                pass
            elif mgr.length(e.slot) != e.start + n:
                raise StepError(f"slot {e.slot}: the cache holds room for {mgr.length(e.slot)} tokens, the step "
                                f"brings tokens {e.start}..{e.start + n - 1}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= spec.vocab_size:
                raise StepError(f"slot {e.slot}: token id {lo if lo < 0 else hi} outside the vocabulary of "
                                f"{spec.vocab_size}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} outside its {n} tokens")

    def build_context(self, entries: Sequence[StepEntry], pad_rows: int = 0, all_logits: bool = False,
                      reserved_ahead: bool = False) -> StepContext:
        """Packs the step into the host buffer, copies it over, returns the views.

        ``pad_rows`` > 0 (decode-only steps): the step is laid out for exactly that many rows and
        segments; rows beyond the entries are padding (segment -1: no cache write, zero attention
        output).  ``all_logits``: every row's logits, whatever the entries want."""
        self.validate(entries, reserved_ahead)
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
        n_real_rows, n_real_segs = T, S
        if pad_rows:
            assert all(len(e.tokens) == 1 for e in entries) and pad_rows >= S
            for name, fill in (("tokens", 0), ("positions", 0), ("row_seq", -1)):
                self._host_view(name, pad_rows)[T:] = fill
            for name in ("seg_slot", "seg_start", "seg_ctx"):
                self._host_view(name, pad_rows)[S:] = 0
            self._host_view("cu_rows", pad_rows + 1)[:] = np.minimum(np.arange(pad_rows + 1), T)
            T = S = pad_rows
        want_rows = (list(range(T)) if all_logits
                     else [row0_of_entry[ei] + w for ei, e in enumerate(entries) for w in e.want])
        R = len(want_rows)
        if R:
            self._host_view("logit_rows", R)[:] = np.asarray(want_rows, dtype=np.int32)
        for g in range(self._n_groups):
            ps, mb = pool.page_size, pool.max_blocks(g)
            sm = self._host_view(f"slot_mapping{g}", T)
            bt = self._host_view(f"block_table{g}", S * mb).reshape(S, mb)
            if pad_rows:
                sm[n_real_rows:] = -1
                bt[n_real_segs:] = -1
            windowed = mgr.window(g) > 0
            for s, ei in enumerate(order):
                e = entries[ei]
                table = self._table(e.slot, g, windowed)
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
        ctx.runner, ctx.max_positions, ctx.fixed_shapes = self, self.model.spec.max_positions, bool(pad_rows)
        ctx.n_rows, ctx.n_segments, ctx.n_logit_rows = T, S, R
        ctx.n_decode = T if pad_rows else sum(1 for e in entries if len(e.tokens) == 1)
        ctx.tokens, ctx.positions, ctx.row_seq = (self._dev_view(n, T) for n in ("tokens", "positions", "row_seq"))
        ctx.seg_slot, ctx.seg_start, ctx.seg_ctx = (self._dev_view(n, S) for n in ("seg_slot", "seg_start", "seg_ctx"))
        ctx.cu_rows = self._dev_view("cu_rows", S + 1)
        ctx.logit_rows = self._dev_view("logit_rows", R)
        ctx.host_seg_rows = [len(entries[ei].tokens) for ei in order] + [1] * (S - n_real_segs)
        ctx.host_seg_ctx = [entries[ei].start + len(entries[ei].tokens) for ei in order] + [0] * (S - n_real_segs)
        ctx.max_seg_rows, ctx.max_ctx = max(ctx.host_seg_rows), max(ctx.host_seg_ctx)
        for g in range(self._n_groups):
            mb = pool.max_blocks(g)
            ctx.groups.append(GroupView(self._dev_view(f"block_table{g}", S * mb).view(S, mb),
                                        self._dev_view(f"slot_mapping{g}", T), mb))
        return ctx

    def _table(self, slot: int, g: int, windowed: bool) -> np.ndarray:
        """The request's block table as an int32 array.  Tables of groups without a window only grow, so a
        copy is kept per (slot, group) and fetched again only when the request or its page count changed."""
        mgr = self.pool.manager
        if windowed:
            return np.asarray(mgr.block_table(slot, g), dtype=np.int32)
        rid, n = mgr.request_id(slot), mgr.table_len(slot, g)
        have = self._table_cache.get((slot, g))
        if have is None or have[0] != rid or have[1] != n:
            have = (rid, n, np.asarray(mgr.block_table(slot, g), dtype=np.int32))
            self._table_cache[(slot, g)] = have
        return have[2]

    def _bucket(self, n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return min(b, self.max_seqs)

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        """Runs one step; returns float32 logits ``[wanted, vocab]`` on the device, in the order
        of the entries and of each entry's ``want``.  The cache manager must already hold room
        for the step's tokens (``manager.append``).  With ``borrow`` the result may be a buffer
        that the next step overwrites (no copy).

        A step of single tokens only (decoding) is captured once per batch-size bucket as a CUDA
        graph and replayed, so its few hundred launches cost one; any other step runs launch by
        launch."""
        if self.use_graphs and all(len(e.tokens) == 1 for e in entries):
            out = self._decode_step_graph(entries)
            return out if borrow else out.clone()
        ctx = self.build_context(entries)
        return self.model.forward(ctx)

    def _decode_step_graph(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        rows = self._bucket(len(entries))
        ctx = self.build_context(entries, pad_rows=rows, all_logits=True)
        if rows not in self._graphs:
            self.model.forward(ctx)                       # warm-up outside the capture (writes the same cache values)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                logits = self.model.forward(ctx)
            self._graphs[rows] = (graph, logits)
        graph, logits = self._graphs[rows]
        graph.replay()
        self.graph_replays += 1
        want = [i for i, e in enumerate(entries) if len(e.want)]
        if len(want) == rows:
            return logits
        return logits[torch.tensor(want, dtype=torch.long, device=logits.device)] if want else logits[:0]

    @torch.no_grad()
    def decode_loop(self, entries: Sequence[StepEntry]) -> "DecodeLoop":
        """A run of greedy decode steps that never leaves the device: see ``DecodeLoop``."""
        return DecodeLoop(self, entries)


class DecodeLoop:
    """Greedy decoding of a fixed batch for many steps without the host in the loop.

    One CUDA graph holds a whole step: the model, the argmax over each row's logits, and the
    kernels that move every row on (the chosen token becomes the input, position + 1, the token
    slot from the request's block table).  The caller reserves the pages of all steps beforehand
    (``manager.append(slot, n_steps)``), so the block tables do not change while it runs."""

    def __init__(self, runner: ModelRunner, entries: Sequence[StepEntry]):
        self.runner = runner
        n = len(entries)
        ctx = runner.build_context(entries, pad_rows=n, all_logits=True, reserved_ahead=True)
        self.ctx = ctx
        self.sampled = torch.zeros(n, dtype=torch.int32, device=runner.device)
        self._one_step()                                  # warm-up, also moves the rows on by one
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._one_step()
        self.steps_done = 1

    def _one_step(self):
        ctx, r = self.ctx, self.runner
        logits = r.model.forward(ctx)
        ops.sample(logits, None, None, self.sampled)
        ops.decode_advance(ctx.tokens, ctx.positions, ctx.seg_start, ctx.seg_ctx, self.sampled, ctx.n_rows)
        for g, view in enumerate(ctx.groups):
            ops.slots_from_table(ctx.positions, ctx.row_seq, view.block_table, r.pool.page_size, view.slot_mapping,
                                 ctx.n_rows)

    def run(self, steps: int) -> None:
        for _ in range(steps):
            self.graph.replay()
        self.steps_done += steps

    def last_tokens(self) -> List[int]:
        return self.sampled.cpu().tolist()
