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

import gc
import os
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CachePool
from ..kernels import ops
from ..kernels.library import host
from ..parts import AttentionLike
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
        self.position_encoding = None          # the model's position encoding: mixers call it if it acts inside them
        self.residual = None                   # while a block runs a part: the 32-bit residual rows, for a part that adds
                                               # its result there itself (it then hands back nothing to be added)
        self.runner = None
        self.fixed_shapes = False              # the step is being captured for replay: no size may depend on this batch
        self.max_positions = 0
        self.ctx_limit = 0                     # no request of the step is longer: the step's own maximum, or, in a step
                                               # captured for replay, the bound of the graph's context class

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
        self._n_groups = len(pool.groups)
        # the native packer validates a step and writes its description into the pinned buffer
        self._packer = host().StepPacker(pool.manager, T, S, model.spec.vocab_size, model.spec.max_positions,
                                         [pool.max_blocks(g) for g in range(self._n_groups)], self._n_groups)
        self._layout: Dict[str, tuple] = dict(self._packer.layout())
        off = self._packer.words()
        self._host = torch.zeros(off, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
            else torch.zeros(off, dtype=torch.int32)
        self._host_np = self._host.numpy()
        self._host_ptr = self._host.data_ptr()
        self._dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._copied = None    # event after the last host->device copy of the packed buffer
        self.feed_tokens = None   # int32 tokens on the device that replace the next packed step's (single-token entries, in order)
        self.last_info = None
        self._stream_obj = None
        # decode-only steps replay a captured CUDA graph unless a part reads device values on the host
        self.use_graphs = all(getattr(part, "capturable", True) for _, part in model.all_parts())
        self._graphs: Dict[tuple, tuple] = {}    # (rows of a decode-only step, context class) -> (graph, logits)
        # Steps with prompt portions: a step's SHAPE (tokens and wanted rows per entry, in order) fixes every launch
        # of it; what differs between two steps of one shape (tokens, positions, block tables, wanted rows) is in
        # the packed buffer on the device.  A shape seen for the eighth time is captured (that costs about 60 ms) and
        # replayed from then on: a 512-token portion then costs the host 0.1 ms instead of 3 (250 launches from Python).
        self.shape_graphs = os.environ.get("CBIS_SHAPE_GRAPHS", "1") != "0"
        self.max_shape_graphs = 24
        self.shape_graph_after = int(os.environ.get("CBIS_SHAPE_GRAPH_AFTER", "8"))
        self.shape_graph_min_host_s = 1e-3
        self._shape_seen: Dict[tuple, int] = {}
        self._shape_graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self.shape_captures = self.shape_replays = 0
        # Small steps with prompt portions (up to small_step_rows rows) whose launches cost the host more than the
        # device needs to run them: one graph per (rows rounded up to a power of two, class of context lengths), laid
        # out for max_num_seqs segments and wanted rows; every segment, of one token too, goes the way of the longer ones.
        self.small_step_graphs = os.environ.get("CBIS_SMALL_STEP_GRAPHS", "1") != "0"
        self.small_step_rows = min(256, self.max_tokens)
        self.small_graph_after = 8
        self.small_graph_host_factor = 1.5      # warm-up keeps a graph whose replay is this many times faster than the launches
        self.small_graph_span_factor = 1.15     # while serving: the device counts as starved if a step's span on it is no longer than this times the host's time to issue it
        self._small_graphs: Dict[tuple, tuple] = {}
        self._small_seen: Dict[tuple, list] = {}
        self._small_pending = None
        self.small_captures = self.small_replays = 0
        # only for models whose mixers are attention over the pages through this package's kernels (they take empty
        # segments and rows that belong to none) and keep no state of their own (a padding segment carries state slot 0)
        self._small_ok = all(isinstance(layer.mixer, AttentionLike) and layer.mixer.state_need() is None
                             for layer in model.layers)
        worst = heads = 0
        for layer in model.layers:
            m = layer.mixer
            if isinstance(m, AttentionLike):
                worst = max(worst, ops.decode_scratch_floats(S, m.n_head, m.head_dim, 32))
                heads = max(heads, m.n_head)
        self._scratch = torch.empty(max(worst, 1), dtype=torch.float32, device=self.device)
        self._counters = torch.zeros(max(S * heads, 1), dtype=torch.int32, device=self.device)
        self.graph_replays = 0

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
            # captured graphs keep the addresses they were recorded with: what is outgrown stays allocated
            self._outgrown = getattr(self, "_outgrown", [])
            if n_floats > self._scratch.numel():
                self._outgrown.append(self._scratch)
                self._scratch = torch.empty(n_floats + n_floats // 2, dtype=torch.float32, device=self.device)
            if n_counters > self._counters.numel():
                self._outgrown.append(self._counters)
                self._counters = torch.zeros(n_counters, dtype=torch.int32, device=self.device)
        return self._scratch, self._counters

    def _pack(self, entries, pad_rows: int, all_logits: bool, reserved_ahead: bool, pad_segments: int = 0):
        """Validates and packs a step (StepEntry objects, or the scheduler's native plan) into the pinned
        buffer and starts its copy to the device; returns the packer's summary."""
        if self._copied is not None:
            self._copied.synchronize()   # the last step's copy must have left the pinned buffer
        try:
            if entries and not isinstance(entries[0], StepEntry):
                info = self._packer.pack_plan(self._host_ptr, entries, pad_rows, all_logits, pad_segments)
            else:
                native = [host().PackEntry(e.slot, e.start, list(e.tokens), list(e.want)) for e in entries]
                info = self._packer.pack(self._host_ptr, native, pad_rows, all_logits, reserved_ahead, pad_segments)
        except ValueError as err:
            raise StepError(str(err)) from None
        self._dev.copy_(self._host, non_blocking=True)
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record(self._current_stream())
        feed = self.feed_tokens   # stays for the whole step: a step that is captured is packed twice
        if feed is not None:      # a step planned ahead: its tokens are the ones the step before sampled, still on the device
            if info.n_decode < feed.shape[0] or info.n_tokens != feed.shape[0]:
                raise StepError("a step fed from the device holds one token for each of the sampled ones")
            self._dev_view("tokens", feed.shape[0]).copy_(feed)
        self.last_info = info
        return info

    def _current_stream(self):
        """torch.cuda.current_stream() costs 5 us of Python layers; the stream object is kept and only looked up
        again when the raw handle of the current stream differs from it."""
        raw = ops.raw_stream_handle()
        if self._stream_obj is None or raw is None or self._stream_obj.cuda_stream != raw:
            self._stream_obj = torch.cuda.current_stream()
        return self._stream_obj

    def validate(self, entries: Sequence[StepEntry], reserved_ahead: bool = False) -> None:
        """Raises StepError if the step does not fit the cache's state or the engine's limits (it is packed
        into the host buffer on the way, which does no harm)."""
        self._pack(entries, 0, False, reserved_ahead)

    def build_context(self, entries, pad_rows: int = 0, all_logits: bool = False,
                      reserved_ahead: bool = False, fixed_shapes: bool = False, ctx_limit: int = 0,
                      pad_segments: int = 0) -> StepContext:
        """Packs the step into the host buffer, copies it over, returns the views.

        ``pad_rows`` > 0 (decode-only steps): the step is laid out for exactly that many rows and
        segments; rows beyond the entries are padding (segment -1: no cache write, zero attention
        output).  ``all_logits``: every row's logits, whatever the entries want.  ``pad_segments`` with ``pad_rows``:
        any step, laid out for exactly that many rows, segments and wanted rows (see the packer)."""
        info = self._pack(entries, pad_rows, all_logits, reserved_ahead, pad_segments)
        pool = self.pool
        T, S, R = info.n_rows, info.n_segments, info.n_logit_rows
        ctx = StepContext()
        ctx.dtype, ctx.pool, ctx.error_flag = self.model.dtype, pool, self.error_flag
        ctx.position_encoding = self.model.position
        ctx.runner, ctx.max_positions, ctx.fixed_shapes = self, self.model.spec.max_positions, bool(pad_rows) or fixed_shapes
        ctx.n_rows, ctx.n_segments, ctx.n_logit_rows, ctx.n_decode = T, S, R, info.n_decode
        ctx.tokens, ctx.positions, ctx.row_seq = (self._dev_view(n, T) for n in ("tokens", "positions", "row_seq"))
        ctx.seg_slot, ctx.seg_start, ctx.seg_ctx = (self._dev_view(n, S) for n in ("seg_slot", "seg_start", "seg_ctx"))
        ctx.cu_rows = self._dev_view("cu_rows", S + 1)
        ctx.logit_rows = self._dev_view("logit_rows", R)
        ctx.host_seg_rows, ctx.host_seg_ctx = list(info.seg_rows), list(info.seg_ctx)
        ctx.max_seg_rows, ctx.max_ctx = (pad_rows if pad_segments else info.max_seg_rows), info.max_ctx
        ctx.ctx_limit = (ctx_limit or ctx.max_positions) if ctx.fixed_shapes else info.max_ctx
        for g in range(self._n_groups):
            mb = pool.max_blocks(g)
            ctx.groups.append(GroupView(self._dev_view(f"block_table{g}", S * mb).view(S, mb),
                                        self._dev_view(f"slot_mapping{g}", T), mb))
        return ctx

    def context_class(self, max_ctx: int) -> int:
        limit = 256
        while limit < max_ctx:
            limit *= 4
        return min(limit, self.model.spec.max_positions)

    def decode_graph_keys(self):
        """Every (rows, class of context lengths) a decode step can be captured for."""
        rows, b = [], 1
        while True:
            rows.append(self._bucket(b))
            if rows[-1] >= self.max_seqs:
                break
            b *= 2
        classes, c = [], 256
        while True:
            classes.append(min(c, self.model.spec.max_positions))
            if c >= self.model.spec.max_positions:
                break
            c *= 4
        return [(r, c) for r in sorted(set(rows)) for c in sorted(set(classes))]

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
        native = bool(entries) and not isinstance(entries[0], StepEntry)
        decode_only = all((e.n_tokens if native else len(e.tokens)) == 1 for e in entries)
        if self.use_graphs and decode_only:
            out = self._decode_step_graph(entries, native)
            return out if borrow else out.clone()
        self._small_pending = None
        if self.use_graphs and self.small_step_graphs and self._small_ok and native and len(entries) <= self.max_seqs:
            rows = sum(e.n_tokens for e in entries)
            if rows <= self.small_step_rows:
                out = self._small_step_graph(entries, rows)
                if out is not None:
                    return out if borrow else out.clone()
        shape = None
        if self.use_graphs and self.shape_graphs and entries:
            shape = self._step_shape(entries, native)
            out = self._shape_step_graph(entries, shape)
            if out is not None:
                return out if borrow else out.clone()
        ctx = self.build_context(entries)
        pending = self._small_pending
        if pending is not None:     # this run is timed on the device too
            pending[2] = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            pending[2][0].record(self._current_stream())
        t0 = time.perf_counter()
        out = self.model.forward(ctx)
        host_s = time.perf_counter() - t0
        if pending is not None:
            pending[2][1].record(self._current_stream())
            pending[1] = host_s
        if shape is not None:      # what issuing this shape's launches costs the host: decides whether a graph pays
            seen = self._shape_seen.get(shape)
            if seen is not None:
                seen[1] = host_s
        return out

    def small_step_bucket(self, rows: int) -> int:
        bucket = 16
        while bucket < rows:
            bucket *= 2
        return min(bucket, self.max_tokens)

    def _small_step_graph(self, entries, rows: int):
        """A small step with prompt portions: replays the graph of its size; or captures it, once steps of that size
        have come often enough and a run timed on both sides has shown the device starved (its span no longer than
        the host took to issue the launches); or returns None: the caller runs it launch by launch.
        ``Engine.warm_up`` decides the same ahead of serving, by measurement (``capture_small_step``)."""
        bucket = self.small_step_bucket(rows)
        seen = self._small_seen.setdefault(bucket, [0, 0.0, None, None])   # times seen, host s, events of the timed run, device ms
        if seen[3] == 0.0:             # measured at warm-up: a graph of this size does not pay
            return None
        seen[0] += 1
        if seen[3] is None:
            if seen[2] is not None and seen[2][1].query():
                seen[3] = max(seen[2][0].elapsed_time(seen[2][1]), 1e-6)
            elif seen[0] >= 2 and seen[2] is None:
                self._small_pending = seen             # the caller times this run
        starved = seen[3] is not None and seen[3] <= self.small_graph_span_factor * seen[1] * 1e3
        have_some = any(k[0] == bucket for k in self._small_graphs)
        if not have_some and (seen[0] < self.small_graph_after or not starved):
            return None
        info = self._pack(entries, bucket, False, False, self.max_seqs)
        limit = self.context_class(info.max_ctx)
        have = self._small_graphs.get((bucket, limit))
        if have is None:
            _, logits = self._capture_small(entries, bucket, limit)      # the step has run, launch by launch
        else:
            graph, logits = have
            graph.replay()
            self.graph_replays += 1
            self.small_replays += 1
        return logits[:self.last_info.n_wanted]

    def _capture_small(self, entries, bucket: int, limit: int):
        ctx = self.build_context(entries, pad_rows=bucket, pad_segments=self.max_seqs, fixed_shapes=True, ctx_limit=limit)
        first = self.model.forward(ctx)                  # runs once, launch by launch; the capture only records
        graph, logits = capture_graph(lambda: self.model.forward(ctx))
        logits.copy_(first)
        self._small_graphs[(bucket, limit)] = (graph, logits)
        self.small_captures += 1
        return graph, logits

    @torch.no_grad()
    def capture_small_step(self, entries, limit: int) -> bool:
        """Warm-up: runs ``entries`` (a step with a prompt portion; every entry wants at most one row) launch by
        launch, captures the graph of its size for the context class ``limit`` and times a replay against the
        launch-by-launch run; keeps the graph if it is at least ``small_graph_host_factor`` times faster, else
        marks the size as not worth a graph.  The step's rows are run more than once: the same keys and values are
        written each time."""
        rows = sum(len(e.tokens) for e in entries)
        bucket = self.small_step_bucket(rows)
        if not (self.use_graphs and self.small_step_graphs and self._small_ok) or rows > self.small_step_rows:
            return False
        seen = self._small_seen.setdefault(bucket, [0, 0.0, None, None])
        if seen[3] == 0.0:
            return False
        for _ in range(2):                  # the second run is the one that counts: the first pays for what is set up once
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            self.model.forward(self.build_context(entries))
            torch.cuda.synchronize()
            eager_s = time.perf_counter() - t0
        graph, logits = self._capture_small(entries, bucket, limit)
        for _ in range(2):
            self._pack(entries, bucket, False, False, self.max_seqs)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            graph.replay()
            torch.cuda.synchronize()
            replay_s = time.perf_counter() - t0
        if eager_s < self.small_graph_host_factor * replay_s:
            for key in [k for k in self._small_graphs if k[0] == bucket]:      # the size is served launch by launch
                del self._small_graphs[key]
            seen[3] = 0.0
            return False
        seen[0], seen[1], seen[3] = max(seen[0], self.small_graph_after), eager_s, 1e-6
        return True

    @staticmethod
    def _step_shape(entries, native: bool) -> tuple:
        if native:
            return tuple((e.n_tokens, 1 if e.sample else 0) for e in entries)
        return tuple((len(e.tokens), len(e.want)) for e in entries)

    def _shape_step_graph(self, entries, shape: tuple):
        """Replays the graph of this step's shape, captures it if the shape has come often enough and issuing its
        launches one by one costs the host a millisecond or more (a capture stalls the engine for tens of
        milliseconds: for a small model that is a hundred steps, and its steps cost the host little anyway), or
        returns None (the caller then runs the step launch by launch)."""
        have = self._shape_graphs.get(shape)
        if have is not None:
            self._shape_graphs.move_to_end(shape)
            self._pack(entries, 0, False, False)
            graph, logits = have
            graph.replay()
            self.graph_replays += 1
            self.shape_replays += 1
            return logits
        if len(self._shape_seen) > 4096:
            self._shape_seen.clear()
        seen = self._shape_seen.setdefault(shape, [0, 0.0])      # [times seen, host seconds of the last launch-by-launch run]
        seen[0] += 1
        if seen[0] < self.shape_graph_after or seen[1] < self.shape_graph_min_host_s:
            return None
        ctx = self.build_context(entries, fixed_shapes=True)
        # The step itself runs ONCE, launch by launch, with the launches the graph will hold; the capture that
        # follows records them without running them, and the recorded step's output buffer takes this run's
        # logits.  (Running it a second time through the fresh graph would be harmless for keys and values,
        # which are written alike both times, but would move a mixer's own per-request state on twice.)
        first = self.model.forward(ctx)
        graph, logits = capture_graph(lambda: self.model.forward(ctx))
        logits.copy_(first)
        while len(self._shape_graphs) >= self.max_shape_graphs:
            self._shape_graphs.popitem(last=False)        # the shape not used for the longest time makes room
        self._shape_graphs[shape] = (graph, logits)
        self.shape_captures += 1
        return logits

    def _decode_step_graph(self, entries, native: bool) -> torch.Tensor:
        rows = self._bucket(len(entries))
        info = self._pack(entries, rows, True, False)     # the captured kernels read the same buffer: no views needed
        # a graph holds for a number of rows and a class of context lengths (256, 1024, 4096, ... up to the model's
        # positions): kernels that split a request's keys over blocks size the split for the class's bound, so short
        # requests of a model with many positions are not cut into pieces that are mostly empty
        limit = self.context_class(info.max_ctx)
        forced = getattr(self, "force_context_class", None)     # warm-up: the class is named, the requests are short
        if forced is not None and forced >= limit:
            limit = forced
        have = self._graphs.get((rows, limit))
        if have is None:
            ctx = self.build_context(entries, pad_rows=rows, all_logits=True, ctx_limit=limit)
            first = self.model.forward(ctx)               # this step runs once, launch by launch; the capture only records
            have = self._graphs[(rows, limit)] = capture_graph(lambda: self.model.forward(ctx))
            graph, logits = have
            logits.copy_(first)
        else:
            graph, logits = have
            graph.replay()
            self.graph_replays += 1
        if info.n_wanting == rows:
            return logits
        if info.n_wanting == len(entries):
            return logits[:len(entries)]      # the entries' rows come first, in their order; the rest is padding
        want = [i for i, e in enumerate(entries) if (e.sample if native else len(e.want))]
        return logits[torch.tensor(want, dtype=torch.long, device=logits.device)] if want else logits[:0]

    @torch.no_grad()
    def decode_loop(self, entries: Sequence[StepEntry]) -> "DecodeLoop":
        """A run of greedy decode steps that never leaves the device: see ``DecodeLoop``."""
        return DecodeLoop(self, entries)


def capture_graph(fn):
    """Captures the launches of ``fn()`` into a CUDA graph on a side stream; returns (graph, what fn returned).
    ``torch.cuda.graph`` does the same but first collects garbage and empties the allocator's cache, which costs
    up to seconds when much memory is cached: too much for a capture in the middle of serving.  What its
    collection is for is done here by switching the cyclic garbage collector off while the capture runs: if it
    came by in the middle and freed another engine's graphs or buffers, the memory calls that this causes would
    end the capture with an error.  Calls of other threads do not touch the capture (thread-local mode)."""
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    gc_was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.stream(side):
            graph.capture_begin(capture_error_mode="thread_local")
            try:
                out = fn()
            finally:
                graph.capture_end()
    finally:
        if gc_was_on:
            gc.enable()
    torch.cuda.current_stream().wait_stream(side)
    return graph, out


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
        self.graph, _ = capture_graph(self._one_step)
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
