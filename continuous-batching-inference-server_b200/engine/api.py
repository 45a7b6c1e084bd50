"""Python entry point: an engine over a model folder or over seeded random weights.

The reference's Python side is its oracle, ``build_model(seed)`` and ``TinyGPT()(idx)``
(python/model.py:63-77); its serving loop lives in C++ ``main`` functions
(src/server_demo.cpp:101-213).  Here ``build_model(config, seed)`` gives an ``Engine`` with
random weights of that configuration, ``Engine(folder)`` loads a model folder, and
``generate`` runs the continuous-batching loop: schedule, one step, sample, update.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..cache import CachePool
from ..config import config_from_dict, load_config
from ..kernels import ops
from ..kernels.library import host
from ..models import Model, load_model, resolve_dtype
from ..sampling import SamplingParams, request_key
from ..weights import InitScheme, random_tensors
from .runner import ModelRunner, StepEntry


@dataclass
class RequestOutput:
    request_id: int
    tokens: List[int]
    finish_reason: str


class Engine:
    def __init__(self, model: Union[str, Model], *, dtype="bfloat16", page_size: int = 16,
                 num_pages: Optional[int] = None, max_tokens: Optional[int] = None, max_num_seqs: int = 16,
                 max_batched_tokens: int = 512, prefill_chunk: Optional[int] = None,
                 memory_fraction: float = 0.85, device: str = "cuda", poison_freed_pages: Optional[bool] = None):
        """``model``: a folder with config.json and model.safetensors, or a loaded ``Model``.
        Engine options in the reference's terms: ``page_size`` = kPageSize (include/config.hpp:20),
        ``num_pages`` = kMaxPages, ``max_num_seqs`` = kMaxSlots, ``max_batched_tokens`` =
        kMaxTotalRows (src/server_demo.cpp:27-29).  ``prefill_chunk`` cuts prompts into portions
        (src/bench_tiering.cpp:78 uses 512); default: the token budget.  ``poison_freed_pages`` (default:
        the environment's CBIS_POISON_FREED_PAGES=1) is a debugging mode: every page that a request gives back
        is filled with NaN before the next step runs, so a read of a page that is no longer held, or of a
        token slot beyond a request's length in a page that was used before, shows as NaN logits."""
        if not torch.cuda.is_available():
            raise RuntimeError("the engine needs a CUDA device (sm_100a); there is no CPU path")
        self.model = load_model(model, dtype, device) if isinstance(model, str) else model
        self.pool = CachePool(self.model, page_size=page_size, num_pages=num_pages, max_tokens=max_tokens,
                              max_requests=max_num_seqs, memory_fraction=memory_fraction, device=device)
        self.runner = ModelRunner(self.model, self.pool, max_batched_tokens=max_batched_tokens,
                                  max_num_seqs=max_num_seqs)
        self.limits = dict(max_num_seqs=max_num_seqs, max_batched_tokens=max_batched_tokens,
                           prefill_chunk=prefill_chunk or max_batched_tokens,
                           max_positions=self.model.spec.max_positions)
        self.scheduler = host().Scheduler(self.pool.manager, host().SchedulerLimits(**self.limits))
        if poison_freed_pages is None:
            poison_freed_pages = os.environ.get("CBIS_POISON_FREED_PAGES", "0") == "1"
        self.poison_freed_pages = bool(poison_freed_pages)
        self.pages_poisoned = 0
        if self.poison_freed_pages:
            self.pool.manager.record_freed(True)
        self._params: Dict[int, SamplingParams] = {}
        self._not_greedy = 0          # live requests that sample with a temperature
        self._sampled = self._sampled_host = self._sampled_event = None
        self._sampled_turn = 0
        self._in_flight = None        # a step launched ahead: (plan, rows, host buffer, had prompt portions)
        self.step_ahead = os.environ.get("CBIS_STEP_AHEAD", "1") != "0"
        self.steps_ahead = 0          # steps launched before the tokens of the step before were read
        self._next_id = 0
        self.steps = 0
        self.tokens_run = 0
        self.last_step_tokens = 0

    # ---- construction from random weights --------------------------------------
    @classmethod
    def from_random(cls, config, seed: int = 1234, *, init: InitScheme = InitScheme(), dtype="bfloat16",
                    weight_dtype: Optional[torch.dtype] = None, device: str = "cuda", draw_on: Optional[str] = None,
                    **options) -> "Engine":
        """Random weights of ``config`` (a typed configuration, a dict of config.json keys, or a path
        to a config.json), drawn on the device; nothing is written to disk.  ``draw_on="cpu"`` draws them
        with the CPU's generator instead (slower): ``weights.random_tensors`` with the same declarations,
        seed and scheme then gives another program the same values."""
        if isinstance(config, str):
            with open(config if config.endswith(".json") else os.path.join(config, "config.json")) as f:
                config = json.load(f)
        if isinstance(config, dict):
            config = config_from_dict(config)
        model = Model(config.model_spec())
        model.config = config
        wd = weight_dtype or (torch.bfloat16 if resolve_dtype(dtype) == torch.bfloat16 else torch.float32)
        tensors = random_tensors(model.declared(), seed, init, wd, device=device, draw_on=draw_on)
        model.load(tensors, dtype, device, where="random weights")
        del tensors
        return cls(model, dtype=dtype, device=device, **options)

    def _poison_freed(self) -> None:
        """Debugging mode: overwrites the pages given back since the last step (queued before the next one)."""
        if not self.poison_freed_pages:
            return
        mgr = self.pool.manager
        for g in range(mgr.num_groups()):
            pages = mgr.take_freed(g)
            self.pages_poisoned += len(pages)
            self.pool.poison_pages(g, pages)

    # ---- requests ---------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        params = params or SamplingParams()
        rid = self._next_id if request_id is None else int(request_id)
        self._next_id = max(self._next_id, rid + 1)
        prompt = [int(t) for t in prompt]
        V = self.model.spec.vocab_size
        bad = [t for t in prompt if not 0 <= t < V]
        if bad:
            raise ValueError(f"request {rid}: token id {bad[0]} outside the vocabulary of {V}")
        eos = -1 if params.eos_token_id is None else int(params.eos_token_id)
        self.scheduler.add(rid, prompt, int(params.max_new_tokens), eos, bool(params.ignore_eos))
        self._params[rid] = params
        self._not_greedy += params.temperature > 0
        return rid

    def has_unfinished(self) -> bool:
        return not self.scheduler.idle()

    def abort(self, request_id: int) -> bool:
        """Drops a request wherever it is (waiting or running); its pages go back at once.  If a step launched ahead
        holds a row of it, that row is computed for nothing and passed over.  False if there is no such request."""
        self._forget(request_id)
        return bool(self.scheduler.abort(int(request_id)))

    @torch.no_grad()
    def step(self) -> List[RequestOutput]:
        """One engine step: plan, run, sample, update.  Returns the requests that finished.

        While the device runs a step, the next one is planned, packed and launched if it is certain but for its tokens
        (``Scheduler.schedule_ahead``: everyone goes on decoding; the sampled tokens stay on the device and feed it),
        and only then are this step's tokens read back: the host's work per step hides behind the device's.  A call
        then returns the results of the step launched by the call before."""
        cur = self._in_flight
        self._in_flight = None
        if cur is None:
            plan = self.scheduler.schedule()
            if not plan:
                return []
            for slot in self.scheduler.take_new_slots():
                self.pool.clear_state(slot)
            cur = self._launch(plan, None)
            if cur is None:
                return []
        if self.step_ahead:
            ahead = self.scheduler.schedule_ahead()
            if ahead:
                feed = self._sampled[:len(ahead)]
                source = self.scheduler.ahead_sources()      # empty: entry i takes the i-th sampled token
                if source:      # a request of the running step has ended meanwhile: the rows no longer line up
                    feed = self._sampled[torch.tensor(source, dtype=torch.long).to(self._sampled.device)]
                self._in_flight = self._launch(ahead, feed)
                self.steps_ahead += 1
        plan, tokens = cur[0], self._read_tokens(cur)
        out = []
        for f in self.scheduler.update_plan(plan, tokens):      # the plan's sampling entries and the tokens, in order
            self._forget(f.request_id)
            out.append(RequestOutput(f.request_id, list(f.output), f.reason))
        if self._in_flight is not None and self.scheduler.idle():
            # every request of the step launched ahead has ended (an end-of-sequence token): it was for nothing,
            # and its tokens go back to the scheduler now, which passes over them, so that nothing is left open
            stale, self._in_flight = self._in_flight, None
            self.scheduler.update_plan(stale[0], self._read_tokens(stale))
        return out

    def _launch(self, plan, feed):
        """Runs the plan's step and its sampling on the device; returns what ``_read_tokens`` needs, None if the
        step samples nothing.  ``feed``: tokens on the device for a step planned ahead."""
        self._poison_freed()
        self.runner.feed_tokens = feed
        try:
            logits = self.runner.step(plan, borrow=True)     # the native plan goes to the native packer as it is
        finally:
            self.runner.feed_tokens = None
        info = self.runner.last_info
        self.steps += 1
        self.last_step_tokens = info.n_tokens
        self.tokens_run += info.n_tokens
        if info.n_wanting == 0:
            return None
        return (plan,) + self._sample(logits, plan)

    def _forget(self, request_id: int) -> None:
        params = self._params.pop(request_id, None)
        if params is not None:
            self._not_greedy -= params.temperature > 0

    @torch.no_grad()
    def warm_up(self, small_steps: bool = True) -> int:
        """Captures ahead of serving, with short requests of its own, the graph of a decode step for every batch-size
        bucket and class of context lengths, so that none is captured in the middle of serving (a capture stalls the
        engine for tens of milliseconds at 48 layers); and, with ``small_steps``, the graphs of small steps with
        prompt portions, each kept only if a replay measured now is faster than the same step launch by launch.
        The engine must be idle.  Returns the number of graphs captured and kept."""
        runner, mgr = self.runner, self.pool.manager
        if not runner.use_graphs:
            return 0
        if not self.scheduler.idle() or self._in_flight is not None:
            raise RuntimeError("warm_up: the engine has requests")
        kept = 0
        keys = [k for k in runner.decode_graph_keys() if k not in runner._graphs]
        classes = sorted({limit for _, limit in runner.decode_graph_keys()})
        slots = []
        try:
            if keys:
                for _ in range(max(rows for rows, _ in keys)):
                    slots.append(self.open_request(-1 - len(slots)))
                per = max(1, runner.max_tokens // 2)
                for i in range(0, len(slots), per):           # a prompt of two tokens each: decode steps follow it
                    self.forward_step([StepEntry(s, 0, [0, 0], []) for s in slots[i:i + per]])
                for rows, limit in keys:
                    runner.force_context_class = limit
                    try:
                        self.forward_step([StepEntry(s, mgr.length(s), [0], [0]) for s in slots[:rows]])
                    finally:
                        runner.force_context_class = None
                kept += len(keys)
            for s in slots:
                self.close_request(s)
            slots = []
            if small_steps and runner.small_step_graphs:
                # one request of its own per size: a prompt portion of that many rows (as many as the positions and the
                # pages allow), whose step is captured for every context class
                bucket = 16
                while bucket <= runner.small_step_rows:
                    n = min(bucket, self.model.spec.max_positions)
                    slot = self.open_request(-1)
                    slots.append(slot)
                    if n > bucket // 2 and mgr.append(slot, n):
                        entries = [StepEntry(slot, 0, [0] * n, [n - 1])]
                        for limit in classes:
                            if (runner.small_step_bucket(n), limit) not in runner._small_graphs:
                                kept += bool(runner.capture_small_step(entries, limit))
                    self.close_request(slot)
                    slots.pop()
                    bucket *= 2
        finally:
            for s in slots:
                self.close_request(s)
        return kept

    def _sample(self, logits: torch.Tensor, plan):
        """One token for every row of ``logits`` (the plan's sampling entries, in order) into ``self._sampled`` on the
        device, and their copy to pinned host memory queued; returns (rows, host buffer, event of the copy, whether
        the step held prompt portions)."""
        R = logits.shape[0]
        if self._sampled is None or self._sampled.shape[0] < R:
            n = max(R, self.pool.max_requests)
            self._sampled = torch.empty(n, dtype=torch.int32, device=logits.device)
            self._sampled_host = [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)]
            self._sampled_event = [torch.cuda.Event() for _ in range(2)]
        out = self._sampled[:R]
        if self._not_greedy == 0:
            ops.sample(logits, None, None, out)
        else:
            sampling = [p for p in plan if p.sample]
            params = [self._params[p.request_id] for p in sampling]
            temps = torch.tensor([float(q.temperature) for q in params], dtype=torch.float32).to(logits.device)
            keys = torch.tensor([request_key(q.seed, p.request_id, p.output_index) for p, q in zip(sampling, params)],
                                dtype=torch.int64).to(logits.device)
            ops.sample(logits, temps, keys, out)
        # two host buffers in turn: the one of the step before may still be unread when this step is launched ahead
        k = self._sampled_turn = 1 - self._sampled_turn
        self._sampled_host[k][:R].copy_(out, non_blocking=True)     # pinned memory: the copy is queued, the event says when it is there
        self._sampled_event[k].record(self.runner._current_stream())
        return R, k, self.last_step_tokens > R

    def _read_tokens(self, launched) -> List[int]:
        _, R, k, had_portions = launched
        self._sampled_event[k].synchronize()
        tokens = self._sampled_host[k][:R].tolist()
        # kernels with bounded waits report through one flag on the device: read after every step with prompt
        # portions (several such kernels) and every 64th decode step (the few-rows tcgen05 product); the host has
        # just waited for the step anyway
        self._unchecked = getattr(self, "_unchecked", 0) + 1
        if had_portions or self._unchecked >= 64:
            self._unchecked = 0
            ops.raise_if_kernel_errors(self.runner.device)
        return tokens

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Runs all prompts to their end under continuous batching; returns each one's new tokens.
        Request i of the call has id ``first_id + i``, the key of its sampling stream."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        try:
            for p, q in zip(prompts, params):
                ids.append(self.add_request(p, q))
        except Exception:
            for rid in ids:                       # a refused prompt leaves nothing of this call behind
                self.scheduler.abort(rid)
                self._forget(rid)
            raise
        results: Dict[int, List[int]] = {}
        while self.has_unfinished():
            for o in self.step():
                results[o.request_id] = o.tokens
        return [results[i] for i in ids]

    # ---- the bare step, for replay and checks -----------------------------------
    def open_request(self, request_id: int = 0) -> int:
        """Takes a request slot outside the scheduler (replay); returns the slot."""
        slot = self.pool.manager.admit(int(request_id))
        if slot < 0:
            raise RuntimeError(f"all {self.pool.max_requests} request slots are taken")
        self.pool.clear_state(slot)
        return slot

    def close_request(self, slot: int) -> None:
        self.pool.manager.release(slot)
        ops.raise_if_kernel_errors(self.runner.device)    # waits for the queued steps: nothing bad goes unreported

    @torch.no_grad()
    def forward_step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Takes pages for the entries' tokens, runs them as ONE step, returns float32 logits
        ``[wanted, vocab]``.  Pages behind a window are given back before the next step."""
        mgr = self.pool.manager
        for e in entries:
            mgr.release_out_of_window(e.slot)
        for e in entries:
            if mgr.length(e.slot) != e.start:
                raise ValueError(f"slot {e.slot}: holds {mgr.length(e.slot)} tokens, the entry starts at {e.start}")
            if not mgr.append(e.slot, len(e.tokens)):
                raise RuntimeError(f"slot {e.slot}: no pages left for {len(e.tokens)} more tokens "
                                   f"(free pages per group: {[mgr.free_pages(g) for g in range(mgr.num_groups())]})")
        self._poison_freed()
        out = self.runner.step(entries)
        if any(len(e.tokens) > 1 for e in entries):
            # a step with prompt portions may have run kernels whose waits are bounded (TMA + tcgen05): a wait that
            # ran out left wrong logits, and says so through a flag on the device (read without stalling the host:
            # a bad step is reported at one of the next calls, or when the request is closed)
            ops.poll_kernel_errors(out.device)
        return out

    @torch.no_grad()
    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """Logits ``[T, vocab]`` of one whole sequence, as the reference's ``model(idx)``
        (python/model.py:63-70), through the step function in portions of the token budget."""
        slot = self.open_request(-1)
        try:
            outs, pos = [], 0
            while pos < len(tokens):
                n = min(self.runner.max_tokens, len(tokens) - pos)
                outs.append(self.forward_step([StepEntry(slot, pos, list(tokens[pos:pos + n]), list(range(n)))]))
                pos += n
            return torch.cat(outs)
        finally:
            self.close_request(slot)


def build_model(config, seed: int = 1234, **options) -> Engine:
    """Engine with seeded random weights of ``config`` (the reference's ``build_model(seed)``,
    python/model.py:73-77, builds its one fixed-size model the same way)."""
    return Engine.from_random(config, seed, **options)
