"""Interfaces of the parts a layer is put together from, and their registries.

A part gets its sizes and constants as constructor parameters (from a ``PartSpec``),
declares the tensors it needs under a name prefix, takes them at load time, and is
run by a block with a ``StepContext``.  No part knows which model or which layer it
is in.  New kinds are added with ``register_mixer`` / ``register_feed_forward`` /
``register_norm`` / ``register_position`` / ``register_block`` / ``register_embedding`` /
``register_head``; a configuration then names them in its ``ModelSpec``.  A part refuses sizes
that no kernel takes in its constructor, so a model that cannot run fails when it is built.

Values that flow between parts:

* the residual stream ``x``: float32 ``[T, width]`` in both precisions;
* a part's input ``h`` (a norm's output): ``[T, width]`` in the compute dtype;
* a part's output: a ``Delta``, the tensor to be added to the residual stream, plus
  an optional bias row that the next norm adds in the same pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Protocol, Tuple, runtime_checkable

import torch

from ..weights.loader import TensorDecl


@dataclass
class Delta:
    """What a mixer or feed-forward adds to the residual stream: value (+ bias per column)."""
    value: torch.Tensor
    bias: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class CacheArray:
    """One array a mixer keeps per token: ``heads`` x ``width`` elements of the compute dtype.  The pool
    stores it in pages ``[num_pages, heads, page_size, width]``, so a (page, head) tile is one run."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token, as a list of named arrays (attention: "k" and "v" of
    ``[n_kv_head, head_dim]``; a mixer with one compressed vector per token: one array of one head).
    ``window`` 0 keeps every token; w > 0 keeps only what queries at later positions can reach.
    Layers whose needs are equal share a group: one pool of pages, one block table per request."""
    arrays: Tuple[CacheArray, ...]
    window: int = 0

    @staticmethod
    def keys_values(n_kv_head: int, head_dim: int, window: int = 0) -> "CacheNeed":
        return CacheNeed((CacheArray("k", n_kv_head, head_dim), CacheArray("v", n_kv_head, head_dim)), window)

    def elements_per_token(self) -> int:
        return sum(a.heads * a.width for a in self.arrays)


@runtime_checkable
class AttentionLike(Protocol):
    """What ``StepContext.attention`` reads off a mixer to choose and run an attention kernel over the
    mixer's "k" and "v" pages.  ``qkv`` handed to it has the columns q (``d_q``), then k and v
    (``d_kv`` each) if ``own_kv``; with ``own_kv`` False only q, and the pages of another layer are read."""
    n_head: int
    n_kv_head: int
    head_dim: int
    d_q: int
    d_kv: int
    own_kv: bool
    window: int
    scale: float


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of a mixer: one tensor of ``shape`` per request slot,
    zeroed when a request is admitted."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Common behaviour: tensor declaration and loading."""

    # False for a part whose forward() reads device values on the host (``.tolist()``, ``.item()``):
    # such a step cannot be captured as a CUDA graph and runs launch by launch.
    capturable = True

    def tensors(self, prefix: str) -> List[TensorDecl]:
        return []

    def load(self, prefix: str, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Takes its tensors (stored dtype, CPU or device) and keeps them on ``device``:
        matrices and tables in ``dtype``, vectors in float32."""

    def streamed_weights(self) -> List[torch.Tensor]:
        """The matrices a decode step reads through this part, in the order it uses them (so that the
        product before can prefetch them)."""
        return []

    @staticmethod
    def _matrix(t: torch.Tensor, dtype, device) -> torch.Tensor:
        return t.to(device=device, dtype=dtype).contiguous()

    @staticmethod
    def _matrix_nk(t: torch.Tensor, dtype, device) -> torch.Tensor:
        """A Conv1D weight [in, out] as the kernels want it: [out, in], the contraction dim contiguous."""
        return t.to(device=device, dtype=dtype).t().contiguous()

    @staticmethod
    def _vector(t: torch.Tensor, device) -> torch.Tensor:
        return t.to(device=device, dtype=torch.float32).contiguous()


class Mixer(Part):
    """Mixes information between the tokens of a request (attention, or anything with a cache or a state)."""

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, ctx, h: torch.Tensor, cache, state: Optional[torch.Tensor]) -> Delta:
        """``cache``: the ``LayerCache`` of this layer (or of the layer it reads), None if it keeps none;
        ``cache.arrays[name]`` are its pages ``[num_pages, heads, page_size, width]``, addressed through
        ``ctx.groups[cache.group]`` (block table per segment, token slot per row).
        ``state``: ``[max_requests, *shape]`` if it declared a state; row ``ctx.seg_slot[s]`` belongs to segment s.
        Returns what is to be added to the residual stream; or None after adding it itself into ``ctx.residual``
        (the 32-bit rows, set while a block runs its parts), which a part is free to ignore."""
        raise NotImplementedError

    # Optional: a mixer may take the residual stream itself, normalise it inside its first kernel and add its result
    # into it.  A block asks ``fuses_norm`` every step and calls ``forward_residual`` only after a yes.
    def fuses_norm(self, ctx, norm: "Norm") -> bool:
        return False

    def forward_residual(self, ctx, x: torch.Tensor, norm: "Norm", cache, state: Optional[torch.Tensor]) -> None:
        """x += mixer(norm(x)), x the 32-bit residual stream, up to date (nothing pending)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor) -> Delta:
        raise NotImplementedError

    def fuses_norm(self, ctx, norm: "Norm") -> bool:      # as Mixer.fuses_norm
        return False

    def forward_residual(self, ctx, x: torch.Tensor, norm: "Norm") -> None:
        """x += feed_forward(norm(x)), x the 32-bit residual stream, up to date."""
        raise NotImplementedError


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, delta: Optional[Delta], rows: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Adds ``delta`` to the residual stream ``x`` in place (32-bit), returns norm(x) in the
        compute dtype.  With ``rows`` (int32 indices) only those rows are produced and x is not changed."""
        raise NotImplementedError

    def as_layernorm(self):
        """(weight, bias, eps) if this norm is exactly a LayerNorm with those (a part that normalises inside its
        own kernel asks for them), else None."""
        return None


class PositionEncoding(Part):
    """Position information.  ``embed`` makes the residual stream of a step from its tokens
    (a lookup in the token table, times ``multiplier`` if the embedding has one, plus whatever the
    encoding adds at the input).  An encoding that acts inside the mixers instead (a rotation of
    queries and keys) sets ``acts_in_mixer`` and defines ``apply_in_mixer``; a mixer finds the
    model's encoding as ``ctx.position_encoding`` and calls it on its queries and keys BEFORE the
    keys go into the cache, so a cached page holds keys as the scores need them."""

    acts_in_mixer = False

    def embed(self, ctx, token_table: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def apply_in_mixer(self, ctx, q: torch.Tensor, k: Optional[torch.Tensor], head_dim: int) -> None:
        """Changes ``q`` ``[T, n_head * head_dim]`` and ``k`` ``[T, n_kv_head * head_dim]`` (views, maybe
        strided; k None for a mixer without keys of its own) in place by ``ctx.positions``."""


class Embedding(Part):
    """The model's input: the residual stream (float32 ``[T, width]``) of a step's tokens.  ``table`` is
    the token table, which a head may share."""

    table: Optional[torch.Tensor] = None

    def forward(self, ctx, position: PositionEncoding) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """The model's output: float32 logits ``[R, vocab]`` at the rows ``ctx.logit_rows``."""

    def tie(self, embedding: Embedding) -> None:
        """Called after the embedding is loaded and before ``load``: a tied head takes the table here."""

    def forward(self, ctx, x: torch.Tensor, pending: Optional[Delta], final_norm: Norm) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of norms, mixer and feed-forward around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norm_mixer: Norm, norm_feed_forward: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norm_mixer, self.norm_feed_forward = norm_mixer, norm_feed_forward

    def forward(self, ctx, x: torch.Tensor, pending: Optional[Delta], cache, state) -> Optional[Delta]:
        """Runs the layer; ``pending`` is the previous layer's output not yet added to x.
        Returns this layer's own pending output (or None if x is up to date)."""
        raise NotImplementedError

    def run_key(self, ctx, cache, state):
        """A block that can run TOGETHER with the blocks after it in one go (one kernel for a run of layers) returns
        a hashable key for this step, else None.  The model hands every maximal run of consecutive layers with equal
        keys to ``forward_run`` of their class; a run of one is allowed."""
        return None

    @classmethod
    def forward_run(cls, ctx, blocks, x: torch.Tensor, pending: Optional[Delta], caches, states) -> Optional[Delta]:
        """Runs ``blocks`` (equal ``run_key``) one after the other; the contract of ``forward`` for the whole run."""
        for block, cache, state in zip(blocks, caches, states):
            pending = block.forward(ctx, x, pending, cache, state)
        return pending


_MIXERS: Dict[str, Callable[..., Mixer]] = {}
_FEED_FORWARDS: Dict[str, Callable[..., FeedForward]] = {}
_NORMS: Dict[str, Callable[..., Norm]] = {}
_POSITIONS: Dict[str, Callable[..., PositionEncoding]] = {}
_BLOCKS: Dict[str, Callable[..., Block]] = {}
_EMBEDDINGS: Dict[str, Callable[..., Embedding]] = {}
_HEADS: Dict[str, Callable[..., Head]] = {}


def register_mixer(kind: str, factory) -> None:
    _MIXERS[kind] = factory


def register_feed_forward(kind: str, factory) -> None:
    _FEED_FORWARDS[kind] = factory


def register_norm(kind: str, factory) -> None:
    _NORMS[kind] = factory


def register_position(kind: str, factory) -> None:
    _POSITIONS[kind] = factory


def register_block(kind: str, factory) -> None:
    _BLOCKS[kind] = factory


def register_embedding(kind: str, factory) -> None:
    _EMBEDDINGS[kind] = factory


def register_head(kind: str, factory) -> None:
    _HEADS[kind] = factory


def _make(table, what, spec, **extra):
    if spec.kind not in table:
        raise KeyError(f"unknown {what} kind {spec.kind!r}; known: {sorted(table)}")
    return table[spec.kind](**spec.params, **extra)


def make_mixer(spec, **extra) -> Mixer:
    return _make(_MIXERS, "mixer", spec, **extra)


def make_feed_forward(spec) -> FeedForward:
    return _make(_FEED_FORWARDS, "feed-forward", spec)


def make_norm(spec) -> Norm:
    return _make(_NORMS, "norm", spec)


def make_position(spec) -> PositionEncoding:
    return _make(_POSITIONS, "position encoding", spec)


def make_embedding(spec) -> Embedding:
    return _make(_EMBEDDINGS, "embedding", spec)


def make_head(spec) -> Head:
    return _make(_HEADS, "head", spec)


def make_block(kind: str, mixer, feed_forward, norm_mixer, norm_feed_forward) -> Block:
    if kind not in _BLOCKS:
        raise KeyError(f"unknown block arrangement {kind!r}; known: {sorted(_BLOCKS)}")
    return _BLOCKS[kind](mixer, feed_forward, norm_mixer, norm_feed_forward)
