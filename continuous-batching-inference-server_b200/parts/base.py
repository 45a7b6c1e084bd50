"""Interfaces of the parts a layer is put together from, and their registries.

A part gets its sizes and constants as constructor parameters (from a ``PartSpec``),
declares the tensors it needs under a name prefix, takes them at load time, and is
run by a block with a ``StepContext``.  No part knows which model or which layer it
is in.  New kinds are added with ``register_mixer`` / ``register_feed_forward`` /
``register_norm`` / ``register_position`` / ``register_block``; a configuration then
names them in its ``ModelSpec``.

Values that flow between parts:

* the residual stream ``x``: float32 ``[T, width]`` in both precisions;
* a part's input ``h`` (a norm's output): ``[T, width]`` in the compute dtype;
* a part's output: a ``Delta``, the tensor to be added to the residual stream, plus
  an optional bias row that the next norm adds in the same pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..weights.loader import TensorDecl


@dataclass
class Delta:
    """What a mixer or feed-forward adds to the residual stream: value (+ bias per column)."""
    value: torch.Tensor
    bias: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per token: pages of ``[n_kv_head, page_size, head_dim]``.
    ``window`` 0 keeps every token; w > 0 keeps only what queries at later positions can reach."""
    n_kv_head: int
    head_dim: int
    window: int = 0


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
        """``cache``: the ``LayerCache`` of this layer (or of the layer it reads), None if it keeps none.
        ``state``: ``[max_requests, *shape]`` if it declared a state; row ``ctx.seg_slot[s]`` belongs to segment s."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor) -> Delta:
        raise NotImplementedError


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, delta: Optional[Delta], rows: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Adds ``delta`` to the residual stream ``x`` in place (32-bit), returns norm(x) in the
        compute dtype.  With ``rows`` (int32 indices) only those rows are produced and x is not changed."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information.  ``embed`` makes the residual stream of a step from its tokens
    (a lookup in the token table plus whatever the encoding adds at the input); encodings that
    act inside a mixer are handed to mixers through ``StepContext.position``."""

    def embed(self, ctx, token_table: torch.Tensor) -> torch.Tensor:
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


_MIXERS: Dict[str, Callable[..., Mixer]] = {}
_FEED_FORWARDS: Dict[str, Callable[..., FeedForward]] = {}
_NORMS: Dict[str, Callable[..., Norm]] = {}
_POSITIONS: Dict[str, Callable[..., PositionEncoding]] = {}
_BLOCKS: Dict[str, Callable[..., Block]] = {}


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


def make_block(kind: str, mixer, feed_forward, norm_mixer, norm_feed_forward) -> Block:
    if kind not in _BLOCKS:
        raise KeyError(f"unknown block arrangement {kind!r}; known: {sorted(_BLOCKS)}")
    return _BLOCKS[kind](mixer, feed_forward, norm_mixer, norm_feed_forward)
