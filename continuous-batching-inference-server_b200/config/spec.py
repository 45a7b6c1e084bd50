"""Architecture-neutral description of a model: which parts stand in which layer.

A typed configuration (one class per architecture, e.g. ``GPT2Config``) turns its
``config.json`` keys into a ``ModelSpec``.  The model builder knows only the spec:
for every layer it looks the named mixer, feed-forward and norm up in the part
registries and hands them their sizes and constants.  Layers need not be alike,
and the order in which layers run (``schedule``) is data: a layer may be named
twice, and a layer may read another layer's cache (``cache_source``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Kind of a part (its registry key) and the parameters its constructor gets."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, tuple(sorted((k, str(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward.

    ``prefix`` is the tensor-name prefix of the layer's weights (``"h.3."``).
    ``cache_source`` names the layer (index into ``ModelSpec.layers``) whose cache
    this layer's mixer reads instead of keeping one; ``None`` means its own.
    """
    prefix: str
    arrangement: str            # key into the block registry, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    norm_mixer: PartSpec
    norm_feed_forward: PartSpec
    cache_source: Optional[int] = None
    norm_prefixes: Tuple[str, str] = ("ln_1.", "ln_2.")   # tensor-name prefixes of the two norms, after `prefix`


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab_size: int
    max_positions: int
    token_embedding: str                    # tensor name of the token table
    position: PartSpec                      # position encoding at the input (or "none")
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]               # layer indices in running order
    final_norm: PartSpec
    final_norm_prefix: str
    head: Optional[str]                     # tensor name of an untied head, None = tied to the token table
    ignored_tensors: Tuple[str, ...] = ()   # regular expressions of tensors a checkpoint may carry unused


class ConfigError(ValueError):
    """A config.json that the architecture cannot be built from."""
