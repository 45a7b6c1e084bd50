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
from typing import Any, Dict, List, Optional, Tuple, Union


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
    """``token_embedding`` and ``head`` are parts like the others: a ``PartSpec`` of the embedding
    registry (built in: "token_table" with ``tensor`` and ``multiplier``) and of the head registry
    (built in: "linear" with ``tensor`` (None: tied to the embedding's table), ``bias`` (a tensor
    name or None), ``logit_scale`` and ``soft_cap``).  As a shorthand a tensor name stands for a
    plain token table, and a tensor name or None for a plain linear head.  ``final_norm`` may be
    ``PartSpec("none", {"width": w})`` for a model that has none."""
    width: int
    vocab_size: int
    max_positions: int
    token_embedding: Union[str, PartSpec]   # the input: token rows (PartSpec of the embedding registry)
    position: PartSpec                      # position encoding at the input (or "none")
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]               # layer indices in running order
    final_norm: PartSpec
    final_norm_prefix: str
    head: Union[None, str, PartSpec]        # the output: logits from the last norm's rows (PartSpec of the head registry)
    ignored_tensors: Tuple[str, ...] = ()   # regular expressions of tensors a checkpoint may carry unused

    def embedding_spec(self) -> PartSpec:
        if isinstance(self.token_embedding, PartSpec):
            return self.token_embedding
        return PartSpec("token_table", {"vocab_size": self.vocab_size, "width": self.width,
                                        "tensor": self.token_embedding})

    def head_spec(self) -> PartSpec:
        if isinstance(self.head, PartSpec):
            return self.head
        return PartSpec("linear", {"vocab_size": self.vocab_size, "width": self.width, "tensor": self.head})


class ConfigError(ValueError):
    """A config.json that the architecture cannot be built from."""
