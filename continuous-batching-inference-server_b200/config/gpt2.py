"""Typed configuration of TinyGPT / GPT-2 folders.

Every size and constant comes from ``config.json``; nothing is fixed in code.
The reference fixes the same quantities at compile time (include/config.hpp:5-21,
mirrored in python/model.py:12-18) with the literal eps of kernels/elementwise.cu:51.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec

_ACTIVATIONS = {"gelu": "gelu_erf", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh"}


def _need_int(d: Dict[str, Any], key: str, minimum: int = 1) -> int:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


@dataclass(frozen=True)
class GPT2Config:
    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int
    n_positions: int
    vocab_size: int
    activation_function: str
    layer_norm_epsilon: float
    tie_word_embeddings: bool
    architecture: str = "GPT2LMHeadModel"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GPT2Config":
        n_embd = _need_int(d, "n_embd")
        n_head = _need_int(d, "n_head")
        if n_embd % n_head:
            raise ConfigError(f"config.json: n_embd={n_embd} is not a multiple of n_head={n_head}")
        n_inner = d.get("n_inner")
        if n_inner is None:
            n_inner = 4 * n_embd            # GPT-2 folders leave it null for 4*n_embd
        elif isinstance(n_inner, bool) or not isinstance(n_inner, int) or n_inner < 1:
            raise ConfigError(f"config.json: 'n_inner' must be a positive integer or null, got {n_inner!r}")
        act = d.get("activation_function", "gelu_new")
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: activation_function {act!r} is not one of {sorted(_ACTIVATIONS)}")
        eps = d.get("layer_norm_epsilon", 1e-5)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not eps > 0:
            raise ConfigError(f"config.json: 'layer_norm_epsilon' must be a positive number, got {eps!r}")
        tie = d.get("tie_word_embeddings", True)
        if not isinstance(tie, bool):
            raise ConfigError(f"config.json: 'tie_word_embeddings' must be true or false, got {tie!r}")
        arch = (d.get("architectures") or [None])[0] or d.get("model_type") or "GPT2LMHeadModel"
        return cls(n_layer=_need_int(d, "n_layer"), n_embd=n_embd, n_head=n_head, n_inner=n_inner,
                   n_positions=_need_int(d, "n_positions"), vocab_size=_need_int(d, "vocab_size"),
                   activation_function=act, layer_norm_epsilon=float(eps),
                   tie_word_embeddings=tie, architecture=str(arch))

    def to_dict(self) -> Dict[str, Any]:
        return {"architectures": [self.architecture], "model_type": "gpt2",
                "n_layer": self.n_layer, "n_embd": self.n_embd, "n_head": self.n_head,
                "n_inner": self.n_inner, "n_positions": self.n_positions,
                "vocab_size": self.vocab_size, "activation_function": self.activation_function,
                "layer_norm_epsilon": self.layer_norm_epsilon,
                "tie_word_embeddings": self.tie_word_embeddings}

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def model_spec(self) -> ModelSpec:
        """Pre-LayerNorm blocks of causal attention and a GELU feed-forward
        (python/model.py:48-51), learned positions added at the input
        (python/model.py:65-66), a last LayerNorm and a head without bias
        (python/model.py:69-70)."""
        d, hd = self.n_embd, self.head_dim
        norm = PartSpec("layernorm", {"width": d, "eps": self.layer_norm_epsilon})
        mixer = PartSpec("attention", {"width": d, "n_head": self.n_head, "n_kv_head": self.n_head,
                                       "head_dim": hd, "scale": hd ** -0.5, "window": 0})
        ffn = PartSpec("dense", {"width": d, "inner": self.n_inner,
                                 "activation": _ACTIVATIONS[self.activation_function]})
        layers = tuple(LayerSpec(prefix=f"h.{i}.", arrangement="pre_norm", mixer=mixer, feed_forward=ffn,
                                 norm_mixer=norm, norm_feed_forward=norm) for i in range(self.n_layer))
        return ModelSpec(width=d, vocab_size=self.vocab_size, max_positions=self.n_positions,
                         token_embedding="wte.weight",
                         position=PartSpec("learned", {"width": d, "n_positions": self.n_positions,
                                                       "tensor": "wpe.weight"}),
                         layers=layers, schedule=tuple(range(self.n_layer)),
                         final_norm=norm, final_norm_prefix="ln_f.",
                         head=None if self.tie_word_embeddings else "lm_head.weight",
                         # buffers that GPT-2 checkpoints carry and no formula uses
                         ignored_tensors=(r"h\.\d+\.attn\.(masked_)?bias$",)
                         + ((r"lm_head\.weight$",) if self.tie_word_embeddings else ()))
