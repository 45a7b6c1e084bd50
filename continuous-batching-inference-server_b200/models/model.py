"""The model: layers put together from registered parts as a ``ModelSpec`` says.

The reference hard-wires one model in ``TransformerRunner::forward_step``
(src/transformer.cpp:65-93): embed, L times (LN, QKV, scatter, attention, O + residual,
LN, FC1, GELU, FC2 + residual), final LN, LM head on all rows.  Here the same order comes
out of the spec's layer list and schedule; the head runs only on the rows whose logits
are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import ModelSpec, load_config
from ..kernels import ops
from ..parts import (make_block, make_embedding, make_feed_forward, make_head, make_mixer, make_norm, make_position)
from ..weights import TensorDecl, check_tensors, read_model_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} is not one of bfloat16, float32")
    return _DTYPES[dtype]


class Layer:
    """A block with its parts and the tensor-name prefix of its weights."""

    def __init__(self, spec, index: int):
        self.spec, self.index = spec, index
        extra = {"own_kv": False} if spec.cache_source is not None and spec.mixer.kind == "attention" else {}
        self.mixer = make_mixer(spec.mixer, **extra)
        self.feed_forward = make_feed_forward(spec.feed_forward)
        self.norm_mixer = make_norm(spec.norm_mixer)
        self.norm_feed_forward = make_norm(spec.norm_feed_forward)
        self.block = make_block(spec.arrangement, self.mixer, self.feed_forward, self.norm_mixer,
                                self.norm_feed_forward)
        self.norm_names = tuple(spec.norm_prefixes)

    def parts(self):
        p = self.spec.prefix
        return [(p, self.mixer), (p, self.feed_forward), (p + self.norm_names[0], self.norm_mixer),
                (p + self.norm_names[1], self.norm_feed_forward)]


class Model:
    """Embedding, layers in the order of the schedule, final norm and head: each a part built from its
    ``PartSpec`` through the registries.  This class decides nothing about the architecture."""

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = make_embedding(spec.embedding_spec())
        self.position = make_position(spec.position)
        self.layers: List[Layer] = [Layer(ls, i) for i, ls in enumerate(spec.layers)]
        for i in spec.schedule:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"schedule names layer {i}; the model has {len(self.layers)} layers")
        for ls in spec.layers:
            if ls.cache_source is not None and not 0 <= ls.cache_source < len(self.layers):
                raise ValueError(f"layer {ls.prefix!r} reads the cache of layer {ls.cache_source}, which does not exist")
        self.final_norm = make_norm(spec.final_norm)
        self.head_part = make_head(spec.head_spec())
        self.dtype: Optional[torch.dtype] = None
        self.device = None

    @property
    def token_table(self) -> Optional[torch.Tensor]:
        return self.embedding.table

    @property
    def head(self) -> Optional[torch.Tensor]:
        """The head's matrix ``[vocab, width]`` (the token table itself when the head is tied)."""
        return getattr(self.head_part, "weight", None)

    def all_parts(self):
        """(tensor-name prefix, part) of every part of the model, in loading order."""
        out = [("", self.embedding), ("", self.position)]
        for layer in self.layers:
            out += layer.parts()
        return out + [(self.spec.final_norm_prefix, self.final_norm), ("", self.head_part)]

    # ---- weights -------------------------------------------------------
    def declared(self) -> List[TensorDecl]:
        decls = []
        for prefix, part in self.all_parts():
            decls += part.tensors(prefix)
        return decls

    def load(self, tensors: Dict[str, torch.Tensor], dtype, device="cuda", where="weights") -> "Model":
        dtype = resolve_dtype(dtype)
        check_tensors(self.declared(), tensors, self.spec.ignored_tensors, where)
        self.dtype, self.device = dtype, torch.device(device)
        for prefix, part in self.all_parts():
            if part is self.head_part:
                part.tie(self.embedding)
            part.load(prefix, tensors, dtype, device)
        self.register_weight_order()
        return self

    def register_weight_order(self) -> None:
        """The order in which a step reads the big matrices, for prefetching one ahead (bfloat16 on a GPU)."""
        if self.dtype != torch.bfloat16 or self.device.type != "cuda":
            return
        order = []
        for li in self.spec.schedule:
            layer = self.layers[li]
            order += layer.mixer.streamed_weights() + layer.feed_forward.streamed_weights()
        ops.add_weight_order(order + self.head_part.streamed_weights())

    def weight_bytes(self) -> int:
        """Bytes of all weights a step reads (each once; a tied head counts once; of the embedding's and the
        position encoding's tables a step reads single rows, which do not count)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for _, part in self.all_parts():
            if part is self.embedding or part is self.position:
                continue
            for v in vars(part).values():
                add(v)
        return total

    # ---- one step ------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Logits (float32 ``[R, vocab]``) at ``ctx.logit_rows`` for the rows of this step."""
        x = self.embedding.forward(ctx, self.position)
        pending = None
        sched = self.spec.schedule
        i = 0
        while i < len(sched):
            li = sched[i]
            block, cache, state = self.layers[li].block, ctx.layer_cache(li), ctx.layer_state(li)
            key = block.run_key(ctx, cache, state)
            if key is None:
                pending = block.forward(ctx, x, pending, cache, state)
                i += 1
                continue
            # a run of consecutive layers whose blocks can go together (for instance one kernel for all of them)
            run = [(block, cache, state)]
            j = i + 1
            while j < len(sched):
                nxt = self.layers[sched[j]].block
                c2, s2 = ctx.layer_cache(sched[j]), ctx.layer_state(sched[j])
                if type(nxt) is not type(block) or nxt.run_key(ctx, c2, s2) != key:
                    break
                run.append((nxt, c2, s2))
                j += 1
            pending = type(block).forward_run(ctx, [r[0] for r in run], x, pending, [r[1] for r in run], [r[2] for r in run])
            i = j
        return self.head_part.forward(ctx, x, pending, self.final_norm)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    return Model(spec).declared()


def load_model(folder: str, dtype="bfloat16", device="cuda") -> Model:
    """Model of ``folder`` (config.json chooses the architecture; model.safetensors by tensor name)."""
    config = load_config(folder)
    model = Model(config.model_spec())
    model.config = config
    model.load(read_model_tensors(folder), dtype, device, where=f"{folder}/model.safetensors")
    return model
