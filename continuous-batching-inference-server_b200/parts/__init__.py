from .base import (AttentionLike, Block, CacheArray, CacheNeed, Delta, Embedding, FeedForward, Head, Mixer, Norm, Part,
                   PositionEncoding, StateNeed, make_block, make_embedding, make_feed_forward, make_head, make_mixer,
                   make_norm, make_position, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position)
from . import attention, blocks, dense, embedding, head, layernorm, positions  # noqa: F401  (register the built-in kinds)
from .attention import PagedAttention
from .blocks import PreNormBlock
from .dense import DenseFeedForward
from .embedding import TokenTable
from .head import LinearHead
from .layernorm import LayerNorm, NoNorm
from .positions import LearnedPositions, NoPositions
