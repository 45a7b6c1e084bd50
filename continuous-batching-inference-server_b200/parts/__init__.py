from .base import (Block, CacheNeed, Delta, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   make_block, make_feed_forward, make_mixer, make_norm, make_position, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import attention, blocks, dense, layernorm, positions  # noqa: F401  (register the built-in kinds)
from .attention import PagedAttention
from .blocks import PreNormBlock
from .dense import DenseFeedForward
from .layernorm import LayerNorm
from .positions import LearnedPositions, NoPositions
