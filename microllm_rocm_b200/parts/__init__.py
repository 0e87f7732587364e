from .base import (Runtime, WeightSpec, PagedKVNeed, FixedStateNeed, PagedKVView, StateView, StepContext, Part, Norm,
                   PositionEncoding, RotaryTable, Mixer, FeedForward, Block, NORMS, POSITION_ENCODINGS, MIXERS,
                   FEED_FORWARDS, BLOCKS, EMBEDDINGS, HEADS, register_norm, register_position_encoding,
                   register_mixer, register_feed_forward, register_block, register_embedding, register_head)
from . import norm, rotary, attention, mlp, embedding, block  # noqa: F401  (register the built-in kinds)
from .build import Model, build_model
