from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv,
                   FeedForward, Mixer, Norm, Part, PositionEncoding, build_part, register_block, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm, register_position_encoding)
from .context import GroupContext, KVCacheView, StateCacheView, StepContext, Workspace
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .model import DecoderModel, expected_tensors

__all__ = [n for n in dir() if not n.startswith("_")]
