from . import attention, block, embedding, feed_forward, norm, rotary  # noqa: F401  (register the built-in parts)
from .base import HostBatch, Part, RunView, StepContext, Stream, Workspace, plan_key_of
from .linear import Linear
from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, register_block,
                       register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                       register_position)

__all__ = ["Part", "RunView", "StepContext", "Stream", "Workspace", "Linear", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS",
           "HEADS", "MIXERS", "NORMS", "POSITIONS", "register_block", "register_embedding", "register_feed_forward",
           "register_head", "register_mixer", "register_norm", "register_position"]
