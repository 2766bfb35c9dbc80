from .base import (
    DeferredProduct, KVRequest, ResidualStream, Runtime, StateRequest, Workspace, part_class,
    register_block, register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
    register_position,
)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .linear import Linear

__all__ = [
    "DeferredProduct", "KVRequest", "Linear", "ResidualStream", "Runtime", "StateRequest", "Workspace", "part_class",
    "register_block", "register_embedding", "register_feed_forward", "register_head", "register_mixer",
    "register_norm", "register_position",
]
