"""Parts: norms, position encodings, mixers, feed-forwards, blocks, and the model made of them.
Importing this package registers the built-in kinds."""

from . import attention, block, rmsnorm, rotary, swiglu  # noqa: F401  (registration)
from .base import (
    Block, FeedForward, Mixer, Norm, PagedKVNeed, PagedView, Part, PositionEncoding,
    ResidualStream, SlotStateNeed, StateView, StepContext,
)
from .linear import Linear
from .model import DecoderModel, build_model, tensor_decls_for_spec
from .registry import (
    build_block, build_part, register_block, register_ffn, register_mixer, register_norm,
    register_position, registered,
)

__all__ = [
    "Block", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "PagedView", "Part", "PositionEncoding",
    "ResidualStream", "SlotStateNeed", "StateView", "StepContext", "Linear", "DecoderModel",
    "build_model", "tensor_decls_for_spec", "build_block", "build_part", "register_block",
    "register_ffn", "register_mixer", "register_norm", "register_position", "registered",
]
