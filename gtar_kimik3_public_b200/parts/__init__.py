"""Parts of a model: norms, position encodings, mixers, feed-forwards, blocks, embedding and head.
Importing the package registers the built-in parts."""

from . import attention, block, delta_rule, embedding, experts, latent_attention, mlp, norms, rope, wide_norm_attention  # noqa: F401
from .base import (  # noqa: F401
    Block, FeedForward, KVRequest, Mixer, Norm, Part, PositionEncoding, RowsRequest, StateRequest, StepContext, TensorSpec,
    build_part, known_parts, register_part,
)
