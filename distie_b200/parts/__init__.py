"""Parts of a block (mixer, feed-forward, norm, position encoding) and their registries."""

from .base import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    BuildContext,
    CacheNeed,
    LayerRun,
    ResidualStream,
    SeqSlice,
    StateNeed,
    TensorSpec,
    build_part,
)
from . import attention, block, mlp, norm, position  # noqa: F401  (register the built-in kinds)

__all__ = [
    "BLOCKS",
    "FEED_FORWARDS",
    "MIXERS",
    "NORMS",
    "POSITION_ENCODINGS",
    "BuildContext",
    "CacheNeed",
    "LayerRun",
    "ResidualStream",
    "SeqSlice",
    "StateNeed",
    "TensorSpec",
    "build_part",
]
