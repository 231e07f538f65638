from . import (  # noqa: F401  (registers the built-in parts)
    attention, block, connection, delta, gated_delta, gla, latent, lightning, matrix_memory, mlp, norm, rotary, routed,
    side_by_side,
)
from .base import (
    Block,
    CacheSpec,
    Connection,
    FeedForward,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    StateSpec,
    TensorSpec,
    build_part,
    part_class,
    register_part,
    registered_parts,
)

__all__ = [
    "Block", "CacheSpec", "Connection", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateSpec", "TensorSpec", "build_part", "part_class", "register_part", "registered_parts",
]
