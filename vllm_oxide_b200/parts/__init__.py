from .base import (NO_ROTATION, Block, CachePlane, CacheSpec, FeedForward, Mixer, Norm, Part, PartSpec, PositionEncoding,
                   RotationRule, StateSpec, Workspace, build_part, known_parts, register_part)
from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .linear import linear

__all__ = ["NO_ROTATION", "Block", "CachePlane", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PartSpec",
           "PositionEncoding", "RotationRule", "StateSpec", "Workspace", "build_part", "known_parts", "register_part",
           "linear"]
