from . import attention, block, mlp, norm, rotary  # noqa: F401  (registers the kinds)
from .base import (Block, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, StateNeed, TensorDecl,
                   build_part, part_factory, register_part)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, straight_schedule

__all__ = ["Block", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding", "StateNeed",
           "TensorDecl", "build_part", "part_factory", "register_part", "LayerSpec", "ModelSpec", "PartSpec",
           "ScheduleEntry", "straight_schedule"]
