"""Model parts; importing the package registers the implementations it ships."""
from .base import (
    Block,
    BuildContext,
    Embedding,
    FeedForward,
    Head,
    KVRequest,
    Mixer,
    Norm,
    ParamSpec,
    Part,
    PartSpec,
    PositionEncoding,
    StateRequest,
    build_part,
    register_part,
    registered_parts,
    unregister_part,
)
from . import norms, rope, attention, mlp, block, ends  # noqa: F401  (registration)
from .model import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry

__all__ = [
    "Block", "BuildContext", "Embedding", "FeedForward", "Head", "KVRequest", "Mixer", "Norm", "ParamSpec", "Part",
    "PartSpec", "PositionEncoding", "StateRequest", "build_part", "register_part",
    "registered_parts", "unregister_part", "DecoderModel", "LayerSpec", "ModelSpec", "ScheduleEntry",
]
