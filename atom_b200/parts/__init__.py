"""Parts a model is put together from; importing the package registers the built-in ones."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, Workspace
from .registry import build, lookup, register
from .spec import CacheNeed, LayerSpec, ModelSpec, ParamSpec, PartSpec, RunEntry

__all__ = [
    "CacheNeed", "FeedForward", "LayerSpec", "Mixer", "ModelSpec", "Norm", "ParamSpec", "Part",
    "PartSpec", "PositionEncoding", "RunEntry", "Runtime", "Workspace", "build", "lookup", "register",
]
