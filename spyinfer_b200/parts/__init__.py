"""The parts a model is put together from, and their registry."""
from .base import Block, BuildContext, FeedForward, Mixer, Norm, NormedDelta, Part, PositionEncoding, ScaledParts
from .block import PreNormBlock, ScaledPreNormBlock, build_block, register_block
from .registry import build_part, known_parts, register_part
from . import attention, conv, embedding, experts, feedforward, norm, parallel, position, recurrent, scan  # noqa: F401  (register the built-in parts)
from .linear import Linear

__all__ = ["Block", "BuildContext", "FeedForward", "Mixer", "Norm", "NormedDelta", "Part", "PositionEncoding", "PreNormBlock", "ScaledParts", "ScaledPreNormBlock", "build_block",
           "register_block", "build_part", "known_parts", "register_part", "Linear"]
