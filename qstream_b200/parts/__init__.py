"""The parts a model is put together from, and their registries."""
from .base import (Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Runtime, add_residuals,
                   part_class, register)
from . import norm, rotary, attention, mlp, block, embedding, head      # register the built-in kinds
from .linear import linear
from .block import build_block

__all__ = ["Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "add_residuals",
           "part_class", "register", "linear", "build_block"]
