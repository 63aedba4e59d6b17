"""Token embedding: x[t] = table[token[t]], no position term, no scale (QStream src/engine.c:710-765)."""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Embedding, register


class TokenEmbedding(Embedding):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.vocab_size, spec.width))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]

    def forward(self, step):
        return ops.embedding(self.weight, step.batch.tokens, self.runtime.dtype)


register("embedding", "embedding", TokenEmbedding)
