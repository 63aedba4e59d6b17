"""Output head: logits = rows W^T + b in 32-bit, for the wanted rows only (QStream src/engine.c:1237-1241
runs it for every token and drops the bias); `tied` takes the embedding table as W (:1200-1236)."""
from __future__ import annotations

import torch

from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import Head, register
from .linear import linear


class LinearHead(Head):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {} if spec.tied else {"weight": TensorDecl((spec.vocab_size, spec.width))}
        if spec.bias:
            d["bias"] = TensorDecl((spec.vocab_size,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = None if spec.tied else tensors["weight"]
        self.bias = tensors["bias"] if spec.bias else None

    def tie(self, embedding):
        weight = getattr(embedding, "weight", None)
        if weight is None or tuple(weight.shape) != (self.spec.vocab_size, self.spec.width):
            raise QStreamError(QsError.INVALID_MODEL, "a tied head needs an embedding with a [vocab, width] table")
        self.weight = weight

    def forward(self, rows):
        return linear(rows, self.weight, self.bias, out_dtype=torch.float32)


register("head", "lm_head", LinearHead)
