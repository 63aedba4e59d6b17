"""LayerNorm with weight and optional bias (QStream src/kernels_scalar.c:151-171)."""
from __future__ import annotations

from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Norm, register


class LayerNorm(Norm):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"weight": TensorDecl((spec.size,), "norm_weight")}
        if spec.bias:
            d["bias"] = TensorDecl((spec.size,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias") if spec.bias else None
        self.eps = float(spec.eps)

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps, settled=True)     # a model's weights are old


register("norm", "layernorm", LayerNorm)
