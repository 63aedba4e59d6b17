"""Dense feed-forward: up projection + bias, activation, down projection + bias
(QStream src/engine.c:1150-1170; the activation's tanh form src/kernels_scalar.c:135-142,
the erf form is GPT-J's 'gelu').  The activation runs on the 32-bit accumulator of the
up projection; residuals are added on the accumulator of the down projection."""
from __future__ import annotations

from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import FeedForward, register
from .linear import linear


class Mlp(FeedForward):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        d = {"up": TensorDecl((spec.inner, spec.width)), "down": TensorDecl((spec.width, spec.inner))}
        if spec.bias:
            d["up_bias"] = TensorDecl((spec.inner,), "bias")
            d["down_bias"] = TensorDecl((spec.width,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.activation not in ops.ACTIVATIONS:
            raise QStreamError(QsError.UNSUPPORTED_ARCH, f"activation '{spec.activation}' has no kernel")
        self.up, self.down = tensors["up"], tensors["down"]
        self.up_bias = tensors.get("up_bias") if spec.bias else None
        self.down_bias = tensors.get("down_bias") if spec.bias else None

    def forward(self, h, step, residuals=()):
        g = self.forward_hidden(h, step)
        return linear(g, self.down, self.down_bias, residuals=residuals)

    # See Attention.output_projection: the same pair for a parallel block that fuses both projections.
    def output_projection(self):
        return self.down, self.down_bias

    def forward_hidden(self, h, step, out=None):
        """The activated up projection: [T, inner], written to `out` if given."""
        return linear(h, self.up, self.up_bias, activation=self.spec.activation, out=out)


register("feed_forward", "mlp", Mlp)
