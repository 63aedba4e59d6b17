"""How a layer's parts are wired: the arrangements.

"parallel": h = norm(x); x + mixer(h) + ffn(h), one norm, both branches read h.  The
reference engine runs the "sequential" form (x += mixer(norm_1 x); x += ffn(norm_2 x),
QStream src/engine.c:936-948,1173-1174); both are here, built from the same parts.
The residual sum is taken in 32-bit inside the last kernel of the branch that ends
the layer.
"""
from __future__ import annotations

import contextlib

from ..errors import QsError, QStreamError
from .base import Part, part_class, register


class Arrangement(Part):
    role = "arrangement"
    norm_names: tuple = ()
    # the arrangements here read nothing of the step but `decode` and, of a decode step, the number of rows
    # and the longest sequence (which a captured decode step is keyed by)
    captures_own_step = True

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, {}, runtime)
        self.mixer = parts["mixer"]
        self.ffn = parts["ffn"]
        self.norms = parts["norms"]
        position = getattr(self.mixer, "position", None)
        self.captures_any_step = self.captures_own_step and all(
            getattr(p, "captures_any_step", False)
            for p in (self.mixer, self.ffn, *self.norms.values(), *([position] if position else [])))
        missing = [n for n in self.norm_names if n not in self.norms]
        if missing:
            raise QStreamError(QsError.INVALID_MODEL,
                               f"arrangement '{spec.arrangement}' needs the norms {self.norm_names}, "
                               f"the layer lacks {missing}")

    def forward(self, x, step, cache_id):
        raise NotImplementedError

    # What a layer is made of is the arrangement's own business.  The three methods below describe the layers
    # of this library (one mixer, one feed-forward, named norms); an arrangement of another make - two mixers,
    # no feed-forward - overrides them and nothing else in the library changes.
    @classmethod
    def part_specs(cls, spec):
        """Yield (role, part spec) for every part of the layer that holds tensors."""
        yield "mixer", spec.mixer
        yield "feed_forward", spec.ffn
        for norm_spec in spec.norms.values():
            yield "norm", norm_spec

    @classmethod
    def build(cls, spec, make, runtime):
        """Build the layer; `make(role, part_spec)` builds one part with its tensors."""
        parts = {"mixer": make("mixer", spec.mixer), "ffn": make("feed_forward", spec.ffn),
                 "norms": {name: make("norm", ns) for name, ns in spec.norms.items()}}
        return cls(spec, parts, runtime)

    def cached_parts(self):
        """The parts that keep something in the cache (keys and values, or state), in the order of the
        cache entries a schedule run names for this layer: `LayerRun.cache` is one id for one such part, a
        tuple of ids for several; `forward` gets it as it stands."""
        return [self.mixer]


# A decode step runs a parallel block's two branches side by side while the keys and values its rows read
# (rows x the longest sequence x the mixer's bytes per key) stay below this share of the feed-forward's
# weights: then the attention kernels are bound by latency, beyond it by memory like the products.
# Up to 8 rows the two streams' products also share the SMs (see `forward`), which moves the limit up.
# Measured on a B200 against the one fused product, tokens a second, GPT-J-6B's sizes: up to 8 rows +1 to +8 %
# up to a share of 0.5 (1 x 2,048 keys ... 8 x 1,024), -10 % at 0.6 (8 x 1,280); 16 rows and more +6 to +7 % up
# to 0.25 (16 x 256), -5 % at 0.5 (16 x 512).  CodeGen-16B's sizes: +5 to +13 % up to 0.33, +1.5 % at 0.67.
# CodeGen-2B's: +11 to +14 % up to 0.4, -1 to -2 % at 0.8.
SIDE_BRANCH_SHARE = 0.5                 # up to SHARED_SM_ROWS rows
SIDE_BRANCH_SHARE_MANY_ROWS = 0.35      # beyond
SHARED_SM_ROWS = 8


class ParallelBlock(Arrangement):
    """x + mixer(h) + ffn(h).  When both parts end in a projection to the width (they offer
    `output_projection()` and `forward_hidden(..., out=view)`) and the weights are bfloat16, the two
    projections become one matrix product over the concatenated hidden vectors:
    x + [o | g] [W_o | W_down]^T + (b_o + b_down), with the residual added on its 32-bit accumulator.

    Decode steps over few keys are bound by the latency of the attention kernels, not by memory: there the
    feed-forward runs whole on a second stream beside the mixer (its two products stream their weights
    while the attention kernels wait for theirs), and the mixer's output product - over its columns of
    the fused matrix - adds x and the feed-forward's result on its 32-bit accumulator."""
    norm_names = ("input",)

    def __init__(self, spec, parts, runtime):
        super().__init__(spec, parts, runtime)
        self.fused_weight = None
        import torch
        fusable = all(hasattr(p, "output_projection") and hasattr(p, "forward_hidden") for p in (self.mixer, self.ffn))
        if fusable and runtime.dtype == torch.bfloat16:
            (wm, bm), (wf, bf) = self.mixer.output_projection(), self.ffn.output_projection()
            if (wm.dtype == wf.dtype == torch.bfloat16 and wm.shape[0] == wf.shape[0]
                    and wm.shape[1] % 8 == 0 and wf.shape[1] % 8 == 0):
                self.k_mixer = wm.shape[1]
                self.fused_weight = torch.cat([wm, wf], dim=1).contiguous()
                biases = [b.float() for b in (bm, bf) if b is not None]
                self.fused_bias = sum(biases[1:], biases[0]) if biases else None
                # the parts keep views of the fused matrix, so the weights are held once
                self.mixer.w_out = self.fused_weight[:, :self.k_mixer]
                self.ffn.down = self.fused_weight[:, self.k_mixer:]
                # the feed-forward's two matrices, taken as equal in size; a mixer that does not say what a key
                # costs it never runs beside the feed-forward
                self.ffn_bytes = 2 * self.ffn.down.numel() * self.fused_weight.element_size()
                self.key_bytes = getattr(self.mixer, "cache_bytes_per_key", None)

    def forward(self, x, step, cache_id):
        h = self.norms["input"].forward(x)
        if self.fused_weight is None:
            a = self.mixer.forward(h, step, cache_id)
            return self.ffn.forward(h, step, residuals=(x, a))
        import torch
        from .linear import linear
        b = step.batch
        side = getattr(step, "side_stream", None)
        share = SIDE_BRANCH_SHARE if h.shape[0] <= SHARED_SM_ROWS else SIDE_BRANCH_SHARE_MANY_ROWS
        if (side is not None and b.decode and self.key_bytes is not None
                and h.shape[0] * (b.max_total or step.cache.max_context) * self.key_bytes <= share * self.ffn_bytes):
            from .linear import beside_main_stream, shared_sms
            # m is read on the main stream, so it comes from the main stream's memory; g lives on the second stream only
            m = torch.empty((h.shape[0], self.fused_weight.shape[0]), dtype=h.dtype, device=h.device)
            # the two streams' products side by side on every SM (up to 8 rows: +1 to +5 % tokens a second; 16 rows: -1 %)
            with shared_sms() if h.shape[0] <= SHARED_SM_ROWS else contextlib.nullcontext():
                with beside_main_stream(side, h.device) as beside:
                    g = self.ffn.forward_hidden(h, step)
                    linear(g, self.fused_weight[:, self.k_mixer:], self.fused_bias, out=m)
                o = self.mixer.forward_hidden(h, step, cache_id)
                beside.join()
                return linear(o, self.fused_weight[:, :self.k_mixer], None, residuals=(x, m))
        hidden = torch.empty((h.shape[0], self.fused_weight.shape[1]), dtype=h.dtype, device=h.device)
        self.mixer.forward_hidden(h, step, cache_id, out=hidden[:, :self.k_mixer])
        self.ffn.forward_hidden(h, step, out=hidden[:, self.k_mixer:])
        return linear(hidden, self.fused_weight, self.fused_bias, residuals=(x,))


class SequentialBlock(Arrangement):
    norm_names = ("input", "post_mixer")

    def forward(self, x, step, cache_id):
        x = self.mixer.forward(self.norms["input"].forward(x), step, cache_id, residuals=(x,))
        return self.ffn.forward(self.norms["post_mixer"].forward(x), step, residuals=(x,))


register("arrangement", "parallel", ParallelBlock)
register("arrangement", "sequential", SequentialBlock)


def build_block(spec, tensors_of, runtime):
    """Build one layer from its `BlockSpec`.  `tensors_of(part_spec, declaration)` returns
    the part's tensors by the part's own names."""
    def make(role, part_spec):
        cls = part_class(role, part_spec.kind)
        return cls(part_spec, tensors_of(part_spec, cls.declare(part_spec)), runtime)

    return part_class("arrangement", spec.arrangement).build(spec, make, runtime)
