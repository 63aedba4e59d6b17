"""Rotary position encoding on the first `rotary_dim` dims of each head, pairs (i, i+1).

theta(pos, i) = pos * base^(-i / rotary_dim), i = 0, 2, ...; (a, b) -> (a cos - b sin,
a sin + b cos): QStream src/engine.c:205-234, which rotates the whole head; here the
rotated width is a parameter.  The angles are computed in float64 and the table
[max_positions, rotary_dim/2, (cos, sin)] is kept in float32.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import PositionEncoding, register


class RotaryInterleaved(PositionEncoding):
    captures_any_step = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec.rotary_dim)
        i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(float(spec.base), dtype=torch.float64), -i / max(self.rotary_dim, 1))
        ang = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * freq[None, :]
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32)
        # Attention fuses the rotation with its cache write when a position part offers this.
        self.fused_table = table.contiguous().to(runtime.device) if self.rotary_dim > 0 else None

    def apply(self, q, k, step, n_heads, n_kv_heads, head_dim):
        """Rotate q and k in place (no cache write); for mixers that do not fuse the rotation with
        their cache write.  A rotary width of 0 rotates nothing."""
        if self.fused_table is None:
            return
        b = step.batch
        for x, heads in ((q, n_heads), (k, n_kv_heads)):
            if x is not None and heads > 0:
                ops.rope_store(x, None, None, heads, 0, head_dim, self.rotary_dim, self.fused_table,
                               b.tok_slot, b.tok_pos, None, 64, None, None, step.status, settled=True)


register("position", "rotary_interleaved", RotaryInterleaved)
