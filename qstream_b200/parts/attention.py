"""Causal softmax attention over the sequence's paged cache.

q/k/v projections (QStream src/engine.c:841-867), position encoding on q and k before
the keys are kept (:871-880), scores q.k / sqrt(dh) over the keys up to the token's own
position, softmax, weighted sum of values (:888-922), heads concatenated, output
projection (:926-934).  Query head j reads key head j // (H / Hkv) (:884,889).  The
three projections are one matrix product over the concatenated weights.
"""
from __future__ import annotations

import torch

from ..cache import KvNeed
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import Mixer, part_class, register
from .linear import linear


class Attention(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hq, hkv = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        d = {"q": TensorDecl((hq, spec.width)), "out": TensorDecl((spec.width, hq))}
        if not spec.shares_cache:
            d["k"] = TensorDecl((hkv, spec.width))
            d["v"] = TensorDecl((hkv, spec.width))
        if spec.qkv_bias:
            d["q_bias"] = TensorDecl((hq,), "bias")
            if not spec.shares_cache:
                d["k_bias"] = TensorDecl((hkv,), "bias")
                d["v_bias"] = TensorDecl((hkv,), "bias")
        if spec.out_bias:
            d["out_bias"] = TensorDecl((spec.width,), "bias")
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_kv_heads:
            raise QStreamError(QsError.INVALID_MODEL,
                               f"{spec.n_heads} query heads are no multiple of {spec.n_kv_heads} key heads")
        if spec.head_dim % 16:
            raise QStreamError(QsError.UNSUPPORTED_ARCH,
                               f"attention kernels take head sizes in steps of 16, not {spec.head_dim}")
        names = ["q"] if spec.shares_cache else ["q", "k", "v"]
        mats = [tensors[n] for n in names]
        if len({m.dtype for m in mats}) != 1:
            raise QStreamError(QsError.INVALID_MODEL, "q/k/v projections are stored in different types")
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.b_qkv = None
        if spec.qkv_bias:
            self.b_qkv = torch.cat([tensors[n + "_bias"].float() for n in names]).contiguous()
        self.w_out = tensors["out"]
        self.b_out = tensors.get("out_bias") if spec.out_bias else None
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position.kind)(spec.position, {}, runtime)

    @property
    def cache_bytes_per_key(self) -> int:
        """What one key of a sequence costs a decode step to read: its key and its value, all heads."""
        return 2 * self.spec.n_kv_heads * self.spec.head_dim * self.w_qkv.element_size()

    def kv_need(self):
        if self.spec.shares_cache:
            return None
        s = self.spec
        return KvNeed(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window)

    def forward(self, h, step, cache_id, residuals=()):
        o = self.forward_hidden(h, step, cache_id)
        return linear(o, self.w_out, self.b_out, residuals=residuals)

    # A parallel block may fuse this part's output projection with the feed-forward's down projection:
    # it takes the projection from `output_projection()` and calls `forward_hidden` with a view to fill.
    def output_projection(self):
        return self.w_out, self.b_out

    def forward_hidden(self, h, step, cache_id, out=None):
        """Everything before the output projection: [T, n_heads * head_dim], written to `out` if given."""
        s = self.spec
        b = step.batch
        view = step.kv(cache_id)
        hq, hkv = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
        qkv = linear(h, self.w_qkv, self.b_qkv)
        q = qkv[:, :hq]
        table = getattr(self.position, "fused_table", None) if self.position is not None else None
        if s.shares_cache:
            if self.position is not None:
                if table is None:
                    self.position.apply(q, None, step, s.n_heads, s.n_kv_heads, s.head_dim)
                else:                                   # rotate q only: no keys of its own
                    ops.rope_store(q, None, None, s.n_heads, 0, s.head_dim, self.position.rotary_dim, table,
                                   b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, None, None,
                                   step.status, settled=True)
        else:
            k = qkv[:, hq:hq + hkv]
            v = qkv[:, hq + hkv:]
            if self.position is not None and table is None:
                self.position.apply(q, k, step, s.n_heads, s.n_kv_heads, s.head_dim)
            ops.rope_store(q, k, v, s.n_heads, s.n_kv_heads, s.head_dim,
                           getattr(self.position, "rotary_dim", 0) if table is not None else 0, table,
                           b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, view.k, view.v,
                           step.status, settled=True)     # a step's slots, positions and pages arrive before its first kernel
        return attend(q, s, step, view, out)


def attend(q, spec, step, view, out=None):
    """Pick the attention kernel for this step: decode and prefill have their own
    bfloat16 kernels; the generic kernel takes every other case."""
    b = step.batch
    if q.dtype == torch.bfloat16:
        from ..csrc import attention_bf16
        done = attention_bf16.attend(q, spec, step, view, out)
        if done is not None:
            return done
    return ops.attention(q, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.scale, spec.window,
                         b.tok_slot, b.tok_pos, view.page_table, view.page_tokens, view.k, view.v,
                         step.status, out=out)


register("mixer", "attention", Attention)
