"""What every part is, and the registries that find a part by its spec's `kind`.

A part is built from a spec (sizes, constants, tensor names) and its tensors; it does
not know which model it sits in.  To add a part: subclass the role's base class,
implement `declare` and `forward`, and `register(role, kind, cls)`; a spec object whose
`kind` names it can then appear in any `ModelSpec`.

Roles and what each must offer:

norm          forward(x) -> y
position      apply(q, k, step, n_heads, n_kv_heads, head_dim): change q [T, H*dh] and k
              in place, from step.batch.tok_pos; a rotary kind may instead offer
              `fused_table` and `rotary_dim`, which attention fuses with its cache write
mixer         kv_need() -> KvNeed | None; state_need() -> StateNeed | None;
              forward(h, step, cache_id, residuals=()) -> [T, width]
feed_forward  forward(h, step, residuals=()) -> [T, width]
arrangement   forward(x, step, cache_id) -> x'; built from the block's parts
embedding     forward(step) -> x [T, width] in the activations' type, from step.batch.tokens (and, for
              position tables, step.batch.tok_pos)
head          forward(rows) -> float32 logits [n, vocab] of the wanted rows (already normalised by the
              model's final norm, if it has one); `tie(embedding)` if its spec says `tied`

`residuals` are tensors to be added to the part's output, in 32-bit, before the one
rounding to the storage type; a part that cannot do that in its last kernel calls
`add_residuals`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from ..cache import KvNeed, StateNeed
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl

_REGISTRY: dict[tuple[str, str], type] = {}
ROLES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")


def register(role: str, kind: str, cls: type) -> None:
    if role not in ROLES:
        raise QStreamError(QsError.INVALID_INPUT, f"unknown part role '{role}' (roles: {ROLES})")
    _REGISTRY[(role, kind)] = cls


def part_class(role: str, kind: str) -> type:
    try:
        return _REGISTRY[(role, kind)]
    except KeyError:
        known = sorted(k for r, k in _REGISTRY if r == role)
        raise QStreamError(QsError.UNSUPPORTED_ARCH,
                           f"no {role} part of kind '{kind}' is registered (known: {known})") from None


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision the parts compute."""
    dtype: torch.dtype                  # storage type of activations: bfloat16 or float32
    device: torch.device


class Part:
    role = ""
    # True if `forward` takes everything that changes from step to step (which tokens, which sequences, how
    # many of each) from the device tensors of `step.batch` and the cache, never from the batch's host lists:
    # a step with prompts can then be captured once per padded size and replayed.  Decode steps are captured
    # for every part; a part that leaves this False only makes steps with prompts run kernel by kernel.
    captures_any_step = False

    @classmethod
    def declare(cls, spec) -> Mapping[str, TensorDecl]:
        """The part's tensors by its own names; `spec.names` maps them to the file's."""
        return {}

    def __init__(self, spec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.runtime = runtime


def add_residuals(out: torch.Tensor, residuals) -> torch.Tensor:
    from ..csrc import ops
    residuals = [r for r in residuals if r is not None]
    if not residuals:
        return out
    if len(residuals) > 2:
        raise QStreamError(QsError.INVALID_INPUT, "at most two residuals")
    return ops.add(out, residuals[0], residuals[1] if len(residuals) > 1 else None)


class Norm(Part):
    role = "norm"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    role = "position"
    fused_table: Optional[torch.Tensor] = None

    def apply(self, q, k, step, n_heads, n_kv_heads, head_dim) -> None:
        raise NotImplementedError


class Mixer(Part):
    role = "mixer"

    def kv_need(self) -> Optional[KvNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h, step, cache_id: int, residuals=()) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    role = "embedding"

    def forward(self, step) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    role = "head"

    def tie(self, embedding: "Embedding") -> None:
        """Take the embedding's table as the weight (specs with `tied`)."""
        raise NotImplementedError

    def forward(self, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"

    def forward(self, h, step, residuals=()) -> torch.Tensor:
        raise NotImplementedError
