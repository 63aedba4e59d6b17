"""Sampling options and the device sampler.

The options and their meanings are QStream's `QSFSamplingConfig`
(include/qsf/sampling.h:23-29, defaults src/sampling.c:41-47): temperature below 0.01
is greedy argmax with the lowest index winning ties; otherwise logits / T, top-k,
top-p, softmax and an inverse-CDF draw; the repeat penalty works on the last 64 tokens
of prompt and output (src/engine.c:1304-1341).  The kernels are in csrc/sampling.cu.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..csrc import ops
from ..errors import QsError, QStreamError
from .rng import XorShift128Plus, request_seed

REPEAT_WINDOW = 64              # src/engine.c:1305
GREEDY_BELOW = 0.01             # src/sampling.c:230


@dataclass(frozen=True)
class SamplingConfig:
    temperature: float = 0.7
    top_k: int = 40             # 0 = off
    top_p: float = 0.9          # >= 1 = off
    repeat_penalty: float = 1.0  # <= 1 = off
    seed: int = 42

    @classmethod
    def greedy(cls) -> "SamplingConfig":
        return cls(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=0)

    @property
    def is_greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW

    def validate(self) -> None:
        if self.temperature < 0 or self.top_k < 0 or self.top_p < 0 or self.repeat_penalty <= 0:
            raise QStreamError(QsError.INVALID_INPUT, f"bad sampling options {self}")


class RequestSamplingState:
    """What sampling remembers of one request: its random stream and recent tokens."""

    def __init__(self, config: SamplingConfig, request_index: int, prompt: Sequence[int]):
        self.rng = XorShift128Plus(request_seed(config.seed, request_index))
        self.recent = list(prompt[-REPEAT_WINDOW:])     # seeded with the prompt's tail (:1309-1313)

    def push(self, token: int) -> None:
        self.recent.append(token)
        if len(self.recent) > REPEAT_WINDOW:
            del self.recent[0]


class Sampler:
    """Picks the next token of every row of a float32 logits tensor on the device."""

    def __init__(self, config: SamplingConfig, device):
        config.validate()
        self.config = config
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, states: Sequence[RequestSamplingState]) -> torch.Tensor:
        """logits [n, V] (may be changed in place by the repeat penalty); returns int32 [n]
        on the device.  The caller feeds the chosen tokens back through `state.push`."""
        cfg = self.config
        n = logits.shape[0]
        if len(states) != n:
            raise QStreamError(QsError.INVALID_INPUT, "sample: one state per logits row")
        if cfg.repeat_penalty > 1.0:
            recent = np.zeros((n, REPEAT_WINDOW), dtype=np.int32)
            count = np.zeros(n, dtype=np.int32)
            for i, st in enumerate(states):
                count[i] = len(st.recent)
                recent[i, :count[i]] = st.recent
            ops.repeat_penalty(logits, self._to_device(recent), self._to_device(count), cfg.repeat_penalty)
        if cfg.is_greedy:
            return ops.argmax(logits)
        draws = np.array([st.rng.next_float() for st in states], dtype=np.float32)
        return ops.sample(logits, cfg.temperature, cfg.top_k, cfg.top_p, self._to_device(draws))

    def _to_device(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(a)
        if self.device.type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t
